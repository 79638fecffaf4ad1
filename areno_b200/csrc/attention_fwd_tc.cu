// Variable-length causal attention forward on the 5th-generation tensor cores (head_dim 64 or 128, GQA).
//
// One CTA per (128 query rows of one sequence, query head), ten warps:
//   warp 0      TMA producer: Q once, then K and V tiles of 128 keys through two-stage rings
//   warp 1      MMA issuer:   S = Q K^T  into TMEM (two S buffers), O_tile = P V into TMEM
//   warps 2-9   softmax:      two threads per query row (64 keys / 64 output channels each).  A thread reads
//                             its part of the S row from TMEM (tcgen05.ld), applies
//                             mask / running max / exp2, writes P (bf16) into a 128-byte-swizzled K-major
//                             shared tile that the second MMA consumes, then reads O_tile back from TMEM and
//                             folds it into the running output kept in registers (o = o * corr + O_tile).
// S of tile i+1 is issued before P V of tile i, so the tensor pipe works on the next scores while the
// softmax warps are busy, and O_tile is double-buffered so that the fold of tile i happens after P of tile
// i+1 has been handed over (the P V latency is not on the softmax warps' critical path).
// TMEM: columns [0,128) and [128,256) hold the two S buffers, [256,384) and [384,512) the two O_tile buffers.
// Shared memory at head_dim 128: Q 32 KB, K 2 x 32 KB, V 2 x 32 KB, P 32 KB (128-byte swizzle, 1024-byte aligned).
//
// Every mbarrier wait is bounded (common.cuh); on expiry the CTA records a status word, lets copies in
// flight land, frees its TMEM and returns.  No multicast loads.
//
// Same contract as areno_attn_fwd (attention_fwd.cu) for head_dim 64 / 128 without a sliding window; role of
// flash_attn_varlen_func in the reference (areno/engine/layers/attention_backend/train.py:135-141).
#include "attention_common.cuh"
#include "launch.h"

namespace areno {

constexpr int kTcBM = 128;      // query rows per CTA
constexpr int kTcBN = 128;      // keys per tile
constexpr uint32_t kTcPTile = 128 * 128 * 2;  // bytes of the 128 x 128 bf16 P tile

struct AttnTcParams {
  __nv_bfloat16* out;
  float* lse;
  const int* cu_q;
  const int* cu_k;
  const int* tile_prefix;  // 128-row query tiles per sequence (prefix sum)
  int num_seqs, hq, hkv;
  long long o_stride;
  float scale;
  int causal;
  int* status;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int kTcD>   // head dim: 64 or 128
__global__ void __launch_bounds__(320, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                   const __grid_constant__ CUtensorMap tma_v, const AttnTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ float s_max[2][2][kTcBM];   // [tile parity][column half][row]: partial row maxima of a warp pair
  __shared__ float s_sum[2][kTcBM];      // [column half][row]: partial row sums, exchanged once at the end
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  constexpr uint32_t kTcTile = 128 * kTcD * 2;   // bytes of a 128 x D bf16 tile (Q, K, V)
  constexpr int kSub = kTcD / 64;                // 64-channel sub-tiles per row
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kTcTile;          // 2 stages
  uint8_t* sV = sK + 2 * kTcTile;      // 2 stages
  uint8_t* sP = sV + 2 * kTcTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kTcPTile);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* s_empty = bars + 11;    // 2
  uint64_t* p_full = bars + 13;
  uint64_t* p_empty = bars + 14;
  uint64_t* o_full = bars + 15;     // 2
  uint64_t* o_empty = bars + 17;    // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();   // before the first global read and before any early return
  // a CTA of this or an earlier launch already gave up on a wait: do not queue up behind the same fault
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) return;
  // ---- work assignment (before any barrier set-up: CTAs without work leave at once)
  // heavy tiles first: under a causal mask the last query tiles of a sequence see the most keys
  const int tile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y;
  const int seq = find_seq(p.tile_prefix, p.num_seqs, tile);
  if (seq < 0) return;
  const int q_beg = p.cu_q[seq], lq = p.cu_q[seq + 1] - q_beg;
  const int k_beg = p.cu_k[seq], lk = p.cu_k[seq + 1] - k_beg;
  const int q0 = (tile - p.tile_prefix[seq]) * kTcBM;
  if (q0 >= lq) return;
  const int shift = lk - lq;
  const int kvh = head / (p.hq / p.hkv);
  int k_end = p.causal ? min(lk, q0 + kTcBM + shift) : lk;
  if (k_end < 0) k_end = 0;
  const int n_tiles = (k_end + kTcBN - 1) / kTcBN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 8);
      mbar_init(&o_full[s], 1);
      mbar_init(&o_empty[s], 8);
    }
    mbar_init(p_full, 8);
    mbar_init(p_empty, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();   // TMEM is held: a dependent kernel that lands on this SM cannot take it from under this CTA

  if (warp == 0) {
    // ------------------------------------ TMA producer ------------------------------------
    if (lane == 0) {
      mbar_expect_tx(q_full, kTcTile);
#pragma unroll
      for (int j = 0; j < kSub; ++j) tma_load_2d(sQ + j * 16384, &tma_q, q_full, head * kTcD + j * 64, q_beg + q0);
    }
    bool ok = true;
    for (int i = 0; i < n_tiles && ok; ++i) {
      const int st = i & 1;
      const uint32_t ph = (i >> 1) & 1;
      const int krow = k_beg + i * kTcBN;
      if (!mbar_wait(&k_empty[st], ph ^ 1u, abort_flag, p.status, 11)) { ok = false; break; }
      if (lane == 0) {
        mbar_expect_tx(&k_full[st], kTcTile);
#pragma unroll
        for (int j = 0; j < kSub; ++j)
          tma_load_2d(sK + st * kTcTile + j * 16384, &tma_k, &k_full[st], kvh * kTcD + j * 64, krow);
      }
      if (!mbar_wait(&v_empty[st], ph ^ 1u, abort_flag, p.status, 12)) { ok = false; break; }
      if (lane == 0) {
        mbar_expect_tx(&v_full[st], kTcTile);
        // MN-major B operand: [key block of 64][head-dim half of 64] boxes of 64 keys x 64 channels
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int nh = 0; nh < kSub; ++nh)
            tma_load_2d(sV + st * kTcTile + kb * (kSub * 8192) + nh * 8192, &tma_v, &v_full[st], kvh * kTcD + nh * 64,
                        krow + kb * 64);
      }
      __syncwarp();
    }
    if (!ok) {
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // let copies in flight land before smem goes away
    }
  } else if (warp == 1) {
    // ------------------------------------- MMA issuer --------------------------------------
    constexpr uint32_t idesc_s = make_idesc_bf16(kTcBM, kTcBN, 0, 0);
    constexpr uint32_t idesc_o = make_idesc_bf16(kTcBM, kTcD, 0, 1);
    bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 13);
    auto issue_s = [&](int i) -> bool {
      const int st = i & 1;
      const uint32_t ph = (i >> 1) & 1;
      if (!mbar_wait(&k_full[st], ph, abort_flag, p.status, 14)) return false;
      if (!mbar_wait(&s_empty[st], ph ^ 1u, abort_flag, p.status, 15)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t a_base = smem_u32(sQ), b_base = smem_u32(sK + st * kTcTile);
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(st * kTcBN);
#pragma unroll
        for (int kb = 0; kb < kSub; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(d_tmem, make_smem_desc_sw128(a_base + kb * 16384 + kk * 32, 0, 1024),
                     make_smem_desc_sw128(b_base + kb * 16384 + kk * 32, 0, 1024), idesc_s, (kb | kk) ? 1u : 0u);
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[st]);
      }
      __syncwarp();
      return true;
    };
    if (ok && n_tiles > 0) ok = issue_s(0);
    for (int i = 0; i < n_tiles && ok; ++i) {
      if (i + 1 < n_tiles && !issue_s(i + 1)) { ok = false; break; }
      const int st = i & 1;
      if (!mbar_wait(&v_full[st], (i >> 1) & 1, abort_flag, p.status, 16)) { ok = false; break; }
      if (!mbar_wait(p_full, i & 1, abort_flag, p.status, 17)) { ok = false; break; }
      if (!mbar_wait(&o_empty[st], ((i >> 1) & 1) ^ 1u, abort_flag, p.status, 18)) { ok = false; break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t a_base = smem_u32(sP), b_base = smem_u32(sV + st * kTcTile);
        const uint32_t d_tmem = tmem_base + 256u + static_cast<uint32_t>(st * kTcD);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(d_tmem, make_smem_desc_sw128(a_base + kb * 16384 + kk * 32, 0, 1024),
                     make_smem_desc_sw128(b_base + kb * (kSub * 8192) + kk * 2048, 8192, 1024), idesc_o,
                     (kb | kk) ? 1u : 0u);
        umma_commit(&v_empty[st]);
        umma_commit(p_empty);
        umma_commit(&o_full[st]);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------ softmax warps ------------------------------------
    // Eight warps: warps w and w + 4 share a TMEM lane quarter (rows) and split the columns, so every
    // scheduler has two softmax warps to interleave.  Thread (row r, half h) handles keys [64 h, 64 h + 64)
    // of each tile and output channels [64 h, 64 h + 64); the two halves of a row exchange their partial
    // maximum through shared memory once per tile and their partial sums once at the end.
    const int qd = warp & 3;                 // TMEM lane quarter of this warp
    const int half = (warp - 2) >> 2;        // 0: warps 2-5, 1: warps 6-9
    const int r = qd * 32 + lane;            // query row inside the tile
    const int qi = q0 + r;                   // query index inside the sequence
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    const float sl2 = p.scale * 1.4426950408889634f;
    const int key_off = half * 64;            // this thread's keys of every tile
    constexpr int kOc = kTcD / 2;             // and its output channels
    const int ch_off = half * kOc;
    float o_reg[kOc];
#pragma unroll
    for (int j = 0; j < kOc; ++j) o_reg[j] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, corr_prev = 0.f;
    bool ok = true;
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + qd) : "memory"); };
    // o = o * c + O_tile(j): runs one tile late, after P of the next tile is on its way
    auto fold = [&](int j, float c) -> bool {
      const int ob = j & 1;
      if (!mbar_wait(&o_full[ob], (j >> 1) & 1, abort_flag, p.status, 21)) return false;
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < kOc; cc += 32) {
        uint32_t v[32];
        tmem_ld_32x32(t_lane + 256u + static_cast<uint32_t>(ob * kTcD + ch_off) + cc, v);
        tmem_ld_wait();
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) o_reg[cc + jj] = o_reg[cc + jj] * c + __uint_as_float(v[jj]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&o_empty[ob]);
      return true;
    };
    for (int i = 0; i < n_tiles && ok; ++i) {
      const int b = i & 1;
      const int kt0 = i * kTcBN;
      if (!mbar_wait(&s_full[b], (i >> 1) & 1, abort_flag, p.status, 19)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_s = t_lane + static_cast<uint32_t>(b * kTcBN + key_off);
      // keys this row may see in this tile: [kt0, limit); this thread's share starts at key_off
      int limit = lk;
      if (p.causal) limit = min(limit, qi + shift + 1);
      const int nvis = max(0, min(64, limit - kt0 - key_off));
      // pass 1: maximum over this thread's 64 keys, then over the row
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(t_s + c, v);
        tmem_ld_wait();
        if (nvis == 64) {   // all visible: no per-element test
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, __uint_as_float(v[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c + j < nvis) mx = fmaxf(mx, __uint_as_float(v[j]));
        }
      }
      s_max[b][half][r] = mx;
      pair_sync();
      mx = fmaxf(mx, s_max[b][half ^ 1][r]);
      const float m_new = fmaxf(m_run, mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float corr = ex2_approx((m_run - m_use) * sl2);   // m_run = -inf -> 0
      if (!mbar_wait(p_empty, (i & 1) ^ 1u, abort_flag, p.status, 20)) { ok = false; break; }
      // pass 2: probabilities -> bf16 P tile (K-major, 128-byte swizzle), partial row sum
      float rs = 0.f;
      uint8_t* sub = sP + half * 16384 + r * 128;   // this thread's 64-key sub-tile, this row
      const float mb = m_use * sl2;
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(t_s + c, v);
        tmem_ld_wait();
        uint32_t pk[16];
        if (nvis == 64) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(v[j]), sl2, -mb));
            const float p1 = ex2_approx(fmaf(__uint_as_float(v[j + 1]), sl2, -mb));
            rs += p0 + p1;
            pk[j >> 1] = pack_bf16x2(p0, p1);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float p0 = c + j < nvis ? ex2_approx(fmaf(__uint_as_float(v[j]), sl2, -mb)) : 0.f;
            const float p1 = c + j + 1 < nvis ? ex2_approx(fmaf(__uint_as_float(v[j + 1]), sl2, -mb)) : 0.f;
            rs += p0 + p1;
            pk[j >> 1] = pack_bf16x2(p0, p1);
          }
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int jc = (c >> 3) + ch;               // 16-byte chunk index within the 128-byte row
          *reinterpret_cast<uint4*>(sub + ((jc ^ (r & 7)) << 4)) =
              make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[b]);
        mbar_arrive(p_full);
      }
      l_run = l_run * corr + rs;
      m_run = m_new;
      if (i > 0 && !fold(i - 1, corr_prev)) { ok = false; break; }
      corr_prev = corr;
    }
    if (ok && n_tiles > 0) ok = fold(n_tiles - 1, corr_prev);
    // total row sum = the two halves' partial sums (both relative to the same final maximum)
    s_sum[half][r] = l_run;
    pair_sync();
    l_run += s_sum[half ^ 1][r];
    if (ok && qi < lq) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = p.out + (long long)(q_beg + qi) * p.o_stride + (long long)head * kTcD + ch_off;
#pragma unroll
      for (int c = 0; c < kOc; c += 8) {
        uint4 o;
        o.x = pack_bf16x2(o_reg[c] * inv, o_reg[c + 1] * inv);
        o.y = pack_bf16x2(o_reg[c + 2] * inv, o_reg[c + 3] * inv);
        o.z = pack_bf16x2(o_reg[c + 4] * inv, o_reg[c + 5] * inv);
        o.w = pack_bf16x2(o_reg[c + 6] * inv, o_reg[c + 7] * inv);
        *reinterpret_cast<uint4*>(dst + c) = o;
      }
      if (p.lse != nullptr && half == 0) {
        const long long total_q = p.cu_q[p.num_seqs];
        p.lse[(long long)head * total_q + q_beg + qi] = l_run > 0.f ? m_run * p.scale + logf(l_run) : -INFINITY;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace areno

using namespace areno;

// Same arguments as areno_attn_fwd plus the row counts of q and k / v (for the tensor maps) and the status
// words.  head_dim must be 64 or 128 and there is no sliding window; returns -2 otherwise (callers fall back to
// areno_attn_fwd).
extern "C" int areno_attn_fwd_tc(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_q,
                                 const int* cu_k, const int* tile_prefix, int num_seqs, int total_tiles, int hq, int hkv,
                                 int head_dim, long long total_q, long long total_k, long long q_stride,
                                 long long k_stride, long long v_stride, long long o_stride, float scale, int causal,
                                 int* status, cudaStream_t stream) {
  if (total_tiles <= 0) return 0;
  if (head_dim != 128 && head_dim != 64) return -2;
  const int kTcD = head_dim;
  if (hq % hkv != 0) return -3;
  if ((q_stride % 8) || (k_stride % 8) || (v_stride % 8) || (o_stride % 8)) return -3;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k) & 15) ||
      (reinterpret_cast<uintptr_t>(v) & 15) || (reinterpret_cast<uintptr_t>(o) & 15))
    return -3;
  CUtensorMap tq, tk, tv;
  int rc = make_tensor_map_2d_bf16(&tq, q, (uint64_t)hq * kTcD, (uint64_t)total_q, (uint64_t)q_stride * 2, 64, 128);
  if (rc != 0) return rc;
  rc = make_tensor_map_2d_bf16(&tk, k, (uint64_t)hkv * kTcD, (uint64_t)total_k, (uint64_t)k_stride * 2, 64, 128);
  if (rc != 0) return rc;
  rc = make_tensor_map_2d_bf16(&tv, v, (uint64_t)hkv * kTcD, (uint64_t)total_k, (uint64_t)v_stride * 2, 64, 64);
  if (rc != 0) return rc;
  AttnTcParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.cu_q = cu_q;
  p.cu_k = cu_k;
  p.tile_prefix = tile_prefix;
  p.num_seqs = num_seqs;
  p.hq = hq;
  p.hkv = hkv;
  p.o_stride = o_stride;
  p.scale = scale;
  p.causal = causal;
  p.status = status;
  const int smem = 5 * 128 * kTcD * 2 + (int)kTcPTile + 256 + 1024;
  static bool cfg_dev[kMaxDevices] = {};
    bool& cfg = per_device_flag(cfg_dev);
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         5 * 128 * 128 * 2 + (int)kTcPTile + 256 + 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_fwd_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               5 * 128 * 64 * 2 + (int)kTcPTile + 256 + 1024);
    if (e != cudaSuccess) return (int)e;
    cfg = true;
  }
  if (kTcD == 128)
    return (int)launch_pdl(attn_fwd_tc_kernel<128>, dim3(total_tiles, hq), dim3(320), smem, stream, tq, tk, tv, p);
  return (int)launch_pdl(attn_fwd_tc_kernel<64>, dim3(total_tiles, hq), dim3(320), smem, stream, tq, tk, tv, p);
}
