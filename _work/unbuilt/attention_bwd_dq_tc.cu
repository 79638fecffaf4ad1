// Attention backward on the 5th-generation tensor cores, head_dim 128: the dQ pass.
//
// One CTA per (128 query rows, query head), ten warps as in attention_fwd_tc.cu:
//   warp 0      TMA producer: Q and dO once, then K and V tiles of 128 keys through a two-stage ring
//   warp 1      MMA issuer:   S = Q K^T and dP = dO V^T into TMEM, then dQ += dS K (accumulated in TMEM
//                             over all key tiles; K is read a second time from the same shared tile,
//                             this time through an MN-major descriptor)
//   warps 2-9   two threads per query row: recompute P = exp(S * scale - lse), form dS = P (dP - delta),
//                             write it as a 128-byte-swizzled bf16 tile for the third MMA; at the end read
//                             dQ from TMEM, scale and store it
// TMEM: S [0,128), dP [128,256), dQ [256,384).  Shared memory: Q, dO, 2 x K, 2 x V, dS = 7 x 32 KB.
// dK / dV stay in attention_bwd.cu (mma.sync), which also computes delta = rowsum(dO * O).
//
// Every mbarrier wait is bounded; on expiry the CTA records a status word, lets copies in flight land, frees
// its TMEM and returns.  No multicast loads.
//
// NOT BUILT: this directory is outside the build's source list and nothing in the package calls the entry
// point below.  State when it was parked: one sequence of 64 rows matched the fp32 oracle and 16 x 1536 rows
// with 28 / 4 heads ran 22 % faster than the mma.sync backward (3.30 vs 4.22 ms), but a packed batch of
// sequence lengths 37, 129 and 5 (4 query heads, 2 KV heads) did not complete on a B200 in two runs; the
// process had to be ended by its time limit and the device stayed usable afterwards.  Reading has not shown
// the cause.  It must not be run on a GPU again before the cause is known; the mma.sync dQ pass in
// attention_bwd.cu is the one in use.
#include "attention_common.cuh"
#include "launch.h"

namespace areno {

constexpr int kBqD = 128;
constexpr uint32_t kBqTile = 128 * 128 * 2;

struct AttnBwdTcParams {
  __nv_bfloat16* dq;
  const float* lse;     // [hq, total_q], natural log of the scaled scores' partition function
  const float* delta;   // [hq, total_q]
  const int* cu_q;
  const int* cu_k;
  const int* tile_prefix;  // 128-row query tiles per sequence (prefix sum)
  int num_seqs, hq, hkv;
  long long dq_stride;
  float scale;
  int causal;
  int* status;
};

__device__ __forceinline__ float ex2_approx_b(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(320, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_do,
                      const __grid_constant__ CUtensorMap tma_k, const __grid_constant__ CUtensorMap tma_v,
                      const AttnBwdTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + kBqTile;
  uint8_t* sK = sdO + kBqTile;         // 2 stages
  uint8_t* sV = sK + 2 * kBqTile;      // 2 stages
  uint8_t* sDS = sV + 2 * kBqTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + kBqTile);
  uint64_t* q_full = bars;           // Q + dO
  uint64_t* kv_full = bars + 1;      // 2
  uint64_t* kv_empty = bars + 3;     // 2
  uint64_t* sp_full = bars + 5;      // S and dP are in TMEM
  uint64_t* sp_empty = bars + 6;     // softmax threads have read them
  uint64_t* ds_full = bars + 7;      // dS tile written
  uint64_t* ds_empty = bars + 8;     // third MMA has consumed it
  uint64_t* dq_full = bars + 9;      // every MMA of the CTA is done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) return;
  const int tile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);   // heavy tiles first
  const int head = blockIdx.y;
  const int seq = find_seq(p.tile_prefix, p.num_seqs, tile);
  if (seq < 0) return;
  const int q_beg = p.cu_q[seq], lq = p.cu_q[seq + 1] - q_beg;
  const int k_beg = p.cu_k[seq], lk = p.cu_k[seq + 1] - k_beg;
  const int q0 = (tile - p.tile_prefix[seq]) * 128;
  if (q0 >= lq) return;
  const int shift = lk - lq;
  const int kvh = head / (p.hq / p.hkv);
  int k_end = p.causal ? min(lk, q0 + 128 + shift) : lk;
  if (k_end < 0) k_end = 0;
  const int n_tiles = (k_end + 127) / 128;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(sp_full, 1);
    mbar_init(sp_empty, 8);
    mbar_init(ds_full, 8);
    mbar_init(ds_empty, 1);
    mbar_init(dq_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_do);
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
  pdl_trigger();

  if (warp == 0) {
    // ------------------------------------ TMA producer ------------------------------------
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * kBqTile);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        tma_load_2d(sQ + j * 16384, &tma_q, q_full, head * kBqD + j * 64, q_beg + q0);
        tma_load_2d(sdO + j * 16384, &tma_do, q_full, head * kBqD + j * 64, q_beg + q0);
      }
    }
    bool ok = true;
    for (int i = 0; i < n_tiles && ok; ++i) {
      const int st = i & 1;
      const uint32_t ph = (i >> 1) & 1;
      const int krow = k_beg + i * 128;
      if (!mbar_wait(&kv_empty[st], ph ^ 1u, abort_flag, p.status, 31)) { ok = false; break; }
      if (lane == 0) {
        mbar_expect_tx(&kv_full[st], 2 * kBqTile);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          tma_load_2d(sK + st * kBqTile + j * 16384, &tma_k, &kv_full[st], kvh * kBqD + j * 64, krow);
          tma_load_2d(sV + st * kBqTile + j * 16384, &tma_v, &kv_full[st], kvh * kBqD + j * 64, krow);
        }
      }
      __syncwarp();
    }
    if (!ok) {
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ------------------------------------- MMA issuer --------------------------------------
    constexpr uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);   // both operands K-major
    constexpr uint32_t idesc_mn = make_idesc_bf16(128, 128, 0, 1);   // B (the K tile) read MN-major
    bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 32);
    for (int i = 0; i < n_tiles && ok; ++i) {
      const int st = i & 1;
      if (!mbar_wait(&kv_full[st], (i >> 1) & 1, abort_flag, p.status, 33)) { ok = false; break; }
      if (!mbar_wait(sp_empty, (i & 1) ^ 1u, abort_flag, p.status, 34)) { ok = false; break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t q_base = smem_u32(sQ), do_base = smem_u32(sdO);
        const uint32_t k_base = smem_u32(sK + st * kBqTile), v_base = smem_u32(sV + st * kBqTile);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem_base, make_smem_desc_sw128(q_base + kb * 16384 + kk * 32, 0, 1024),
                     make_smem_desc_sw128(k_base + kb * 16384 + kk * 32, 0, 1024), idesc_kk, (kb | kk) ? 1u : 0u);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem_base + 128u, make_smem_desc_sw128(do_base + kb * 16384 + kk * 32, 0, 1024),
                     make_smem_desc_sw128(v_base + kb * 16384 + kk * 32, 0, 1024), idesc_kk, (kb | kk) ? 1u : 0u);
        umma_commit(sp_full);
      }
      __syncwarp();
      if (!mbar_wait(ds_full, i & 1, abort_flag, p.status, 35)) { ok = false; break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t a_base = smem_u32(sDS), k_base = smem_u32(sK + st * kBqTile);
        // dQ[q, d] += sum_key dS[q, key] K[key, d]: the K tile is [key rows][two 64-channel halves 16 KB apart]
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)      // 64-key block
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)    // 16 keys
            umma_f16(tmem_base + 256u, make_smem_desc_sw128(a_base + kb * 16384 + kk * 32, 0, 1024),
                     make_smem_desc_sw128(k_base + kb * 8192 + kk * 2048, 16384, 1024), idesc_mn,
                     (i | kb | kk) ? 1u : 0u);
        umma_commit(ds_empty);
        umma_commit(&kv_empty[st]);
        if (i == n_tiles - 1) umma_commit(dq_full);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------ softmax warps ------------------------------------
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = qd * 32 + lane;
    const int qi = q0 + r;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    const float sl2 = p.scale * 1.4426950408889634f;
    const int key_off = half * 64;
    const long long total_q = p.cu_q[p.num_seqs];
    float lse_l2 = INFINITY, delta_r = 0.f;   // rows past the sequence: p = exp2(-inf) = 0
    if (qi < lq) {
      const float l = p.lse[(long long)head * total_q + q_beg + qi];
      lse_l2 = l == -INFINITY ? INFINITY : l * 1.4426950408889634f;
      delta_r = p.delta[(long long)head * total_q + q_beg + qi];
    }
    bool ok = true;
    for (int i = 0; i < n_tiles && ok; ++i) {
      const int kt0 = i * 128;
      if (!mbar_wait(sp_full, i & 1, abort_flag, p.status, 36)) { ok = false; break; }
      tc_fence_after();
      int limit = lk;
      if (p.causal) limit = min(limit, qi + shift + 1);
      const int nvis = max(0, min(64, limit - kt0 - key_off));
      if (!mbar_wait(ds_empty, (i & 1) ^ 1u, abort_flag, p.status, 37)) { ok = false; break; }
      uint8_t* sub = sDS + half * 16384 + r * 128;
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(t_lane + static_cast<uint32_t>(key_off + c), sv);
        tmem_ld_32x32(t_lane + 128u + static_cast<uint32_t>(key_off + c), dv);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float d0 = 0.f, d1 = 0.f;
          if (c + j < nvis) {
            const float pr = ex2_approx_b(fmaf(__uint_as_float(sv[j]), sl2, -lse_l2));
            d0 = pr * (__uint_as_float(dv[j]) - delta_r);
          }
          if (c + j + 1 < nvis) {
            const float pr = ex2_approx_b(fmaf(__uint_as_float(sv[j + 1]), sl2, -lse_l2));
            d1 = pr * (__uint_as_float(dv[j + 1]) - delta_r);
          }
          pk[j >> 1] = pack_bf16x2(d0, d1);
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int jc = (c >> 3) + ch;
          *reinterpret_cast<uint4*>(sub + ((jc ^ (r & 7)) << 4)) =
              make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(sp_empty);
        mbar_arrive(ds_full);
      }
    }
    if (ok && n_tiles > 0) ok = mbar_wait(dq_full, 0, abort_flag, p.status, 38);
    if (ok && qi < lq) {
      tc_fence_after();
      __nv_bfloat16* dst = p.dq + (long long)(q_beg + qi) * p.dq_stride + (long long)head * kBqD + key_off;
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t v[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(t_lane + 256u + static_cast<uint32_t>(key_off + c), v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(v[j]) * p.scale, __uint_as_float(v[j + 1]) * p.scale);
          o.y = pack_bf16x2(__uint_as_float(v[j + 2]) * p.scale, __uint_as_float(v[j + 3]) * p.scale);
          o.z = pack_bf16x2(__uint_as_float(v[j + 4]) * p.scale, __uint_as_float(v[j + 5]) * p.scale);
          o.w = pack_bf16x2(__uint_as_float(v[j + 6]) * p.scale, __uint_as_float(v[j + 7]) * p.scale);
          *reinterpret_cast<uint4*>(dst + c + j) = o;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace areno

using namespace areno;

// dQ of areno_attn_bwd on the tcgen05 path (head_dim 128, no sliding window; -2 otherwise).  lse / delta: fp32
// [hq, total_q] as produced by the forward and by areno_attn_bwd's delta kernel.  tile_prefix: 128-row query tiles.
extern "C" int areno_attn_bwd_dq_tc(const void* q, const void* k, const void* v, const void* d_o, const float* lse,
                                    const float* delta, void* dq, const int* cu_q, const int* cu_k,
                                    const int* tile_prefix, int num_seqs, int total_tiles, int hq, int hkv, int head_dim,
                                    long long total_q, long long total_k, long long q_stride, long long k_stride,
                                    long long v_stride, long long do_stride, long long dq_stride, float scale,
                                    int causal, int* status, cudaStream_t stream) {
  if (total_tiles <= 0) return 0;
  if (head_dim != kBqD) return -2;
  if (hq % hkv != 0) return -3;
  if ((q_stride % 8) || (k_stride % 8) || (v_stride % 8) || (do_stride % 8) || (dq_stride % 8)) return -3;
  const void* ptrs[5] = {q, k, v, d_o, dq};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return -3;
  CUtensorMap tq, tdo, tk, tv;
  int rc = make_tensor_map_2d_bf16(&tq, q, (uint64_t)hq * kBqD, (uint64_t)total_q, (uint64_t)q_stride * 2, 64, 128);
  if (rc != 0) return rc;
  rc = make_tensor_map_2d_bf16(&tdo, d_o, (uint64_t)hq * kBqD, (uint64_t)total_q, (uint64_t)do_stride * 2, 64, 128);
  if (rc != 0) return rc;
  rc = make_tensor_map_2d_bf16(&tk, k, (uint64_t)hkv * kBqD, (uint64_t)total_k, (uint64_t)k_stride * 2, 64, 128);
  if (rc != 0) return rc;
  rc = make_tensor_map_2d_bf16(&tv, v, (uint64_t)hkv * kBqD, (uint64_t)total_k, (uint64_t)v_stride * 2, 64, 128);
  if (rc != 0) return rc;
  AttnBwdTcParams p;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq);
  p.lse = lse;
  p.delta = delta;
  p.cu_q = cu_q;
  p.cu_k = cu_k;
  p.tile_prefix = tile_prefix;
  p.num_seqs = num_seqs;
  p.hq = hq;
  p.hkv = hkv;
  p.dq_stride = dq_stride;
  p.scale = scale;
  p.causal = causal;
  p.status = status;
  constexpr int smem = 7 * (int)kBqTile + 256 + 1024;
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    cfg = true;
  }
  return (int)launch_pdl(attn_bwd_dq_tc_kernel, dim3(total_tiles, hq), dim3(320), smem, stream, tq, tdo, tk, tv, p);
}
