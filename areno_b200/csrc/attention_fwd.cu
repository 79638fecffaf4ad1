// Variable-length causal attention forward (training + prefill), GQA, head_dim 64/128.
// Flash-style online softmax; bf16 tensor-core MMAs with fp32 accumulation; K/V tiles are
// double-buffered in swizzled shared memory with cp.async.  One CTA = 64 query rows of one
// (sequence, q-head); 4 warps x 16 rows.  Query i of a sequence with lq queries and lk keys
// sees keys j <= i + (lk - lq) (bottom-right aligned causal mask, so a prefill chunk can
// attend to earlier keys), optionally limited to a sliding window.
// Replaces flash_attn_varlen_func as used by the reference
// (areno/engine/layers/attention_backend/train.py:135-141, infer.py:163-169) and the scalar
// "native" kernel (areno/accel/csrc/attention.cu:145-242).
#include "attention_common.cuh"
#include "launch.h"

namespace areno {

template <int D>
__global__ void __launch_bounds__(128)
attn_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ o, float* __restrict__ lse,
                const int* __restrict__ cu_q, const int* __restrict__ cu_k, const int* __restrict__ tile_prefix,
                int num_seqs, int hq, int hkv, long long q_stride, long long k_stride, long long v_stride,
                long long o_stride, float scale, int causal, int window) {
  constexpr int BM = 64, BN = 64;
  constexpr int CH = D / 8;            // 16-byte chunks per row
  constexpr int TILE = BM * D;         // elements per tile
  extern __shared__ __align__(128) uint8_t smem_attn[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_attn);
  __nv_bfloat16* sK = sQ + TILE;       // 2 buffers
  __nv_bfloat16* sV = sK + 2 * TILE;   // 2 buffers

  const int tile = blockIdx.x;
  const int head = blockIdx.y;
  const int kvh = head / (hq / hkv);
  const int seq = find_seq(tile_prefix, num_seqs, tile);
  if (seq < 0) return;
  const int q_tile = tile - tile_prefix[seq];
  const int q_beg = cu_q[seq], lq = cu_q[seq + 1] - q_beg;
  const int k_beg = cu_k[seq], lk = cu_k[seq + 1] - k_beg;
  const int q0 = q_tile * BM;
  if (q0 >= lq) return;
  const int shift = lk - lq;  // key index visible to query i: j <= i + shift

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  // key range for this q tile
  int k_end = causal ? min(lk, q0 + BM + shift) : lk;
  int k_start = 0;
  if (window > 0) k_start = max(0, q0 + shift - window + 1) / BN * BN;
  if (k_end < 0) k_end = 0;
  const int n_tiles = (k_end - k_start + BN - 1) / BN;

  const __nv_bfloat16* qp = q + (long long)(q_beg + q0) * q_stride + (long long)head * D;
  const __nv_bfloat16* kp = k + (long long)k_beg * k_stride + (long long)kvh * D;
  const __nv_bfloat16* vp = v + (long long)k_beg * v_stride + (long long)kvh * D;

  load_tile_async<D, BM>(sQ, qp, q_stride, lq - q0);
  if (n_tiles > 0) {
    load_tile_async<D, BN>(sK, kp + (long long)k_start * k_stride, k_stride, lk - k_start);
    load_tile_async<D, BN>(sV, vp + (long long)k_start * v_stride, v_stride, lk - k_start);
  }
  cp_async_commit();

  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const float scale_log2 = scale * 1.4426950408889634f;

  uint32_t qf[D / 16][4];
  const int row_a = q0 + warp * 16 + g;  // rows row_a and row_a + 8 (within the sequence)

  for (int it = 0; it < n_tiles; ++it) {
    const int buf = it & 1;
    const int kt0 = k_start + it * BN;
    if (it + 1 < n_tiles) {
      const int kn = kt0 + BN;
      load_tile_async<D, BN>(sK + (buf ^ 1) * TILE, kp + (long long)kn * k_stride, k_stride, lk - kn);
      load_tile_async<D, BN>(sV + (buf ^ 1) * TILE, vp + (long long)kn * v_stride, v_stride, lk - kn);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) ldsm_a<CH>(qf[ks], sQ, warp * 16, ks * 2, lane);
    }
    const __nv_bfloat16* cK = sK + buf * TILE;
    const __nv_bfloat16* cV = sV + buf * TILE;

    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int nt = 0; nt < BN / 16; ++nt) {
        uint32_t b[4];
        ldsm_b_nt<CH>(b, cK, nt * 16, ks * 2, lane);
        mma_bf16(s[2 * nt], qf[ks], b[0], b[1]);
        mma_bf16(s[2 * nt + 1], qf[ks], b[2], b[3]);
      }
    }
    // mask + online softmax
    const bool need_mask = (kt0 + BN > lk) || (causal && kt0 + BN - 1 > q0 + warp * 16 + shift) || window > 0;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = row_a + (e >> 1) * 8;
        const int c = kt0 + nt * 8 + t4 * 2 + (e & 1);
        if (need_mask) {
          bool ok = c < lk;
          if (causal) ok = ok && (c <= r + shift);
          if (window > 0) ok = ok && (c > r + shift - window);
          if (!ok) s[nt][e] = -INFINITY;
        }
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      }
    }
    float corr[2], m_new[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      m_new[h] = fmaxf(m_run[h], mx[h]);
      const float m_use = m_new[h] == -INFINITY ? 0.f : m_new[h];
      corr[h] = exp2f((m_run[h] - m_use) * scale_log2);
      m_run[h] = m_new[h];
      m_new[h] = m_use;
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pf[BN / 16][4];
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
      float p0 = exp2f((s[nt][0] - m_new[0]) * scale_log2);
      float p1 = exp2f((s[nt][1] - m_new[0]) * scale_log2);
      float p2 = exp2f((s[nt][2] - m_new[1]) * scale_log2);
      float p3 = exp2f((s[nt][3] - m_new[1]) * scale_log2);
      rs[0] += p0 + p1;
      rs[1] += p2 + p3;
      pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(p0, p1);
      pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(p2, p3);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * corr[h] + rs[h];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o_acc[i][0] *= corr[0]; o_acc[i][1] *= corr[0];
      o_acc[i][2] *= corr[1]; o_acc[i][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
      for (int dt = 0; dt < D / 16; ++dt) {
        uint32_t b[4];
        ldsm_b_t<CH>(b, cV, kk * 16, dt * 2, lane);
        mma_bf16(o_acc[2 * dt], pf[kk], b[0], b[1]);
        mma_bf16(o_acc[2 * dt + 1], pf[kk], b[2], b[3]);
      }
    }
    __syncthreads();
  }
  if (n_tiles == 0) cp_async_wait<0>();

  // finalize
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_a + h * 8;
    if (r < lq) {
      const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
      __nv_bfloat16* op = o + (long long)(q_beg + r) * o_stride + (long long)head * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        *reinterpret_cast<uint32_t*>(op + i * 8 + t4 * 2) =
            pack_bf16x2(o_acc[i][h * 2] * inv, o_acc[i][h * 2 + 1] * inv);
      }
      if (lse != nullptr && t4 == 0) {
        // natural-log LSE of the scaled scores
        lse[(long long)head * cu_q[num_seqs] + q_beg + r] =
            l_run[h] > 0.f ? m_run[h] * scale + logf(l_run[h]) : -INFINITY;
      }
    }
  }
}

}  // namespace areno

using namespace areno;

extern "C" int areno_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_q,
                              const int* cu_k, const int* tile_prefix, int num_seqs, int total_tiles, int hq,
                              int hkv, int head_dim, long long q_stride, long long k_stride, long long v_stride,
                              long long o_stride, float scale, int causal, int window, cudaStream_t stream) {
  if (total_tiles <= 0) return 0;
  if (hq % hkv != 0) return -3;
  dim3 grid(total_tiles, hq);
  if (head_dim == 128) {
    constexpr int smem = 5 * 64 * 128 * 2;
    static bool cfg_dev[kMaxDevices] = {};
    bool& cfg = per_device_flag(cfg_dev);
    if (!cfg) { cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); cfg = true; }
    attn_fwd_kernel<128><<<grid, 128, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
        (const __nv_bfloat16*)v, (__nv_bfloat16*)o, lse, cu_q, cu_k, tile_prefix, num_seqs, hq, hkv, q_stride,
        k_stride, v_stride, o_stride, scale, causal, window);
  } else if (head_dim == 64) {
    constexpr int smem = 5 * 64 * 64 * 2;
    static bool cfg_dev[kMaxDevices] = {};
    bool& cfg = per_device_flag(cfg_dev);
    if (!cfg) { cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); cfg = true; }
    attn_fwd_kernel<64><<<grid, 128, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
        (const __nv_bfloat16*)v, (__nv_bfloat16*)o, lse, cu_q, cu_k, tile_prefix, num_seqs, hq, hkv, q_stride,
        k_stride, v_stride, o_stride, scale, causal, window);
  } else if (head_dim == 256) {
    constexpr int smem = 5 * 64 * 256 * 2;
    static bool cfg_dev[kMaxDevices] = {};
    bool& cfg = per_device_flag(cfg_dev);
    if (!cfg) { cudaFuncSetAttribute(attn_fwd_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); cfg = true; }
    attn_fwd_kernel<256><<<grid, 128, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
        (const __nv_bfloat16*)v, (__nv_bfloat16*)o, lse, cu_q, cu_k, tile_prefix, num_seqs, hq, hkv, q_stride,
        k_stride, v_stride, o_stride, scale, causal, window);
  } else {
    return -2;
  }
  return (int)cudaGetLastError();
}
