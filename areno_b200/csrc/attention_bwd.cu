// Variable-length causal attention backward (GQA, head_dim 64/128/256), deterministic (no atomics):
//   1. delta[h, t] = sum_d dO * O
//   2. dK/dV kernel: one CTA per (key tile, kv head); loops over the q heads of the group and
//      the query tiles that can see the key tile; works on transposed scores S^T = K Q^T so
//      that P^T and dS^T come out of the MMA in A-fragment layout for dV = P^T dO, dK = dS^T Q.
//   3. dQ kernel: one CTA per (query tile, q head); loops over key tiles; dQ = dS K.
// Both recompute P from the saved log-sum-exp.  The reference gets this from flash-attn's
// autograd (areno/engine/layers/attention_backend/train.py:126-141); its own scalar backward
// (areno/accel/csrc/attention.cu:389-524) uses fp32 atomics.
#include "attention_common.cuh"
#include "launch.h"

namespace areno {

__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                  float* __restrict__ delta, long long total_q, int hq, int D, long long o_stride,
                  long long do_stride) {
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= total_q * hq) return;
  const int lane = threadIdx.x & 31;
  const long long t = w / hq;
  const int h = (int)(w % hq);
  const __nv_bfloat16* po = o + t * o_stride + (long long)h * D;
  const __nv_bfloat16* pd = d_o + t * do_stride + (long long)h * D;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(po + i));
    float2 b = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(pd + i));
    acc += a.x * b.x + a.y * b.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[(long long)h * total_q + t] = acc;
}

// DO = output columns owned by one CTA: head_dim 256 runs as two CTAs (blockIdx.z) that each recompute
// S and dP over the full head dimension and accumulate one 128-column half of dK / dV (dQ below), so
// the accumulators stay at the register budget of the 128 case.
template <int D, int DO>
__global__ void __launch_bounds__(128)
attn_bwd_dkv_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                    const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ d_o,
                    const float* __restrict__ lse, const float* __restrict__ delta,
                    __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, const int* __restrict__ cu_q,
                    const int* __restrict__ cu_k, const int* __restrict__ tile_prefix_k, int num_seqs, int hq,
                    int hkv, long long q_stride, long long k_stride, long long v_stride, long long do_stride,
                    long long dk_stride, long long dv_stride, float scale, int causal, int window,
                    float* __restrict__ ws, long long total_k) {
  constexpr int BT = 64;
  constexpr int CH = D / 8;
  constexpr int TILE = BT * D;
  extern __shared__ __align__(128) uint8_t smem_attn[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_attn);
  __nv_bfloat16* sV = sK + TILE;
  __nv_bfloat16* sQ = sV + TILE;        // 2 buffers
  __nv_bfloat16* sdO = sQ + 2 * TILE;   // 2 buffers
  float* sLse = reinterpret_cast<float*>(sdO + 2 * TILE);  // 2 x 64
  float* sDelta = sLse + 2 * BT;                           // 2 x 64

  // With a workspace every CTA takes ONE query head of the group (blockIdx.y = kv head * group + head in group) and
  // stores its fp32 partial of dK / dV; attn_dkv_reduce_kernel adds the heads of a group in a fixed order.  A key
  // tile then costs a seventh of the loop at 28 / 4 heads, and the longest CTA no longer sets the kernel's time.
  const int tile = blockIdx.x;
  const int group = hq / hkv;
  const int hsplit = ws != nullptr ? group : 1;
  const int kvh = blockIdx.y / hsplit;
  const int h_first = blockIdx.y % hsplit;
  const int heads_here = group / hsplit;
  const int seq = find_seq(tile_prefix_k, num_seqs, tile);
  if (seq < 0) return;
  const int k_tile = tile - tile_prefix_k[seq];
  const int q_beg = cu_q[seq], lq = cu_q[seq + 1] - q_beg;
  const int k_beg = cu_k[seq], lk = cu_k[seq + 1] - k_beg;
  const long long total_q = cu_q[num_seqs];
  const int kt0 = k_tile * BT;
  if (kt0 >= lk) return;
  const int shift = lk - lq;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  int q_lo = causal ? max(0, kt0 - shift) : 0;
  int q_hi = lq;
  if (window > 0) q_hi = min(lq, kt0 + BT - 1 - shift + window);
  const int qt_lo = q_lo / BT;
  const int qt_hi = (q_hi + BT - 1) / BT;           // exclusive
  const int n_qt = max(0, qt_hi - qt_lo);
  const int n_iter = n_qt * heads_here;

  const __nv_bfloat16* kp = k + (long long)(k_beg + kt0) * k_stride + (long long)kvh * D;
  const __nv_bfloat16* vp = v + (long long)(k_beg + kt0) * v_stride + (long long)kvh * D;
  load_tile_async<D, BT>(sK, kp, k_stride, lk - kt0);
  load_tile_async<D, BT>(sV, vp, v_stride, lk - kt0);

  auto issue = [&](int it, int buf) {
    const int hh = kvh * group + h_first + it / n_qt;
    const int qs = (qt_lo + it % n_qt) * BT;
    const __nv_bfloat16* qp = q + (long long)(q_beg + qs) * q_stride + (long long)hh * D;
    const __nv_bfloat16* dop = d_o + (long long)(q_beg + qs) * do_stride + (long long)hh * D;
    load_tile_async<D, BT>(sQ + buf * TILE, qp, q_stride, lq - qs);
    load_tile_async<D, BT>(sdO + buf * TILE, dop, do_stride, lq - qs);
    if (threadIdx.x < BT) {
      const int r = qs + threadIdx.x;
      sLse[buf * BT + threadIdx.x] = r < lq ? lse[(long long)hh * total_q + q_beg + r] : INFINITY;
      sDelta[buf * BT + threadIdx.x] = r < lq ? delta[(long long)hh * total_q + q_beg + r] : 0.f;
    }
  };
  if (n_iter > 0) issue(0, 0);
  cp_async_commit();

  const int c0 = blockIdx.z * (DO / 8);  // first 8-column chunk of this CTA's output slice
  float dk_acc[DO / 8][4], dv_acc[DO / 8][4];
#pragma unroll
  for (int i = 0; i < DO / 8; ++i) {
    dk_acc[i][0] = dk_acc[i][1] = dk_acc[i][2] = dk_acc[i][3] = 0.f;
    dv_acc[i][0] = dv_acc[i][1] = dv_acc[i][2] = dv_acc[i][3] = 0.f;
  }
  const float scale_log2 = scale * 1.4426950408889634f;
  const int key_a = kt0 + warp * 16 + g;  // keys key_a, key_a + 8

  for (int it = 0; it < n_iter; ++it) {
    const int buf = it & 1;
    if (it + 1 < n_iter) {
      issue(it + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* cQ = sQ + buf * TILE;
    const __nv_bfloat16* cdO = sdO + buf * TILE;
    const float* cLse = sLse + buf * BT;
    const float* cDelta = sDelta + buf * BT;
    const int qs = (qt_lo + it % n_qt) * BT;

    float st[BT / 8][4], dpt[BT / 8][4];
#pragma unroll
    for (int i = 0; i < BT / 8; ++i) {
      st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.f;
      dpt[i][0] = dpt[i][1] = dpt[i][2] = dpt[i][3] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t kf[4], vf[4];
      ldsm_a<CH>(kf, sK, warp * 16, ks * 2, lane);
      ldsm_a<CH>(vf, sV, warp * 16, ks * 2, lane);
#pragma unroll
      for (int nt = 0; nt < BT / 16; ++nt) {
        uint32_t b[4];
        ldsm_b_nt<CH>(b, cQ, nt * 16, ks * 2, lane);
        mma_bf16(st[2 * nt], kf, b[0], b[1]);
        mma_bf16(st[2 * nt + 1], kf, b[2], b[3]);
        ldsm_b_nt<CH>(b, cdO, nt * 16, ks * 2, lane);
        mma_bf16(dpt[2 * nt], vf, b[0], b[1]);
        mma_bf16(dpt[2 * nt + 1], vf, b[2], b[3]);
      }
    }
    // P^T and dS^T in A-fragment layout (m = key, k = query)
    uint32_t pf[BT / 16][4], dsf[BT / 16][4];
#pragma unroll
    for (int nt = 0; nt < BT / 8; ++nt) {
      float pv[4], dsv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key_a + (e >> 1) * 8;
        const int qc = nt * 8 + t4 * 2 + (e & 1);
        const int qi = qs + qc;
        bool ok = key < lk && qi < lq;
        if (causal) ok = ok && (key <= qi + shift);
        if (window > 0) ok = ok && (key > qi + shift - window);
        const float p = ok ? exp2f(st[nt][e] * scale_log2 - cLse[qc] * 1.4426950408889634f) : 0.f;
        pv[e] = p;
        dsv[e] = p * (dpt[nt][e] - cDelta[qc]);
      }
      pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(pv[0], pv[1]);
      pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(pv[2], pv[3]);
      dsf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(dsv[0], dsv[1]);
      dsf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(dsv[2], dsv[3]);
    }
#pragma unroll
    for (int kk = 0; kk < BT / 16; ++kk) {
#pragma unroll
      for (int dt = 0; dt < DO / 16; ++dt) {
        uint32_t b[4];
        ldsm_b_t<CH>(b, cdO, kk * 16, c0 + dt * 2, lane);
        mma_bf16(dv_acc[2 * dt], pf[kk], b[0], b[1]);
        mma_bf16(dv_acc[2 * dt + 1], pf[kk], b[2], b[3]);
        ldsm_b_t<CH>(b, cQ, kk * 16, c0 + dt * 2, lane);
        mma_bf16(dk_acc[2 * dt], dsf[kk], b[0], b[1]);
        mma_bf16(dk_acc[2 * dt + 1], dsf[kk], b[2], b[3]);
      }
    }
    __syncthreads();
  }
  if (n_iter == 0) cp_async_wait<0>();

  if (ws != nullptr) {
    const long long row_w = (long long)hkv * D;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int key = key_a + h * 8;
      if (key < lk) {
        float* pk = ws + ((long long)h_first * total_k + k_beg + key) * row_w + (long long)kvh * D + c0 * 8;
        float* pv = pk + (long long)group * total_k * row_w;
#pragma unroll
        for (int i = 0; i < DO / 8; ++i) {
          *reinterpret_cast<float2*>(pk + i * 8 + t4 * 2) = make_float2(dk_acc[i][h * 2] * scale, dk_acc[i][h * 2 + 1] * scale);
          *reinterpret_cast<float2*>(pv + i * 8 + t4 * 2) = make_float2(dv_acc[i][h * 2], dv_acc[i][h * 2 + 1]);
        }
      }
    }
    return;
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int key = key_a + h * 8;
    if (key < lk) {
      __nv_bfloat16* pk = dk + (long long)(k_beg + key) * dk_stride + (long long)kvh * D + c0 * 8;
      __nv_bfloat16* pv = dv + (long long)(k_beg + key) * dv_stride + (long long)kvh * D + c0 * 8;
#pragma unroll
      for (int i = 0; i < DO / 8; ++i) {
        *reinterpret_cast<uint32_t*>(pk + i * 8 + t4 * 2) =
            pack_bf16x2(dk_acc[i][h * 2] * scale, dk_acc[i][h * 2 + 1] * scale);
        *reinterpret_cast<uint32_t*>(pv + i * 8 + t4 * 2) = pack_bf16x2(dv_acc[i][h * 2], dv_acc[i][h * 2 + 1]);
      }
    }
  }
}

// dK / dV = sum over the query heads of a group of the fp32 partials written by attn_bwd_dkv_kernel
// (ws: [2][group][total_k][hkv * D]); one thread per four columns, heads added in index order.
__global__ void __launch_bounds__(256)
attn_dkv_reduce_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                       long long total_k, int group, int row_w, int D, long long dk_stride, long long dv_stride) {
  const long long per = total_k * (row_w / 4);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < 2 * per; i += (long long)gridDim.x * blockDim.x) {
    const int which = i >= per;
    const long long j = which ? i - per : i;
    const long long token = j / (row_w / 4);
    const int col = (int)(j % (row_w / 4)) * 4;
    const float* p = ws + ((long long)which * group * total_k + token) * row_w + col;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int g = 0; g < group; ++g) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(p + (long long)g * total_k * row_w));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    __nv_bfloat16* out = (which ? dv + token * dv_stride : dk + token * dk_stride) + col;
    uint2 o;
    o.x = pack_bf16x2(acc.x, acc.y);
    o.y = pack_bf16x2(acc.z, acc.w);
    *reinterpret_cast<uint2*>(out) = o;
  }
}

template <int D, int DO>
__global__ void __launch_bounds__(128)
attn_bwd_dq_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                   const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ d_o,
                   const float* __restrict__ lse, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dq,
                   const int* __restrict__ cu_q, const int* __restrict__ cu_k, const int* __restrict__ tile_prefix,
                   int num_seqs, int hq, int hkv, long long q_stride, long long k_stride, long long v_stride,
                   long long do_stride, long long dq_stride, float scale, int causal, int window) {
  constexpr int BM = 64, BN = 64;
  constexpr int CH = D / 8;
  constexpr int TILE = BM * D;
  extern __shared__ __align__(128) uint8_t smem_attn[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_attn);
  __nv_bfloat16* sdO = sQ + TILE;
  __nv_bfloat16* sK = sdO + TILE;      // 2 buffers
  __nv_bfloat16* sV = sK + 2 * TILE;   // 2 buffers

  // causal: later query tiles see more keys, so the grid walks the tiles from the last to the first and the
  // long CTAs start first (the short ones fill the tail of the last wave)
  const int tile = causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  const int head = blockIdx.y;
  const int kvh = head / (hq / hkv);
  const int seq = find_seq(tile_prefix, num_seqs, tile);
  if (seq < 0) return;
  const int q_tile = tile - tile_prefix[seq];
  const int q_beg = cu_q[seq], lq = cu_q[seq + 1] - q_beg;
  const int k_beg = cu_k[seq], lk = cu_k[seq + 1] - k_beg;
  const long long total_q = cu_q[num_seqs];
  const int q0 = q_tile * BM;
  if (q0 >= lq) return;
  const int shift = lk - lq;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  int k_end = causal ? min(lk, q0 + BM + shift) : lk;
  int k_start = 0;
  if (window > 0) k_start = max(0, q0 + shift - window + 1) / BN * BN;
  if (k_end < 0) k_end = 0;
  const int n_tiles = (k_end - k_start + BN - 1) / BN;

  const __nv_bfloat16* qp = q + (long long)(q_beg + q0) * q_stride + (long long)head * D;
  const __nv_bfloat16* dop = d_o + (long long)(q_beg + q0) * do_stride + (long long)head * D;
  const __nv_bfloat16* kp = k + (long long)k_beg * k_stride + (long long)kvh * D;
  const __nv_bfloat16* vp = v + (long long)k_beg * v_stride + (long long)kvh * D;
  load_tile_async<D, BM>(sQ, qp, q_stride, lq - q0);
  load_tile_async<D, BM>(sdO, dop, do_stride, lq - q0);
  if (n_tiles > 0) {
    load_tile_async<D, BN>(sK, kp + (long long)k_start * k_stride, k_stride, lk - k_start);
    load_tile_async<D, BN>(sV, vp + (long long)k_start * v_stride, v_stride, lk - k_start);
  }
  cp_async_commit();

  const int row_a = q0 + warp * 16 + g;
  float lse_r[2], delta_r[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_a + h * 8;
    lse_r[h] = r < lq ? lse[(long long)head * total_q + q_beg + r] * 1.4426950408889634f : INFINITY;
    delta_r[h] = r < lq ? delta[(long long)head * total_q + q_beg + r] : 0.f;
  }
  const int c0 = blockIdx.z * (DO / 8);
  float dq_acc[DO / 8][4];
#pragma unroll
  for (int i = 0; i < DO / 8; ++i) dq_acc[i][0] = dq_acc[i][1] = dq_acc[i][2] = dq_acc[i][3] = 0.f;
  const float scale_log2 = scale * 1.4426950408889634f;

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
    const __nv_bfloat16* cK = sK + buf * TILE;
    const __nv_bfloat16* cV = sV + buf * TILE;
    float s[BN / 8][4], dp[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t qf[4], dof[4];
      ldsm_a<CH>(qf, sQ, warp * 16, ks * 2, lane);
      ldsm_a<CH>(dof, sdO, warp * 16, ks * 2, lane);
#pragma unroll
      for (int nt = 0; nt < BN / 16; ++nt) {
        uint32_t b[4];
        ldsm_b_nt<CH>(b, cK, nt * 16, ks * 2, lane);
        mma_bf16(s[2 * nt], qf, b[0], b[1]);
        mma_bf16(s[2 * nt + 1], qf, b[2], b[3]);
        ldsm_b_nt<CH>(b, cV, nt * 16, ks * 2, lane);
        mma_bf16(dp[2 * nt], dof, b[0], b[1]);
        mma_bf16(dp[2 * nt + 1], dof, b[2], b[3]);
      }
    }
    uint32_t dsf[BN / 16][4];
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
      float dsv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = row_a + (e >> 1) * 8;
        const int c = kt0 + nt * 8 + t4 * 2 + (e & 1);
        bool ok = c < lk && r < lq;
        if (causal) ok = ok && (c <= r + shift);
        if (window > 0) ok = ok && (c > r + shift - window);
        const float p = ok ? exp2f(s[nt][e] * scale_log2 - lse_r[e >> 1]) : 0.f;
        dsv[e] = p * (dp[nt][e] - delta_r[e >> 1]);
      }
      dsf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(dsv[0], dsv[1]);
      dsf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(dsv[2], dsv[3]);
    }
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
      for (int dt = 0; dt < DO / 16; ++dt) {
        uint32_t b[4];
        ldsm_b_t<CH>(b, cK, kk * 16, c0 + dt * 2, lane);
        mma_bf16(dq_acc[2 * dt], dsf[kk], b[0], b[1]);
        mma_bf16(dq_acc[2 * dt + 1], dsf[kk], b[2], b[3]);
      }
    }
    __syncthreads();
  }
  if (n_tiles == 0) cp_async_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_a + h * 8;
    if (r < lq) {
      __nv_bfloat16* p = dq + (long long)(q_beg + r) * dq_stride + (long long)head * D + c0 * 8;
#pragma unroll
      for (int i = 0; i < DO / 8; ++i)
        *reinterpret_cast<uint32_t*>(p + i * 8 + t4 * 2) =
            pack_bf16x2(dq_acc[i][h * 2] * scale, dq_acc[i][h * 2 + 1] * scale);
    }
  }
}

template <int D>
static int launch_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                      float* delta, void* dq, void* dk, void* dv, const int* cu_q, const int* cu_k,
                      const int* tile_prefix_q, const int* tile_prefix_k, int num_seqs, int total_q_tiles,
                      int total_k_tiles, long long total_q, int hq, int hkv, long long q_stride, long long k_stride,
                      long long v_stride, long long o_stride, long long do_stride, long long dq_stride,
                      long long dk_stride, long long dv_stride, float scale, int causal, int window, float* dkv_ws,
                      long long total_k, cudaStream_t stream) {
  constexpr int smem_kv = 6 * 64 * D * 2 + 4 * 64 * 4;
  constexpr int smem_q = 6 * 64 * D * 2;
  constexpr int DO = D > 128 ? 128 : D;
  constexpr int NZ = D / DO;
  static bool cfg_dev[kMaxDevices] = {};
    bool& cfg = per_device_flag(cfg_dev);
  if (!cfg) {
    cudaFuncSetAttribute(attn_bwd_dkv_kernel<D, DO>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_kv);
    cudaFuncSetAttribute(attn_bwd_dq_kernel<D, DO>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_q);
    cfg = true;
  }
  const long long nw = total_q * hq;
  attn_delta_kernel<<<(unsigned)((nw + 7) / 8), 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o,
                                                                  delta, total_q, hq, D, o_stride, do_stride);
  const int group = hq / hkv;
  if (group == 1 || total_k <= 0) dkv_ws = nullptr;
  attn_bwd_dkv_kernel<D, DO><<<dim3(total_k_tiles, dkv_ws != nullptr ? hq : hkv, NZ), 128, smem_kv, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)d_o, lse,
      delta, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, cu_q, cu_k, tile_prefix_k, num_seqs, hq, hkv, q_stride,
      k_stride, v_stride, do_stride, dk_stride, dv_stride, scale, causal, window, dkv_ws, total_k);
  if (dkv_ws != nullptr) {
    const long long work = 2 * total_k * (hkv * D / 4);
    long long blocks = (work + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    attn_dkv_reduce_kernel<<<(unsigned)blocks, 256, 0, stream>>>(dkv_ws, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, total_k,
                                                                 group, hkv * D, D, dk_stride, dv_stride);
  }
  attn_bwd_dq_kernel<D, DO><<<dim3(total_q_tiles, hq, NZ), 128, smem_q, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)d_o, lse,
      delta, (__nv_bfloat16*)dq, cu_q, cu_k, tile_prefix_q, num_seqs, hq, hkv, q_stride, k_stride, v_stride,
      do_stride, dq_stride, scale, causal, window);
  return (int)cudaGetLastError();
}

}  // namespace areno

using namespace areno;

// `delta` is fp32 scratch of hq * total_q elements.  `dkv_ws` (optional): fp32 scratch of
// 2 * (hq / hkv) * total_k * hkv * head_dim elements; with it the dK / dV kernel runs one CTA per (key tile, query
// head) and a second kernel adds the heads of every group (grouped-query attention only).
extern "C" int areno_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                              const float* lse, float* delta, void* dq, void* dk, void* dv, const int* cu_q,
                              const int* cu_k, const int* tile_prefix_q, const int* tile_prefix_k, int num_seqs,
                              int total_q_tiles, int total_k_tiles, long long total_q, int hq, int hkv, int head_dim,
                              long long q_stride, long long k_stride, long long v_stride, long long o_stride,
                              long long do_stride, long long dq_stride, long long dk_stride, long long dv_stride,
                              float scale, int causal, int window, float* dkv_ws, long long total_k,
                              cudaStream_t stream) {
  if (total_q <= 0) return 0;
  if (hq % hkv != 0) return -3;
  if (head_dim == 128)
    return launch_bwd<128>(q, k, v, o, d_o, lse, delta, dq, dk, dv, cu_q, cu_k, tile_prefix_q, tile_prefix_k,
                           num_seqs, total_q_tiles, total_k_tiles, total_q, hq, hkv, q_stride, k_stride, v_stride,
                           o_stride, do_stride, dq_stride, dk_stride, dv_stride, scale, causal, window, dkv_ws, total_k, stream);
  if (head_dim == 256)
    return launch_bwd<256>(q, k, v, o, d_o, lse, delta, dq, dk, dv, cu_q, cu_k, tile_prefix_q, tile_prefix_k,
                           num_seqs, total_q_tiles, total_k_tiles, total_q, hq, hkv, q_stride, k_stride, v_stride,
                           o_stride, do_stride, dq_stride, dk_stride, dv_stride, scale, causal, window, dkv_ws, total_k, stream);
  if (head_dim == 64)
    return launch_bwd<64>(q, k, v, o, d_o, lse, delta, dq, dk, dv, cu_q, cu_k, tile_prefix_q, tile_prefix_k,
                          num_seqs, total_q_tiles, total_k_tiles, total_q, hq, hkv, q_stride, k_stride, v_stride,
                          o_stride, do_stride, dq_stride, dk_stride, dv_stride, scale, causal, window, dkv_ws, total_k, stream);
  return -2;
}
