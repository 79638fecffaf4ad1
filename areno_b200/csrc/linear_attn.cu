// Kernels of the hybrid (linear-attention) layers: depthwise causal conv1d + SiLU over packed
// sequences (forward, backward, single-token decode with a rolling window cache), the gated
// delta-rule recurrence (forward, with per-slot state cache), and RMSNorm fused with a SiLU gate
// (forward / backward).  Roles of areno/accel/csrc/conv.cu, normalization.cu:84-178 and of the FLA
// fused_recurrent_gated_delta_rule kernel in the reference.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "launch.h"

namespace areno {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float dsilu_f(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

// ----------------------------------------------------------------------------------
// Depthwise causal conv1d + SiLU on packed rows.
//   pre[t, c] = sum_{j=0}^{K-1} w[c, j] * x[t - (K-1) + j, c]   (rows before the sequence start
//   come from `hist` when given: hist[seq, c, j] holds the K-1 inputs preceding the chunk)
//   y = silu(pre)
// seq_start[t] = first row of the sequence that row t belongs to; seq_id[t] = its index.
// ----------------------------------------------------------------------------------
template <int K>
__global__ void __launch_bounds__(256)
conv1d_silu_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride, const float* __restrict__ w,
                       const int* __restrict__ seq_start, const int* __restrict__ seq_id,
                       const float* __restrict__ hist, long long tokens, int C, __nv_bfloat16* __restrict__ y,
                       long long y_stride) {
  const long long total = tokens * C;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / C;
    const int c = (int)(i % C);
    const int s0 = seq_start[t];
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const long long src = t - (K - 1) + j;
      float v = 0.f;
      if (src >= s0) v = __bfloat162float(x[src * x_stride + c]);
      else if (hist != nullptr) {
        const int h = (int)(src - s0) + (K - 1);  // index into the K-1 history slots
        if (h >= 0) v = hist[((size_t)seq_id[t] * C + c) * (K - 1) + h];
      }
      acc += w[c * K + j] * v;
    }
    y[t * y_stride + c] = __float2bfloat16_rn(silu_f(acc));
  }
}

// dx[t, c] = sum_j w[c, j] * dpre[t + (K-1) - j, c] over rows of the same sequence; dpre = dy * silu'(pre)
// (pre recomputed).  dw accumulated per block into dw_partial[block, C*K] (folded by the caller).
template <int K>
__global__ void __launch_bounds__(256)
conv1d_silu_bwd_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride, const float* __restrict__ w,
                       const int* __restrict__ seq_start, const int* __restrict__ seq_end,
                       const __nv_bfloat16* __restrict__ dy, long long dy_stride, long long tokens, int C,
                       __nv_bfloat16* __restrict__ dx, long long dx_stride, float* __restrict__ dw) {
  // one thread per channel, blocks stride over row ranges: dw stays in registers
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float wv[K], dwv[K];
#pragma unroll
  for (int j = 0; j < K; ++j) { wv[j] = w[c * K + j]; dwv[j] = 0.f; }
  const long long rows_per = (tokens + gridDim.y - 1) / gridDim.y;
  const long long lo = (long long)blockIdx.y * rows_per;
  const long long hi = lo + rows_per < tokens ? lo + rows_per : tokens;
  for (long long t = lo; t < hi; ++t) {
    // dx[t] needs dpre at rows t .. t+K-1 (same sequence)
    const int s0 = seq_start[t];
    const int s1 = seq_end[t];
    float acc = 0.f;
#pragma unroll
    for (int d = 0; d < K; ++d) {
      const long long r = t + d;  // row whose pre-activation used x[t] with tap j = K-1-d
      if (r >= s1) break;
      float pre = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        const long long src = r - (K - 1) + j;
        if (src >= s0) pre += wv[j] * __bfloat162float(x[src * x_stride + c]);
      }
      const float dpre = __bfloat162float(dy[r * dy_stride + c]) * dsilu_f(pre);
      acc += wv[K - 1 - d] * dpre;
      if (d == 0) {
        // weight gradient of row t: dw[j] += dpre[t] * x[t-(K-1)+j]
#pragma unroll
        for (int j = 0; j < K; ++j) {
          const long long src = t - (K - 1) + j;
          if (src >= s0) dwv[j] += dpre * __bfloat162float(x[src * x_stride + c]);
        }
      }
    }
    dx[t * dx_stride + c] = __float2bfloat16_rn(acc);
  }
#pragma unroll
  for (int j = 0; j < K; ++j) dw[((size_t)blockIdx.y * C + c) * K + j] = dwv[j];
}

// After a prefill chunk: hist[slot[seq], c, :] = last K-1 inputs of the sequence (older history
// shifts in when the chunk is shorter than K-1).
template <int K>
__global__ void __launch_bounds__(256)
conv1d_update_hist_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride, const int* __restrict__ cu,
                          const int* __restrict__ slots, const int* __restrict__ fresh, int num_seqs, int C,
                          float* __restrict__ hist) {
  const long long total = (long long)num_seqs * C;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int s = (int)(i / C), c = (int)(i % C);
    const int lo = cu[s], hi = cu[s + 1];
    float* h = hist + ((size_t)slots[s] * C + c) * (K - 1);
    float old[K - 1];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) old[j] = (fresh != nullptr && fresh[s]) ? 0.f : h[j];
    const int n = hi - lo;
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
      const int back = (K - 1) - j;  // slot j holds the input `back` rows before the end of the sequence so far
      float v = 0.f;
      if (back <= n) {
        v = __bfloat162float(x[(long long)(hi - back) * x_stride + c]);
      } else {
#pragma unroll
        for (int m = 0; m < K - 1; ++m)
          if (m == j + n) v = old[m];  // older than this chunk: shifts in from the previous window
      }
      h[j] = v;
    }
  }
}

// Decode: one new row per slot; y = silu(w . [hist, x]); hist shifts by one.  Rows with active == 0
// leave the cache untouched.
template <int K>
__global__ void __launch_bounds__(256)
conv1d_silu_decode_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride, const float* __restrict__ w,
                          const int* __restrict__ active, int rows, int C, float* __restrict__ hist,
                          __nv_bfloat16* __restrict__ y, long long y_stride) {
  const long long total = (long long)rows * C;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / C), c = (int)(i % C);
    float* h = hist + ((size_t)r * C + c) * (K - 1);
    const float xv = __bfloat162float(x[(long long)r * x_stride + c]);
    float acc = w[c * K + K - 1] * xv;
    float win[K - 1];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) { win[j] = h[j]; acc += w[c * K + j] * win[j]; }
    y[(long long)r * y_stride + c] = __float2bfloat16_rn(silu_f(acc));
    if (active == nullptr || active[r] > 0) {
#pragma unroll
      for (int j = 0; j < K - 2; ++j) h[j] = win[j + 1];
      h[K - 2] = xv;
    }
  }
}

// ----------------------------------------------------------------------------------
// Gated delta rule, recurrent form.  One block per (sequence, value head); thread j owns column j
// of the state S[dk, dv] (dk registers), so the per-token products k^T S and q^T S are
// thread-local and k / q are broadcast from shared memory.
//   S <- exp(g_t) S;  u = k_t^T S;  d = beta_t (v_t - u);  S <- S + k_t d^T;  o_t = scale * q_t^T S
// With DELTA == false (beta unused) the delta correction is dropped (d = v_t): decayed linear ("lightning") attention,
// S <- exp(g) S + k_t v_t^T.  g is read at g[t * g_stride + head]; g_stride == 0 gives a per-head constant.
// q, k arrive l2-normalised.  state: fp32 [slots, Hv, DK, DV]; a sequence starts from its slot's
// state unless fresh[seq] != 0 and writes the final state back (when state != nullptr).
// ----------------------------------------------------------------------------------
template <int DK, bool DELTA>
__global__ void __launch_bounds__(128)
gdn_recurrent_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, long long qk_stride,
                     const __nv_bfloat16* __restrict__ v, long long v_stride, const float* __restrict__ g,
                     long long g_stride, const float* __restrict__ beta, const int* __restrict__ cu,
                     const int* __restrict__ slots, const int* __restrict__ fresh, const int* __restrict__ active,
                     float* __restrict__ state, int Hk, int Hv, int DV, float scale, __nv_bfloat16* __restrict__ out,
                     long long out_stride) {
  const int seq = blockIdx.x / Hv;
  const int hv = blockIdx.x % Hv;
  const int hk = hv / (Hv / Hk);
  const int j = threadIdx.x;  // value column
  const int lo = cu[seq], hi = cu[seq + 1];
  if (active != nullptr && active[seq] <= 0) return;
  __shared__ float sk[DK], sq[DK];
  float S[DK];
  const int slot = slots != nullptr ? slots[seq] : seq;
  float* st = state != nullptr ? state + (((size_t)slot * Hv + hv) * DK) * DV : nullptr;
  const bool start_zero = st == nullptr || (fresh != nullptr && fresh[seq] != 0);
#pragma unroll
  for (int i = 0; i < DK; ++i) S[i] = (!start_zero && j < DV) ? st[(size_t)i * DV + j] : 0.f;
  for (int t = lo; t < hi; ++t) {
    __syncthreads();
    for (int i = threadIdx.x; i < DK; i += blockDim.x) {
      sk[i] = __bfloat162float(k[(long long)t * qk_stride + hk * DK + i]);
      sq[i] = __bfloat162float(q[(long long)t * qk_stride + hk * DK + i]);
    }
    __syncthreads();
    if (j < DV) {
      const float a = __expf(g[(long long)t * g_stride + hv]);
      float d = __bfloat162float(v[(long long)t * v_stride + hv * DV + j]);
      if constexpr (DELTA) {
        float u = 0.f;
#pragma unroll
        for (int i = 0; i < DK; ++i) { S[i] *= a; u += sk[i] * S[i]; }
        d = beta[(long long)t * Hv + hv] * (d - u);
      } else {
#pragma unroll
        for (int i = 0; i < DK; ++i) S[i] *= a;
      }
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i) { S[i] += sk[i] * d; o += sq[i] * S[i]; }
      out[(long long)t * out_stride + hv * DV + j] = __float2bfloat16_rn(o * scale);
    }
  }
  if (st != nullptr && j < DV) {
#pragma unroll
    for (int i = 0; i < DK; ++i) st[(size_t)i * DV + j] = S[i];
  }
}

// ----------------------------------------------------------------------------------
// y = x * rsqrt(mean x^2 + eps) * w * silu(gate), rows of D <= 256 (one warp per row).
// ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rmsnorm_silu_gate_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate,
                             long long gate_stride, int gate_group, const float* __restrict__ w, long long rows, int D,
                             float eps, __nv_bfloat16* __restrict__ y, float* __restrict__ inv_rms) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  // gate rows: token = row / gate_group, head = row % gate_group, laid out [token, gate_stride] + head * D
  const __nv_bfloat16* grow = gate + (row / gate_group) * gate_stride + (row % gate_group) * D;
  float xv[8], ss = 0.f;
  const int n = D / 32;  // elements per lane (D multiple of 32, <= 256)
  for (int i = 0; i < n; ++i) {
    xv[i] = __bfloat162float(x[row * D + lane + i * 32]);
    ss += xv[i] * xv[i];
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)D + eps);
  if (lane == 0 && inv_rms != nullptr) inv_rms[row] = inv;
  for (int i = 0; i < n; ++i) {
    const int c = lane + i * 32;
    y[row * D + c] = __float2bfloat16_rn(xv[i] * inv * w[c] * silu_f(__bfloat162float(grow[c])));
  }
}

// dx, dgate, per-block dw partials.
__global__ void __launch_bounds__(256)
rmsnorm_silu_gate_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                             const __nv_bfloat16* __restrict__ gate, long long gate_stride, int gate_group,
                             const float* __restrict__ w, const float* __restrict__ inv_rms, long long rows, int D,
                             __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dgate, long long dgate_stride,
                             float* __restrict__ dw_partial) {
  __shared__ float sdw[8][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = D / 32;
  float dwacc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) dwacc[i] = 0.f;
  for (long long row = (long long)blockIdx.x * 8 + warp; row < rows; row += (long long)gridDim.x * 8) {
    const long long tok = row / gate_group;
    const int hd = (int)(row % gate_group);
    const __nv_bfloat16* grow = gate + tok * gate_stride + (long long)hd * D;
    __nv_bfloat16* dgrow = dgate + tok * dgate_stride + (long long)hd * D;
    const float inv = inv_rms[row];
    float xv[8], gm[8], dot = 0.f;
    for (int i = 0; i < n; ++i) {
      const int c = lane + i * 32;
      xv[i] = __bfloat162float(x[row * D + c]);
      const float gt = __bfloat162float(grow[c]);
      const float d = __bfloat162float(dy[row * D + c]);
      const float nx = xv[i] * inv;
      dgrow[c] = __float2bfloat16_rn(d * nx * w[c] * dsilu_f(gt));
      const float dn = d * silu_f(gt);       // gradient w.r.t. (nx * w)
      dwacc[i] += dn * nx;
      gm[i] = dn * w[c];                      // gradient w.r.t. nx
      dot += gm[i] * xv[i];
    }
    dot = warp_sum(dot);
    const float cst = dot / (float)D * inv * inv;
    for (int i = 0; i < n; ++i) dx[row * D + lane + i * 32] = __float2bfloat16_rn(inv * (gm[i] - xv[i] * cst));
  }
  for (int i = 0; i < n; ++i) sdw[warp][lane + i * 32] = dwacc[i];
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += 256) {
    float s = 0.f;
#pragma unroll
    for (int ww = 0; ww < 8; ++ww) s += sdw[ww][c];
    dw_partial[(size_t)blockIdx.x * D + c] = s;
  }
}

// ----------------------------------------------------------------------------------
// Backward of decayed linear attention  S_t = a S_{t-1} + k_t v_t^T,  o_t = scale q_t^T S_t  (a = exp(-slope_h),
// state starts at zero).  With G_t = scale q_t dO_t^T + a G_{t+1}:
//   dq_t = scale S_t dO_t        (forward scan, thread i owns row i of S)
//   dk_t = G_t v_t               (reverse scan, thread i owns row i of G)
//   dv_t = G_t^T k_t             (reverse scan, thread j owns column j of G)
// All three are the same loop  R <- a R + own * A;  out = scale * <R, B>  with different operands, so one
// kernel runs them as blockIdx.y = 0, 1, 2.  One block per (sequence, head); D = head_dim (q, k, v alike).
// The broadcast vectors A, B are double-buffered in shared memory: one barrier per token.
// ----------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128)
lightning_bwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                     const __nv_bfloat16* __restrict__ v, long long qkv_stride, const __nv_bfloat16* __restrict__ d_o,
                     long long do_stride, const float* __restrict__ slope, const int* __restrict__ cu, int H, float scale,
                     __nv_bfloat16* __restrict__ dq, __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                     long long dqkv_stride) {
  const int seq = blockIdx.x / H, h = blockIdx.x % H;
  const int role = blockIdx.y;
  const int lo = cu[seq], hi = cu[seq + 1];
  const int n = hi - lo;
  if (n <= 0) return;
  const float a = __expf(-slope[h]);
  const __nv_bfloat16 *own_p, *a_p, *b_p;
  long long own_s, a_s, b_s;
  __nv_bfloat16* out_p;
  if (role == 0) { own_p = k; own_s = qkv_stride; a_p = v; a_s = qkv_stride; b_p = d_o; b_s = do_stride; out_p = dq; }
  else if (role == 1) { own_p = q; own_s = qkv_stride; a_p = d_o; a_s = do_stride; b_p = v; b_s = qkv_stride; out_p = dk; }
  else { own_p = d_o; own_s = do_stride; a_p = q; a_s = qkv_stride; b_p = k; b_s = qkv_stride; out_p = dv; }
  __shared__ float sA[2][D], sB[2][D];
  float R[D];
#pragma unroll
  for (int i = 0; i < D; ++i) R[i] = 0.f;
  const int tid = threadIdx.x;
  const long long col = (long long)h * D + tid;
  for (int s = 0; s < n; ++s) {
    const long long t = role == 0 ? lo + s : hi - 1 - s;
    const int buf = s & 1;
    float own = 0.f;
    if (tid < D) {
      sA[buf][tid] = __bfloat162float(a_p[t * a_s + col]);
      sB[buf][tid] = __bfloat162float(b_p[t * b_s + col]);
      own = __bfloat162float(own_p[t * own_s + col]);
    }
    __syncthreads();
    if (tid < D) {
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < D; ++i) {
        R[i] = a * R[i] + own * sA[buf][i];
        acc += R[i] * sB[buf][i];
      }
      out_p[t * dqkv_stride + col] = __float2bfloat16_rn(acc * scale);
    }
  }
}

// ----------------------------------------------------------------------------------
// Group RMSNorm with a sigmoid gate: the hidden dimension is G groups of W channels, each group is
// normalised on its own:  y[r, g, c] = x * rsqrt(mean_c x^2 + eps) * w[g, c] * sigmoid(gate[r, g, c]).
// One warp per (row, group).  Role of areno/engine/layers/norm.py:60-105 in the reference.
// ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
group_rmsnorm_gate_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate,
                              long long gate_stride, const float* __restrict__ w, long long rows, int G, int W,
                              float eps, __nv_bfloat16* __restrict__ y, float* __restrict__ inv_rms) {
  const int lane = threadIdx.x & 31;
  const long long total = rows * G;
  for (long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); wid < total; wid += (long long)gridDim.x * 8) {
    const long long r = wid / G;
    const int g = (int)(wid % G);
    const __nv_bfloat16* xr = x + (r * G + g) * W;
    const __nv_bfloat16* gr = gate + r * gate_stride + (long long)g * W;
    float ss = 0.f;
    for (int c = lane; c < W; c += 32) { const float xv = __bfloat162float(xr[c]); ss += xv * xv; }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)W + eps);
    if (lane == 0 && inv_rms != nullptr) inv_rms[wid] = inv;
    __nv_bfloat16* yr = y + (r * G + g) * W;
    for (int c = lane; c < W; c += 32) {
      const float sg = 1.f / (1.f + __expf(-__bfloat162float(gr[c])));
      yr[c] = __float2bfloat16_rn(__bfloat162float(xr[c]) * inv * w[g * W + c] * sg);
    }
  }
}

// dx and dgate (one warp per (row, group)).
__global__ void __launch_bounds__(256)
group_rmsnorm_gate_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                              const __nv_bfloat16* __restrict__ gate, long long gate_stride,
                              const float* __restrict__ w, const float* __restrict__ inv_rms, long long rows, int G,
                              int W, __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dgate) {
  const int lane = threadIdx.x & 31;
  const long long total = rows * G;
  for (long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); wid < total; wid += (long long)gridDim.x * 8) {
    const long long r = wid / G;
    const int g = (int)(wid % G);
    const long long base = (r * G + g) * W;
    const __nv_bfloat16* gr = gate + r * gate_stride + (long long)g * W;
    const float inv = inv_rms[wid];
    float dot = 0.f;
    for (int c = lane; c < W; c += 32) {
      const float sg = 1.f / (1.f + __expf(-__bfloat162float(gr[c])));
      const float nx = __bfloat162float(x[base + c]) * inv;
      const float d = __bfloat162float(dy[base + c]);
      const float wv = w[g * W + c];
      dgate[base + c] = __float2bfloat16_rn(d * nx * wv * sg * (1.f - sg));
      dot += d * sg * wv * nx;          // <dn, n>
    }
    dot = warp_sum(dot) / (float)W;
    for (int c = lane; c < W; c += 32) {
      const float sg = 1.f / (1.f + __expf(-__bfloat162float(gr[c])));
      const float nx = __bfloat162float(x[base + c]) * inv;
      const float dn = __bfloat162float(dy[base + c]) * sg * w[g * W + c];
      dx[base + c] = __float2bfloat16_rn(inv * (dn - nx * dot));
    }
  }
}

// dw partials: thread = channel (of G*W), blockIdx.y = row range; part[blockIdx.y, G*W].
__global__ void __launch_bounds__(256)
group_rmsnorm_gate_dw_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                             const __nv_bfloat16* __restrict__ gate, long long gate_stride,
                             const float* __restrict__ inv_rms, long long rows, int G, int W,
                             float* __restrict__ part) {
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const int GW = G * W;
  if (ch >= GW) return;
  const int g = ch / W;
  const long long per = (rows + gridDim.y - 1) / gridDim.y;
  const long long lo = (long long)blockIdx.y * per;
  const long long hi = lo + per < rows ? lo + per : rows;
  float acc = 0.f;
  for (long long r = lo; r < hi; ++r) {
    const float sg = 1.f / (1.f + __expf(-__bfloat162float(gate[r * gate_stride + ch])));
    acc += __bfloat162float(dy[r * GW + ch]) * sg * __bfloat162float(x[r * GW + ch]) * inv_rms[r * G + g];
  }
  part[(size_t)blockIdx.y * GW + ch] = acc;
}

static inline int grid_for_elems(long long work, int per_block, int cap = 148 * 16) {
  long long g = (work + per_block - 1) / per_block;
  if (g > cap) g = cap;
  return (int)(g < 1 ? 1 : g);
}

}  // namespace areno

using namespace areno;

#define CONV_K_DISPATCH(K, ...)        \
  switch (K) {                         \
    case 2: { constexpr int KK = 2; __VA_ARGS__; break; } \
    case 3: { constexpr int KK = 3; __VA_ARGS__; break; } \
    case 4: { constexpr int KK = 4; __VA_ARGS__; break; } \
    default: return -2;                \
  }

extern "C" int areno_conv1d_silu_fwd(const void* x, long long x_stride, const float* w, const int* seq_start,
                                     const int* seq_id, const float* hist, long long tokens, int C, int K, void* y,
                                     long long y_stride, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  CONV_K_DISPATCH(K, (conv1d_silu_fwd_kernel<KK><<<grid_for_elems(tokens * C, 256), 256, 0, stream>>>(
                         (const __nv_bfloat16*)x, x_stride, w, seq_start, seq_id, hist, tokens, C, (__nv_bfloat16*)y,
                         y_stride)));
  return (int)cudaGetLastError();
}

// dw_partial: fp32 [row_blocks, C, K]; returns through *row_blocks_out how many were written.
extern "C" int areno_conv1d_silu_bwd_blocks(long long tokens) {
  long long b = (tokens + 255) / 256;
  if (b > 64) b = 64;
  return (int)(b < 1 ? 1 : b);
}
extern "C" int areno_conv1d_silu_bwd(const void* x, long long x_stride, const float* w, const int* seq_start,
                                     const int* seq_end, const void* dy, long long dy_stride, long long tokens, int C,
                                     int K, void* dx, long long dx_stride, float* dw_partial, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  dim3 grid((C + 127) / 128, areno_conv1d_silu_bwd_blocks(tokens));
  CONV_K_DISPATCH(K, (conv1d_silu_bwd_kernel<KK><<<grid, 128, 0, stream>>>(
                         (const __nv_bfloat16*)x, x_stride, w, seq_start, seq_end, (const __nv_bfloat16*)dy, dy_stride,
                         tokens, C, (__nv_bfloat16*)dx, dx_stride, dw_partial)));
  return (int)cudaGetLastError();
}

extern "C" int areno_conv1d_update_hist(const void* x, long long x_stride, const int* cu, const int* slots,
                                        const int* fresh, int num_seqs, int C, int K, float* hist,
                                        cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  CONV_K_DISPATCH(K, (conv1d_update_hist_kernel<KK><<<grid_for_elems((long long)num_seqs * C, 256), 256, 0, stream>>>(
                         (const __nv_bfloat16*)x, x_stride, cu, slots, fresh, num_seqs, C, hist)));
  return (int)cudaGetLastError();
}

extern "C" int areno_conv1d_silu_decode(const void* x, long long x_stride, const float* w, const int* active, int rows,
                                        int C, int K, float* hist, void* y, long long y_stride, cudaStream_t stream) {
  if (rows <= 0) return 0;
  CONV_K_DISPATCH(K, (conv1d_silu_decode_kernel<KK><<<grid_for_elems((long long)rows * C, 256), 256, 0, stream>>>(
                         (const __nv_bfloat16*)x, x_stride, w, active, rows, C, hist, (__nv_bfloat16*)y, y_stride)));
  return (int)cudaGetLastError();
}

extern "C" int areno_gdn_recurrent(const void* q, const void* k, long long qk_stride, const void* v, long long v_stride,
                                   const float* g, const float* beta, const int* cu, const int* slots,
                                   const int* fresh, const int* active, float* state, int num_seqs, int Hk, int Hv,
                                   int DK, int DV, float scale, void* out, long long out_stride, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (DV > 128 || Hv % Hk != 0) return -3;
  const int grid = num_seqs * Hv;
  const long long g_stride = Hv;
#define GDN_LAUNCH(D)                                                                                             \
  gdn_recurrent_kernel<D, true><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, qk_stride, \
                                                    (const __nv_bfloat16*)v, v_stride, g, g_stride, beta, cu, slots, \
                                                    fresh, active, state, Hk, Hv, DV, scale, (__nv_bfloat16*)out,  \
                                                    out_stride)
  if (DK == 128) GDN_LAUNCH(128);
  else if (DK == 64) GDN_LAUNCH(64);
  else if (DK == 32) GDN_LAUNCH(32);
  else return -2;
#undef GDN_LAUNCH
  return (int)cudaGetLastError();
}

extern "C" int areno_rmsnorm_silu_gate_fwd(const void* x, const void* gate, long long gate_stride, int gate_group,
                                           const float* w, long long rows, int D, float eps, void* y, float* inv_rms,
                                           cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D % 32 != 0 || D > 256) return -3;
  rmsnorm_silu_gate_fwd_kernel<<<(int)((rows + 7) / 8), 256, 0, stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, gate_stride, gate_group, w, rows, D, eps, (__nv_bfloat16*)y,
      inv_rms);
  return (int)cudaGetLastError();
}

extern "C" int areno_rmsnorm_silu_gate_bwd_blocks(long long rows) {
  long long b = (rows + 7) / 8;
  if (b > 592) b = 592;
  return (int)(b < 1 ? 1 : b);
}
extern "C" int areno_rmsnorm_silu_gate_bwd(const void* dy, const void* x, const void* gate, long long gate_stride,
                                           int gate_group, const float* w, const float* inv_rms, long long rows, int D,
                                           void* dx, void* dgate, long long dgate_stride, float* dw_partial,
                                           cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D % 32 != 0 || D > 256) return -3;
  rmsnorm_silu_gate_bwd_kernel<<<areno_rmsnorm_silu_gate_bwd_blocks(rows), 256, 0, stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, gate_stride, gate_group, w, inv_rms,
      rows, D, (__nv_bfloat16*)dx, (__nv_bfloat16*)dgate, dgate_stride, dw_partial);
  return (int)cudaGetLastError();
}

// Decayed linear attention forward (prefill chunks and decode rows; training forward with state == nullptr).
// log_decay: fp32 [H] = -slope.  q, k, v: [T, H, D] views sharing `qkv_stride`.
extern "C" int areno_lightning_recurrent(const void* q, const void* k, const void* v, long long qkv_stride,
                                         const float* log_decay, const int* cu, const int* slots, const int* fresh,
                                         const int* active, float* state, int num_seqs, int H, int D, float scale,
                                         void* out, long long out_stride, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (D > 128) return -3;
  const int grid = num_seqs * H;
#define LA_LAUNCH(DD)                                                                                                \
  gdn_recurrent_kernel<DD, false><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, qkv_stride,  \
                                                     (const __nv_bfloat16*)v, qkv_stride, log_decay, 0, nullptr, cu, \
                                                     slots, fresh, active, state, H, H, DD, scale,                   \
                                                     (__nv_bfloat16*)out, out_stride)
  if (D == 128) LA_LAUNCH(128);
  else if (D == 64) LA_LAUNCH(64);
  else if (D == 32) LA_LAUNCH(32);
  else return -2;
#undef LA_LAUNCH
  return (int)cudaGetLastError();
}

extern "C" int areno_lightning_bwd(const void* q, const void* k, const void* v, long long qkv_stride, const void* d_o,
                                   long long do_stride, const float* slope, const int* cu, int num_seqs, int H, int D,
                                   float scale, void* dq, void* dk, void* dv, long long dqkv_stride,
                                   cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  const dim3 grid(num_seqs * H, 3);
#define LB_LAUNCH(DD)                                                                                               \
  lightning_bwd_kernel<DD><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k,              \
                                                     (const __nv_bfloat16*)v, qkv_stride, (const __nv_bfloat16*)d_o, \
                                                     do_stride, slope, cu, H, scale, (__nv_bfloat16*)dq,             \
                                                     (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, dqkv_stride)
  if (D == 128) LB_LAUNCH(128);
  else if (D == 64) LB_LAUNCH(64);
  else if (D == 32) LB_LAUNCH(32);
  else return -2;
#undef LB_LAUNCH
  return (int)cudaGetLastError();
}

extern "C" int areno_group_rmsnorm_gate_fwd(const void* x, const void* gate, long long gate_stride, const float* w,
                                            long long rows, int G, int W, float eps, void* y, float* inv_rms,
                                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  group_rmsnorm_gate_fwd_kernel<<<grid_for_elems(rows * G, 8), 256, 0, stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, gate_stride, w, rows, G, W, eps, (__nv_bfloat16*)y, inv_rms);
  return (int)cudaGetLastError();
}

extern "C" int areno_group_rmsnorm_gate_dw_blocks(long long rows) {
  long long b = (rows + 63) / 64;
  if (b > 64) b = 64;
  return (int)(b < 1 ? 1 : b);
}

// dw_partial: fp32 [areno_group_rmsnorm_gate_dw_blocks(rows), G * W], folded by the caller.
extern "C" int areno_group_rmsnorm_gate_bwd(const void* dy, const void* x, const void* gate, long long gate_stride,
                                            const float* w, const float* inv_rms, long long rows, int G, int W,
                                            void* dx, void* dgate, float* dw_partial, cudaStream_t stream) {
  if (rows <= 0) return 0;
  group_rmsnorm_gate_bwd_kernel<<<grid_for_elems(rows * G, 8), 256, 0, stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, gate_stride, w, inv_rms, rows, G, W,
      (__nv_bfloat16*)dx, (__nv_bfloat16*)dgate);
  const dim3 grid((G * W + 255) / 256, areno_group_rmsnorm_gate_dw_blocks(rows));
  group_rmsnorm_gate_dw_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                         (const __nv_bfloat16*)gate, gate_stride, inv_rms, rows, G, W,
                                                         dw_partial);
  return (int)cudaGetLastError();
}
