// Bandwidth-bound fused elementwise / normalisation kernels (sm_100a).
// All tensors are bf16 with 16-byte vector accesses (row length a multiple of 8) and fp32
// math.  Covers the reference's normalization.cu, activation.cu and embedding.cu, plus RoPE
// and the residual add that the reference leaves to a tracing compiler.
#include "common.cuh"
#include "launch.h"

namespace areno {

struct alignas(16) bf16x8 {
  uint32_t u[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  bf16x8 v = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = unpack_bf16x2(v.u[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  bf16x8 v;
#pragma unroll
  for (int i = 0; i < 4; ++i) v.u[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = v;
}
__device__ __forceinline__ void load8w(const void* w, int wf32, int idx, float (&f)[8]) {
  if (w == nullptr) {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = 1.f;
  } else if (wf32) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + idx);
    float4 a = p[0], b = p[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    load8(reinterpret_cast<const __nv_bfloat16*>(w) + idx, f);
  }
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// ---------------------------------------------------------------------------------
// RMSNorm forward, optional fused residual add.  One block per row, row cached in
// registers (VPT vectors of 8 per thread), single pass over HBM.
//   h = x (+ residual);  y = h * rsqrt(mean(h^2) + eps) * (w + w_offset)
// Writes y, optionally h (new residual stream) and inv_rms (fp32, for backward).
// ---------------------------------------------------------------------------------
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                   const void* __restrict__ w, int wf32, float w_offset, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ inv_rms, int rows, int H,
                   float eps) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = (size_t)row * H;
    float v[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        load8(x + base + vi * 8, v[i]);
        if (residual != nullptr) {
          float r[8];
          load8(residual + base + vi * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j] + r[j]));
          if (h_out != nullptr) store8(h_out + base + vi * 8, v[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    const float tot = block_sum<THREADS>(ss, red);
    const float inv = rsqrtf(tot / (float)H + eps);
    if (threadIdx.x == 0 && inv_rms != nullptr) inv_rms[row] = inv;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        float wv[8], o[8];
        load8w(w, wf32, vi * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j] * inv * (wv[j] + w_offset);
        store8(y + base + vi * 8, o);
      }
    }
  }
}

// Warp-per-row variant for short rows (per-head q/k norm, H <= 256).
__global__ void __launch_bounds__(256)
rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const void* __restrict__ w, int wf32,
                        float w_offset, __nv_bfloat16* __restrict__ y, float* __restrict__ inv_rms,
                        long long rows, int H, float eps) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float ss = 0.f;
  if (lane < nvec) {
    load8(x + row * H + lane * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)H + eps);
  if (lane == 0 && inv_rms != nullptr) inv_rms[row] = inv;
  if (lane < nvec) {
    float wv[8], o[8];
    load8w(w, wf32, lane * 8, wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = v[j] * inv * (wv[j] + w_offset);
    store8(y + row * H + lane * 8, o);
  }
}

// Per-head RMSNorm on strided [token, head, D] views (q/k norm inside a packed QKV buffer):
// row r -> token r / heads, head r % heads; element offset token * stride + head * D.  D <= 256.
__global__ void __launch_bounds__(256)
headnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride, const void* __restrict__ w, int wf32,
                    float w_offset, __nv_bfloat16* __restrict__ y, long long y_stride, float* __restrict__ inv_rms,
                    long long rows, int heads, int D, float eps) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long t = row / heads;
  const int hd = (int)(row % heads);
  const int nvec = D >> 3;
  float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float ss = 0.f;
  if (lane < nvec) {
    load8(x + t * x_stride + (long long)hd * D + lane * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)D + eps);
  if (lane == 0 && inv_rms != nullptr) inv_rms[row] = inv;
  if (lane < nvec) {
    float wv[8], o[8];
    load8w(w, wf32, lane * 8, wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = v[j] * inv * (wv[j] + w_offset);
    store8(y + t * y_stride + (long long)hd * D + lane * 8, o);
  }
}

// Backward of the per-head norm.  dx may alias dy (in place).  dW partials: one row of
// `dw_partial[gridDim.x, D]` per block (warps of a block are folded through shared memory).
__global__ void __launch_bounds__(256)
headnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, long long dy_stride, const __nv_bfloat16* __restrict__ x,
                    long long x_stride, const void* __restrict__ w, int wf32, float w_offset,
                    const float* __restrict__ inv_rms, __nv_bfloat16* __restrict__ dx, long long dx_stride,
                    float* __restrict__ dw_partial, long long rows, int heads, int D) {
  __shared__ float sdw[8][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = D >> 3;
  float wv[8], dwacc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { dwacc[j] = 0.f; wv[j] = 0.f; }
  if (lane < nvec) {
    load8w(w, wf32, lane * 8, wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) wv[j] += w_offset;
  }
  for (long long row = (long long)blockIdx.x * 8 + warp; row < rows; row += (long long)gridDim.x * 8) {
    const long long t = row / heads;
    const int hd = (int)(row % heads);
    const float inv = inv_rms[row];
    float d[8], xv[8], g[8];
    float dot = 0.f;
    if (lane < nvec) {
      load8(dy + t * dy_stride + (long long)hd * D + lane * 8, d);
      load8(x + t * x_stride + (long long)hd * D + lane * 8, xv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dwacc[j] += d[j] * xv[j] * inv;
        g[j] = d[j] * wv[j];
        dot += g[j] * xv[j];
      }
    }
    dot = warp_sum(dot);
    const float c = dot / (float)D * inv * inv;
    if (lane < nvec) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = inv * (g[j] - xv[j] * c);
      store8(dx + t * dx_stride + (long long)hd * D + lane * 8, o);
    }
  }
  if (dw_partial != nullptr) {
    if (lane < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) sdw[warp][lane * 8 + j] = dwacc[j];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < D; c += 256) {
      float s = 0.f;
#pragma unroll
      for (int ww = 0; ww < 8; ++ww) s += sdw[ww][c];
      dw_partial[(size_t)blockIdx.x * D + c] = s;
    }
  }
}

// RMSNorm backward.  Persistent blocks; each block keeps a partial dW in registers over
// its rows and writes it to `dw_partial[block, H]` (fp32 scratch); a second kernel folds
// the partials, so the result does not depend on atomics ordering.
//   g = dy * (w + off);  dx = inv * (g - h * inv^2 * mean(g*h)) (+ dres_in)
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                   const void* __restrict__ w, int wf32, float w_offset, const float* __restrict__ inv_rms,
                   const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int rows, int H) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  float dwacc[VPT][8];
  float wv[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    if (vi < nvec) {
      load8w(w, wf32, vi * 8, wv[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[i][j] += w_offset;
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = (size_t)row * H;
    const float inv = inv_rms[row];
    float g[VPT][8], hv[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        float d[8];
        load8(dy + base + vi * 8, d);
        load8(h + base + vi * 8, hv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dwacc[i][j] += d[j] * hv[i][j] * inv;
          g[i][j] = d[j] * wv[i][j];
          dot += g[i][j] * hv[i][j];
        }
      }
    }
    const float tot = block_sum<THREADS>(dot, red);
    const float c = tot / (float)H * inv * inv;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = inv * (g[i][j] - hv[i][j] * c);
        if (dres_in != nullptr) {
          float r[8];
          load8(dres_in + base + vi * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + base + vi * 8, o);
      }
    }
  }
  if (dw_partial != nullptr) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        float* p = dw_partial + (size_t)blockIdx.x * H + vi * 8;
        *reinterpret_cast<float4*>(p) = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
      }
    }
  }
}

// out[c] (+)= sum_b partial[b, c]
__global__ void colsum_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, int nblocks,
                                       int H, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[(size_t)b * H + c];
  out[c] = accumulate ? out[c] + s : s;
}

// ---------------------------------------------------------------------------------
// Gated activations: out[r, :I] = act(x[r, :I]) * x[r, I:2I]     (act: 0 = SiLU, 1 = GELU-tanh)
// ---------------------------------------------------------------------------------
__device__ __forceinline__ float act_fwd(float g, int kind) {
  if (kind == 0) return g / (1.f + __expf(-g));
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanhf(k0 * (g + k1 * g * g * g));
  return 0.5f * g * (1.f + t);
}
__device__ __forceinline__ float act_bwd(float g, int kind) {
  if (kind == 0) {
    const float s = 1.f / (1.f + __expf(-g));
    return s * (1.f + g * (1.f - s));
  }
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float u = k0 * (g + k1 * g * g * g);
  const float t = tanhf(u);
  const float du = k0 * (1.f + 3.f * k1 * g * g);
  return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * du;
}

__global__ void __launch_bounds__(256)
gated_act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, long long rows, int I,
                     int kind) {
  pdl_trigger();
  pdl_wait();
  const int nvec = I >> 3;
  const long long total = rows * nvec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / nvec;
    const int c = (int)(idx % nvec) * 8;
    float g[8], u[8], o[8];
    load8(x + r * 2 * I + c, g);
    load8(x + r * 2 * I + I + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = act_fwd(g[j], kind) * u[j];
    store8(out + r * I + c, o);
  }
}

// The same activation for an expert-sorted row buffer at inference: rows without a route (padding up to whole
// tiles; a decode step of 256 routes over 128 experts is 98 % padding) are neither read nor written.  Their
// content only ever reaches output rows that nobody gathers.
__global__ void __launch_bounds__(256)
gated_act_fwd_rows_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                          const int* __restrict__ row_route, long long rows, int I, int kind) {
  pdl_trigger();
  pdl_wait();
  const int nvec = I >> 3;
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += nwarps) {
    if (row_route[r] < 0) continue;
    for (int v = lane; v < nvec; v += 32) {
      float g[8], u[8], o[8];
      load8(x + r * 2 * I + v * 8, g);
      load8(x + r * 2 * I + I + v * 8, u);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = act_fwd(g[j], kind) * u[j];
      store8(out + r * I + v * 8, o);
    }
  }
}

__global__ void __launch_bounds__(256)
gated_act_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ x,
                     __nv_bfloat16* __restrict__ dx, long long rows, int I, int kind) {
  const int nvec = I >> 3;
  const long long total = rows * nvec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / nvec;
    const int c = (int)(idx % nvec) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(x + r * 2 * I + c, g);
    load8(x + r * 2 * I + I + c, u);
    load8(dout + r * I + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg[j] = d[j] * u[j] * act_bwd(g[j], kind);
      du[j] = d[j] * act_fwd(g[j], kind);
    }
    store8(dx + r * 2 * I + c, dg);
    store8(dx + r * 2 * I + I + c, du);
  }
}

// Plain unary activations: 0 silu, 1 sigmoid, 2 softplus (threshold 20).  mode 0 = fwd (y = f(x)),
// mode 1 = bwd (y = dy * f'(x)).
__global__ void __launch_bounds__(256)
unary_act_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                 __nv_bfloat16* __restrict__ y, long long n, int kind, int mode) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(x[i]);
    float o;
    if (mode == 0) {
      if (kind == 0) o = v / (1.f + __expf(-v));
      else if (kind == 1) o = 1.f / (1.f + __expf(-v));
      else o = v > 20.f ? v : log1pf(__expf(v));
    } else {
      const float s = 1.f / (1.f + __expf(-v));
      float d;
      if (kind == 0) d = s * (1.f + v * (1.f - s));
      else if (kind == 1) d = s * (1.f - s);
      else d = v > 20.f ? 1.f : s;
      o = __bfloat162float(dy[i]) * d;
    }
    y[i] = __float2bfloat16_rn(o);
  }
}

// ---------------------------------------------------------------------------------
// Rotary embedding (neox "rotate half" over the first rot_dim channels of each head), in place on
// a packed [tokens, heads, head_dim] view with row stride `row_stride` elements.  `sign` = -1 gives
// the backward (inverse rotation).  cos/sin computed on the fly from position and theta; optional
// `inv_freq` table overrides theta (scaled RoPE variants).  `interleaved` selects GPT-J pairing.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ positions, const float* __restrict__ inv_freq,
            long long tokens, int heads, int head_dim, int rot_dim, long long row_stride, float theta,
            float sign, int interleaved) {
  const int half = rot_dim >> 1;
  const long long total = tokens * heads * half;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int i = (int)(idx % half);
    const long long th = idx / half;
    const int hd = (int)(th % heads);
    const long long t = th / heads;
    const float f = inv_freq != nullptr ? inv_freq[i] : __powf(theta, -2.f * (float)i / (float)rot_dim);
    float s, c;
    sincosf((float)positions[t] * f, &s, &c);
    s *= sign;
    __nv_bfloat16* p = x + t * row_stride + (long long)hd * head_dim;
    const int i0 = interleaved ? 2 * i : i;
    const int i1 = interleaved ? 2 * i + 1 : i + half;
    const float a = __bfloat162float(p[i0]);
    const float b = __bfloat162float(p[i1]);
    p[i0] = __float2bfloat16_rn(a * c - b * s);
    p[i1] = __float2bfloat16_rn(b * c + a * s);
  }
}

// The same rotation for the usual layout (rotate-half pairing, 16-byte aligned heads, rot_dim a multiple of 16):
// one thread owns eight consecutive frequencies of one token, computes their sines and cosines once and applies
// them to `kHeadsPerThread` heads with 16-byte loads and stores.  The sine / cosine expressions are the ones of
// rope_kernel, so both kernels give the same bits.
constexpr int kRopeHeadsPerThread = 4;
__global__ void __launch_bounds__(256)
rope_vec_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                long long tokens, int heads, int head_dim, int rot_dim, long long row_stride, float theta, float sign) {
  const int half = rot_dim >> 1;
  const int chunks = half >> 3;
  const int hgroups = (heads + kRopeHeadsPerThread - 1) / kRopeHeadsPerThread;
  const long long total = tokens * hgroups * chunks;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(idx % chunks);
    const long long r = idx / chunks;
    const int hg = (int)(r % hgroups);
    const long long t = r / hgroups;
    const float pos = (float)positions[t];
    float c[8], sn[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = ch * 8 + j;
      const float f = inv_freq != nullptr ? inv_freq[i] : __powf(theta, -2.f * (float)i / (float)rot_dim);
      sincosf(pos * f, &sn[j], &c[j]);
      sn[j] *= sign;
    }
    const int h_end = min(heads, (hg + 1) * kRopeHeadsPerThread);
    for (int hd = hg * kRopeHeadsPerThread; hd < h_end; ++hd) {
      __nv_bfloat16* p = x + t * row_stride + (long long)hd * head_dim + ch * 8;
      float a[8], b[8], oa[8], ob[8];
      load8(p, a);
      load8(p + half, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        oa[j] = a[j] * c[j] - b[j] * sn[j];
        ob[j] = b[j] * c[j] + a[j] * sn[j];
      }
      store8(p, oa);
      store8(p + half, ob);
    }
  }
}

// ---------------------------------------------------------------------------------
// Vocab-parallel embedding: out[t] = ids[t] in [v0, v1) ? table[ids[t]-v0] : 0
// backward: dtable[ids[t]-v0] += dout[t]  (fp32 atomics into the main-grad buffer)
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                     __nv_bfloat16* __restrict__ out, long long tokens, int H, long long v0, long long v1,
                     float scale) {
  const int nvec = H >> 3;
  const long long total = tokens * nvec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int c = (int)(idx % nvec) * 8;
    const long long id = ids[t];
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (id >= v0 && id < v1) {
      load8(table + (id - v0) * H + c, f);
      if (scale != 1.f) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= scale;
      }
    }
    store8(out + t * H + c, f);
  }
}

__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                     float* __restrict__ dtable, long long tokens, int H, long long v0, long long v1, float scale) {
  const int nvec = H >> 3;
  const long long total = tokens * nvec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int c = (int)(idx % nvec) * 8;
    const long long id = ids[t];
    if (id < v0 || id >= v1) continue;
    float f[8];
    load8(dout + t * H + c, f);
    float* p = dtable + (id - v0) * H + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(p + j, f[j] * scale);
  }
}

// fp32 accumulate of a bf16 gradient: acc += g   (main-grad accumulation for non-GEMM params)
__global__ void __launch_bounds__(256)
accumulate_bf16_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ g, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    acc[i] += __bfloat162float(g[i]);
}

static inline int grid_for(long long work, int threads, int cap = 148 * 16) {
  long long g = (work + threads - 1) / threads;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace areno

using namespace areno;

#define RMS_DISPATCH(KERNEL, H, ...)                                             \
  do {                                                                           \
    const int nvec_ = (H) >> 3;                                                  \
    if (nvec_ <= 128) KERNEL<128, 1><<<grid, 128, 0, stream>>>(__VA_ARGS__);     \
    else if (nvec_ <= 256) KERNEL<128, 2><<<grid, 128, 0, stream>>>(__VA_ARGS__); \
    else if (nvec_ <= 512) KERNEL<256, 2><<<grid, 256, 0, stream>>>(__VA_ARGS__); \
    else if (nvec_ <= 1024) KERNEL<256, 4><<<grid, 256, 0, stream>>>(__VA_ARGS__); \
    else if (nvec_ <= 2048) KERNEL<512, 4><<<grid, 512, 0, stream>>>(__VA_ARGS__); \
    else return -2;                                                              \
  } while (0)

// Same dispatch through launch_pdl (kernels that start with pdl_trigger / pdl_wait).
#define RMS_DISPATCH_PDL(KERNEL, H, ...)                                                                  \
  do {                                                                                                    \
    const int nvec_ = (H) >> 3;                                                                           \
    cudaError_t e_ = cudaSuccess;                                                                         \
    if (nvec_ <= 128) e_ = launch_pdl(KERNEL<128, 1>, dim3(grid), dim3(128), 0, stream, __VA_ARGS__);     \
    else if (nvec_ <= 256) e_ = launch_pdl(KERNEL<128, 2>, dim3(grid), dim3(128), 0, stream, __VA_ARGS__); \
    else if (nvec_ <= 512) e_ = launch_pdl(KERNEL<256, 2>, dim3(grid), dim3(256), 0, stream, __VA_ARGS__); \
    else if (nvec_ <= 1024) e_ = launch_pdl(KERNEL<256, 4>, dim3(grid), dim3(256), 0, stream, __VA_ARGS__); \
    else if (nvec_ <= 2048) e_ = launch_pdl(KERNEL<512, 4>, dim3(grid), dim3(512), 0, stream, __VA_ARGS__); \
    else return -2;                                                                                       \
    if (e_ != cudaSuccess) return (int)e_;                                                                \
  } while (0)

extern "C" int areno_rmsnorm_fwd(const void* x, const void* residual, const void* w, int wf32, float w_offset,
                                 void* y, void* h_out, float* inv_rms, long long rows, int H, float eps,
                                 cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H % 8 != 0) return -3;
  if (H <= 256 && residual == nullptr) {
    const int grid = (int)((rows + 7) / 8);
    rmsnorm_fwd_warp_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, w, wf32, w_offset,
                                                      (__nv_bfloat16*)y, inv_rms, rows, H, eps);
    return (int)cudaGetLastError();
  }
  const int grid = (int)(rows < 148 * 32 ? rows : 148 * 32);
  RMS_DISPATCH(rmsnorm_fwd_kernel, H, (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, w, wf32, w_offset,
               (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, inv_rms, (int)rows, H, eps);
  return (int)cudaGetLastError();
}

// Number of persistent blocks (= rows of the fp32 scratch `dw_partial[blocks, H]`).
extern "C" int areno_rmsnorm_bwd_blocks(long long rows) {
  long long b = rows < 296 ? rows : 296;
  return (int)(b < 1 ? 1 : b);
}

extern "C" int areno_rmsnorm_bwd(const void* dy, const void* h, const void* w, int wf32, float w_offset,
                                 const float* inv_rms, const void* dres_in, void* dx, float* dw_partial,
                                 float* dw, int dw_accumulate, long long rows, int H, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H % 8 != 0) return -3;
  const int grid = areno_rmsnorm_bwd_blocks(rows);
  RMS_DISPATCH(rmsnorm_bwd_kernel, H, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, w, wf32, w_offset,
               inv_rms, (const __nv_bfloat16*)dres_in, (__nv_bfloat16*)dx, dw_partial, (int)rows, H);
  if (dw_partial != nullptr && dw != nullptr)
    colsum_partials_kernel<<<(H + 255) / 256, 256, 0, stream>>>(dw_partial, dw, grid, H, dw_accumulate);
  return (int)cudaGetLastError();
}

extern "C" int areno_gated_act_fwd(const void* x, void* out, long long rows, int I, int kind, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (I % 8 != 0) return -3;
  return (int)launch_pdl(gated_act_fwd_kernel, dim3(grid_for(rows * (I / 8), 256)), dim3(256), 0, stream,
                         (const __nv_bfloat16*)x, (__nv_bfloat16*)out, rows, I, kind);
}

extern "C" int areno_gated_act_fwd_rows(const void* x, void* out, const int* row_route, long long rows, int I, int kind,
                                        cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (I % 8 != 0 || row_route == nullptr) return -3;
  return (int)launch_pdl(gated_act_fwd_rows_kernel, dim3(grid_for(rows * 32, 256, 148 * 8)), dim3(256), 0, stream,
                         (const __nv_bfloat16*)x, (__nv_bfloat16*)out, row_route, rows, I, kind);
}

extern "C" int areno_gated_act_bwd(const void* dout, const void* x, void* dx, long long rows, int I, int kind,
                                   cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (I % 8 != 0) return -3;
  gated_act_bwd_kernel<<<grid_for(rows * (I / 8), 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)dout, (const __nv_bfloat16*)x, (__nv_bfloat16*)dx, rows, I, kind);
  return (int)cudaGetLastError();
}

extern "C" int areno_unary_act(const void* x, const void* dy, void* y, long long n, int kind, int mode,
                               cudaStream_t stream) {
  if (n <= 0) return 0;
  unary_act_kernel<<<grid_for(n, 256), 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                         (__nv_bfloat16*)y, n, kind, mode);
  return (int)cudaGetLastError();
}

extern "C" int areno_rope(void* x, const int* positions, const float* inv_freq, long long tokens, int heads,
                          int head_dim, int rot_dim, long long row_stride, float theta, float sign,
                          int interleaved, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (!interleaved && rot_dim % 16 == 0 && head_dim % 8 == 0 && row_stride % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const long long threads = tokens * ((heads + kRopeHeadsPerThread - 1) / kRopeHeadsPerThread) * (rot_dim / 16);
    rope_vec_kernel<<<grid_for(threads, 256), 256, 0, stream>>>((__nv_bfloat16*)x, positions, inv_freq, tokens, heads,
                                                                head_dim, rot_dim, row_stride, theta, sign);
    return (int)cudaGetLastError();
  }
  rope_kernel<<<grid_for(tokens * heads * (rot_dim / 2), 256), 256, 0, stream>>>(
      (__nv_bfloat16*)x, positions, inv_freq, tokens, heads, head_dim, rot_dim, row_stride, theta, sign,
      interleaved);
  return (int)cudaGetLastError();
}

extern "C" int areno_embedding_fwd(const long long* ids, const void* table, void* out, long long tokens, int H,
                                   long long v0, long long v1, float scale, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H % 8 != 0) return -3;
  embedding_fwd_kernel<<<grid_for(tokens * (H / 8), 256), 256, 0, stream>>>(
      ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, tokens, H, v0, v1, scale);
  return (int)cudaGetLastError();
}

extern "C" int areno_embedding_bwd(const long long* ids, const void* dout, float* dtable, long long tokens, int H,
                                   long long v0, long long v1, float scale, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H % 8 != 0) return -3;
  embedding_bwd_kernel<<<grid_for(tokens * (H / 8), 256), 256, 0, stream>>>(
      ids, (const __nv_bfloat16*)dout, dtable, tokens, H, v0, v1, scale);
  return (int)cudaGetLastError();
}

extern "C" int areno_accumulate_bf16(float* acc, const void* g, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  accumulate_bf16_kernel<<<grid_for(n, 256), 256, 0, stream>>>(acc, (const __nv_bfloat16*)g, n);
  return (int)cudaGetLastError();
}

extern "C" int areno_headnorm_fwd(const void* x, long long x_stride, const void* w, int wf32, float w_offset, void* y,
                                  long long y_stride, float* inv_rms, long long tokens, int heads, int D, float eps,
                                  cudaStream_t stream) {
  const long long rows = tokens * heads;
  if (rows <= 0) return 0;
  if (D % 8 != 0 || D > 256) return -3;
  headnorm_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(
      (const __nv_bfloat16*)x, x_stride, w, wf32, w_offset, (__nv_bfloat16*)y, y_stride, inv_rms, rows, heads, D, eps);
  return (int)cudaGetLastError();
}

extern "C" int areno_headnorm_bwd_blocks(long long rows) {
  long long b = (rows + 7) / 8;
  if (b > 592) b = 592;
  return (int)(b < 1 ? 1 : b);
}

extern "C" int areno_headnorm_bwd(const void* dy, long long dy_stride, const void* x, long long x_stride,
                                  const void* w, int wf32, float w_offset, const float* inv_rms, void* dx,
                                  long long dx_stride, float* dw_partial, float* dw, int dw_accumulate,
                                  long long tokens, int heads, int D, cudaStream_t stream) {
  const long long rows = tokens * heads;
  if (rows <= 0) return 0;
  if (D % 8 != 0 || D > 256) return -3;
  const int grid = areno_headnorm_bwd_blocks(rows);
  headnorm_bwd_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dy, dy_stride, (const __nv_bfloat16*)x, x_stride,
                                                w, wf32, w_offset, inv_rms, (__nv_bfloat16*)dx, dx_stride, dw_partial,
                                                rows, heads, D);
  if (dw_partial != nullptr && dw != nullptr)
    colsum_partials_kernel<<<(D + 255) / 256, 256, 0, stream>>>(dw_partial, dw, grid, D, dw_accumulate);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------
// Fold of split-K partials fused with the residual add and the RMSNorm that follows a
// row-parallel projection in a decoder block:
//   h = residual + sum_s ws[s];  y = h * rsqrt(mean h^2 + eps) * (w + w_offset)
// ws: fp32 [splits, rows, H] as left by areno_gemm_bf16_partials.  One block per row.
// ---------------------------------------------------------------------------------
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
splitk_residual_rmsnorm_kernel(const float* __restrict__ ws, int splits, long long split_stride,
                               const __nv_bfloat16* __restrict__ residual, const void* __restrict__ w, int wf32,
                               float w_offset, __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out,
                               int rows, int H, float eps) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const int nvec = H >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = (size_t)row * H;
    float v[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        if (residual != nullptr) {
          load8(residual + base + vi * 8, v[i]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
        }
        // batches of 8 splits: 16 independent 16-byte loads in flight before the first add (the
        // partials sit in L2; a one-split-at-a-time loop is a chain of L2 round trips)
        for (int s0 = 0; s0 < splits; s0 += 8) {
          float4 a[8], b[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (s0 + u < splits) {
              const float* p = ws + (size_t)(s0 + u) * split_stride + base + vi * 8;
              a[u] = __ldcg(reinterpret_cast<const float4*>(p));
              b[u] = __ldcg(reinterpret_cast<const float4*>(p + 4));
            } else {
              a[u] = make_float4(0.f, 0.f, 0.f, 0.f);
              b[u] = a[u];
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {   // fixed order: the sum does not depend on the batch size
            v[i][0] += a[u].x; v[i][1] += a[u].y; v[i][2] += a[u].z; v[i][3] += a[u].w;
            v[i][4] += b[u].x; v[i][5] += b[u].y; v[i][6] += b[u].z; v[i][7] += b[u].w;
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j]));
        if (h_out != nullptr) store8(h_out + base + vi * 8, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    const float tot = block_sum<THREADS>(ss, red);
    const float inv = rsqrtf(tot / (float)H + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        float wv[8], o[8];
        load8w(w, wf32, vi * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j] * inv * (wv[j] + w_offset);
        store8(y + base + vi * 8, o);
      }
    }
  }
}

extern "C" int areno_splitk_residual_rmsnorm(const float* ws, int splits, long long split_stride, const void* residual,
                                             const void* w, int wf32, float w_offset, void* y, void* h_out,
                                             long long rows, int H, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H % 8 != 0 || splits < 1 || w == nullptr) return -3;
  const int grid = (int)(rows < 148 * 32 ? rows : 148 * 32);
  RMS_DISPATCH_PDL(splitk_residual_rmsnorm_kernel, H, ws, splits, split_stride, (const __nv_bfloat16*)residual, w, wf32,
                   w_offset, (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, (int)rows, H, eps);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------
// RMSNorm backward with library-owned scratch (declared in no_alloc.h).
// The partial-dW rows go to a fixed device array instead of a caller buffer, so the call
// needs no allocator.  `g_rmsnorm_bwd_scratch` below is the host-side handle of that array,
// not a device address: the address differs per device and is looked up once per device with
// cudaGetSymbolAddress while that device is current, then cached in g_scratch_addr[].
// ---------------------------------------------------------------------------------
#include <mutex>

#include "no_alloc.h"

static __device__ __align__(256) float
    g_rmsnorm_bwd_scratch[(size_t)ARENO_RMSNORM_BWD_STATIC_BLOCKS * ARENO_RMSNORM_BWD_STATIC_MAX_H];

namespace {
float* g_scratch_addr[areno::kMaxDevices] = {};  // filled lazily, one slot per device ordinal
std::mutex g_scratch_mutex;

// Returns 0 and the device address of the scratch on the current device, or an error code.
int static_scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess) return (int)rc;
  if (dev < 0 || dev >= areno::kMaxDevices) return ARENO_NOALLOC_ERR_DEVICE;
  std::lock_guard<std::mutex> guard(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    rc = cudaGetSymbolAddress((void**)&p, g_rmsnorm_bwd_scratch);
    if (rc != cudaSuccess) return (int)rc;
    if (p == nullptr) return ARENO_NOALLOC_ERR_SYMBOL;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}
}  // namespace

extern "C" const char* areno_no_alloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -2: return "hidden size not supported by the RMSNorm kernels";
    case -3: return "hidden size must be a multiple of 8 and dy, h, inv_rms, dx must not be null";
    case ARENO_NOALLOC_ERR_H_TOO_LARGE:
      return "hidden size exceeds ARENO_RMSNORM_BWD_STATIC_MAX_H (8192): the fixed scratch cannot hold it; "
             "use areno_rmsnorm_bwd with caller-provided scratch";
    case ARENO_NOALLOC_ERR_SYMBOL: return "could not resolve the device address of the fixed scratch array";
    case ARENO_NOALLOC_ERR_DEVICE: return "device ordinal is outside the per-device table (64 entries)";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error code";
  }
}

extern "C" int areno_rmsnorm_bwd_static(const void* dy, const void* h, const void* w, int wf32, float w_offset,
                                        const float* inv_rms, const void* dres_in, void* dx, float* dw,
                                        int dw_accumulate, long long rows, int H, cudaStream_t stream) {
  if (H % 8 != 0) return -3;
  if (H > ARENO_RMSNORM_BWD_STATIC_MAX_H) return ARENO_NOALLOC_ERR_H_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);  // set-up on the first call per device
  if (rc != 0) return rc;
  if (rows <= 0) return 0;
  if (dy == nullptr || h == nullptr || inv_rms == nullptr || dx == nullptr) return -3;  // w, dres_in, dw may be null
  const int grid = (int)(rows < ARENO_RMSNORM_BWD_STATIC_BLOCKS ? rows : ARENO_RMSNORM_BWD_STATIC_BLOCKS);
  // Each of the `grid` blocks writes its whole H-wide row of the scratch (zeros included), and the
  // fold reads exactly those rows, so leftovers of earlier calls are never read.
  RMS_DISPATCH(rmsnorm_bwd_kernel, H, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, w, wf32, w_offset,
               inv_rms, (const __nv_bfloat16*)dres_in, (__nv_bfloat16*)dx, scratch, (int)rows, H);
  if (dw != nullptr)
    colsum_partials_kernel<<<(H + 255) / 256, 256, 0, stream>>>(scratch, dw, grid, H, dw_accumulate);
  return (int)cudaGetLastError();
}
