// Fused optimizer kernels on flat fp32 shards (sm_100a):
//   * AdamW with fp32 master weights: one pass reads grad/master/m/v, writes master/m/v and the
//     bf16 parameter shard.  Decoupled weight decay, eps outside the sqrt, bias correction
//     (semantics of areno/engine/optim/adamw_fp32_master.py:239-303).
//   * AdamW with block-scaled 8-bit moments (one fp32 scale per 32 elements; m as signed int8,
//     sqrt(v) as uint8), replacing the one-scale-per-shard scheme of
//     areno/engine/optim/adamw_8bit.py:263-292.
//   * sum of squares (two-stage, deterministic) for the gradient norm, and in-place scaling.
#include "common.cuh"
#include "launch.h"

namespace areno {

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale;
  const float* scale_ptr;  // optional device scalar multiplied into grad_scale (clip coefficient)
};

__global__ void __launch_bounds__(256)
adamw_fp32_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                  const float* __restrict__ grad, __nv_bfloat16* __restrict__ param_out, long long n, AdamArgs a) {
  if (a.scale_ptr != nullptr) a.grad_scale *= a.scale_ptr[0];
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 4 <= n) {
      float4 g4 = *reinterpret_cast<const float4*>(grad + i);
      float4 p4 = *reinterpret_cast<float4*>(master + i);
      float4 m4 = *reinterpret_cast<float4*>(m + i);
      float4 v4 = *reinterpret_cast<float4*>(v + i);
      float g[4] = {g4.x, g4.y, g4.z, g4.w}, p[4] = {p4.x, p4.y, p4.z, p4.w};
      float mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = g[j] * a.grad_scale;
        mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gj;
        vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gj * gj;
        const float mh = mm[j] / a.bc1, vh = vv[j] / a.bc2;
        p[j] = p[j] * (1.f - a.lr * a.weight_decay) - a.lr * mh / (sqrtf(vh) + a.eps);
      }
      *reinterpret_cast<float4*>(master + i) = make_float4(p[0], p[1], p[2], p[3]);
      *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      if (param_out != nullptr)
        *reinterpret_cast<uint2*>(param_out + i) = make_uint2(pack_bf16x2(p[0], p[1]), pack_bf16x2(p[2], p[3]));
    } else {
      for (long long k = i; k < n; ++k) {
        const float gj = grad[k] * a.grad_scale;
        const float mj = a.beta1 * m[k] + (1.f - a.beta1) * gj;
        const float vj = a.beta2 * v[k] + (1.f - a.beta2) * gj * gj;
        const float pj = master[k] * (1.f - a.lr * a.weight_decay) - a.lr * (mj / a.bc1) / (sqrtf(vj / a.bc2) + a.eps);
        m[k] = mj; v[k] = vj; master[k] = pj;
        if (param_out != nullptr) param_out[k] = __float2bfloat16_rn(pj);
      }
    }
  }
}

// 8-bit moments, blocks of 32 elements: one warp lane per element, warp = block.
// When `master` is null the bf16 parameter itself is the state that is updated.
__global__ void __launch_bounds__(256)
adamw_8bit_kernel(float* __restrict__ master, signed char* __restrict__ mq, unsigned char* __restrict__ vq,
                  float* __restrict__ m_scale, float* __restrict__ v_scale, const float* __restrict__ grad,
                  __nv_bfloat16* __restrict__ param, long long n, AdamArgs a) {
  if (a.scale_ptr != nullptr) a.grad_scale *= a.scale_ptr[0];
  const long long nblocks = (n + 31) / 32;
  const int lane = threadIdx.x & 31;
  for (long long blk = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); blk < nblocks; blk += (long long)gridDim.x * 8) {
    const long long i = blk * 32 + lane;
    const bool ok = i < n;
    const float ms = m_scale[blk], vs = v_scale[blk];
    float mj = ok ? (float)mq[i] * ms : 0.f;
    float sv = ok ? (float)vq[i] * vs : 0.f;  // sqrt(v)
    float vj = sv * sv;
    const float gj = ok ? grad[i] * a.grad_scale : 0.f;
    mj = a.beta1 * mj + (1.f - a.beta1) * gj;
    vj = a.beta2 * vj + (1.f - a.beta2) * gj * gj;
    if (ok) {
      float pj = master != nullptr ? master[i] : __bfloat162float(param[i]);
      pj = pj * (1.f - a.lr * a.weight_decay) - a.lr * (mj / a.bc1) / (sqrtf(vj / a.bc2) + a.eps);
      if (master != nullptr) master[i] = pj;
      if (param != nullptr) param[i] = __float2bfloat16_rn(pj);
    }
    const float m_abs = warp_max(fabsf(mj));
    const float sv_new = sqrtf(vj);
    const float v_max = warp_max(sv_new);
    const float nms = fmaxf(m_abs, 1e-30f) / 127.f;
    const float nvs = fmaxf(v_max, 1e-30f) / 255.f;
    if (ok) {
      mq[i] = (signed char)__float2int_rn(fminf(fmaxf(mj / nms, -127.f), 127.f));
      // round sqrt(v) up so a non-zero second moment never quantises to zero
      vq[i] = (unsigned char)min(255, (int)ceilf(sv_new / nvs));
    }
    if (lane == 0) { m_scale[blk] = nms; v_scale[blk] = nvs; }
  }
}

__global__ void __launch_bounds__(256)
sumsq_partial_kernel(const float* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float red[8];
  float acc = 0.f;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 4 <= n) {
      const float4 v = *reinterpret_cast<const float4*>(x + i);
      acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    } else {
      for (long long k = i; k < n; ++k) acc += x[k] * x[k];
    }
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
  }
}
__global__ void __launch_bounds__(256)
sumsq_final_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out, int accumulate) {
  __shared__ float red[8];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nparts; i += 256) acc += partial[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + t : t;
  }
}

__global__ void __launch_bounds__(256)
scale_kernel(float* __restrict__ x, long long n, const float* __restrict__ scale_ptr, float scale) {
  const float s = scale_ptr != nullptr ? scale_ptr[0] * scale : scale;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] *= s;
}

__global__ void __launch_bounds__(256)
cast_f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = __float2bfloat16_rn(x[i]);
}

static inline int grid_cap(long long work, int per_block, int cap) {
  long long g = (work + per_block - 1) / per_block;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace areno

using namespace areno;

extern "C" int areno_adamw_fp32(float* master, float* m, float* v, const float* grad, void* param_out, long long n,
                                float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                                float grad_scale, const float* scale_ptr, cudaStream_t stream) {
  if (n <= 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step),
             grad_scale, scale_ptr};
  adamw_fp32_kernel<<<grid_cap(n, 1024, 148 * 16), 256, 0, stream>>>(master, m, v, grad, (__nv_bfloat16*)param_out, n, a);
  return (int)cudaGetLastError();
}

extern "C" int areno_adamw_8bit(float* master, void* mq, void* vq, float* m_scale, float* v_scale, const float* grad,
                                void* param, long long n, float lr, float beta1, float beta2, float eps,
                                float weight_decay, int step, float grad_scale, const float* scale_ptr,
                                cudaStream_t stream) {
  if (n <= 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step),
             grad_scale, scale_ptr};
  adamw_8bit_kernel<<<grid_cap((n + 31) / 32, 8, 148 * 16), 256, 0, stream>>>(
      master, (signed char*)mq, (unsigned char*)vq, m_scale, v_scale, grad, (__nv_bfloat16*)param, n, a);
  return (int)cudaGetLastError();
}

// partial: fp32 scratch of at least areno_sumsq_blocks() elements.
extern "C" int areno_sumsq_blocks() { return 148 * 8; }
extern "C" int areno_sumsq(const float* x, long long n, float* partial, float* out, int accumulate,
                           cudaStream_t stream) {
  if (n <= 0) {
    if (!accumulate) cudaMemsetAsync(out, 0, sizeof(float), stream);
    return 0;
  }
  const int blocks = grid_cap(n, 1024, areno_sumsq_blocks());
  sumsq_partial_kernel<<<blocks, 256, 0, stream>>>(x, n, partial);
  sumsq_final_kernel<<<1, 256, 0, stream>>>(partial, blocks, out, accumulate);
  return (int)cudaGetLastError();
}

extern "C" int areno_scale_f32(float* x, long long n, const float* scale_ptr, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  scale_kernel<<<grid_cap(n, 256, 148 * 16), 256, 0, stream>>>(x, n, scale_ptr, scale);
  return (int)cudaGetLastError();
}

extern "C" int areno_cast_f32_bf16(const float* x, void* y, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_cap(n, 256, 148 * 16), 256, 0, stream>>>(x, (__nv_bfloat16*)y, n);
  return (int)cudaGetLastError();
}
