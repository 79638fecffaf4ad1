// Fused token-level clipped policy loss (PPO dual-clip / GRPO) forward + gradient in one pass.
// Per token t (fp32 vectors):
//   d      = clamp(lp - old, -20, 20)          (old == nullptr: on-policy surrogate, d = 0)
//   r      = exp(d);  rc = clamp(r, 1-eps, 1+eps)
//   l1     = -r A;  l2 = -rc A;  lc = max(l1, l2)
//   loss   = A < 0 && dual_c > 0 ? min(-A dual_c, lc) : lc
//   kl     = estimator(lp, ref) when kl_type >= 0      (0 k1, 1 abs, 2 k2, 3 k3)
// Outputs: loss[t], kl[t], dloss/dlp[t], dkl/dlp[t], flags[t] (bit0: upper clip active,
// bit1: dual-clip active).  Masked means are taken by the caller.
// Math of areno/api/loss_fns/ppo.py:42-99 and grpo.py:25-31 in the reference.
#include "common.cuh"
#include "launch.h"

namespace areno {

__global__ void __launch_bounds__(256)
policy_loss_kernel(const float* __restrict__ lp, const float* __restrict__ old_lp, const float* __restrict__ adv,
                   const float* __restrict__ ref_lp, float* __restrict__ loss, float* __restrict__ kl,
                   float* __restrict__ dloss, float* __restrict__ dkl, int* __restrict__ flags, long long n,
                   float clip_lo, float clip_hi, float dual_c, int kl_type) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float x = lp[i];
    const float a = adv[i];
    float d = old_lp != nullptr ? x - old_lp[i] : 0.f;
    const bool d_clamped = d < -20.f || d > 20.f;
    d = fminf(fmaxf(d, -20.f), 20.f);
    const float r = __expf(d);
    const float dr = d_clamped ? 0.f : r;  // dr/dlp
    const float rc = fminf(fmaxf(r, 1.f - clip_lo), 1.f + clip_hi);
    const bool rc_active = (r < 1.f - clip_lo) || (r > 1.f + clip_hi);
    const float l1 = -r * a, l2 = -rc * a;
    float l, g;
    int f = 0;
    if (l2 > l1) { l = l2; g = rc_active ? 0.f : -a * dr; f |= 1; }
    else { l = l1; g = -a * dr; }
    if (a < 0.f && dual_c > 0.f) {
      const float l3 = -a * dual_c;
      if (l > l3) { l = l3; g = 0.f; f |= 2; }
    }
    loss[i] = l;
    dloss[i] = g;
    if (flags != nullptr) flags[i] = f;
    if (kl != nullptr) {
      float k = 0.f, gk = 0.f;
      if (kl_type >= 0 && ref_lp != nullptr) {
        const float e = x - ref_lp[i];
        if (kl_type == 0) { k = e; gk = 1.f; }
        else if (kl_type == 1) { k = fabsf(e); gk = e > 0.f ? 1.f : (e < 0.f ? -1.f : 0.f); }
        else if (kl_type == 2) { k = 0.5f * e * e; gk = e; }
        else {
          const bool c = (-e) < -20.f || (-e) > 20.f;
          const float ne = fminf(fmaxf(-e, -20.f), 20.f);
          const float ex = __expf(ne);
          const float raw = ex - ne - 1.f;
          k = fminf(fmaxf(raw, -10.f), 10.f);
          gk = (c || raw < -10.f || raw > 10.f) ? 0.f : (1.f - ex);  // d/dlp of exp(-e) + e - 1
        }
      }
      kl[i] = k;
      if (dkl != nullptr) dkl[i] = gk;
    }
  }
}

}  // namespace areno

using namespace areno;

extern "C" int areno_policy_loss(const float* lp, const float* old_lp, const float* adv, const float* ref_lp,
                                 float* loss, float* kl, float* dloss, float* dkl, int* flags, long long n,
                                 float clip_lo, float clip_hi, float dual_c, int kl_type, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long g = (n + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  policy_loss_kernel<<<(unsigned)g, 256, 0, stream>>>(lp, old_lp, adv, ref_lp, loss, kl, dloss, dkl, flags, n, clip_lo,
                                                      clip_hi, dual_c, kl_type);
  return (int)cudaGetLastError();
}
