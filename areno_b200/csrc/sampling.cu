// Vocabulary-wide reductions (sm_100a): token log-prob / entropy for training, and the decode
// sampler.  One CTA per row, single pass with online log-sum-exp, 16-byte loads.
//
//   * logprob_stats : per row (max, sum exp(x-max), sum exp(x-max)*x, x[target]) over a vocab
//     shard; shards combine with three tiny reductions, the [T, V] probabilities are never
//     materialised (the reference keeps an fp32 probability shard for backward,
//     areno/engine/runtime/logprobs.py:172-235).
//   * logprob_bwd   : in place, logits <- d(loss)/d(logits) from d/d(logprob) and d/d(entropy).
//   * sample        : greedy / temperature / top-k / top-p sampling by the Gumbel-max trick with
//     counter-based Philox noise keyed on (seed, row uid, step, global token id).  Every TP rank
//     that runs it on its shard with the same key draws consistent noise, so shards combine with
//     one small gather and no token-id broadcast.  The returned log-prob is the raw-logit
//     log-softmax at temperature 1 (areno/engine/data/sampling.py:154-160).
#include "common.cuh"
#include "launch.h"

namespace areno {

struct OnlineLse {
  float m, s, sx;  // running max, sum exp(x-m), sum exp(x-m)*x
  __device__ __forceinline__ void init() { m = -INFINITY; s = 0.f; sx = 0.f; }
  __device__ __forceinline__ void add(float x) {
    if (x == -INFINITY) return;
    if (x > m) {
      const float c = __expf(m - x);
      s = s * c + 1.f;
      sx = sx * c + x;
      m = x;
    } else {
      const float e = __expf(x - m);
      s += e;
      sx += e * x;
    }
  }
  __device__ __forceinline__ void merge(const OnlineLse& o) {
    if (o.m == -INFINITY) return;
    if (m == -INFINITY) { *this = o; return; }
    const float mn = fmaxf(m, o.m);
    const float a = __expf(m - mn), b = __expf(o.m - mn);
    s = s * a + o.s * b;
    sx = sx * a + o.sx * b;
    m = mn;
  }
};

__device__ __forceinline__ OnlineLse warp_merge(OnlineLse v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    OnlineLse t;
    t.m = __shfl_xor_sync(0xffffffffu, v.m, o);
    t.s = __shfl_xor_sync(0xffffffffu, v.s, o);
    t.sx = __shfl_xor_sync(0xffffffffu, v.sx, o);
    v.merge(t);
  }
  return v;
}

template <typename T>
__device__ __forceinline__ float load_logit(const T* p, long long i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}

// Load 8 consecutive logits starting at element i (i multiple of 8, row base 16-byte aligned).
template <typename T>
__device__ __forceinline__ void load_logits8(const T* p, long long i, float (&f)[8]);
template <>
__device__ __forceinline__ void load_logits8<float>(const float* p, long long i, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p + i);
  const float4 b = *reinterpret_cast<const float4*>(p + i + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load_logits8<__nv_bfloat16>(const __nv_bfloat16* p, long long i, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p + i);
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = unpack_bf16x2(u[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}

constexpr int kRowThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
logprob_stats_kernel(const T* __restrict__ logits, long long ld, int V, const long long* __restrict__ targets,
                     long long vocab_start, float* __restrict__ out_max, float* __restrict__ out_sum,
                     float* __restrict__ out_sumx, float* __restrict__ out_tgt) {
  __shared__ OnlineLse red[kRowThreads / 32];
  const long long row = blockIdx.x;
  const T* p = logits + row * ld;
  OnlineLse acc;
  acc.init();
  const int nvec = V >> 3;
  for (int v = threadIdx.x; v < nvec; v += kRowThreads) {
    float f[8];
    load_logits8<T>(p, (long long)v * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc.add(f[j]);
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += kRowThreads) acc.add(load_logit<T>(p, i));
  acc = warp_merge(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    OnlineLse t;
    t.init();
    if (threadIdx.x < kRowThreads / 32) t = red[threadIdx.x];
    t = warp_merge(t);
    if (threadIdx.x == 0) {
      out_max[row] = t.m;
      out_sum[row] = t.s;
      if (out_sumx != nullptr) out_sumx[row] = t.sx;
      const long long tg = targets[row] - vocab_start;
      out_tgt[row] = (tg >= 0 && tg < V) ? load_logit<T>(p, tg) : 0.f;
    }
  }
}

// logits[row, i] <- dlp[row] * (onehot_i - p_i) + dent[row] * (-p_i * (x_i - ex[row]))
// with p_i = exp(x_i - lse[row]).  Rows with both gradients zero are zero-filled.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
logprob_bwd_kernel(T* __restrict__ logits, long long ld, int V, const long long* __restrict__ targets,
                   long long vocab_start, const float* __restrict__ lse, const float* __restrict__ ex,
                   const float* __restrict__ dlp, const float* __restrict__ dent) {
  const long long row = blockIdx.x;
  T* p = logits + row * ld;
  const float l = lse[row];
  const float g = dlp[row];
  const float ge = dent != nullptr ? dent[row] : 0.f;
  const float e = ex != nullptr ? ex[row] : 0.f;
  const long long tg = targets[row] - vocab_start;
  for (int i = threadIdx.x; i < V; i += kRowThreads) {
    const float x = load_logit<T>(p, i);
    const float pr = __expf(x - l);
    float d = -g * pr - ge * pr * (x - e);
    if (i == tg) d += g;
    if constexpr (sizeof(T) == 2) p[i] = __float2bfloat16_rn(d);
    else p[i] = d;
  }
}

// ------------------------------- Philox4x32-10 -----------------------------------
__device__ __forceinline__ uint4 philox4x32(uint4 ctr, uint2 key) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}
__device__ __forceinline__ float gumbel_from_bits(uint32_t bits) {
  const float u = ((float)(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
  return -__logf(-__logf(u));
}

struct Best {
  float v;
  int idx;
  __device__ __forceinline__ void take(float nv, int ni) {
    if (nv > v || (nv == v && ni < idx)) { v = nv; idx = ni; }
  }
};
__device__ __forceinline__ Best warp_best(Best b) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, b.idx, o);
    b.take(ov, oi);
  }
  return b;
}

__device__ __forceinline__ uint32_t float_to_ordered(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ordered_to_float(uint32_t o) {
  const uint32_t u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
  return __uint_as_float(u);
}

template <int THREADS>
__device__ __forceinline__ float block_sum_f(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < THREADS / 32 ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
    t = warp_sum(t);
    if (threadIdx.x == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// part (optional, TP mode): float[rows, 6] = {best score, best global id, raw logit at best, raw max,
// raw sum-exp, unused}; when part == nullptr the kernel finalises token + logprob itself.
// With gridDim.y > 1 the vocabulary of a row is cut into slices of `slice_len` tokens (a multiple of 4, so
// the random counters do not move): block (row, slice) writes its record to slice_part[slice][row] and
// sample_combine_kernel picks the winner - one CTA per row cannot keep a B200 busy at 64 rows.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
sample_kernel(const T* __restrict__ logits, long long ld, int V, int vocab_start, const signed char* __restrict__ cls,
              const int* __restrict__ gen_count, int min_new, float temperature, int top_k, float top_p,
              unsigned long long seed, const long long* __restrict__ row_uid, long long* __restrict__ out_token,
              float* __restrict__ out_logprob, float* __restrict__ part, int slice_len, float* __restrict__ slice_part) {
  __shared__ OnlineLse red_lse[kRowThreads / 32];
  __shared__ Best red_best[kRowThreads / 32];
  __shared__ float red_f[32];
  __shared__ float sh_thresh;
  const long long row = blockIdx.x;
  const T* p = logits + row * ld;
  if (gridDim.y > 1) {
    const int v0 = (int)blockIdx.y * slice_len;
    p += v0;
    vocab_start += v0;
    V = min(slice_len, V - v0);
    part = slice_part + (long long)blockIdx.y * gridDim.x * 6;
  }
  const int step = gen_count != nullptr ? gen_count[row] : 0;
  const bool mask_eos = step < min_new;
  const bool greedy = temperature <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temperature;
  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  const unsigned long long uid = row_uid != nullptr ? (unsigned long long)row_uid[row] : (unsigned long long)row;

  auto masked = [&](int i, float x) -> float {
    if (x != x) return -INFINITY;  // NaN
    if (cls != nullptr) {
      const signed char c = cls[vocab_start + i];
      if (c == 1 || (c == 2 && mask_eos)) return -INFINITY;
    }
    return x;
  };

  // ---- optional truncation threshold (top-k / top-p) on the masked, tempered distribution ----
  float thresh = -INFINITY;
  const bool truncate = !greedy && (top_k > 0 || top_p < 1.f);
  if (truncate) {
    // masked max and partition function at temperature T
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += kRowThreads) mx = fmaxf(mx, masked(i, load_logit<T>(p, i)));
    mx = warp_max(mx);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red_f[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = -INFINITY;
    for (int w = 0; w < kRowThreads / 32; ++w) mx = fmaxf(mx, red_f[w]);
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += kRowThreads) {
      const float x = masked(i, load_logit<T>(p, i));
      if (x != -INFINITY) z += __expf((x - mx) * inv_t);
    }
    z = block_sum_f<kRowThreads>(z, red_f);
    // bisection over the order-preserving integer image of fp32: lo fails the keep test, hi passes
    uint32_t lo = float_to_ordered(-INFINITY), hi = float_to_ordered(mx);
    // keep-test(t): count(x >= t) <= k  and  mass(x > t_prev...) handled as: elements kept are x >= t
    // top-k: smallest t with count(x >= t) <= k  -> kept = {x >= t}
    // top-p: kept = {x : mass(y > x) <= p}; with g(t) = mass(y >= t), kept = {x >= t*}, t* smallest t with
    //        mass(y > t) <= p.  Both tests are monotone in t, so one bisection finds max of the two.
    for (int it = 0; it < 33 && hi - lo > 1; ++it) {
      const uint32_t mid = lo + ((hi - lo) >> 1);
      const float t = ordered_to_float(mid);
      float cnt = 0.f, mass_gt = 0.f;
      for (int i = threadIdx.x; i < V; i += kRowThreads) {
        const float x = masked(i, load_logit<T>(p, i));
        if (x >= t) cnt += 1.f;
        if (x > t) mass_gt += __expf((x - mx) * inv_t);
      }
      cnt = block_sum_f<kRowThreads>(cnt, red_f);
      mass_gt = block_sum_f<kRowThreads>(mass_gt, red_f);
      bool pass = true;
      if (top_k > 0 && cnt > (float)top_k) pass = false;   // too many kept at this threshold: raise it
      if (pass && top_p < 1.f && mass_gt > top_p * z) {
        // elements equal to t would be preceded by more than p of the mass: t is still too low
        pass = false;
      }
      if (pass) hi = mid; else lo = mid;
    }
    if (threadIdx.x == 0) sh_thresh = ordered_to_float(hi);
    __syncthreads();
    thresh = sh_thresh;
  }

  // ---- main pass: raw log-sum-exp and (perturbed) argmax ----
  OnlineLse acc;
  acc.init();
  Best best;
  best.v = -INFINITY;
  best.idx = 0x7fffffff;
  for (int i0 = threadIdx.x * 4; i0 < V; i0 += kRowThreads * 4) {
    uint4 rnd = make_uint4(0, 0, 0, 0);
    if (!greedy) {
      const uint32_t gidx = (uint32_t)(vocab_start + i0) >> 2;
      rnd = philox4x32(make_uint4(gidx, (uint32_t)step, (uint32_t)uid, (uint32_t)(uid >> 32)), key);
    }
    const uint32_t rb[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = i0 + j;
      if (i >= V) break;
      const float raw = load_logit<T>(p, i);
      if (raw == raw) acc.add(fminf(raw, 3.0e38f));
      float x = masked(i, raw);
      if (x == -INFINITY || x < thresh) continue;
      x = fminf(x, 3.0e38f);
      const float score = greedy ? x : x * inv_t + gumbel_from_bits(rb[j]);
      best.take(score, i);
    }
  }
  acc = warp_merge(acc);
  best = warp_best(best);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    red_lse[threadIdx.x >> 5] = acc;
    red_best[threadIdx.x >> 5] = best;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    OnlineLse t;
    t.init();
    Best b;
    b.v = -INFINITY;
    b.idx = 0x7fffffff;
    if (threadIdx.x < kRowThreads / 32) { t = red_lse[threadIdx.x]; b = red_best[threadIdx.x]; }
    t = warp_merge(t);
    b = warp_best(b);
    if (threadIdx.x == 0) {
      if (b.idx == 0x7fffffff) b.idx = 0;  // fully masked row: deterministic fallback
      const float raw_best = load_logit<T>(p, b.idx);
      if (part != nullptr) {
        float* q = part + row * 6;
        q[0] = b.v;
        q[1] = __int_as_float(vocab_start + b.idx);
        q[2] = raw_best;
        q[3] = t.m;
        q[4] = t.s;
        q[5] = 0.f;
      } else {
        out_token[row] = (long long)(vocab_start + b.idx);
        if (out_logprob != nullptr) out_logprob[row] = raw_best - (t.m + __logf(t.s));
      }
    }
  }
}

// Winner over the vocabulary slices of a row (records as written by sample_kernel); one thread per row.
__global__ void sample_combine_kernel(const float* __restrict__ slice_part, int slices, long long rows,
                                      long long* __restrict__ out_token, float* __restrict__ out_logprob,
                                      float* __restrict__ part) {
  const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  Best best;
  best.v = -INFINITY;
  best.idx = 0x7fffffff;
  float raw_best = 0.f, m = -INFINITY, sum = 0.f;
  for (int s = 0; s < slices; ++s) {
    const float* q = slice_part + ((long long)s * rows + row) * 6;
    const int id = __float_as_int(q[1]);
    const float bv = q[0];
    if (bv > best.v || (bv == best.v && id < best.idx)) { best.v = bv; best.idx = id; raw_best = q[2]; }
    const float om = q[3], os = q[4];
    if (om != -INFINITY) {
      if (m == -INFINITY) { m = om; sum = os; }
      else {
        const float mn = fmaxf(m, om);
        sum = sum * __expf(m - mn) + os * __expf(om - mn);
        m = mn;
      }
    }
  }
  if (part != nullptr) {
    float* q = part + row * 6;
    q[0] = best.v; q[1] = __int_as_float(best.idx); q[2] = raw_best; q[3] = m; q[4] = sum; q[5] = 0.f;
  } else {
    out_token[row] = (long long)best.idx;
    if (out_logprob != nullptr) out_logprob[row] = raw_best - (m + __logf(sum));
  }
}

}  // namespace areno

using namespace areno;

extern "C" int areno_logprob_stats(const void* logits, int is_bf16, long long ld, long long rows, int V,
                                   const long long* targets, long long vocab_start, float* out_max, float* out_sum,
                                   float* out_sumx, float* out_tgt, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (is_bf16) {
    if (ld % 8 != 0) return -3;
    logprob_stats_kernel<__nv_bfloat16><<<(unsigned)rows, kRowThreads, 0, stream>>>(
        (const __nv_bfloat16*)logits, ld, V, targets, vocab_start, out_max, out_sum, out_sumx, out_tgt);
  } else {
    if (ld % 4 != 0) return -3;
    logprob_stats_kernel<float><<<(unsigned)rows, kRowThreads, 0, stream>>>((const float*)logits, ld, V, targets,
                                                                           vocab_start, out_max, out_sum, out_sumx,
                                                                           out_tgt);
  }
  return (int)cudaGetLastError();
}

extern "C" int areno_logprob_bwd(void* logits, int is_bf16, long long ld, long long rows, int V,
                                 const long long* targets, long long vocab_start, const float* lse, const float* ex,
                                 const float* dlp, const float* dent, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (is_bf16)
    logprob_bwd_kernel<__nv_bfloat16><<<(unsigned)rows, kRowThreads, 0, stream>>>((__nv_bfloat16*)logits, ld, V, targets,
                                                                                 vocab_start, lse, ex, dlp, dent);
  else
    logprob_bwd_kernel<float><<<(unsigned)rows, kRowThreads, 0, stream>>>((float*)logits, ld, V, targets, vocab_start,
                                                                         lse, ex, dlp, dent);
  return (int)cudaGetLastError();
}

// slice_scratch: optional fp32 [slices, rows, 6]; with slices > 1 (and no top-k / top-p truncation, which needs
// the whole row in one block) every row is sampled by `slices` blocks and a second tiny kernel picks the winner.
extern "C" int areno_sample(const void* logits, int is_bf16, long long ld, long long rows, int V, int vocab_start,
                            const signed char* cls, const int* gen_count, int min_new, float temperature, int top_k,
                            float top_p, long long seed, const long long* row_uid, long long* out_token,
                            float* out_logprob, float* part, float* slice_scratch, int slices, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const bool truncate = temperature > 0.f && (top_k > 0 || top_p < 1.f);
  int slice_len = V;
  if (slice_scratch == nullptr || truncate || slices <= 1 || V < 4096) slices = 1;
  if (slices > 1) slice_len = ((V + slices - 1) / slices + 3) / 4 * 4;
  if (slices > 1 && (long long)slice_len * (slices - 1) >= V) slices = (V + slice_len - 1) / slice_len;
  const dim3 grid((unsigned)rows, (unsigned)slices);
  if (is_bf16)
    sample_kernel<__nv_bfloat16><<<grid, kRowThreads, 0, stream>>>(
        (const __nv_bfloat16*)logits, ld, V, vocab_start, cls, gen_count, min_new, temperature, top_k, top_p,
        (unsigned long long)seed, row_uid, out_token, out_logprob, part, slice_len, slice_scratch);
  else
    sample_kernel<float><<<grid, kRowThreads, 0, stream>>>((const float*)logits, ld, V, vocab_start, cls, gen_count,
                                                           min_new, temperature, top_k, top_p, (unsigned long long)seed,
                                                           row_uid, out_token, out_logprob, part, slice_len, slice_scratch);
  if (slices > 1)
    sample_combine_kernel<<<(unsigned)((rows + 127) / 128), 128, 0, stream>>>(slice_scratch, slices, rows, out_token,
                                                                             out_logprob, part);
  return (int)cudaGetLastError();
}
