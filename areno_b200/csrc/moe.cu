// Mixture-of-experts routing kernels: top-k softmax router (fwd/bwd), grouped sigmoid router,
// route alignment (expert-sorted, tile-padded row plan built entirely on the device), row
// permute / weighted combine and their backward pieces.  The expert GEMMs themselves are the
// grouped modes of the tcgen05 kernel in gemm_tcgen05.cu, driven by the plan built here.
//
// Plan layout (all int32, device memory, sized from static upper bounds so that nothing is read
// back to the host):
//   expert_rows[2*E]   : {offset, padded_count} of every local expert in the sorted row space
//                        (offsets and padded counts are multiples of 128 = GEMM M tile)
//   tile_expert[tiles] : local expert id owning each 128-row tile, or -1 for tiles past the end
//   row_route[P]       : route id (token * k + slot) stored at each sorted row, or -1 for padding
//   route_row[T*k]     : sorted row of each route, or -1 if its expert is not local
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <stdint.h>

#include "common.cuh"
#include "launch.h"

namespace areno {

constexpr int kMoeTile = 128;

// ----------------------------------------------------------------------------------
// Top-k softmax router.  One warp per token; E <= 1024, k <= 32.
//   probs = softmax(logits);  ids = top-k(probs) (ties: lower index);  w = probs[ids]
//   renorm: w /= sum(w)
// ----------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, int i);
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, int i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, int i) { return __bfloat162float(p[i]); }

template <typename T>
__global__ void __launch_bounds__(256)
topk_softmax_fwd_kernel(const T* __restrict__ logits, int tokens, int E, int k, int renorm,
                        float* __restrict__ weights, int* __restrict__ ids) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= tokens) return;
  const T* row = logits + (size_t)t * E;
  constexpr int PER = 32;  // up to 1024 experts
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + i * 32;
    v[i] = e < E ? ld_logit<T>(row, e) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float z = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + i * 32;
    v[i] = e < E ? __expf(v[i] - mx) : -1.f;  // -1 marks "not a candidate"
    if (e < E) z += v[i];
  }
  z = warp_sum(z);
  const float inv_z = 1.f / z;
  float picked_sum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + i * 32;
      if (v[i] > best) { best = v[i]; best_e = e; }  // ascending e within a lane: first max wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (lane + i * 32 == best_e) v[i] = -1.f;
    }
    const float pw = best * inv_z;
    picked_sum += pw;
    if (lane == j) { my_w = pw; my_id = best_e; }
  }
  if (lane < k) {
    weights[(size_t)t * k + lane] = renorm ? my_w / picked_sum : my_w;
    ids[(size_t)t * k + lane] = my_id;
  }
}

// dlogits from dweights.  With p = softmax(x), S = sum_j p[id_j], w_j = p[id_j] / (renorm ? S : 1):
//   dL/dp[id_j] = (dw_j - (renorm ? sum_i dw_i w_i : 0)) / (renorm ? S : 1);  dL/dp elsewhere 0
//   dx = p * (dL/dp - sum_e p_e dL/dp_e)
template <typename T>
__global__ void __launch_bounds__(256)
topk_softmax_bwd_kernel(const T* __restrict__ logits, const int* __restrict__ ids, const float* __restrict__ weights,
                        const float* __restrict__ dweights, int tokens, int E, int k, int renorm,
                        float* __restrict__ dlogits) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= tokens) return;
  const T* row = logits + (size_t)t * E;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, ld_logit<T>(row, e));
  mx = warp_max(mx);
  float z = 0.f;
  for (int e = lane; e < E; e += 32) z += __expf(ld_logit<T>(row, e) - mx);
  z = warp_sum(z);
  const float inv_z = 1.f / z;
  // per-lane copy of the k selections
  float w = 0.f, dw = 0.f;
  int id = -1;
  if (lane < k) {
    w = weights[(size_t)t * k + lane];
    dw = dweights[(size_t)t * k + lane];
    id = ids[(size_t)t * k + lane];
  }
  const float dot = warp_sum(w * dw);
  float S = 1.f;
  if (renorm) {
    float p_sel = lane < k ? __expf(ld_logit<T>(row, id) - mx) * inv_z : 0.f;
    S = warp_sum(p_sel);
  }
  const float g_sel = lane < k ? (dw - (renorm ? dot : 0.f)) / S : 0.f;  // dL/dp at my selection
  float p_sel2 = lane < k ? __expf(ld_logit<T>(row, id) - mx) * inv_z : 0.f;
  const float pg = warp_sum(p_sel2 * g_sel);  // sum_e p_e dL/dp_e
  for (int e0 = 0; e0 < E; e0 += 32) {
    const int e = e0 + lane;
    float g = 0.f;
    for (int j = 0; j < k; ++j) {
      const int idj = __shfl_sync(0xffffffffu, id, j);
      const float gj = __shfl_sync(0xffffffffu, g_sel, j);
      if (idj == e) g = gj;
    }
    if (e < E) {
      const float pe = __expf(ld_logit<T>(row, e) - mx) * inv_z;
      dlogits[(size_t)t * E + e] = pe * (g - pg);
    }
  }
}

// ----------------------------------------------------------------------------------
// Grouped sigmoid router ("noaux_tc"): scores = sigmoid(logits); choice scores = scores + bias;
// group score = sum of the top-2 choice scores of each group; keep `topk_group` groups; pick the
// top-k experts among the kept groups by choice score; weights = scores[ids] (unbiased),
// optionally renormalised, times `scale`.  One warp per token, E <= 512, groups <= 32.
// ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
grouped_sigmoid_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int tokens, int E,
                            int n_group, int topk_group, int k, int renorm, float scale,
                            float* __restrict__ weights, int* __restrict__ ids) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= tokens) return;
  __shared__ float sh_choice[8][512];
  __shared__ float sh_score[8][512];
  float* choice = sh_choice[warp];
  float* score = sh_score[warp];
  const int per_group = E / n_group;
  for (int e = lane; e < E; e += 32) {
    const float s = 1.f / (1.f + __expf(-logits[(size_t)t * E + e]));
    score[e] = s;
    choice[e] = s + (bias != nullptr ? bias[e] : 0.f);
  }
  __syncwarp();
  // group scores: lane g handles group g
  float gscore = -INFINITY;
  if (lane < n_group) {
    float a = -INFINITY, b = -INFINITY;
    for (int i = 0; i < per_group; ++i) {
      const float c = choice[lane * per_group + i];
      if (c > a) { b = a; a = c; } else if (c > b) { b = c; }
    }
    gscore = per_group > 1 ? a + b : a;
  }
  // select topk_group groups (mask of kept groups, same on every lane)
  uint32_t kept = 0;
  for (int j = 0; j < topk_group; ++j) {
    float best = (lane < n_group && !((kept >> lane) & 1u)) ? gscore : -INFINITY;
    int bi = lane;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    kept |= 1u << bi;
  }
  // top-k experts among kept groups
  float picked_sum = 0.f, my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float c = ((kept >> (e / per_group)) & 1u) ? choice[e] : -INFINITY;
      if (c > best) { best = c; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    const float s = score[be];
    __syncwarp();
    if (lane == 0) choice[be] = -INFINITY;
    __syncwarp();
    picked_sum += s;
    if (lane == j) { my_w = s; my_id = be; }
  }
  if (lane < k) {
    weights[(size_t)t * k + lane] = (renorm ? my_w / (picked_sum + 1e-20f) : my_w) * scale;
    ids[(size_t)t * k + lane] = my_id;
  }
}

// ----------------------------------------------------------------------------------
// Alignment.  One block; warp w handles local experts w, w+32, ... : it walks the route list in
// order (so rows of an expert keep token order: deterministic) and assigns positions.
// Pass 1 counts, a serial scan over E (thread 0) lays out padded segments, pass 2 writes rows.
// ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ ids, int routes, int e_lo, int e_count, int max_rows,
                 int* __restrict__ expert_rows, int* __restrict__ tile_expert, int* __restrict__ row_route,
                 int* __restrict__ route_row, int* __restrict__ counts_out, int* __restrict__ dropped_out) {
  extern __shared__ int sh[];  // [e_count] counts, [e_count] offsets, [e_count] rows that fit
  int* cnt = sh;
  int* off = sh + e_count;
  int* fit = sh + 2 * e_count;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < max_rows; i += blockDim.x) row_route[i] = -1;
  for (int i = threadIdx.x; i < max_rows / kMoeTile; i += blockDim.x) tile_expert[i] = -1;
  for (int e = warp; e < e_count; e += nwarps) {
    int c = 0;
    for (int r0 = 0; r0 < routes; r0 += 32) {
      const int r = r0 + lane;
      const bool hit = r < routes && ids[r] == e_lo + e;
      c += __popc(__ballot_sync(0xffffffffu, hit));
    }
    if (lane == 0) cnt[e] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // max_rows covers every case when it was sized from the static bound (routes + experts * 127).  A caller
    // that sizes it from an expected load instead (expert parallelism: a capacity factor over the mean) may
    // see more routes than fit: the surplus routes of an expert are dropped (their route_row stays -1, the
    // token simply gets no contribution from that expert) and counted in dropped_out.
    int o = 0, dropped = 0;
    for (int e = 0; e < e_count; ++e) {
      int padded = (cnt[e] + kMoeTile - 1) / kMoeTile * kMoeTile;
      if (o + padded > max_rows) padded = (max_rows - o) / kMoeTile * kMoeTile;
      fit[e] = min(cnt[e], padded);
      dropped += cnt[e] - fit[e];
      off[e] = o;
      expert_rows[2 * e] = o;
      expert_rows[2 * e + 1] = padded;
      if (counts_out != nullptr) counts_out[e] = fit[e];
      for (int tile = o / kMoeTile; tile < (o + padded) / kMoeTile; ++tile) tile_expert[tile] = e;
      o += padded;
    }
    if (dropped_out != nullptr) *dropped_out = dropped;
  }
  __syncthreads();
  for (int e = warp; e < e_count; e += nwarps) {
    int pos = off[e];
    for (int r0 = 0; r0 < routes; r0 += 32) {
      const int r = r0 + lane;
      const bool hit = r < routes && ids[r] == e_lo + e;
      const uint32_t m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int row = pos + __popc(m & ((1u << lane) - 1u));
        if (row < off[e] + fit[e]) {
          row_route[row] = r;
          route_row[r] = row;
        } else {
          route_row[r] = -1;
        }
      }
      pos += __popc(m);
    }
  }
  // routes whose expert lives on another rank
  for (int r = threadIdx.x; r < routes; r += blockDim.x) {
    const int e = ids[r] - e_lo;
    if (e < 0 || e >= e_count) route_row[r] = -1;
  }
}

// ----------------------------------------------------------------------------------
// The same plan from three launches, for many routes (a training micro-batch of an expert-parallel group has
// 8 x 32768 of them, and the single-CTA kernel above walks all of them once per expert at one dependent
// load per step).  Every warp owns a chunk of kAlignChunk consecutive routes:
//   count   per-chunk histogram over the local experts (chunk_cnt[chunk][e]); row_route / tile_expert reset
//   scan    one CTA: per-expert totals -> padded segments (capacity as above), then every chunk's counter is
//           replaced by the first row of that chunk inside the expert's segment (exclusive prefix in chunk order)
//   place   every warp walks its chunk again and hands out rows in route order
// Rows are assigned in route order inside every expert, exactly as the single-CTA kernel does, so both give
// the same plan.
// ----------------------------------------------------------------------------------
constexpr int kAlignChunk = 512;

__global__ void __launch_bounds__(256)
moe_align_count_kernel(const int* __restrict__ ids, int routes, int e_lo, int e_count, int max_rows,
                       int* __restrict__ chunk_cnt, int* __restrict__ row_route, int* __restrict__ tile_expert) {
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x, gsize = gridDim.x * blockDim.x;
  for (int i = gtid; i < max_rows; i += gsize) row_route[i] = -1;
  for (int i = gtid; i < max_rows / kMoeTile; i += gsize) tile_expert[i] = -1;
  const int lane = threadIdx.x & 31;
  const int nchunks = (routes + kAlignChunk - 1) / kAlignChunk;
  for (int chunk = gtid >> 5; chunk < nchunks; chunk += gsize >> 5) {
    int* cnt = chunk_cnt + (size_t)chunk * e_count;
    for (int e = lane; e < e_count; e += 32) cnt[e] = 0;
    __syncwarp();
    const int base = chunk * kAlignChunk;
    for (int r0 = 0; r0 < kAlignChunk; r0 += 32) {
      const int r = base + r0 + lane;
      int e = r < routes ? ids[r] - e_lo : -1;
      if (e >= e_count) e = -1;
      const uint32_t m = __match_any_sync(0xffffffffu, e);
      if (e >= 0 && lane == __ffs(m) - 1) cnt[e] += __popc(m);     // one writer per expert and step
      __syncwarp();
    }
  }
}

__global__ void __launch_bounds__(1024)
moe_align_scan_kernel(int routes, int e_count, int max_rows, int* __restrict__ chunk_cnt, int* __restrict__ limit,
                      int* __restrict__ expert_rows, int* __restrict__ tile_expert, int* __restrict__ counts_out,
                      int* __restrict__ dropped_out) {
  extern __shared__ int sh[];  // [e_count] totals, [e_count] offsets
  int* tot = sh;
  int* off = sh + e_count;
  const int nchunks = (routes + kAlignChunk - 1) / kAlignChunk;
  for (int e = threadIdx.x; e < e_count; e += blockDim.x) {
    int c = 0;
    for (int ch = 0; ch < nchunks; ++ch) c += chunk_cnt[(size_t)ch * e_count + e];
    tot[e] = c;
  }
  __syncthreads();
  // Segment layout.  Common case (at most 1024 experts, everything fits): an exclusive scan of the padded sizes,
  // every thread writes its own expert.  Otherwise thread 0 walks the experts and applies the capacity.
  __shared__ int scan[1024];
  __shared__ int sh_fits;
  bool laid_out = false;
  if (e_count <= 1024) {
    const int e = threadIdx.x;
    const int padded = e < e_count ? (tot[e] + kMoeTile - 1) / kMoeTile * kMoeTile : 0;
    scan[e] = padded;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {
      const int v = e >= d ? scan[e - d] : 0;
      __syncthreads();
      scan[e] += v;
      __syncthreads();
    }
    if (e == 0) sh_fits = scan[1023] <= max_rows;
    __syncthreads();
    if (sh_fits) {
      laid_out = true;
      if (e < e_count) {
        const int o = scan[e] - padded;
        off[e] = o;
        limit[e] = o + tot[e];
        expert_rows[2 * e] = o;
        expert_rows[2 * e + 1] = padded;
        if (counts_out != nullptr) counts_out[e] = tot[e];
        for (int tile = o / kMoeTile; tile < (o + padded) / kMoeTile; ++tile) tile_expert[tile] = e;
      }
      if (e == 0 && dropped_out != nullptr) *dropped_out = 0;
    }
  }
  if (!laid_out && threadIdx.x == 0) {
    int o = 0, dropped = 0;
    for (int e = 0; e < e_count; ++e) {
      int padded = (tot[e] + kMoeTile - 1) / kMoeTile * kMoeTile;
      if (o + padded > max_rows) padded = (max_rows - o) / kMoeTile * kMoeTile;
      const int fit = min(tot[e], padded);
      dropped += tot[e] - fit;
      off[e] = o;
      limit[e] = o + fit;
      expert_rows[2 * e] = o;
      expert_rows[2 * e + 1] = padded;
      if (counts_out != nullptr) counts_out[e] = fit;
      for (int tile = o / kMoeTile; tile < (o + padded) / kMoeTile; ++tile) tile_expert[tile] = e;
      o += padded;
    }
    if (dropped_out != nullptr) *dropped_out = dropped;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < e_count; e += blockDim.x) {
    int run = off[e];
    for (int ch = 0; ch < nchunks; ++ch) {
      const size_t i = (size_t)ch * e_count + e;
      const int c = chunk_cnt[i];
      chunk_cnt[i] = run;
      run += c;
    }
  }
}

__global__ void __launch_bounds__(256)
moe_align_place_kernel(const int* __restrict__ ids, int routes, int e_lo, int e_count, int* __restrict__ chunk_cnt,
                       const int* __restrict__ limit, int* __restrict__ row_route, int* __restrict__ route_row) {
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x, gsize = gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  const int nchunks = (routes + kAlignChunk - 1) / kAlignChunk;
  for (int chunk = gtid >> 5; chunk < nchunks; chunk += gsize >> 5) {
    int* next = chunk_cnt + (size_t)chunk * e_count;       // next free row of every expert for this chunk
    const int base = chunk * kAlignChunk;
    for (int r0 = 0; r0 < kAlignChunk; r0 += 32) {
      const int r = base + r0 + lane;
      int e = r < routes ? ids[r] - e_lo : -1;
      if (e >= e_count) e = -1;
      const uint32_t m = __match_any_sync(0xffffffffu, e);
      const int leader = __ffs(m) - 1;
      int first = (e >= 0 && lane == leader) ? next[e] : 0;
      first = __shfl_sync(0xffffffffu, first, leader);
      if (e >= 0) {
        const int row = first + __popc(m & ((1u << lane) - 1u));
        if (row < limit[e]) {
          row_route[row] = r;
          route_row[r] = row;
        } else {
          route_row[r] = -1;
        }
        if (lane == leader) next[e] = first + __popc(m);
      } else if (r < routes) {
        route_row[r] = -1;      // the expert lives on another rank
      }
      __syncwarp();
    }
  }
}

// xs[row] = x[row_route[row] / k]  (zeros for padding rows)
__global__ void __launch_bounds__(256)
moe_permute_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_route, int k, int max_rows, int H,
                   __nv_bfloat16* __restrict__ xs) {
  const int nvec = H >> 3;
  const long long total = (long long)max_rows * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / nvec), v = (int)(i % nvec);
    const int route = row_route[row];
    uint4 val = make_uint4(0, 0, 0, 0);
    if (route >= 0) val = *reinterpret_cast<const uint4*>(x + (size_t)(route / k) * H + v * 8);
    *reinterpret_cast<uint4*>(xs + (size_t)row * H + v * 8) = val;
  }
}

// Inference variant: one warp per row, padding rows are left untouched (a GEMM row only feeds its own output row,
// and nobody gathers the output of a padding row), so a decode step copies its few hundred real rows instead
// of zero-filling a tile per expert.
__global__ void __launch_bounds__(256)
moe_permute_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_route, int k, int max_rows,
                        int H, __nv_bfloat16* __restrict__ xs) {
  const int nvec = H >> 3;
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int row = warp; row < max_rows; row += nwarps) {
    const int route = row_route[row];
    if (route < 0) continue;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(route / k) * H);
    uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)row * H);
    for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
  }
}

// Router logits for a handful of tokens: logits[t, e] = sum_h x[t, h] * w[e, h] with fp32 weights and fp32
// accumulation.  One CTA per (token, block of 16 experts) keeps the token in shared memory as fp32; every warp
// takes two experts and keeps four 16-byte loads of the weight row in flight.  Replaces a cast kernel + a library
// SGEMM + its split-K reduction (30 us for 32 tokens x 128 experts) in the decode step.
constexpr int kRouterExpertsPerCta = 16;
__global__ void __launch_bounds__(256)
router_logits_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, float* __restrict__ logits, int H,
                     int E) {
  extern __shared__ float sx[];
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < H; i += blockDim.x) sx[i] = __bfloat162float(x[(size_t)t * H + i]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float4* s4 = reinterpret_cast<const float4*>(sx);
  const int n4 = H >> 2;
  for (int e = blockIdx.y * kRouterExpertsPerCta + warp; e < min(E, (int)(blockIdx.y + 1) * kRouterExpertsPerCta);
       e += blockDim.x >> 5) {
    const float4* w4 = reinterpret_cast<const float4*>(w + (size_t)e * H);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i0 = lane; i0 < n4; i0 += 128) {
      float4 b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) b[u] = i0 + u * 32 < n4 ? __ldg(w4 + i0 + u * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i0 + u * 32 < n4) {
          const float4 a = s4[i0 + u * 32];
          acc[u] += a.x * b[u].x + a.y * b[u].y + a.z * b[u].z + a.w * b[u].w;
        }
      }
    }
    float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) logits[(size_t)t * E + e] = sum;
  }
}

// out[t] = sum_j w[t, j] * ys[route_row[t*k + j]]   (missing routes contribute nothing).
// weights == nullptr: plain sum (backward of permute).
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ route_row,
                   const float* __restrict__ weights, int tokens, int k, int H, __nv_bfloat16* __restrict__ out) {
  const int nvec = H >> 3;
  const long long total = (long long)tokens * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / nvec), v = (int)(i % nvec);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < k; ++s) {
      const int row = route_row[(size_t)t * k + s];
      if (row < 0) continue;
      const float w = weights != nullptr ? weights[(size_t)t * k + s] : 1.f;
      const uint4 val = *reinterpret_cast<const uint4*>(ys + (size_t)row * H + v * 8);
      const uint32_t u[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += w * __uint_as_float(u[j] << 16);
        acc[2 * j + 1] += w * __uint_as_float(u[j] & 0xffff0000u);
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + (size_t)t * H + v * 8) = o;
  }
}

// Backward of combine: dys[row] = w[route] * dout[token(route)] (zeros for padding rows) and
// dw[route] = <ys[row], dout[token]>.  One warp per sorted row.
__global__ void __launch_bounds__(256)
moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ ys,
                       const int* __restrict__ row_route, const float* __restrict__ weights, int k, int max_rows, int H,
                       __nv_bfloat16* __restrict__ dys, float* __restrict__ dweights) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int row = blockIdx.x * 8 + warp; row < max_rows; row += gridDim.x * 8) {
    const int route = row_route[row];
    if (route < 0) {
      for (int v = lane; v < nvec; v += 32)
        *reinterpret_cast<uint4*>(dys + (size_t)row * H + v * 8) = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int t = route / k;
    const float w = weights[route];
    float dot = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 g = *reinterpret_cast<const uint4*>(dout + (size_t)t * H + v * 8);
      const uint4 yv = *reinterpret_cast<const uint4*>(ys + (size_t)row * H + v * 8);
      const uint32_t gu[4] = {g.x, g.y, g.z, g.w};
      const uint32_t yu[4] = {yv.x, yv.y, yv.z, yv.w};
      float o[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float g0 = __uint_as_float(gu[j] << 16), g1 = __uint_as_float(gu[j] & 0xffff0000u);
        dot += g0 * __uint_as_float(yu[j] << 16) + g1 * __uint_as_float(yu[j] & 0xffff0000u);
        o[2 * j] = w * g0;
        o[2 * j + 1] = w * g1;
      }
      uint4 ov;
      ov.x = pack_bf16x2(o[0], o[1]);
      ov.y = pack_bf16x2(o[2], o[3]);
      ov.z = pack_bf16x2(o[4], o[5]);
      ov.w = pack_bf16x2(o[6], o[7]);
      *reinterpret_cast<uint4*>(dys + (size_t)row * H + v * 8) = ov;
    }
    dot = warp_sum(dot);
    if (lane == 0) dweights[route] = dot;
  }
}

__global__ void moe_fill_kernel(float* __restrict__ p, long long n, float v) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) p[i] = v;
}

static inline int grid_1d(long long work, int per_block, int cap = 148 * 16) {
  long long g = (work + per_block - 1) / per_block;
  if (g > cap) g = cap;
  return (int)(g < 1 ? 1 : g);
}

}  // namespace areno

using namespace areno;

extern "C" int areno_topk_softmax_fwd(const void* logits, int bf16, long long tokens, int E, int k, int renorm,
                                      float* weights, int* ids, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (E < 1 || E > 1024 || k < 1 || k > 32 || k > E) return -3;
  const int grid = (int)((tokens + 7) / 8);
  if (bf16) topk_softmax_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)logits, (int)tokens, E, k, renorm, weights, ids);
  else topk_softmax_fwd_kernel<float><<<grid, 256, 0, stream>>>((const float*)logits, (int)tokens, E, k, renorm, weights, ids);
  return (int)cudaGetLastError();
}

extern "C" int areno_topk_softmax_bwd(const void* logits, int bf16, const int* ids, const float* weights,
                                      const float* dweights, long long tokens, int E, int k, int renorm,
                                      float* dlogits, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (E < 1 || E > 1024 || k < 1 || k > 32) return -3;
  const int grid = (int)((tokens + 7) / 8);
  if (bf16) topk_softmax_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)logits, ids, weights, dweights, (int)tokens, E, k, renorm, dlogits);
  else topk_softmax_bwd_kernel<float><<<grid, 256, 0, stream>>>((const float*)logits, ids, weights, dweights, (int)tokens, E, k, renorm, dlogits);
  return (int)cudaGetLastError();
}

extern "C" int areno_grouped_sigmoid_topk(const float* logits, const float* bias, long long tokens, int E, int n_group,
                                          int topk_group, int k, int renorm, float scale, float* weights, int* ids,
                                          cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (E < 1 || E > 512 || n_group < 1 || n_group > 32 || E % n_group != 0 || topk_group < 1 || topk_group > n_group ||
      k < 1 || k > 32)
    return -3;
  grouped_sigmoid_topk_kernel<<<(int)((tokens + 7) / 8), 256, 0, stream>>>(logits, bias, (int)tokens, E, n_group,
                                                                           topk_group, k, renorm, scale, weights, ids);
  return (int)cudaGetLastError();
}

// Upper bound of sorted rows for `routes` routes over `experts` local experts (multiple of 128).
extern "C" long long areno_moe_max_rows(long long routes, int experts) {
  const long long raw = routes + (long long)experts * (kMoeTile - 1);
  return (raw + kMoeTile - 1) / kMoeTile * kMoeTile;
}

extern "C" int areno_moe_align(const int* ids, long long routes, int e_lo, int e_count, long long max_rows,
                               int* expert_rows, int* tile_expert, int* row_route, int* route_row, int* counts,
                               cudaStream_t stream) {
  if (e_count < 1 || e_count > 4096 || max_rows % kMoeTile != 0) return -3;
  moe_align_kernel<<<1, 1024, 3 * e_count * sizeof(int), stream>>>(ids, (int)routes, e_lo, e_count, (int)max_rows,
                                                                  expert_rows, tile_expert, row_route, route_row, counts,
                                                                  nullptr);
  return (int)cudaGetLastError();
}

// The plan from the three-launch path above.  scratch: int32 [areno_moe_align_scratch_ints(routes, e_count)];
// dropped may be null (then max_rows must cover every case).
extern "C" long long areno_moe_align_scratch_ints(long long routes, int e_count) {
  return ((routes + kAlignChunk - 1) / kAlignChunk + 1) * (long long)e_count;
}

extern "C" int areno_moe_align_par(const int* ids, long long routes, int e_lo, int e_count, long long max_rows,
                                   int* expert_rows, int* tile_expert, int* row_route, int* route_row, int* counts,
                                   int* dropped, int* scratch, cudaStream_t stream) {
  if (e_count < 1 || e_count > 4096 || max_rows % kMoeTile != 0 || max_rows < kMoeTile || routes < 1 ||
      scratch == nullptr)
    return -3;
  const long long nchunks = (routes + kAlignChunk - 1) / kAlignChunk;
  int* chunk_cnt = scratch;
  int* limit = scratch + nchunks * e_count;
  const int warps = (int)std::min<long long>(nchunks, 148 * 16);
  const int grid = std::max((warps + 7) / 8, std::min<int>(148, (int)((max_rows + 255) / 256)));
  moe_align_count_kernel<<<grid, 256, 0, stream>>>(ids, (int)routes, e_lo, e_count, (int)max_rows, chunk_cnt, row_route,
                                                   tile_expert);
  moe_align_scan_kernel<<<1, 1024, 2 * e_count * sizeof(int), stream>>>((int)routes, e_count, (int)max_rows, chunk_cnt,
                                                                        limit, expert_rows, tile_expert, counts, dropped);
  moe_align_place_kernel<<<(warps + 7) / 8, 256, 0, stream>>>(ids, (int)routes, e_lo, e_count, chunk_cnt, limit, row_route,
                                                             route_row);
  return (int)cudaGetLastError();
}

// Same plan, for a row buffer that is smaller than the static bound: routes that do not fit are dropped and
// *dropped (device int) receives their number.
extern "C" int areno_moe_align_capped(const int* ids, long long routes, int e_lo, int e_count, long long max_rows,
                                      int* expert_rows, int* tile_expert, int* row_route, int* route_row, int* counts,
                                      int* dropped, cudaStream_t stream) {
  if (e_count < 1 || e_count > 4096 || max_rows % kMoeTile != 0 || max_rows < kMoeTile) return -3;
  moe_align_kernel<<<1, 1024, 3 * e_count * sizeof(int), stream>>>(ids, (int)routes, e_lo, e_count, (int)max_rows,
                                                                  expert_rows, tile_expert, row_route, route_row, counts,
                                                                  dropped);
  return (int)cudaGetLastError();
}

extern "C" int areno_moe_permute(const void* x, const int* row_route, int k, long long max_rows, int H, void* xs,
                                 cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if (H % 8 != 0) return -3;
  moe_permute_kernel<<<grid_1d(max_rows * (H / 8), 256), 256, 0, stream>>>((const __nv_bfloat16*)x, row_route, k,
                                                                            (int)max_rows, H, (__nv_bfloat16*)xs);
  return (int)cudaGetLastError();
}

// Inference: copy only the rows that have a route (see moe_permute_rows_kernel).
extern "C" int areno_moe_permute_rows(const void* x, const int* row_route, int k, long long max_rows, int H, void* xs,
                                      cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if (H % 8 != 0) return -3;
  moe_permute_rows_kernel<<<grid_1d(max_rows * 32, 256), 256, 0, stream>>>((const __nv_bfloat16*)x, row_route, k,
                                                                           (int)max_rows, H, (__nv_bfloat16*)xs);
  return (int)cudaGetLastError();
}

// x: bf16 [tokens, H]; w: fp32 [E, H]; logits: fp32 [tokens, E].  For a few hundred tokens at most.
extern "C" int areno_router_logits(const void* x, const float* w, float* logits, long long tokens, int H, int E,
                                   cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H % 4 != 0 || H > 12288 || E < 1 || (reinterpret_cast<uintptr_t>(w) & 15)) return -3;
  static bool cfg_dev[kMaxDevices] = {};
  bool& cfg = per_device_flag(cfg_dev);
  if (!cfg) {
    cudaFuncSetAttribute(router_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 12288 * 4);
    cfg = true;
  }
  const dim3 grid((unsigned)tokens, (unsigned)((E + kRouterExpertsPerCta - 1) / kRouterExpertsPerCta));
  router_logits_kernel<<<grid, 256, H * sizeof(float), stream>>>((const __nv_bfloat16*)x, w, logits, H, E);
  return (int)cudaGetLastError();
}

extern "C" int areno_moe_combine(const void* ys, const int* route_row, const float* weights, long long tokens, int k,
                                 int H, void* out, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H % 8 != 0) return -3;
  moe_combine_kernel<<<grid_1d(tokens * (H / 8), 256), 256, 0, stream>>>((const __nv_bfloat16*)ys, route_row, weights,
                                                                         (int)tokens, k, H, (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}

extern "C" int areno_moe_combine_bwd(const void* dout, const void* ys, const int* row_route, const float* weights, int k,
                                     long long max_rows, long long routes, int H, void* dys, float* dweights,
                                     cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if (H % 8 != 0) return -3;
  moe_fill_kernel<<<grid_1d(routes, 256), 256, 0, stream>>>(dweights, routes, 0.f);
  moe_combine_bwd_kernel<<<grid_1d(max_rows, 8), 256, 0, stream>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)ys,
                                                                    row_route, weights, k, (int)max_rows, H,
                                                                    (__nv_bfloat16*)dys, dweights);
  return (int)cudaGetLastError();
}
