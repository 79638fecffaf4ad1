// Paged-KV decode attention and the RoPE + KV-append kernel that feeds it (sm_100a).
//
// Cache layout (per layer): K and V pages [num_pages, kv_heads, page_size, head_dim], either
// bf16 or fp8-e4m3 with one fp32 scale per (page, kv_head, slot) stored in a parallel
// [num_pages, kv_heads, page_size] table (the scale of a token never changes once written, so
// appends never requantise a page).
//
// Decode: one CTA per (sequence, kv head, split).  All q heads of the GQA group share each K/V
// tile (padded to the 16-row MMA tile), so the cache is read once per group rather than once
// per q head.  Pages stream through a 3-stage cp.async pipeline; fp8 pages are expanded to fp16 in
// shared memory (e4m3 -> fp16 is exact: one conversion and one fp16 multiply by the token's scale per
// pair) and the MMAs of that variant run on fp16 operands.  Split partials are merged by a second kernel.
// Everything is driven by device-side `seq_lens` / `block_table`, so the launch shape is static
// and the kernel is CUDA-graph friendly.
//
// Replaces flash_attn_with_kvcache (areno/engine/layers/attention_backend/infer.py:172-178) and the
// reference's scalar paged kernels (areno/accel/csrc/attention.cu:526-702).
#include "attention_common.cuh"
#include "launch.h"

#include <cuda_fp8.h>

namespace areno {

constexpr int kPage = 64;  // tokens per page (also the key tile)

// ---------------------------------------------------------------------------------
// RoPE (neox / interleaved, partial allowed) on q and k in place + append k, v to the cache.
// One warp per (token, head).  Heads [0, hq) are q (rotate only), [hq, hq+hkv) are k (rotate,
// write back, append), [hq+hkv, hq+2hkv) are v (append).  slot_mapping[t] < 0 skips the append.
// ---------------------------------------------------------------------------------
// Per-warp work on one (token, head) row `p` (D bf16 values already in global memory): rotate q / k
// heads in place, append k / v heads to the paged cache.
template <bool FP8>
__device__ __forceinline__ void rope_append_row(__nv_bfloat16* p, int lane, long long t, int h, const int* positions,
                                                const int* slot_mapping, const float* inv_freq, void* k_cache,
                                                void* v_cache, float* k_scale, float* v_scale, int hq, int hkv, int D,
                                                int rot_dim, float theta, int interleaved, int page_size) {
  const bool is_v = h >= hq + hkv;
  const bool is_k = !is_v && h >= hq;
  if (!is_v && rot_dim > 0) {
    const int half = rot_dim >> 1;
    const float pos = (float)positions[t];
    for (int i = lane; i < half; i += 32) {
      const float f = inv_freq != nullptr ? inv_freq[i] : __powf(theta, -2.f * (float)i / (float)rot_dim);
      float s, c;
      sincosf(pos * f, &s, &c);
      const int i0 = interleaved ? 2 * i : i;
      const int i1 = interleaved ? 2 * i + 1 : i + half;
      const float a = __bfloat162float(p[i0]), b = __bfloat162float(p[i1]);
      p[i0] = __float2bfloat16_rn(a * c - b * s);
      p[i1] = __float2bfloat16_rn(b * c + a * s);
    }
    __syncwarp();
  }
  if (!is_k && !is_v) return;
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const int kvh = is_k ? h - hq : h - hq - hkv;
  const int page = slot / page_size, off = slot % page_size;
  const long long row = ((long long)page * hkv + kvh) * page_size + off;
  void* cache = is_k ? k_cache : v_cache;
  if constexpr (FP8) {
    float amax = 0.f;
    for (int i = lane; i < D; i += 32) amax = fmaxf(amax, fabsf(__bfloat162float(p[i])));
    amax = warp_max(amax);
    const float sc = fmaxf(amax, 1e-8f) / 448.f;
    const float inv = 1.f / sc;
    __nv_fp8_e4m3* dst = reinterpret_cast<__nv_fp8_e4m3*>(cache) + row * D;
    for (int i = lane; i < D; i += 32) dst[i] = __nv_fp8_e4m3(__bfloat162float(p[i]) * inv);
    if (lane == 0) (is_k ? k_scale : v_scale)[row] = sc;
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(cache) + row * D;
    for (int i = lane * 2; i < D; i += 64)
      *reinterpret_cast<uint32_t*>(dst + i) = *reinterpret_cast<const uint32_t*>(p + i);
  }
}

template <bool FP8>
__global__ void __launch_bounds__(256)
rope_append_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                   const int* __restrict__ slot_mapping, const float* __restrict__ inv_freq, void* __restrict__ k_cache,
                   void* __restrict__ v_cache, float* __restrict__ k_scale, float* __restrict__ v_scale, long long tokens,
                   int hq, int hkv, int D, int rot_dim, float theta, int interleaved, int page_size) {
  pdl_trigger();
  pdl_wait();
  const int heads = hq + 2 * hkv;
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= tokens * heads) return;
  const int lane = threadIdx.x & 31;
  const long long t = w / heads;
  const int h = (int)(w % heads);
  __nv_bfloat16* p = qkv + t * (long long)heads * D + (long long)h * D;
  rope_append_row<FP8>(p, lane, t, h, positions, slot_mapping, inv_freq, k_cache, v_cache, k_scale, v_scale, hq, hkv, D,
                       rot_dim, theta, interleaved, page_size);
}

// Decode-sized fused form: the q/k/v projection left split-K partials ws[splits, tokens, heads * D]
// (fp32); one warp per (token, head) folds them in split order, adds the bias, rounds to bf16 into
// `qkv`, applies the optional per-head RMSNorm of q / k heads, then rotates and appends as above.
// Every intermediate passes through the same bf16 rounding as the separate kernels it replaces
// (split-K fold, head norm, rope + append), so the results are identical.
template <bool FP8>
__global__ void __launch_bounds__(256)
fold_rope_append_kernel(const float* __restrict__ ws, int splits, long long split_stride,
                        const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ qkv,
                        const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                        const float* __restrict__ inv_freq, void* __restrict__ k_cache, void* __restrict__ v_cache,
                        float* __restrict__ k_scale, float* __restrict__ v_scale, long long tokens, int hq, int hkv, int D,
                        int rot_dim, float theta, int interleaved, int page_size, const void* __restrict__ q_norm_w,
                        const void* __restrict__ k_norm_w, int norm_wf32, float norm_offset, float norm_eps) {
  pdl_trigger();
  pdl_wait();
  const int heads = hq + 2 * hkv;
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= tokens * heads) return;
  const int lane = threadIdx.x & 31;
  const long long t = w / heads;
  const int h = (int)(w % heads);
  const long long row_off = t * (long long)heads * D + (long long)h * D;
  __nv_bfloat16* p = qkv + row_off;
  for (int i = lane * 4; i < D; i += 128) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < splits; s0 += 4) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        v[u] = s0 + u < splits ? __ldcg(reinterpret_cast<const float4*>(ws + (s0 + u) * split_stride + row_off + i))
                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 4; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
    }
    if (bias != nullptr) {
      const __nv_bfloat16* b = bias + (long long)h * D + i;
      acc.x += __bfloat162float(b[0]); acc.y += __bfloat162float(b[1]);
      acc.z += __bfloat162float(b[2]); acc.w += __bfloat162float(b[3]);
    }
    uint2 o;
    o.x = pack_bf16x2(acc.x, acc.y);
    o.y = pack_bf16x2(acc.z, acc.w);
    *reinterpret_cast<uint2*>(p + i) = o;
  }
  __syncwarp();
  const void* nw = h < hq ? q_norm_w : (h < hq + hkv ? k_norm_w : nullptr);
  if (nw != nullptr) {
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) { const float x = __bfloat162float(p[i]); ss += x * x; }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)D + norm_eps);
    for (int i = lane; i < D; i += 32) {
      const float wv = norm_wf32 ? reinterpret_cast<const float*>(nw)[i]
                                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(nw)[i]);
      p[i] = __float2bfloat16_rn(__bfloat162float(p[i]) * inv * (wv + norm_offset));
    }
    __syncwarp();
  }
  rope_append_row<FP8>(p, lane, t, h, positions, slot_mapping, inv_freq, k_cache, v_cache, k_scale, v_scale, hq, hkv, D,
                       rot_dim, theta, interleaved, page_size);
}

// ---------------------------------------------------------------------------------
// Decode attention.
// ---------------------------------------------------------------------------------
template <int D, bool FP8>
struct DecodeSmem {
  // fp8 pages stay as bytes in shared memory and are expanded to fp16 in registers, fragment by fragment, so there
  // is no second copy of a page and no extra barrier: a stage is half the size of a bf16 stage
  // fp8: the kernel is bound by the dependent instruction chain of a page, not by bytes, so a CTA runs TWO groups
  // of four warps that take alternate pages (own stages, own named barrier) and twice the warps hide the chain
  static constexpr int kGroups = FP8 ? 2 : 1;
  static constexpr int kStages = 3;
  static constexpr int kTile = kPage * D * 2;                 // bf16 tile bytes
  static constexpr int kRaw = FP8 ? kPage * D : 0;            // fp8 page bytes (K or V)
  static constexpr int kStageBytes = FP8 ? 2 * kRaw + 2 * kPage * 4 : 2 * kTile;   // fp8: K, V, k scales, v scales
  static constexpr int kQ = FP8 ? 0 : 16 * D * 2;             // fp8: q lives in registers
  static constexpr int kMerge = 4 * kGroups * 16 * (D + 2) * 4;   // per-warp partial O, m, l (fp32)
  // the merge buffer aliases the (by then idle) pipeline stages
  static_assert(kMerge <= kGroups * kStages * kStageBytes, "merge buffer must fit in the stage area");
  static constexpr int kTotal = kGroups * kStages * kStageBytes + kQ;
};

// Position of 16-byte chunk `c` of row `r` inside a row of an fp8 page in shared memory: the XOR spreads the eight
// rows that one quarter-warp (K fragments) or one ldmatrix phase (V fragments) touches over all banks.
template <int CHB>
__device__ __forceinline__ int fp8_chunk(int r, int c) {
  return CHB >= 8 ? (c ^ (((r & 1) << 2) | ((r >> 1) & 3))) : c;
}
__device__ __forceinline__ uint32_t prmt_u32(uint32_t a, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %1, %2;" : "=r"(r) : "r"(a), "r"(sel));
  return r;
}

template <int D, bool FP8>
__global__ void __launch_bounds__(FP8 ? 256 : 128, FP8 && D <= 128 ? 2 : 1)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const void* __restrict__ k_cache,
                    const void* __restrict__ v_cache, const float* __restrict__ k_scale,
                    const float* __restrict__ v_scale, const int* __restrict__ block_table,
                    const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int hq, int hkv, int max_pages, long long q_stride,
                    long long o_stride, float scale, int pages_per_split, int nsplit, int window) {
  using SM = DecodeSmem<D, FP8>;
  constexpr int CH = D / 8;
  extern __shared__ __align__(128) uint8_t smem_attn[];
  pdl_trigger();
  pdl_wait();
  constexpr int NWG = SM::kGroups;
  const int wg = threadIdx.x >> 7;                 // warp group (0 unless fp8)
  const int tid = threadIdx.x & 127;               // thread inside its group
  uint8_t* stage_base = smem_attn + wg * SM::kStages * SM::kStageBytes;
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_attn + NWG * SM::kStages * SM::kStageBytes);   // bf16 path only
  float* sMerge = reinterpret_cast<float*>(smem_attn);
  auto group_sync = [&]() {
    if constexpr (NWG == 1) __syncthreads();
    else if (wg == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
    else asm volatile("bar.sync 2, 128;" ::: "memory");
  };
  constexpr int CHB = D / 16;      // 16-byte chunks per row of an fp8 page

  const int b = blockIdx.x;
  const int group = hq / hkv;
  const int gtiles = (group + 15) / 16;
  const int kvh = blockIdx.y / gtiles;
  const int gt = blockIdx.y % gtiles;
  const int split = blockIdx.z;
  const int ctx = seq_lens[b];
  const int warp = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31;      // warp inside its group
  const int g = lane >> 2, t4 = lane & 3;
  const int rows_valid = min(16, group - gt * 16);
  const int head0 = kvh * group + gt * 16;

  int first_key = 0;
  if (window > 0) first_key = max(0, ctx - window);
  const int total_pages = (ctx + kPage - 1) / kPage;
  const int page_lo = max(split * pages_per_split, first_key / kPage);
  const int page_hi = min(total_pages, (split + 1) * pages_per_split);
  const int n_pages_all = max(0, page_hi - page_lo);
  const int n_pages = n_pages_all > wg ? (n_pages_all - wg + NWG - 1) / NWG : 0;   // pages wg, wg + NWG, ... of the range

  // Q tile: 16 rows (q heads of the group, zero padded) x D
  // fp8: q goes to registers as fp16 A fragments (e4m3 expands to fp16 exactly, so the MMAs run on fp16).  The
  // contraction index is permuted so that one 16-byte load of a K row feeds four MMA steps: step (j, s) of lane
  // quarter t4 covers channels j * 64 + 16 * t4 + 4 * s + {0, 1} (first half of k) and + {2, 3} (second half).
  uint32_t qf[FP8 ? D / 64 : 1][4][4];
  if constexpr (FP8) {
#pragma unroll
    for (int j = 0; j < D / 64; ++j) {
#pragma unroll
      for (int hr = 0; hr < 2; ++hr) {
        const int r = g + hr * 8;
        uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
        if (r < rows_valid) {
          const __nv_bfloat16* qp = q + (long long)b * q_stride + (long long)(head0 + r) * D + j * 64 + 16 * t4;
          lo = *reinterpret_cast<const uint4*>(qp);
          hi = *reinterpret_cast<const uint4*>(qp + 8);
        }
        const uint32_t u[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int sidx = 0; sidx < 4; ++sidx) {
          const float2 f0 = unpack_bf16x2(u[2 * sidx]), f1 = unpack_bf16x2(u[2 * sidx + 1]);
          qf[j][sidx][hr] = pack_f16x2(f0.x, f0.y);
          qf[j][sidx][2 + hr] = pack_f16x2(f1.x, f1.y);
        }
      }
    }
  } else {
    for (int idx = tid; idx < 16 * CH; idx += 128) {
      const int r = idx / CH, ch = idx % CH;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r < rows_valid) val = *reinterpret_cast<const uint4*>(q + (long long)b * q_stride + (long long)(head0 + r) * D + ch * 8);
      *reinterpret_cast<uint4*>(sQ + swz<CH>(r, ch)) = val;
    }
  }

  // Page ids come from the block table in global memory; a load inside the loop would put its latency in front
  // of every copy.  The ids of the first pages are fetched together, later ones one iteration before their use.
  const int* bt = block_table + (long long)b * max_pages + page_lo;
  auto issue = [&](int page, int st) {
    uint8_t* sb = stage_base + st * SM::kStageBytes;
    if constexpr (FP8) {
      const uint8_t* kp = reinterpret_cast<const uint8_t*>(k_cache) + ((long long)page * hkv + kvh) * kPage * D;
      const uint8_t* vp = reinterpret_cast<const uint8_t*>(v_cache) + ((long long)page * hkv + kvh) * kPage * D;
      for (int idx = tid; idx < kPage * CHB; idx += 128) {
        const int r = idx / CHB, c = idx % CHB;
        const int off = r * D + fp8_chunk<CHB>(r, c) * 16;
        cp_async16(sb + off, kp + idx * 16);
        cp_async16(sb + SM::kRaw + off, vp + idx * 16);
      }
      if (tid < kPage / 4) {
        const long long srow = ((long long)page * hkv + kvh) * kPage;
        cp_async16(sb + 2 * SM::kRaw + tid * 16, k_scale + srow + tid * 4);
        cp_async16(sb + 2 * SM::kRaw + kPage * 4 + tid * 16, v_scale + srow + tid * 4);
      }
    } else {
      const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(k_cache) + ((long long)page * hkv + kvh) * kPage * D;
      const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(v_cache) + ((long long)page * hkv + kvh) * kPage * D;
      load_tile_async<D, kPage>(reinterpret_cast<__nv_bfloat16*>(sb), kp, D, kPage);
      load_tile_async<D, kPage>(reinterpret_cast<__nv_bfloat16*>(sb + SM::kTile), vp, D, kPage);
    }
  };

  int first_pages[SM::kStages];
#pragma unroll
  for (int s = 0; s < SM::kStages; ++s) first_pages[s] = s < n_pages ? bt[s * NWG + wg] : 0;
#pragma unroll
  for (int s = 0; s < SM::kStages - 1; ++s) {
    if (s < n_pages) issue(first_pages[s], s);
    cp_async_commit();
  }
  int page_next = first_pages[SM::kStages - 1];      // id of page pi + kStages - 1 at the top of iteration pi

  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float scale_log2 = scale * 1.4426950408889634f;

  for (int pi = 0; pi < n_pages; ++pi) {
    const int st = pi % SM::kStages;
    if constexpr (FP8) {
      // one barrier per page: after it every thread has left page pi - 1, whose stage the next copy overwrites
      cp_async_wait<SM::kStages - 2>();
      group_sync();
      const int page_now = page_next;
      if (pi + SM::kStages < n_pages) page_next = bt[(pi + SM::kStages) * NWG + wg];
      if (pi + SM::kStages - 1 < n_pages) issue(page_now, (pi + SM::kStages - 1) % SM::kStages);
      cp_async_commit();
    } else {
      const int page_now = page_next;
      if (pi + SM::kStages < n_pages) page_next = bt[(pi + SM::kStages) * NWG + wg];
      if (pi + SM::kStages - 1 < n_pages) issue(page_now, (pi + SM::kStages - 1) % SM::kStages);
      cp_async_commit();
      cp_async_wait<SM::kStages - 1>();
      __syncthreads();
    }
    const uint8_t* sb = stage_base + st * SM::kStageBytes;
    const __nv_bfloat16* cK = reinterpret_cast<const __nv_bfloat16*>(sb);
    const __nv_bfloat16* cV = reinterpret_cast<const __nv_bfloat16*>(sb + SM::kTile);
    const float* ksc = reinterpret_cast<const float*>(sb + 2 * SM::kRaw);      // fp8: per-token scales of the page
    const float* vsc = ksc + kPage;

    // this warp: keys [warp*16, warp*16+16) of the page
    const int key0 = (page_lo + pi * NWG + wg) * kPage + warp * 16;
    if (key0 < ctx && key0 + 16 > first_key) {
      float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
      if constexpr (FP8) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int r = warp * 16 + nt * 8 + g;
#pragma unroll
          for (int j = 0; j < D / 64; ++j) {
            const uint4 kw = *reinterpret_cast<const uint4*>(sb + r * D + fp8_chunk<CHB>(r, j * 4 + t4) * 16);
            const uint32_t w[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
            for (int sidx = 0; sidx < 4; ++sidx)
              mma_f16(s[nt], qf[j][sidx], cvt_e4m3x2_f16x2(w[sidx]), cvt_e4m3x2_f16x2(w[sidx] >> 16));
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) s[nt][e] *= ksc[warp * 16 + nt * 8 + t4 * 2 + (e & 1)];
        }
      } else {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          uint32_t a[4], bb[4];
          ldsm_a<CH>(a, sQ, 0, ks * 2, lane);
          ldsm_b_nt<CH>(bb, cK, warp * 16, ks * 2, lane);
          mma_bf16(s[0], a, bb[0], bb[1]);
          mma_bf16(s[1], a, bb[2], bb[3]);
        }
      }
      if (key0 + 16 > ctx || key0 < first_key) {      // only the pages at the two ends of the range have masked keys
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = key0 + nt * 8 + t4 * 2 + (e & 1);
            if (c >= ctx || c < first_key) s[nt][e] = -INFINITY;
          }
      }
      float mx[2];
      mx[0] = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
      mx[1] = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
      float corr[2], m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float mn = fmaxf(m_run[h], mx[h]);
        m_use[h] = mn == -INFINITY ? 0.f : mn;
        corr[h] = exp2f((m_run[h] - m_use[h]) * scale_log2);
        m_run[h] = mn;
      }
      uint32_t pf[4];
      float rs[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float p0 = exp2f((s[nt][0] - m_use[0]) * scale_log2);
        const float p1 = exp2f((s[nt][1] - m_use[0]) * scale_log2);
        const float p2 = exp2f((s[nt][2] - m_use[1]) * scale_log2);
        const float p3 = exp2f((s[nt][3] - m_use[1]) * scale_log2);
        rs[0] += p0 + p1;
        rs[1] += p2 + p3;
        if constexpr (FP8) {
          // the per-token scale of V rides on P (the row sums above use the unscaled probabilities)
          const float v0 = vsc[warp * 16 + nt * 8 + t4 * 2], v1 = vsc[warp * 16 + nt * 8 + t4 * 2 + 1];
          pf[nt * 2 + 0] = pack_f16x2(p0 * v0, p1 * v1);
          pf[nt * 2 + 1] = pack_f16x2(p2 * v0, p3 * v1);
        } else {
          pf[nt * 2 + 0] = pack_bf16x2(p0, p1);
          pf[nt * 2 + 1] = pack_bf16x2(p2, p3);
        }
      }
      l_run[0] = l_run[0] * corr[0] + rs[0];
      l_run[1] = l_run[1] * corr[1] + rs[1];
      // the running maxima settle after the first pages; the accumulators are rescaled only when one moved
      if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          o_acc[i][0] *= corr[0]; o_acc[i][1] *= corr[0];
          o_acc[i][2] *= corr[1]; o_acc[i][3] *= corr[1];
        }
      }
      if constexpr (FP8) {
        // V fragments: a transposing ldmatrix over the page's BYTES read as 16-bit elements hands every lane, for
        // its two keys, the byte pair of channels (2g, 2g + 1) of a 16-channel chunk; a byte permute separates the
        // even and the odd channel, which become two n-tiles.  Accumulator tile 2c + par, element e of lane
        // quarter t4 therefore holds channel c * 16 + 4 * t4 + 2 * (e & 1) + par.
        const uint8_t* sV8 = sb + SM::kRaw;
        const int mat = lane >> 3;
        const int vrow = warp * 16 + (mat & 1) * 8 + (lane & 7);
#pragma unroll
        for (int cp = 0; cp < CHB / 2; ++cp) {
          uint32_t rr[4];
          ldsm_x4_t(rr, sV8 + vrow * D + fp8_chunk<CHB>(vrow, cp * 2 + (mat >> 1)) * 16);
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            const int c = cp * 2 + hc;
            const uint32_t u0 = prmt_u32(rr[hc * 2], 0x3120u), u1 = prmt_u32(rr[hc * 2 + 1], 0x3120u);
            mma_f16(o_acc[2 * c], pf, cvt_e4m3x2_f16x2(u0), cvt_e4m3x2_f16x2(u1));
            mma_f16(o_acc[2 * c + 1], pf, cvt_e4m3x2_f16x2(u0 >> 16), cvt_e4m3x2_f16x2(u1 >> 16));
          }
        }
      } else {
#pragma unroll
        for (int dt = 0; dt < D / 16; ++dt) {
          uint32_t bb[4];
          ldsm_b_t<CH>(bb, cV, warp * 16, dt * 2, lane);
          mma_bf16(o_acc[2 * dt], pf, bb[0], bb[1]);
          mma_bf16(o_acc[2 * dt + 1], pf, bb[2], bb[3]);
        }
      }
    }
    if constexpr (!FP8) __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the 4 warps' partials (each covered different keys) ----
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  constexpr int NW = 4 * NWG;                      // partials to merge: one per warp of the CTA
  float* wbuf = sMerge + (wg * 4 + warp) * 16 * (D + 2);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + h * 8;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      // channel of element 0 of this tile (bf16: consecutive pairs; fp8: see the V fragments above)
      const int d0 = FP8 ? (i >> 1) * 16 + 4 * t4 + (i & 1) : i * 8 + t4 * 2;
      wbuf[r * (D + 2) + d0] = o_acc[i][h * 2];
      wbuf[r * (D + 2) + d0 + (FP8 ? 2 : 1)] = o_acc[i][h * 2 + 1];
    }
    if (t4 == 0) {
      wbuf[r * (D + 2) + D] = m_run[h];
      wbuf[r * (D + 2) + D + 1] = l_run[h];
    }
  }
  __syncthreads();
  // thread -> (row r, column group cg covering D / (8 NWG) columns)
  {
    constexpr int CG = 8 * NWG, COLS = D / CG;
    const int r = threadIdx.x / CG, cg = threadIdx.x % CG;
    if (r < rows_valid) {
      float mw[NW], lw[NW], mmax = -INFINITY;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        mw[w] = sMerge[(w * 16 + r) * (D + 2) + D];
        lw[w] = sMerge[(w * 16 + r) * (D + 2) + D + 1];
        mmax = fmaxf(mmax, mw[w]);
      }
      float wgt[NW], ltot = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        wgt[w] = mw[w] == -INFINITY ? 0.f : exp2f((mw[w] - mmax) * scale_log2);
        ltot += lw[w] * wgt[w];
      }
      const int head = head0 + r;
      if (nsplit == 1) {
        const float inv = ltot > 0.f ? 1.f / ltot : 0.f;
        __nv_bfloat16* op = out + (long long)b * o_stride + (long long)head * D;
        for (int c = cg * COLS; c < (cg + 1) * COLS; ++c) {
          float acc = 0.f;
#pragma unroll
          for (int w = 0; w < NW; ++w) acc += sMerge[(w * 16 + r) * (D + 2) + c] * wgt[w];
          op[c] = __float2bfloat16_rn(acc * inv);
        }
      } else {
        float* po = part_o + (((long long)b * hq + head) * nsplit + split) * D;
        for (int c = cg * COLS; c < (cg + 1) * COLS; ++c) {
          float acc = 0.f;
#pragma unroll
          for (int w = 0; w < NW; ++w) acc += sMerge[(w * 16 + r) * (D + 2) + c] * wgt[w];
          po[c] = acc;
        }
        if (cg == 0) {
          float* pml = part_ml + (((long long)b * hq + head) * nsplit + split) * 2;
          pml[0] = mmax;
          pml[1] = ltot;
        }
      }
    }
  }
}

// Merge split partials: one warp per (sequence, q head).
__global__ void __launch_bounds__(256)
decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                    int batch, int hq, int D, int nsplit, long long o_stride, float scale) {
  pdl_trigger();
  pdl_wait();
  const int w = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= batch * hq) return;
  const int lane = threadIdx.x & 31;
  const int b = w / hq, head = w % hq;
  const float* pml = part_ml + (long long)w * nsplit * 2;
  const float scale_log2 = scale * 1.4426950408889634f;
  float mmax = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mmax = fmaxf(mmax, pml[s * 2]);
  float ltot = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float m = pml[s * 2];
    ltot += m == -INFINITY ? 0.f : pml[s * 2 + 1] * exp2f((m - mmax) * scale_log2);
  }
  const float inv = ltot > 0.f ? 1.f / ltot : 0.f;
  for (int c = lane; c < D; c += 32) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float m = pml[s * 2];
      if (m == -INFINITY) continue;
      acc += part_o[((long long)w * nsplit + s) * D + c] * exp2f((m - mmax) * scale_log2);
    }
    out[(long long)b * o_stride + (long long)head * D + c] = __float2bfloat16_rn(acc * inv);
  }
}

template <int D, bool FP8>
static int launch_decode(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                         const float* v_scale, const int* block_table, const int* seq_lens, void* out, float* part_o,
                         float* part_ml, int batch, int hq, int hkv, int max_pages, long long q_stride,
                         long long o_stride, float scale, int pages_per_split, int nsplit, int window,
                         cudaStream_t stream) {
  using SM = DecodeSmem<D, FP8>;
  static bool cfg_dev[kMaxDevices] = {};
    bool& cfg = per_device_flag(cfg_dev);
  if (!cfg) {
    cudaFuncSetAttribute(paged_decode_kernel<D, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kTotal);
    cfg = true;
  }
  const int group = hq / hkv;
  dim3 grid(batch, hkv * ((group + 15) / 16), nsplit);
  cudaError_t e = launch_pdl(paged_decode_kernel<D, FP8>, grid, dim3(128 * SM::kGroups), SM::kTotal, stream, (const __nv_bfloat16*)q,
                             k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, (__nv_bfloat16*)out, part_o,
                             part_ml, hq, hkv, max_pages, q_stride, o_stride, scale, pages_per_split, nsplit, window);
  if (e == cudaSuccess && nsplit > 1)
    e = launch_pdl(decode_merge_kernel, dim3((batch * hq + 7) / 8), dim3(256), 0, stream, (const float*)part_o,
                   (const float*)part_ml, (__nv_bfloat16*)out, batch, hq, D, nsplit, o_stride, scale);
  return (int)e;
}

}  // namespace areno

using namespace areno;

extern "C" int areno_page_size() { return kPage; }

extern "C" int areno_rope_append_kv(void* qkv, const int* positions, const int* slot_mapping, const float* inv_freq,
                                    void* k_cache, void* v_cache, float* k_scale, float* v_scale, long long tokens,
                                    int hq, int hkv, int head_dim, int rot_dim, float theta, int interleaved,
                                    int page_size, int fp8, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const long long nw = tokens * (hq + 2 * hkv);
  const unsigned grid = (unsigned)((nw + 7) / 8);
  cudaError_t e;
  if (fp8)
    e = launch_pdl(rope_append_kernel<true>, dim3(grid), dim3(256), 0, stream, (__nv_bfloat16*)qkv, positions,
                   slot_mapping, inv_freq, k_cache, v_cache, k_scale, v_scale, tokens, hq, hkv, head_dim, rot_dim, theta,
                   interleaved, page_size);
  else
    e = launch_pdl(rope_append_kernel<false>, dim3(grid), dim3(256), 0, stream, (__nv_bfloat16*)qkv, positions,
                   slot_mapping, inv_freq, k_cache, v_cache, k_scale, v_scale, tokens, hq, hkv, head_dim, rot_dim, theta,
                   interleaved, page_size);
  return (int)e;
}

// Split-K fold + bias + optional q/k head norm + rope + KV append in one launch (decode).  ws: fp32
// [splits, tokens, (hq + 2 hkv) * head_dim] partials; qkv: bf16 output of the same row layout.
extern "C" int areno_fold_rope_append_kv(const float* ws, int splits, long long split_stride, const void* bias, void* qkv,
                                         const int* positions, const int* slot_mapping, const float* inv_freq,
                                         void* k_cache, void* v_cache, float* k_scale, float* v_scale, long long tokens,
                                         int hq, int hkv, int head_dim, int rot_dim, float theta, int interleaved,
                                         int page_size, int fp8, const void* q_norm_w, const void* k_norm_w,
                                         int norm_wf32, float norm_offset, float norm_eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (splits < 1 || (head_dim % 4) != 0) return -3;
  const long long nw = tokens * (hq + 2 * hkv);
  const unsigned grid = (unsigned)((nw + 7) / 8);
  cudaError_t e;
  if (fp8)
    e = launch_pdl(fold_rope_append_kernel<true>, dim3(grid), dim3(256), 0, stream, ws, splits, split_stride,
                   (const __nv_bfloat16*)bias, (__nv_bfloat16*)qkv, positions, slot_mapping, inv_freq, k_cache, v_cache,
                   k_scale, v_scale, tokens, hq, hkv, head_dim, rot_dim, theta, interleaved, page_size, q_norm_w, k_norm_w,
                   norm_wf32, norm_offset, norm_eps);
  else
    e = launch_pdl(fold_rope_append_kernel<false>, dim3(grid), dim3(256), 0, stream, ws, splits, split_stride,
                   (const __nv_bfloat16*)bias, (__nv_bfloat16*)qkv, positions, slot_mapping, inv_freq, k_cache, v_cache,
                   k_scale, v_scale, tokens, hq, hkv, head_dim, rot_dim, theta, interleaved, page_size, q_norm_w, k_norm_w,
                   norm_wf32, norm_offset, norm_eps);
  return (int)e;
}

// part_o: fp32 [batch, hq, nsplit, D]; part_ml: fp32 [batch, hq, nsplit, 2] (only used when nsplit > 1).
extern "C" int areno_paged_decode(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                                  const float* v_scale, const int* block_table, const int* seq_lens, void* out,
                                  float* part_o, float* part_ml, int batch, int hq, int hkv, int head_dim,
                                  int max_pages, long long q_stride, long long o_stride, float scale,
                                  int pages_per_split, int nsplit, int window, int fp8, cudaStream_t stream) {
  if (batch <= 0) return 0;
  if (hq % hkv != 0) return -3;
  if (head_dim == 128) {
    if (fp8)
      return launch_decode<128, true>(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, out, part_o,
                                      part_ml, batch, hq, hkv, max_pages, q_stride, o_stride, scale, pages_per_split,
                                      nsplit, window, stream);
    return launch_decode<128, false>(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, out, part_o, part_ml,
                                     batch, hq, hkv, max_pages, q_stride, o_stride, scale, pages_per_split, nsplit,
                                     window, stream);
  }
  if (head_dim == 256) {
    if (fp8)
      return launch_decode<256, true>(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, out, part_o,
                                      part_ml, batch, hq, hkv, max_pages, q_stride, o_stride, scale, pages_per_split,
                                      nsplit, window, stream);
    return launch_decode<256, false>(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, out, part_o, part_ml,
                                     batch, hq, hkv, max_pages, q_stride, o_stride, scale, pages_per_split, nsplit,
                                     window, stream);
  }
  if (head_dim == 64) {
    if (fp8)
      return launch_decode<64, true>(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, out, part_o, part_ml,
                                     batch, hq, hkv, max_pages, q_stride, o_stride, scale, pages_per_split, nsplit,
                                     window, stream);
    return launch_decode<64, false>(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, out, part_o, part_ml,
                                    batch, hq, hkv, max_pages, q_stride, o_stride, scale, pages_per_split, nsplit,
                                    window, stream);
  }
  return -2;
}
