// bf16 GEMM family for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma with the
// fp32 accumulator in TMEM -> tcgen05.ld epilogue.  Persistent, warp-specialised:
//   warp 0      TMA producer          (one lane issues)
//   warp 1      MMA issuer + TMEM owner (one lane issues)
//   warps 2..5  epilogue (each warp reads its own 32-lane quarter of TMEM)
// The accumulator is double-buffered in TMEM so the epilogue of tile i overlaps the main
// loop of tile i+1.
//
// Logical problem: D[M,N] = sum_k A(m,k) * B(n,k), with each operand either K-major
// (memory [rows, K]) or MN-major (memory [K, rows]).  That covers the three linear-layer
// products without any transpose pass:
//   forward  Y  = X  W^T   : A = X  (K-major),  B = W (K-major)
//   dgrad    dX = dY W     : A = dY (K-major),  B = W (MN-major)
//   wgrad    dW = dY^T X   : A = dY (MN-major), B = X (MN-major), fp32 accumulate epilogue
// Replaces the cublasGemmEx wrapper of the reference (areno/accel/csrc/linear.cu:73-249).
#include "common.cuh"
#include "launch.h"

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

namespace areno {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const void* bias;  // bf16 [N] or nullptr
  int* status;
  int tiles_m, tiles_n;
  int epi;
  int splits;         // split-K factor (1 = none); split s covers k-blocks [s*kb_per_split, ...)
  int kb_per_split;
  long long split_stride;  // elements between consecutive split partials in C (fp32 workspace)
  // Extra destinations of a bf16 result (epi 0/1): the same tile is also stored at the same
  // (row, col) of each of these buffers, which may live in a peer GPU's memory (plain st.global
  // over NVLink).  Used by row-parallel TP linears to deliver their partial to every rank.
  int n_extra;
  void* extra[7];
  // Grouped (mixture-of-experts) modes, driven by the device-side plan of moe.cu:
  //   1: every 128-row M tile belongs to one expert (tile_expert[m_tile], -1 = unused tile); the B
  //      operand of expert e starts b_group_rows further along B's outer TMA coordinate.
  //   2: work item = (expert, output tile); the K range of expert e is rows
  //      [expert_rows[2e], expert_rows[2e] + expert_rows[2e+1]) of A and B (multiples of 128) and
  //      its output starts c_group_stride elements further into C (per-expert weight gradients).
  int group_mode;
  const int* tile_expert;
  const int* expert_rows;
  long long b_group_rows;
  long long c_group_stride;
  int num_groups;
  // Tile order: 0 = consecutive work items walk M first, 1 = N first.  The CTAs running at the same
  // time then span all tiles of the SHORT dimension and a few of the long one, which keeps both
  // operand working sets inside L2 (otherwise a weight-gradient GEMM re-reads dY from DRAM once per
  // N tile).
  int n_fast;
  // Gated-activation epilogue (epi 4 = SiLU, 5 = GELU-tanh; 256-wide tiles, K-major operands): B is a
  // merged [2 * gate_rows, K] weight (gate rows first, then up rows).  A tile pairs 128 gate rows
  // with the 128 up rows of the same channels, so both halves of a channel land in one
  // accumulator and the epilogue stores act(gate) * up: C is [M, gate_rows].
  long long gate_rows;
  // Tail splitting (plain mode, splits == 1): the persistent grid walks `tail_first` whole tiles, then the
  // remaining `tail_tiles` tiles (less than a wave) are cut into `tail_splits` K ranges of `tail_kb`
  // k-blocks each so that the last round keeps every SM busy with a fraction of a tile instead of leaving
  // most of them idle for a whole tile.  Tail partials go to tail_ws[tail tile][split][128][BN] (fp32)
  // and a small kernel folds them with the requested epilogue.
  int tail_first, tail_tiles, tail_splits, tail_kb;
  float* tail_ws;
  // Weight-streaming GEMMs (few rows): number of B boxes (one k-block of one N tile) every CTA asks L2 to fetch
  // for its own first work items BEFORE it waits for the previous kernel of the stream.  The weights do not depend
  // on that kernel, so HBM keeps streaming while a short latency-bound kernel (norm, activation, rope) runs.
  int b_prefetch;
  // Log-sum-exp epilogue (epi 6; LM head): nothing is stored for the [M, N] product.  Every row of a tile is
  // reduced on the fly to (max, sum exp(x - max), sum exp(x - max) x, x[target]) over the tile's columns below
  // `lse_valid`, with x rounded to bf16 first (and soft-capped when lse_softcap > 0), and written to
  // lse_out[(n_tile * M + row) * 4 ...]; a small kernel merges the tiles of a row.
  const long long* lse_targets;   // global token id per row
  long long lse_vocab_start;      // id of column 0
  int lse_valid;                  // columns >= lse_valid are padding
  float lse_softcap;
  float* lse_out;
};

struct WorkItem {
  int m0, n0, kb_lo, kb_hi, split;
  int tail;         // index among the tail tiles, or -1 for a whole tile
  int b_off;        // added to B's outer TMA coordinate
  long long c_off;  // elements added to the C pointer
  bool skip;        // nothing to do for any role
  bool zero;        // no K range: the epilogue stores zeros, the other roles skip
};

template <int BN>
__device__ __forceinline__ WorkItem decode_work(const GemmParams& p, int work, int num_kb) {
  WorkItem w;
  w.b_off = 0;
  w.c_off = 0;
  w.skip = false;
  w.zero = false;
  w.tail = -1;
  if (p.tail_splits > 0 && work >= p.tail_first) {
    const int r = work - p.tail_first;
    w.tail = r / p.tail_splits;
    w.split = r - w.tail * p.tail_splits;
    const int tile = p.tail_first + w.tail;
    w.m0 = (p.n_fast ? tile / p.tiles_n : tile % p.tiles_m) * kBM;
    w.n0 = (p.n_fast ? tile % p.tiles_n : tile / p.tiles_m) * BN;
    w.kb_lo = w.split * p.tail_kb;
    w.kb_hi = min(num_kb, w.kb_lo + p.tail_kb);
    return w;
  }
  if (p.group_mode == 2) {
    const int tiles = p.tiles_m * p.tiles_n;
    const int e = work / tiles;
    const int tile = work - e * tiles;
    w.m0 = (p.n_fast ? tile / p.tiles_n : tile % p.tiles_m) * kBM;
    w.n0 = (p.n_fast ? tile % p.tiles_n : tile / p.tiles_m) * BN;
    w.split = 0;
    w.kb_lo = p.expert_rows[2 * e] / kBK;
    w.kb_hi = w.kb_lo + p.expert_rows[2 * e + 1] / kBK;
    w.c_off = (long long)e * p.c_group_stride;
    if (w.kb_hi == w.kb_lo) {
      if (p.epi == 3) w.skip = true;  // accumulate: adding nothing
      else w.zero = true;
    }
    return w;
  }
  const int tile = work / p.splits;
  w.split = work - tile * p.splits;
  const int m_tile = p.n_fast ? tile / p.tiles_n : tile % p.tiles_m;
  w.m0 = m_tile * kBM;
  w.n0 = (p.n_fast ? tile % p.tiles_n : tile / p.tiles_m) * BN;
  w.kb_lo = w.split * p.kb_per_split;
  w.kb_hi = min(num_kb, w.kb_lo + p.kb_per_split);
  if (p.group_mode == 1) {
    const int e = p.tile_expert[m_tile];
    if (e < 0) w.skip = true;
    else w.b_off = (int)(e * p.b_group_rows);
  }
  return w;
}

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr uint32_t kABytes = kBM * kBK * 2;
  static constexpr uint32_t kBBytes = BN * kBK * 2;
  static constexpr uint32_t kBarOffset = STAGES * (kABytes + kBBytes);
  static constexpr uint32_t kTotal = kBarOffset + (2 * STAGES + 4) * 8 + 16 + 1024;  // + align slack
};

__device__ __forceinline__ void store_row_bf16(__nv_bfloat16* dst, const uint32_t (&r)[32], int ncols,
                                               const __nv_bfloat16* bias) {
  // dst points at 32 consecutive output columns of one row; ncols (<=32) of them are valid.
  if (ncols == 32) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a = __uint_as_float(r[v * 8 + 2 * j]);
        float b = __uint_as_float(r[v * 8 + 2 * j + 1]);
        if (bias != nullptr) {
          a += __bfloat162float(bias[v * 8 + 2 * j]);
          b += __bfloat162float(bias[v * 8 + 2 * j + 1]);
        }
        o[j] = pack_bf16x2(a, b);
      }
      *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < ncols) {
        float a = __uint_as_float(r[j]);
        if (bias != nullptr) a += __bfloat162float(bias[j]);
        dst[j] = __float2bfloat16_rn(a);
      }
    }
  }
}

__device__ __forceinline__ void store_row_f32(float* dst, const uint32_t (&r)[32], int ncols,
                                              bool accumulate) {
  if (ncols == 32) {
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      float4 o = make_float4(__uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]),
                             __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
      float4* p = reinterpret_cast<float4*>(dst + v * 4);
      if (accumulate) {
        float4 c = *p;
        o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
      }
      *p = o;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < ncols) {
        float a = __uint_as_float(r[j]);
        dst[j] = accumulate ? dst[j] + a : a;
      }
    }
  }
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One 32-column chunk of a row for the log-sum-exp epilogue: x = accumulator rounded to bf16 (soft-capped and rounded
// again when CAP), online update of (max, sum exp(x - max), sum exp(x - max) * x) and pick-up of the target logit.
// The accumulations run as four independent chains and the exponent is one FMA + ex2; columns beyond `ncols`
// (vocabulary padding) take a large negative finite value so that they add exact zeros.  `tj` is the target's column
// relative to this chunk (outside [0, 32) when it lies elsewhere).
template <bool CAP>
__device__ __forceinline__ void lse_chunk(const uint32_t (&r)[32], int ncols, int tj, float cap, float& m, float& s,
                                          float& sx, float& tg) {
  constexpr float kLog2e = 1.4426950408889634f, kMasked = -1e30f;
  float x[32];
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    float a = __uint_as_float(r[j]), b = __uint_as_float(r[j + 1]);
    if constexpr (CAP) {
      const float inv = 1.f / cap;
      a = cap * tanhf(__bfloat162float(__float2bfloat16_rn(a)) * inv);
      b = cap * tanhf(__bfloat162float(__float2bfloat16_rn(b)) * inv);
    }
    const __nv_bfloat162 pk = __floats2bfloat162_rn(a, b);       // .x = a (low half), .y = b
    const uint32_t u = *reinterpret_cast<const uint32_t*>(&pk);
    x[j] = __uint_as_float(u << 16);
    x[j + 1] = __uint_as_float(u & 0xffff0000u);
  }
  if (ncols < 32) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j >= ncols) x[j] = kMasked;
  }
  float c0 = fmaxf(x[0], x[1]), c1 = fmaxf(x[2], x[3]), c2 = fmaxf(x[4], x[5]), c3 = fmaxf(x[6], x[7]);
#pragma unroll
  for (int j = 8; j < 32; j += 4) {
    c0 = fmaxf(c0, x[j]);
    c1 = fmaxf(c1, x[j + 1]);
    c2 = fmaxf(c2, x[j + 2]);
    c3 = fmaxf(c3, x[j + 3]);
  }
  const float mn = fmaxf(m, fmaxf(fmaxf(c0, c1), fmaxf(c2, c3)));
  const float ml2 = mn * kLog2e;
  const float rescale = m == -INFINITY ? 0.f : ex2_approx(fmaf(m, kLog2e, -ml2));
  float s0 = s * rescale, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  float t0 = sx * rescale, t1 = 0.f, t2 = 0.f, t3 = 0.f;
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float e0 = ex2_approx(fmaf(x[j], kLog2e, -ml2)), e1 = ex2_approx(fmaf(x[j + 1], kLog2e, -ml2));
    const float e2 = ex2_approx(fmaf(x[j + 2], kLog2e, -ml2)), e3 = ex2_approx(fmaf(x[j + 3], kLog2e, -ml2));
    s0 += e0;
    s1 += e1;
    s2 += e2;
    s3 += e3;
    t0 = fmaf(e0, x[j], t0);
    t1 = fmaf(e1, x[j + 1], t1);
    t2 = fmaf(e2, x[j + 2], t2);
    t3 = fmaf(e3, x[j + 3], t3);
  }
  s = (s0 + s1) + (s2 + s3);
  sx = (t0 + t1) + (t2 + t3);
  m = mn;
  if (__any_sync(0xffffffffu, static_cast<unsigned>(tj) < 32u)) {   // rare: 32 rows, one target column each
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (tj == j) tg = x[j];
  }
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmParams p) {
  using S = GemmSmem<BN, STAGES>;
  constexpr uint32_t NCOLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128
                             : (2 * BN <= 256) ? 256 : 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * S::kABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, NCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // barriers, TMEM and descriptors are set up: let the next kernel start its own prologue, then wait for
  // the previous kernel's results (everything below reads or writes global memory)
  pdl_trigger();
  const int num_kb = (p.K + kBK - 1) / kBK;
  const int num_work = p.tail_splits > 0 ? p.tail_first + p.tail_tiles * p.tail_splits
                                         : p.tiles_m * p.tiles_n * p.splits * (p.group_mode == 2 ? p.num_groups : 1);
  if constexpr (!B_MN) {
    if (threadIdx.x == 0 && p.b_prefetch > 0) {
      // plain mode only (the host sets b_prefetch for nothing else): decode_work reads nothing but `p`
      int left = p.b_prefetch;
      for (int work = blockIdx.x; work < num_work && left > 0; work += gridDim.x) {
        const WorkItem wi = decode_work<BN>(p, work, num_kb);
        for (int kb = wi.kb_lo; kb < wi.kb_hi && left > 0; ++kb, --left)
          tma_prefetch_l2_2d(&tma_b, kb * kBK, wi.n0);
      }
    }
  }
  pdl_wait();

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
      const WorkItem wi = decode_work<BN>(p, work, num_kb);
      if (wi.skip || wi.zero) continue;
      const int m0 = wi.m0, n0 = wi.n0, kb_lo = wi.kb_lo, kb_hi = wi.kb_hi;
      for (int kb = kb_lo; kb < kb_hi; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(&full_bar[stage], S::kABytes + S::kBBytes);
          uint8_t* a_dst = sA + stage * S::kABytes;
          uint8_t* b_dst = sB + stage * S::kBBytes;
          const int k0 = kb * kBK;
          if constexpr (A_MN) {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j)
              tma_load_2d(a_dst + j * 8192, &tma_a, &full_bar[stage], m0 + j * 64, k0);
          } else {
            tma_load_2d(a_dst, &tma_a, &full_bar[stage], k0, m0);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * 8192, &tma_b, &full_bar[stage], n0 + j * 64, k0 + wi.b_off);
          } else if (p.gate_rows > 0) {
            // two 128-row boxes (gate, up) stacked into one 256-row K-major tile
            tma_load_2d(b_dst, &tma_b, &full_bar[stage], k0, n0 / 2);
            tma_load_2d(b_dst + 128 * 128, &tma_b, &full_bar[stage], k0, static_cast<int>(p.gate_rows) + n0 / 2);
          } else {
            tma_load_2d(b_dst, &tma_b, &full_bar[stage], k0, n0 + wi.b_off);
          }
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
    if (!ok) {
      // Give copies already in flight time to land before the CTA's shared memory goes away.
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t acc_phase[2] = {0, 0};
    int acc = 0;
    bool ok = true;
    for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
      const WorkItem wi = decode_work<BN>(p, work, num_kb);
      if (wi.skip || wi.zero) continue;
      const int kb_lo = wi.kb_lo, kb_hi = wi.kb_hi;
      if (!mbar_wait(&tempty_bar[acc], acc_phase[acc] ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
      for (int kb = kb_lo; kb < kb_hi; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 3)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_base = smem_u32(sA + stage * S::kABytes);
          const uint32_t b_base = smem_u32(sB + stage * S::kBBytes);
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_base + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(a_base + kk * 32, 0, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_base + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(b_base + kk * 32, 0, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb != kb_lo || kk != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (lane == 0) umma_commit(&tfull_bar[acc]);
      __syncwarp();
      acc_phase[acc] ^= 1u;
      acc ^= 1;
    }
  } else {
    // ------------------------------- epilogue ----------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint32_t acc_phase[2] = {0, 0};
    int acc = 0;
    bool ok = true;
    for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
      const WorkItem wi = decode_work<BN>(p, work, num_kb);
      if (wi.skip) continue;
      const int split = wi.split, m0 = wi.m0, n0 = wi.n0;
      if (wi.zero) {
        // an expert without rows: its gradient tile is zero (no accumulator was produced)
        const int zrow = m0 + q * 32 + lane;
        uint32_t z[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) z[j] = 0u;
        for (int c = 0; c < BN && zrow < p.M; c += 32) {
          const int col = n0 + c;
          const int ncols = min(32, p.N - col);
          if (ncols <= 0) break;
          if (p.epi <= 1)
            store_row_bf16(reinterpret_cast<__nv_bfloat16*>(p.C) + wi.c_off + (long long)zrow * p.ldc + col, z, ncols, nullptr);
          else
            store_row_f32(reinterpret_cast<float*>(p.C) + wi.c_off + (long long)zrow * p.ldc + col, z, ncols, false);
        }
        continue;
      }
      if (!mbar_wait(&tfull_bar[acc], acc_phase[acc], abort_flag, p.status, 4)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(acc * BN);
      if (wi.tail >= 0) {
        // a K slice of a tail tile: the raw fp32 accumulator goes to the compact tail workspace
        float* tw = p.tail_ws + ((size_t)(wi.tail * p.tail_splits + wi.split) * kBM + (q * 32 + lane)) * BN;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c, r);
          tmem_ld_wait();
          store_row_f32(tw + c, r, 32, false);
        }
      } else if (p.epi == 6) {
        const long long tgt = row < p.M ? p.lse_targets[row] - p.lse_vocab_start - n0 : -1;
        const int tcol = tgt >= 0 && tgt < BN ? (int)tgt : -1;      // target column inside this tile, if any
        float m = -INFINITY, s = 0.f, sx = 0.f, tg = 0.f;
        const bool capped = p.lse_softcap > 0.f;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          const int ncols = min(32, p.lse_valid - (n0 + c));
          if (ncols <= 0) break;      // the same for the whole warp
          uint32_t r[32];
          tmem_ld_32x32(t_row + c, r);
          tmem_ld_wait();
          if (capped) lse_chunk<true>(r, ncols, tcol - c, p.lse_softcap, m, s, sx, tg);
          else lse_chunk<false>(r, ncols, tcol - c, 0.f, m, s, sx, tg);
        }
        if (row < p.M)
          *reinterpret_cast<float4*>(p.lse_out + ((size_t)(n0 / BN) * p.M + row) * 4) = make_float4(m, s, sx, tg);
      } else if (p.epi >= 4) {
        if constexpr (BN == 256) {
#pragma unroll 1
          for (int c = 0; c < 128; c += 32) {
            uint32_t rg[32], ru[32];
            tmem_ld_32x32(t_row + c, rg);
            tmem_ld_32x32(t_row + 128 + c, ru);
            tmem_ld_wait();
            const int col = n0 / 2 + c;
            const int ncols = min(32, static_cast<int>(p.gate_rows) - col);
            if (row < p.M && ncols > 0) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                // both halves pass through bf16 first: the same values the unfused path reads back
                const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(rg[j])));
                const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(ru[j])));
                float a;
                if (p.epi == 4) {
                  a = g / (1.f + __expf(-g));
                } else {
                  const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
                  a = 0.5f * g * (1.f + t);
                }
                rg[j] = __float_as_uint(a * u);
              }
              store_row_bf16(reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col, rg, ncols, nullptr);
            }
          }
        }
      } else
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c, r);
        tmem_ld_wait();
        const int col = n0 + c;
        const int ncols = min(32, p.N - col);
        if (row < p.M && ncols > 0) {
          if (p.epi == 0 || p.epi == 1) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + wi.c_off + (long long)row * p.ldc + col;
            const __nv_bfloat16* bias =
                p.epi == 1 ? reinterpret_cast<const __nv_bfloat16*>(p.bias) + col : nullptr;
            store_row_bf16(dst, r, ncols, bias);
            for (int e = 0; e < p.n_extra; ++e)
              store_row_bf16(reinterpret_cast<__nv_bfloat16*>(p.extra[e]) + (long long)row * p.ldc + col, r, ncols,
                             bias);
          } else {
            float* dst = reinterpret_cast<float*>(p.C) + wi.c_off + split * p.split_stride + (long long)row * p.ldc + col;
            store_row_f32(dst, r, ncols, p.epi == 3);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc_phase[acc] ^= 1u;
      acc ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, NCOLS);
}

// ------------------------------- host side ---------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

int make_tensor_map_2d_bf16(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer,
                            uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

static int num_sms() {
  static int n_dev[kMaxDevices] = {};
  int& n = n_dev[current_device_slot()];
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

// ARENO_GEMM_L2_PREFETCH=0 switches the pre-wait weight prefetch off (for A/B timing).
static bool l2_prefetch_enabled() {
  static const bool on = [] {
    const char* v = getenv("ARENO_GEMM_L2_PREFETCH");
    return v == nullptr || v[0] != '0';
  }();
  return on;
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES>;
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
  static bool configured_dev[kMaxDevices] = {};
  bool& configured = per_device_flag(configured_dev);
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int grid = p.tiles_m * p.tiles_n * p.splits;
  if (grid > num_sms()) grid = num_sms();
  GemmParams q = p;
  q.b_prefetch = 0;
  if (!B_MN && p.group_mode == 0 && p.gate_rows == 0 && p.M <= 4 * kBM && l2_prefetch_enabled()) {
    // at most ~40 MB per launch: what L2 keeps beside the running kernel's own stream
    const long long box = (long long)BN * kBK * 2;
    q.b_prefetch = (int)std::min<long long>(4096, (40ll << 20) / (box * grid));
  }
  return static_cast<int>(launch_pdl(kern, dim3(grid), dim3(kGemmThreads), S::kTotal, stream, ta, tb, q));
}

template <bool A_MN, bool B_MN>
static int dispatch_bn(int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                       cudaStream_t stream) {
  switch (bn) {
    case 256: return launch_gemm<256, 4, A_MN, B_MN>(ta, tb, p, stream);
    case 128: return launch_gemm<128, 6, A_MN, B_MN>(ta, tb, p, stream);
    case 64: return launch_gemm<64, 8, A_MN, B_MN>(ta, tb, p, stream);
    case 32:
      if constexpr (!B_MN) return launch_gemm<32, 10, A_MN, B_MN>(ta, tb, p, stream);
      return -2;
    default: return -2;
  }
}

static int pick_bn(int M, int N, bool b_mn) {
  // Measured on B200: the 128x256 tile wins whenever N allows it (smaller N-tiles are bound by
  // shared-memory operand bandwidth); narrower tiles only serve narrow outputs.  Exception: skinny
  // split-K problems (one M tile, few N tiles) run 10-20 % faster with 128-wide tiles, which
  // double the number of CTAs streaming the weight for the same number of K splits.
  if (M <= kBM && !b_mn && N > 128 && (N + 255) / 256 <= 37) return 128;
  if (N > 128) return 256;
  if (N > 64) return 128;
  if (N > 32 || b_mn) return 64;
  return 32;
}

struct ExtraDst {
  int n;
  void* p[7];
};

// Folds the K slices of the tail tiles (see GemmParams::tail_*) in split order and applies the epilogue the
// GEMM was asked for: 0 bf16, 1 bf16 + bias, 2 fp32 store, 3 fp32 accumulate.  One thread per 4 columns.
__global__ void __launch_bounds__(256)
tail_reduce_kernel(const float* __restrict__ ws, void* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M,
                   int N, long long ldc, int epi, int bn, int tiles_m, int tiles_n, int n_fast, int tail_first,
                   int tail_tiles, int tail_splits) {
  pdl_trigger();
  pdl_wait();
  const int vec_per_tile = kBM * bn / 4;
  const long long total = (long long)tail_tiles * vec_per_tile;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int tt = (int)(idx / vec_per_tile);
    const int v = (int)(idx % vec_per_tile);
    const int r = v / (bn / 4), c = (v % (bn / 4)) * 4;
    const int tile = tail_first + tt;
    const int row = (n_fast ? tile / tiles_n : tile % tiles_m) * kBM + r;
    const int col = (n_fast ? tile % tiles_n : tile / tiles_m) * bn + c;
    if (row >= M || col >= N) continue;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* base = ws + ((size_t)tt * tail_splits * kBM + r) * bn + c;
    for (int s0 = 0; s0 < tail_splits; s0 += 4) {
      float4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        x[u] = s0 + u < tail_splits ? __ldcg(reinterpret_cast<const float4*>(base + (size_t)(s0 + u) * kBM * bn))
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 4; ++u) { acc.x += x[u].x; acc.y += x[u].y; acc.z += x[u].z; acc.w += x[u].w; }
    }
    float o[4] = {acc.x, acc.y, acc.z, acc.w};
    const int ncols = min(4, N - col);
    if (epi <= 1) {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(C) + (long long)row * ldc + col;
      for (int j = 0; j < ncols; ++j)
        dst[j] = __float2bfloat16_rn(o[j] + (epi == 1 ? __bfloat162float(bias[col + j]) : 0.f));
    } else {
      float* dst = reinterpret_cast<float*>(C) + (long long)row * ldc + col;
      for (int j = 0; j < ncols; ++j) dst[j] = epi == 3 ? dst[j] + o[j] : o[j];
    }
  }
}

// out[m, n] = bf16(sum_s ws[s, m, n] (+ bias[n])), fixed summation order; the result is also
// written to every extra destination (peer inboxes of a TP group).
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ bias,
                     int M, int N, long long ldc, long long split_stride, int splits, ExtraDst extra) {
  pdl_trigger();
  pdl_wait();
  const int nvec = N >> 2;
  const long long total = (long long)M * nvec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(idx / nvec);
    const int c = (int)(idx % nvec) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < splits; s0 += 4) {   // four loads in flight, summed in split order
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        v[u] = s0 + u < splits ? __ldcg(reinterpret_cast<const float4*>(ws + (s0 + u) * split_stride + (long long)m * N + c))
                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 4; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
    }
    if (bias != nullptr) {
      acc.x += __bfloat162float(bias[c]); acc.y += __bfloat162float(bias[c + 1]);
      acc.z += __bfloat162float(bias[c + 2]); acc.w += __bfloat162float(bias[c + 3]);
    }
    uint2 o = make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
    *reinterpret_cast<uint2*>(out + (long long)m * ldc + c) = o;
    for (int e = 0; e < extra.n; ++e)
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(extra.p[e]) + (long long)m * ldc + c) = o;
  }
}

// Merge the per-tile log-sum-exp statistics of every row (see GemmParams::lse_*): one warp per row.
__global__ void __launch_bounds__(256)
lse_combine_kernel(const float* __restrict__ part, int tiles_n, int M, float* __restrict__ out_max,
                   float* __restrict__ out_sum, float* __restrict__ out_sumx, float* __restrict__ out_tgt) {
  pdl_wait();
  const int row = (int)((blockIdx.x * (unsigned)blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  float m = -INFINITY, s = 0.f, sx = 0.f, tg = 0.f;
  for (int t = lane; t < tiles_n; t += 32) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(part + ((size_t)t * M + row) * 4));
    tg += v.w;
    if (v.x == -INFINITY) continue;
    const float mn = fmaxf(m, v.x);
    const float a = m == -INFINITY ? 0.f : __expf(m - mn), b = __expf(v.x - mn);
    s = s * a + v.y * b;
    sx = sx * a + v.z * b;
    m = mn;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    const float osx = __shfl_xor_sync(0xffffffffu, sx, o);
    tg += __shfl_xor_sync(0xffffffffu, tg, o);
    const float mn = fmaxf(m, om);
    if (mn != -INFINITY) {
      const float a = m == -INFINITY ? 0.f : __expf(m - mn), b = om == -INFINITY ? 0.f : __expf(om - mn);
      s = s * a + os * b;
      sx = sx * a + osx * b;
    }
    m = mn;
  }
  if (lane == 0) {
    out_max[row] = m;
    out_sum[row] = s;
    out_sumx[row] = sx;
    out_tgt[row] = tg;
  }
}

}  // namespace areno

using namespace areno;

// Bytes of fp32 scratch that a split-K launch of this shape may use (0 when no split applies).
extern "C" long long areno_gemm_workspace_bytes(int M, int N, int K) {
  if (M > kBM || (N % 4) != 0) return 0;
  return 16ll * M * N * 4;  // at most 16 splits
}

struct GroupArgs {
  int mode;
  const int* tile_expert;
  const int* expert_rows;
  long long b_group_rows;
  long long c_group_stride;
  int num_groups;
};

struct LseArgs {
  const long long* targets;
  long long vocab_start;
  int valid;
  float softcap;
  float* out;
};

static int gemm_bf16_impl(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                          long long lda, long long ldb, long long ldc, int a_mn, int b_mn, int epi, int bn,
                          void* workspace, long long workspace_bytes, int* status, cudaStream_t stream,
                          void* const* extra, int n_extra, const GroupArgs* group = nullptr, int b_groups = 1,
                          int* splits_out = nullptr, long long gate_rows = 0, const LseArgs* lse = nullptr) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((epi == 6) != (lse != nullptr)) return -3;
  if (epi == 6) {
    if (a_mn || b_mn || group != nullptr || n_extra != 0 || lse->out == nullptr || lse->targets == nullptr ||
        lse->valid < 1 || lse->valid > N)
      return -3;
    bn = 256;
    workspace = nullptr;
  }
  if (epi == 4 || epi == 5) {  // gated activation: merged weight, 256-wide tiles only
    if (a_mn || b_mn || group != nullptr || n_extra != 0 || gate_rows <= 0 || N != 2 * gate_rows || (gate_rows % 8) != 0)
      return -3;
    bn = 256;
    workspace = nullptr;
  }
  if (n_extra < 0 || n_extra > 7 || (n_extra > 0 && epi > 1)) return -3;
  for (int e = 0; e < n_extra; ++e)
    if (reinterpret_cast<uintptr_t>(extra[e]) & 15) return -3;
  if ((lda % 8) != 0 || (ldb % 8) != 0) return -3;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15))
    return -3;
  if (epi != 6 && ((epi <= 1 || epi >= 4) ? (ldc % 8) != 0 : (ldc % 4) != 0)) return -3;
  {
    // cuTensorMapEncodeTiled needs a current driver context; threads that have not yet made a
    // runtime call (e.g. autograd workers) get the primary context bound here.
    static thread_local bool bound = false;
    if (!bound) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaSetDevice(dev);
      cudaFree(nullptr);
      bound = true;
    }
  }
  if (bn <= 0) bn = pick_bn(M, N, b_mn != 0);
  if (b_mn && bn < 64) bn = 64;
  CUtensorMap ta, tb;
  int rc;
  if (a_mn) rc = make_tensor_map_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, 64);
  else rc = make_tensor_map_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, 64, kBM);
  if (rc != 0) return rc;
  // grouped mode 1: B holds `b_groups` experts stacked along its outer dimension
  const uint64_t b_mult = (group != nullptr && group->mode == 1) ? (uint64_t)b_groups : 1u;
  if (b_mn) rc = make_tensor_map_2d_bf16(&tb, B, (uint64_t)N, (uint64_t)K * b_mult, (uint64_t)ldb * 2, 64, 64);
  else rc = make_tensor_map_2d_bf16(&tb, B, (uint64_t)K, (uint64_t)N * b_mult, (uint64_t)ldb * 2, 64,
                                    (epi == 4 || epi == 5) ? 128u : (uint32_t)bn);
  if (rc != 0) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.bias = bias; p.status = status;
  p.tiles_m = (M + kBM - 1) / kBM;
  p.tiles_n = (N + bn - 1) / bn;
  p.epi = epi;
  p.n_fast = p.tiles_n < p.tiles_m ? 1 : 0;
  p.splits = 1;
  p.kb_per_split = (K + kBK - 1) / kBK;
  p.split_stride = 0;
  p.n_extra = n_extra;
  for (int e = 0; e < 7; ++e) p.extra[e] = e < n_extra ? extra[e] : nullptr;
  p.gate_rows = (epi == 4 || epi == 5) ? gate_rows : 0;
  p.tail_first = p.tail_tiles = p.tail_splits = p.tail_kb = 0;
  p.tail_ws = nullptr;
  p.lse_targets = lse != nullptr ? lse->targets : nullptr;
  p.lse_vocab_start = lse != nullptr ? lse->vocab_start : 0;
  p.lse_valid = lse != nullptr ? lse->valid : 0;
  p.lse_softcap = lse != nullptr ? lse->softcap : 0.f;
  p.lse_out = lse != nullptr ? lse->out : nullptr;
  p.group_mode = 0;
  p.tile_expert = nullptr;
  p.expert_rows = nullptr;
  p.b_group_rows = 0;
  p.c_group_stride = 0;
  p.num_groups = 1;
  if (group != nullptr && group->mode != 0) {
    p.group_mode = group->mode;
    p.tile_expert = group->tile_expert;
    p.expert_rows = group->expert_rows;
    p.b_group_rows = group->b_group_rows;
    p.c_group_stride = group->c_group_stride;
    p.num_groups = group->num_groups;
    workspace = nullptr;  // no split-K in grouped modes
  }
  // Split-K for problems with too few output tiles to fill the GPU and a long K: decode (one M tile), and
  // the few-hundred-row batches of a tensor-parallel decode step, whose per-rank N or K is a fraction of the
  // layer's (two to four M tiles).
  const int num_kb = (K + kBK - 1) / kBK;
  const int tiles = p.tiles_m * p.tiles_n;
  bool split = false;
  if (epi <= 1 && M <= 4 * kBM && tiles * 2 <= num_sms() && num_kb >= 8 && workspace != nullptr && (N % 4) == 0) {
    int want = num_sms() / tiles;
    if (want > 16) want = 16;
    if (M > kBM && want > 8) want = 8;   // the fold reads every partial back: keep it a fraction of the GEMM
    int kbps = (num_kb + want - 1) / want;
    if (kbps < 4) kbps = 4;
    const int splits = (num_kb + kbps - 1) / kbps;
    if (splits > 1 && (long long)splits * M * N * 4 <= workspace_bytes) {
      p.splits = splits;
      p.kb_per_split = kbps;
      p.split_stride = (long long)M * N;
      p.C = workspace;
      p.ldc = N;
      p.epi = 2;
      p.bias = nullptr;
      p.n_extra = 0;  // partials go to the workspace; the fold kernel delivers the result
      split = true;
    }
  }
  // Tail splitting: more than one wave of whole tiles and a small remainder.
  bool tail = false;
  if (!split && group == nullptr && epi <= 3 && n_extra == 0 && workspace != nullptr && tiles > num_sms()) {
    const int rem = tiles % num_sms();
    if (rem > 0 && rem * 3 <= num_sms()) {
      const int want = num_sms() / rem;
      const int tkb = (num_kb + want - 1) / want;
      const int tsplits = (num_kb + tkb - 1) / tkb;
      if (tsplits >= 3 && (long long)rem * tsplits * kBM * bn * 4 <= workspace_bytes) {
        p.tail_first = tiles - rem;
        p.tail_tiles = rem;
        p.tail_splits = tsplits;
        p.tail_kb = tkb;
        p.tail_ws = reinterpret_cast<float*>(workspace);
        tail = true;
      }
    }
  }
  if (a_mn) {
    if (b_mn) rc = dispatch_bn<true, true>(bn, ta, tb, p, stream);
    else rc = dispatch_bn<true, false>(bn, ta, tb, p, stream);
  } else {
    if (b_mn) rc = dispatch_bn<false, true>(bn, ta, tb, p, stream);
    else rc = dispatch_bn<false, false>(bn, ta, tb, p, stream);
  }
  if (splits_out != nullptr) *splits_out = split ? p.splits : 1;
  if (rc == 0 && tail) {
    const long long total = (long long)p.tail_tiles * kBM * bn / 4;
    int rgrid = (int)((total + 255) / 256);
    if (rgrid > 148 * 8) rgrid = 148 * 8;
    return (int)launch_pdl(tail_reduce_kernel, dim3(rgrid), dim3(256), 0, stream, (const float*)p.tail_ws, C,
                           reinterpret_cast<const __nv_bfloat16*>(bias), M, N, ldc, epi, bn, p.tiles_m, p.tiles_n, p.n_fast,
                           p.tail_first, p.tail_tiles, p.tail_splits);
  }
  if (rc != 0 || !split) return rc;
  if (splits_out != nullptr) return 0;  // the caller folds the partials itself (fused consumer)
  ExtraDst xd;
  xd.n = n_extra;
  for (int e = 0; e < 7; ++e) xd.p[e] = e < n_extra ? extra[e] : nullptr;
  const long long total = (long long)M * (N / 4);
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  return (int)launch_pdl(splitk_reduce_kernel, dim3(grid), dim3(256), 0, stream,
                         reinterpret_cast<const float*>(workspace), reinterpret_cast<__nv_bfloat16*>(C),
                         epi == 1 ? reinterpret_cast<const __nv_bfloat16*>(bias) : nullptr, M, N, ldc, p.split_stride,
                         p.splits, xd);
}

extern "C" int areno_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                               long long lda, long long ldb, long long ldc, int a_mn, int b_mn, int epi, int bn,
                               void* workspace, long long workspace_bytes, int* status, cudaStream_t stream) {
  return gemm_bf16_impl(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, epi, bn, workspace, workspace_bytes, status,
                        stream, nullptr, 0);
}

// Same GEMM (K-major operands, bf16 result with optional bias), with the result ALSO stored at the
// same offsets of `n_extra` (<= 7) further buffers given as a host array of device pointers; these
// are typically the inbox lanes of the other ranks of a TP group, written over NVLink from the
// epilogue while later tiles are still being multiplied.
extern "C" int areno_gemm_bf16_push(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                                    long long lda, long long ldb, long long ldc, void* const* extra, int n_extra,
                                    void* workspace, long long workspace_bytes, int* status, cudaStream_t stream) {
  return gemm_bf16_impl(A, B, C, bias, M, N, K, lda, ldb, ldc, 0, 0, bias != nullptr ? 1 : 0, 0, workspace,
                        workspace_bytes, status, stream, extra, n_extra);
}

// Gate / up projection with the gated activation in the epilogue (inference: the pre-activation is not
// kept).  B: merged weight [2 * I, K] (gate rows, then up rows); C: bf16 [M, I] = act(A Bg^T) * (A Bu^T).
// act: 0 = SiLU, 1 = GELU-tanh.  Both products are rounded to bf16 before the activation, so the result
// equals areno_gemm_bf16 followed by areno_gated_act_fwd.
extern "C" int areno_gemm_bf16_gated(const void* A, const void* B, void* C, int M, int I, int K, long long lda,
                                     long long ldb, long long ldc, int act, int* status, cudaStream_t stream) {
  if (act != 0 && act != 1) return -3;
  return gemm_bf16_impl(A, B, C, nullptr, M, 2 * I, K, lda, ldb, ldc, 0, 0, 4 + act, 256, nullptr, 0, status, stream,
                        nullptr, 0, nullptr, 1, nullptr, I);
}

// ---- grouped (mixture-of-experts) entry points; plans come from areno_moe_align -------------------
// Forward / input-gradient: C[P, N] = A[P, K] * B_e, rows grouped by expert in 128-row tiles.
//   b_mn = 0: B is [E, N, K] (K contiguous)  -> C = A * B_e^T          (forward)
//   b_mn = 1: B is [E, K, N] (N contiguous)  -> C = A * B_e            (input gradient of the above)
extern "C" int areno_grouped_gemm_bf16(const void* A, const void* B, void* C, int P, int N, int K, int E, int b_mn,
                                       const int* tile_expert, int* status, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (P % kBM != 0 || E < 1) return -3;
  GroupArgs g{1, tile_expert, nullptr, b_mn ? (long long)K : (long long)N, 0, E};
  // B flattened over experts: [E*N, K] (K-major) or [E*K, N] (MN-major)
  return gemm_bf16_impl(A, B, C, nullptr, P, N, K, K, b_mn ? N : K, N, 0, b_mn, 0, 0, nullptr, 0, status, stream, nullptr,
                        0, &g, E);
}

// Weight gradient: dW[e][N, K] (+)= dY_e^T[N, rows_e] * X_e[rows_e, K]; dY is [P, N], X is [P, K].
// out_f32_accumulate = 1: fp32 accumulate into dW (main-grad buffers); 0: bf16 store.
extern "C" int areno_grouped_wgrad_bf16(const void* dY, const void* X, void* dW, int P, int N, int K, int E,
                                        const int* expert_rows, int out_f32_accumulate, int* status,
                                        cudaStream_t stream) {
  if (P <= 0 || E < 1) return 0;
  if (P % kBM != 0) return -3;
  GroupArgs g{2, nullptr, expert_rows, 0, (long long)N * K, E};
  return gemm_bf16_impl(dY, X, dW, nullptr, N, K, P, N, K, K, 1, 1, out_f32_accumulate ? 3 : 0, 0, nullptr, 0, status,
                        stream, nullptr, 0, &g, E);
}

// Skinny GEMM that leaves its split-K partials in `workspace` (fp32 [splits, M, N]) for a fused
// consumer (areno_splitk_residual_rmsnorm) instead of folding them.  *splits_out receives the number
// of partials; 1 means no split was applied and C holds the finished bf16 result.
extern "C" int areno_gemm_bf16_partials(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                        long long ldb, long long ldc, void* workspace, long long workspace_bytes,
                                        int* splits_out, int* status, cudaStream_t stream) {
  if (splits_out == nullptr) return -3;
  *splits_out = 1;
  return gemm_bf16_impl(A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, 0, 0, 0, workspace, workspace_bytes, status, stream,
                        nullptr, 0, nullptr, 1, splits_out);
}

// LM head fused with the per-row log-sum-exp statistics of the selected-token log-prob (and entropy): the
// [M, N] logits are never written.  A: hidden [M, K], B: head weight [N, K] (row n = token vocab_start + n),
// columns >= valid are padding.  Logits are rounded to bf16 (and soft-capped when softcap > 0) before they are
// reduced, exactly as if they had been stored and read back.  partials: fp32 scratch of
// areno_gemm_lse_partials_elems(M, N) elements.  Outputs (fp32 [M] each): row max, sum exp(x - max),
// sum exp(x - max) x, x[target] (0 when the target is outside [vocab_start, vocab_start + valid)).
extern "C" long long areno_gemm_lse_partials_elems(int M, int N) { return (long long)((N + 255) / 256) * M * 4; }

extern "C" int areno_gemm_bf16_lse(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                                   const long long* targets, long long vocab_start, int valid, float softcap,
                                   float* partials, float* out_max, float* out_sum, float* out_sumx, float* out_tgt,
                                   int* status, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (partials == nullptr || out_max == nullptr || out_sum == nullptr || out_sumx == nullptr || out_tgt == nullptr)
    return -3;
  LseArgs lse{targets, vocab_start, valid, softcap, partials};
  const int rc = gemm_bf16_impl(A, B, partials, nullptr, M, N, K, lda, ldb, 8, 0, 0, 6, 256, nullptr, 0, status, stream,
                                nullptr, 0, nullptr, 1, nullptr, 0, &lse);
  if (rc != 0) return rc;
  const int tiles_n = (N + 255) / 256;
  const long long threads = (long long)M * 32;
  return (int)launch_pdl(lse_combine_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, stream,
                         (const float*)partials, tiles_n, M, out_max, out_sum, out_sumx, out_tgt);
}
