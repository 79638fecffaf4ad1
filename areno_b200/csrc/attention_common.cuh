// Fragment-level helpers shared by the attention kernels: swizzled shared-memory tiles filled
// by cp.async, ldmatrix fragment loads and the bf16 m16n8k16 MMA.
#pragma once
#include "common.cuh"

namespace areno {

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Tile of ROWS x D bf16, rows of D/8 16-byte chunks, chunk index XOR-swizzled with (row & 7).
template <int CH>
__device__ __forceinline__ int swz(int row, int chunk) {
  return (row * CH + (chunk ^ (row & 7))) * 8;
}

// Cooperative async load by `NT` threads; rows >= valid_rows are zero-filled.
template <int D, int ROWS, int NT = 128>
__device__ __forceinline__ void load_tile_async(__nv_bfloat16* dst, const __nv_bfloat16* src, long long stride,
                                                int valid_rows) {
  constexpr int CH = D / 8;
#pragma unroll
  for (int i = 0; i < ROWS * CH / NT; ++i) {
    const int idx = threadIdx.x + i * NT;
    const int row = idx / CH, ch = idx % CH;
    __nv_bfloat16* d = dst + swz<CH>(row, ch);
    if (row < valid_rows) cp_async16(d, src + (long long)row * stride + ch * 8);
    else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
  }
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}

// A fragment (16 rows x 16 k) of a row-major [row][k] tile: rows row0..row0+15, chunks chunk0, chunk0+1.
template <int CH>
__device__ __forceinline__ void ldsm_a(uint32_t (&r)[4], const __nv_bfloat16* tile, int row0, int chunk0, int lane) {
  const int row = row0 + (lane & 15);
  const int ch = chunk0 + (lane >> 4);
  ldsm_x4(r, tile + swz<CH>(row, ch));
}
// B fragments for two adjacent n-tiles from a [n][k] row-major tile (K for Q.K^T):
// r[0], r[1] = (b0, b1) of n-tile n0..n0+7;  r[2], r[3] = n-tile n0+8..n0+15.
template <int CH>
__device__ __forceinline__ void ldsm_b_nt(uint32_t (&r)[4], const __nv_bfloat16* tile, int n0, int chunk0, int lane) {
  const int row = n0 + (lane & 7) + ((lane >> 4) << 3);
  const int ch = chunk0 + ((lane >> 3) & 1);
  ldsm_x4(r, tile + swz<CH>(row, ch));
}
// B fragments for two adjacent n-tiles from a [k][n] row-major tile (V for P.V), transposed load:
// r[0], r[1] = (b0, b1) of n-chunk chunk0;  r[2], r[3] = n-chunk chunk0+1.  k rows k0..k0+15.
template <int CH>
__device__ __forceinline__ void ldsm_b_t(uint32_t (&r)[4], const __nv_bfloat16* tile, int k0, int chunk0, int lane) {
  const int row = k0 + (lane & 7) + (((lane >> 3) & 1) << 3);
  const int ch = chunk0 + (lane >> 4);
  ldsm_x4_t(r, tile + swz<CH>(row, ch));
}
// A fragment (16 m x 16 k) from a [k][m] row-major tile (transposed load): m rows m0.., k rows k0..
// Used when the contraction index is the tile's row index (e.g. dS^T, P^T products).
template <int CH>
__device__ __forceinline__ void ldsm_a_t(uint32_t (&r)[4], const __nv_bfloat16* tile, int k0, int mchunk0, int lane) {
  // matrices: m0 = (m lo, k lo), m1 = (m hi, k lo), m2 = (m lo, k hi), m3 = (m hi, k hi);
  // stored as [k][m]: 8x8 block rows = k, cols = m; .trans yields (m, k) fragments.
  const int row = k0 + (lane & 7) + ((lane >> 4) << 3);
  const int ch = mchunk0 + ((lane >> 3) & 1);
  ldsm_x4_t(r, tile + swz<CH>(row, ch));
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Same tile shape with fp16 operands (used where an operand was expanded from fp8: e4m3 converts to fp16 exactly).
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Two e4m3 values (low 16 bits of `v`) to two fp16 values.
__device__ __forceinline__ uint32_t cvt_e4m3x2_f16x2(uint32_t v) {
  uint32_t r;
  asm("{\n\t.reg .b16 lo;\n\tcvt.u16.u32 lo, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\t}" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Largest s with prefix[s] <= tile, or -1 if tile >= prefix[num_seqs].
__device__ __forceinline__ int find_seq(const int* prefix, int num_seqs, int tile) {
  if (tile >= prefix[num_seqs]) return -1;
  int lo = 0, hi = num_seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (prefix[mid] <= tile) lo = mid; else hi = mid - 1;
  }
  return lo;
}

}  // namespace areno
