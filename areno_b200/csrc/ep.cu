// Expert-parallel token exchange over peer memory (NVLink / NVSwitch): the all-to-all that moves every
// token to the ranks that own its experts and brings the expert outputs back, written as row gathers
// and scatters over the symmetric heap.  No NCCL, no host read-back, no atomics.
//
// Every rank of the group owns E / n experts and its own tokens.  One MoE layer call:
//
//   publish   each rank copies its tokens into its own `pub` buffer and stores its routing table
//             (expert id per (token, slot)) into EVERY rank's `ids_all[rank]` section        -> barrier
//   align     (moe.cu, local) the routes of all ranks that hit a local expert are sorted by expert and
//             padded to 128-row tiles; row_route[row] is the global route g = rank * cap * k + token * k + slot
//   pull      ep_pull_rows_kernel: row `row` of the expert-sorted activation buffer is loaded from the
//             publishing rank's `pub` buffer with plain peer loads (one warp per row, 16 bytes per lane)
//   experts   grouped tcgen05 GEMMs on the local rows (gemm_tcgen05.cu)
//   push      ep_push_rows_kernel: every output row goes to the `inbox` of the rank that owns the token,
//             at [token * k + slot] (peer stores, one warp per row)                           -> barrier
//   combine   (moe.cu, local) weighted sum of the k rows of every token
//
// Backward runs the same two kernels with the roles swapped (the gradient of a gather is a scatter).
// Only the rows a rank needs cross NVLink, once in each direction, as in an all-to-all; the row counts
// live on the device (the plan), buffers are sized from the static bound cap * k * n routes.
//
// The reference shards experts over TP with replicated tokens and an all-reduce
// (areno/models/qwen3/model.py:99-116); it has no expert-parallel all-to-all.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "launch.h"

namespace areno {

constexpr int kEpMax = 8;

struct EpBases {
  int n;
  char* base[kEpMax];   // the same buffer of every rank, as mapped on this rank
};

// Routing table of this rank to every rank: dst[r][my_rank * cap_routes + i] = ids[i] (i < routes), -1 beyond.
__global__ void __launch_bounds__(256)
ep_publish_ids_kernel(EpBases out, int my_rank, const int* __restrict__ ids, int routes, int cap_routes) {
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < cap_routes; i += gridDim.x * blockDim.x) {
    const int v = i < routes ? ids[i] : -1;
    for (int r = 0; r < out.n; ++r)
      reinterpret_cast<int*>(out.base[r])[(size_t)my_rank * cap_routes + i] = v;
  }
}

// dst[row, :] = src[s][index, :] with g = row_route[row], s = g / cap_routes, l = g % cap_routes and
// index = l / k (per_token: the source holds one row per token) or l (one row per route).
// Rows without a route (g < 0, tile padding) are zero-filled.
__global__ void __launch_bounds__(256)
ep_pull_rows_kernel(EpBases src, const int* __restrict__ row_route, int cap_routes, int k, int per_token,
                    __nv_bfloat16* __restrict__ dst, int max_rows, int H) {
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int nvec = H >> 3;
  for (int row = warp; row < max_rows; row += nwarps) {
    const int g = row_route[row];
    uint4* d = reinterpret_cast<uint4*>(dst + (size_t)row * H);
    if (g < 0) {
      for (int v = lane; v < nvec; v += 32) d[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int s = g / cap_routes, l = g - s * cap_routes;
    const size_t index = per_token ? (size_t)(l / k) : (size_t)l;
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src.base[s]) + index * H);
    for (int v0 = lane; v0 < nvec; v0 += 128) {   // four loads in flight per lane: NVLink latency is microseconds
      uint4 t[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + u * 32 < nvec) t[u] = __ldcg(p + v0 + u * 32);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + u * 32 < nvec) d[v0 + u * 32] = t[u];
    }
  }
}

// dst[s][l, :] = src[row, :] for every row with a route g = row_route[row] (s = g / cap_routes, l = g % cap_routes).
__global__ void __launch_bounds__(256)
ep_push_rows_kernel(EpBases dst, const int* __restrict__ row_route, int cap_routes,
                    const __nv_bfloat16* __restrict__ src, int max_rows, int H) {
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int nvec = H >> 3;
  for (int row = warp; row < max_rows; row += nwarps) {
    const int g = row_route[row];
    if (g < 0) continue;
    const int s = g / cap_routes, l = g - s * cap_routes;
    const uint4* p = reinterpret_cast<const uint4*>(src + (size_t)row * H);
    uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.base[s]) + (size_t)l * H);
    for (int v = lane; v < nvec; v += 32) d[v] = __ldcg(p + v);
  }
}

}  // namespace areno

using namespace areno;

static int fill_bases(EpBases* b, int n, void* const* ptrs) {
  if (n < 1 || n > kEpMax || ptrs == nullptr) return -3;
  b->n = n;
  for (int i = 0; i < kEpMax; ++i) {
    b->base[i] = i < n ? reinterpret_cast<char*>(ptrs[i]) : nullptr;
    if (i < n && b->base[i] == nullptr) return -3;
  }
  return 0;
}

static int row_grid(long long rows) {
  long long blocks = (rows + 7) / 8;      // eight warps (rows) per block
  if (blocks > 148 * 8) blocks = 148 * 8;
  return blocks < 1 ? 1 : (int)blocks;
}

// ids_all_ptrs: the `ids_all` buffer (int32 [n][cap_routes]) of every rank as mapped here.
extern "C" int areno_ep_publish_ids(int n, int rank, void* const* ids_all_ptrs, const int* ids, long long routes,
                                    long long cap_routes, cudaStream_t stream) {
  EpBases b;
  const int rc = fill_bases(&b, n, ids_all_ptrs);
  if (rc != 0) return rc;
  if (rank < 0 || rank >= n || routes < 0 || routes > cap_routes || cap_routes < 1) return -3;
  int grid = (int)((cap_routes + 255) / 256);
  if (grid > 148 * 4) grid = 148 * 4;
  return (int)launch_pdl(ep_publish_ids_kernel, dim3(grid), dim3(256), 0, stream, b, rank, ids, (int)routes,
                         (int)cap_routes);
}

// src_ptrs: the published buffer (bf16 rows of H) of every rank as mapped here.
extern "C" int areno_ep_pull_rows(int n, void* const* src_ptrs, const int* row_route, long long cap_routes, int k,
                                  int per_token, void* dst, long long max_rows, int H, cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  EpBases b;
  const int rc = fill_bases(&b, n, src_ptrs);
  if (rc != 0) return rc;
  if (H % 8 != 0 || k < 1 || cap_routes < 1 || (reinterpret_cast<uintptr_t>(dst) & 15)) return -3;
  return (int)launch_pdl(ep_pull_rows_kernel, dim3(row_grid(max_rows)), dim3(256), 0, stream, b, row_route,
                         (int)cap_routes, k, per_token, reinterpret_cast<__nv_bfloat16*>(dst), (int)max_rows, H);
}

// dst_ptrs: the inbox (bf16 [cap_routes, H]) of every rank as mapped here.
extern "C" int areno_ep_push_rows(int n, void* const* dst_ptrs, const int* row_route, long long cap_routes,
                                  const void* src, long long max_rows, int H, cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  EpBases b;
  const int rc = fill_bases(&b, n, dst_ptrs);
  if (rc != 0) return rc;
  if (H % 8 != 0 || cap_routes < 1 || (reinterpret_cast<uintptr_t>(src) & 15)) return -3;
  return (int)launch_pdl(ep_push_rows_kernel, dim3(row_grid(max_rows)), dim3(256), 0, stream, b, row_route,
                         (int)cap_routes, reinterpret_cast<const __nv_bfloat16*>(src), (int)max_rows, H);
}
