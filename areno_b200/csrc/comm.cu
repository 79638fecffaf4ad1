// Tensor-parallel communication over peer memory (NVLink / NVSwitch), no NCCL on this path.
//
// Each rank owns one "symmetric" region (plain cudaMalloc, exported with CUDA IPC and mapped by
// every peer of its TP group):
//
//   flags  : uint32 [kMaxBlocks][8]      one row per thread block, one column per source rank
//   inbox  : bf16   [2 slots][tp][rows_cap][H]
//
// A row-parallel GEMM (o_proj, down_proj) writes its partial product straight into slot s, lane
// `my_rank`, of EVERY rank's inbox from its epilogue (areno_gemm_bf16_push in gemm_tcgen05.cu: the
// NVLink stores of one tile overlap the tensor-core work of the next).  The consumer kernel below
// then (1) tells its peers "my partial has landed" and waits for theirs through the flag rows, and
// (2) sums the tp lanes of its LOCAL inbox in rank order, adds the residual stream, and applies
// the RMSNorm that follows in the model - all-reduce, residual add and norm in one pass over HBM,
// with every rank computing bit-identical results.
//
// Slot discipline: consecutive calls alternate slots.  A rank may overwrite slot s (call n+2) only
// after all peers finished reading it (call n); they have, because this rank passed the barrier of
// call n+1, which a peer joins only after its kernel of call n has completed.
//
// Every wait is bounded: on expiry the block records a status word and carries on with whatever is
// in the inbox, so a lost peer produces a reported error, never a hung GPU.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "launch.h"

namespace areno {

constexpr int kMaxTp = 8;
constexpr int kMaxBlocks = 1024;
constexpr unsigned kSpinLimit = 1u << 22;  // x ~50 ns backoff: a fraction of a second

struct TpPeers {
  int tp, rank;
  uint32_t* flags[kMaxTp];  // flags[p] = base of rank p's flag array (peer-mapped for p != rank)
  uint32_t* epoch;          // local uint32 [kMaxBlocks]
  int* status;              // local int [4]: {code, block, peer, epoch}
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Cross-rank rendezvous of block `blockIdx.x` on every rank.  Returns false if a peer never showed up.
__device__ __forceinline__ bool tp_block_barrier(const TpPeers& c) {
  __shared__ uint32_t sh_epoch;
  __shared__ int sh_ok;
  if (threadIdx.x == 0) {
    const uint32_t e = c.epoch[blockIdx.x] + 1u;
    c.epoch[blockIdx.x] = e;
    sh_epoch = e;
    sh_ok = 1;
  }
  __syncthreads();
  const uint32_t e = sh_epoch;
  const int p = threadIdx.x;
  if (p < c.tp && p != c.rank) {
    __threadfence_system();
    st_release_sys(c.flags[p] + blockIdx.x * kMaxTp + c.rank, e);
    const uint32_t* mine = c.flags[c.rank] + blockIdx.x * kMaxTp + p;
    unsigned spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - e) < 0) {
      if (++spins > kSpinLimit) {
        if (atomicCAS(c.status, 0, 7) == 0) {  // 7: peer wait timed out
          c.status[1] = blockIdx.x;
          c.status[2] = p;
          c.status[3] = (int)e;
        }
        sh_ok = 0;
        break;
      }
      __nanosleep(40);
    }
  }
  __syncthreads();
  return sh_ok != 0;
}

__device__ __forceinline__ void load8_cg(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 v = __ldcg(reinterpret_cast<const uint4*>(p));
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = __uint_as_float(u[j] << 16);
    f[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
  }
}
__device__ __forceinline__ void store8_bf16(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

// h = residual + sum_r inbox[r];  y = h * rsqrt(mean h^2 + eps) * (w + w_offset)
// inbox: this rank's slot base, lanes `lane_stride` elements apart.  One block per row (grid-stride).
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
tp_reduce_rmsnorm_kernel(TpPeers c, const __nv_bfloat16* __restrict__ inbox, long long lane_stride,
                         const __nv_bfloat16* __restrict__ residual, const void* __restrict__ w, int wf32,
                         float w_offset, __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out, int rows,
                         int H, float eps) {
  __shared__ float red[32];
  tp_block_barrier(c);
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
          load8_cg(residual + base + vi * 8, v[i]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
        }
        for (int r = 0; r < c.tp; ++r) {
          float t[8];
          load8_cg(inbox + (size_t)r * lane_stride + base + vi * 8, t);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += t[j];
        }
        // the stream is kept in bf16: norm statistics are taken on the rounded values
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j]));
        if (h_out != nullptr) store8_bf16(h_out + base + vi * 8, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    ss = warp_sum(ss);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < THREADS / 32; ++k) tot += red[k];
    const float inv = rsqrtf(tot / (float)H + eps);
    if (y != nullptr) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = threadIdx.x + i * THREADS;
        if (vi < nvec) {
          float o[8];
          if (w != nullptr) {
            float wv[8];
            if (wf32) {
              const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + vi * 8);
              const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + vi * 8 + 4);
              wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w;
              wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
            } else {
              load8_cg(reinterpret_cast<const __nv_bfloat16*>(w) + vi * 8, wv);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = v[i][j] * inv * (wv[j] + w_offset);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = v[i][j] * inv;
          }
          store8_bf16(y + base + vi * 8, o);
        }
      }
    }
  }
}

// Barrier only (used to keep the slot alternation even, and by tests).
__global__ void tp_barrier_kernel(TpPeers c) { tp_block_barrier(c); }

// ----------------------------------------------------------------------------------
// Data-parallel gradient reduce-scatter over peer memory.
//
// Every rank keeps its fp32 gradient buckets in one symmetric region (same layout on every rank).
// When the gradients of bucket b are final on a rank (its last micro-batch's backward has passed
// them), that rank raises ready[b][rank] = epoch on every rank (grad_ready_kernel, on the compute
// stream).  The owner of shard r of bucket b then runs grad_reduce_scatter_kernel on a side stream:
// it waits until all ranks' ready[b] reached the epoch and sums the shard from every rank's
// bucket in rank order (peer loads over NVLink), in place into its own bucket - while the compute
// stream is still producing the gradients of earlier layers.  A cross-rank barrier before the
// buckets are zeroed for the next step keeps a slow reader safe.
// ready: uint32 [kMaxBuckets][8] inside the symmetric region of every rank.
// ----------------------------------------------------------------------------------
constexpr int kMaxBuckets = 4096;

struct DpPeers {
  int n, rank;
  uint32_t* ready[kMaxTp];   // ready[p] = rank p's ready array as mapped here
  const float* grads[kMaxTp];  // grads[p] = rank p's gradient region as mapped here
  int* status;
};

__global__ void grad_ready_kernel(DpPeers c, int bucket, uint32_t epoch) {
  const int p = threadIdx.x;
  if (p < c.n) {
    __threadfence_system();  // gradient stores of earlier kernels of this stream are ordered before the flag
    st_release_sys(c.ready[p] + bucket * kMaxTp + c.rank, epoch);
  }
}

template <int UNROLL, int NP>
__global__ void __launch_bounds__(256)
grad_reduce_scatter_kernel(DpPeers c, int bucket, uint32_t epoch, long long offset, long long elems, float* out,
                           unsigned spin_limit) {
  __shared__ int sh_ok;
  if (threadIdx.x == 0) sh_ok = 1;
  __syncthreads();
  if (threadIdx.x < c.n) {
    const uint32_t* mine = c.ready[c.rank] + bucket * kMaxTp + threadIdx.x;
    unsigned spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if (++spins > spin_limit) {
        if (atomicCAS(c.status, 0, 8) == 0) {  // 8: a peer's gradients never became ready
          c.status[1] = bucket;
          c.status[2] = threadIdx.x;
          c.status[3] = (int)epoch;
        }
        sh_ok = 0;
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  if (!sh_ok) return;  // reported; the host refuses to step on this result
  // NVLink latency is microseconds: every thread keeps UNROLL x n 16-byte loads in flight
  const long long nvec = elems >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * UNROLL) {
    float4 v[UNROLL][NP];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
#pragma unroll
      for (int p = 0; p < NP; ++p)
        if (p < c.n && i < nvec) v[u][p] = __ldcg(reinterpret_cast<const float4*>(c.grads[p] + offset) + i);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) break;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int p = 0; p < NP; ++p)   // rank order: the sum is the same whoever computes it
        if (p < c.n) { acc.x += v[u][p].x; acc.y += v[u][p].y; acc.z += v[u][p].z; acc.w += v[u][p].w; }
      reinterpret_cast<float4*>(out)[i] = acc;
    }
  }
}

}  // namespace areno

using namespace areno;

// ------------------------------- symmetric memory --------------------------------------
extern "C" int areno_symm_alloc(void** out, long long bytes) {
  void* p = nullptr;
  cudaError_t rc = cudaMalloc(&p, (size_t)bytes);
  if (rc != cudaSuccess) return (int)rc;
  rc = cudaMemset(p, 0, (size_t)bytes);
  if (rc != cudaSuccess) return (int)rc;
  *out = p;
  return 0;
}
extern "C" int areno_symm_free(void* p) { return (int)cudaFree(p); }
extern "C" int areno_ipc_export(void* p, unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  const cudaError_t rc = cudaIpcGetMemHandle(&h, p);
  if (rc != cudaSuccess) return (int)rc;
  static_assert(sizeof(h) == 64, "IPC handle size");
  for (int i = 0; i < 64; ++i) handle64[i] = reinterpret_cast<unsigned char*>(&h)[i];
  return 0;
}
extern "C" int areno_ipc_import(const unsigned char* handle64, void** out) {
  cudaIpcMemHandle_t h;
  for (int i = 0; i < 64; ++i) reinterpret_cast<unsigned char*>(&h)[i] = handle64[i];
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int areno_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }
extern "C" int areno_tp_max_blocks() { return kMaxBlocks; }
extern "C" long long areno_tp_flags_bytes() { return (long long)kMaxBlocks * kMaxTp * 4; }

static int fill_peers(TpPeers* c, int tp, int rank, void* const* flag_ptrs, uint32_t* epoch, int* status) {
  if (tp < 1 || tp > kMaxTp || rank < 0 || rank >= tp) return -3;
  c->tp = tp;
  c->rank = rank;
  for (int i = 0; i < kMaxTp; ++i) c->flags[i] = i < tp ? reinterpret_cast<uint32_t*>(flag_ptrs[i]) : nullptr;
  c->epoch = epoch;
  c->status = status;
  return 0;
}

// flag_ptrs: host array of tp pointers (rank order) to every rank's flag array as mapped HERE.
extern "C" int areno_tp_reduce_rmsnorm(int tp, int rank, void* const* flag_ptrs, void* epoch, int* status,
                                       const void* inbox_slot, long long lane_stride, const void* residual,
                                       const void* w, int wf32, float w_offset, void* y, void* h_out, long long rows,
                                       int H, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H % 8 != 0) return -3;
  TpPeers c;
  const int rc = fill_peers(&c, tp, rank, flag_ptrs, reinterpret_cast<uint32_t*>(epoch), status);
  if (rc != 0) return rc;
  const int grid = (int)(rows < kMaxBlocks ? rows : kMaxBlocks);
  const int nvec = H >> 3;
#define TP_LAUNCH(T, V)                                                                                      \
  tp_reduce_rmsnorm_kernel<T, V><<<grid, T, 0, stream>>>(                                                    \
      c, (const __nv_bfloat16*)inbox_slot, lane_stride, (const __nv_bfloat16*)residual, w, wf32, w_offset,   \
      (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, (int)rows, H, eps)
  if (nvec <= 128) TP_LAUNCH(128, 1);
  else if (nvec <= 256) TP_LAUNCH(128, 2);
  else if (nvec <= 512) TP_LAUNCH(256, 2);
  else if (nvec <= 1024) TP_LAUNCH(256, 4);
  else if (nvec <= 2048) TP_LAUNCH(512, 4);
  else return -2;
#undef TP_LAUNCH
  return (int)cudaGetLastError();
}

extern "C" int areno_tp_barrier(int tp, int rank, void* const* flag_ptrs, void* epoch, int* status, int blocks,
                                cudaStream_t stream) {
  TpPeers c;
  const int rc = fill_peers(&c, tp, rank, flag_ptrs, reinterpret_cast<uint32_t*>(epoch), status);
  if (rc != 0) return rc;
  if (blocks < 1 || blocks > kMaxBlocks) return -3;
  tp_barrier_kernel<<<blocks, 32, 0, stream>>>(c);
  return (int)cudaGetLastError();
}

// ------------------------------- DP gradient reduce-scatter ----------------------------
extern "C" int areno_dp_max_buckets() { return kMaxBuckets; }
extern "C" long long areno_dp_ready_bytes() { return (long long)kMaxBuckets * kMaxTp * 4; }

static int fill_dp(DpPeers* c, int n, int rank, void* const* ready_ptrs, void* const* grad_ptrs, int* status) {
  if (n < 1 || n > kMaxTp || rank < 0 || rank >= n) return -3;
  c->n = n;
  c->rank = rank;
  for (int i = 0; i < kMaxTp; ++i) {
    c->ready[i] = i < n ? reinterpret_cast<uint32_t*>(ready_ptrs[i]) : nullptr;
    c->grads[i] = i < n ? reinterpret_cast<const float*>(grad_ptrs[i]) : nullptr;
  }
  c->status = status;
  return 0;
}

// Announce to every rank that this rank's gradients of `bucket` are final for `epoch`.
extern "C" int areno_dp_grad_ready(int n, int rank, void* const* ready_ptrs, void* const* grad_ptrs, int* status,
                                   int bucket, unsigned epoch, cudaStream_t stream) {
  DpPeers c;
  const int rc = fill_dp(&c, n, rank, ready_ptrs, grad_ptrs, status);
  if (rc != 0) return rc;
  if (bucket < 0 || bucket >= kMaxBuckets) return -3;
  // ordinary launch: starts only after every earlier kernel of the stream (the gradient producers) completed
  grad_ready_kernel<<<1, 32, 0, stream>>>(c, bucket, (uint32_t)epoch);
  return (int)cudaGetLastError();
}

// out[i] = sum over ranks of grads[rank][offset + i] for i < elems (fp32, rank order), after every rank
// announced `bucket` for `epoch`.  offset / elems in elements, multiples of 4; out may alias this
// rank's own region at the same offset.  wait_ms bounds the wait for the slowest peer.
extern "C" int areno_dp_grad_reduce_scatter(int n, int rank, void* const* ready_ptrs, void* const* grad_ptrs,
                                            int* status, int bucket, unsigned epoch, long long offset, long long elems,
                                            void* out, int blocks, int wait_ms, cudaStream_t stream) {
  if (elems <= 0) return 0;
  DpPeers c;
  const int rc = fill_dp(&c, n, rank, ready_ptrs, grad_ptrs, status);
  if (rc != 0) return rc;
  if (bucket < 0 || bucket >= kMaxBuckets || (offset & 3) || (elems & 3) || blocks < 1) return -3;
  if (wait_ms < 1) wait_ms = 1;
  if (wait_ms > 20000) wait_ms = 20000;
  const unsigned spin_limit = (unsigned)wait_ms * 4000u;  // ~250 ns per poll (200 ns sleep + the load)
  float* o = reinterpret_cast<float*>(out);
  if (n <= 2) grad_reduce_scatter_kernel<8, 2><<<blocks, 256, 0, stream>>>(c, bucket, (uint32_t)epoch, offset, elems, o, spin_limit);
  else if (n <= 4) grad_reduce_scatter_kernel<4, 4><<<blocks, 256, 0, stream>>>(c, bucket, (uint32_t)epoch, offset, elems, o, spin_limit);
  else grad_reduce_scatter_kernel<2, 8><<<blocks, 256, 0, stream>>>(c, bucket, (uint32_t)epoch, offset, elems, o, spin_limit);
  return (int)cudaGetLastError();
}
