// Tensor-parallel and data-parallel communication over peer memory (NVLink / NVSwitch); no NCCL on
// these paths.
//
// Tensor parallel: fused all-reduce + residual add + RMSNorm after a row-parallel GEMM
// -------------------------------------------------------------------------------------
// Every rank of a TP group owns one region of the symmetric heap (symm_heap.cu) with the same
// layout, mapped by every peer and, when the fabric supports it, bound to an NVLink multicast object:
//
//   flags   : uint32 [64]                      [0] call counter, [1] finished-CTA counter,
//                                              [8 + r] "partial ready" of rank r, [16 + r] "rows published" of rank r,
//                                              [24 + r] row count of rank r's current call (cross-checked)
//   partial : bf16 [2 slots][max_rows][H]      written locally by the row-parallel GEMM of this rank
//   h_out   : bf16 [2 slots][max_rows][H]      new residual stream, written by the owner of each row
//   y_out   : bf16 [2 slots][max_rows][H]      normalised rows, written by the owner of each row
//
// The o_proj / down_proj GEMM stores its partial product into `partial` of its own rank (ordinary
// local stores).  tp_reduce_norm_kernel then does a two-shot all-reduce with the residual add and
// the RMSNorm of the next block folded in:
//   1. tell every peer "my partial is complete" and wait for theirs (flag per source rank);
//   2. the rank that owns a row (rows are dealt out in contiguous blocks) sums the row over all ranks:
//      one multimem.ld_reduce per 16 bytes (the switch adds, fp32 accumulation) or, without
//      multicast, tp plain peer loads summed in rank order; adds the residual, rounds the new stream
//      to bf16, normalises;
//   3. it publishes both rows to EVERY rank: multimem.st, or one plain store per peer;
//   4. the last CTA to finish tells every peer "my rows are published" and waits for theirs, so that
//      when the kernel completes the local h_out / y_out hold all rows.
// Each element crosses NVLink once in each direction per rank (reduce-scatter + all-gather), every
// row is normalised once, and all ranks see bit-identical results.
//
// One-shot variant (the default wherever it moves no more bytes, and for every decode-sized call): after step 1
// every rank reduces ALL rows for itself and keeps the results locally; there is nothing to publish and no second
// flag exchange.  With multimem the switch hands each rank the finished sums (rows x H bf16 inbound whatever the
// group size); with plain loads a rank reads tp - 1 remote partials, which is the cheaper choice for two ranks
// and for a few hundred rows, where the call is bound by the flag round trip and not by bytes.  This replaces GEMM + NCCL
// all-reduce + residual RMSNorm of the reference (areno/engine/parallel/collectives.py:143-155,
// areno/engine/layers/linear.py:235-244).
//
// Slot discipline: consecutive calls alternate slots.  A rank writes slot s of a peer (call n + 2)
// only after that peer has sent its "partial ready" of call n + 2, which it does after all of its own
// kernels that read slot s of call n have completed.
//
// Every wait is bounded by wall time (wait_ns, measured with %globaltimer).  A CTA whose wait runs out (status
// code 7 or 9), or that finds a peer running the same call with another row count (code 10: the ranks' control
// flow has diverged), records {code, block, peer, call} in the status words, publishes nothing, and the kernel still
// counts itself finished, so a lost peer becomes a reported error and never a hung GPU or a sum of
// half-written data.  Nothing here uses a TMA load, and nothing uses cluster multicast.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "launch.h"

namespace areno {

constexpr int kMaxTp = 8;
constexpr int kFlagWords = 64;
constexpr int kFlagCall = 0, kFlagDone = 1, kFlagReady = 8, kFlagPublished = 16, kFlagRows = 24;

struct TpCtx {
  int tp, rank;
  uint32_t* flags[kMaxTp];            // flags[r]: rank r's flag block as mapped here ([rank] is local)
  const __nv_bfloat16* part[kMaxTp];  // partial buffers (slot 0) of every rank as mapped here
  __nv_bfloat16* h_out[kMaxTp];       // h_out buffers (slot 0) of every rank as mapped here
  __nv_bfloat16* y_out[kMaxTp];       // y_out buffers (slot 0) of every rank as mapped here
  const __nv_bfloat16* part_mc;       // multicast addresses of the same three buffers, or null
  __nv_bfloat16* h_mc;
  __nv_bfloat16* y_mc;
  int* status;                        // local int [4]: {code, block, peer, call}
  unsigned long long wait_ns;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Poll `flag` until it reaches `want` (wrap-safe) or `wait_ns` of wall time have passed.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want, unsigned long long wait_ns) {
  if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
  const unsigned long long t0 = globaltimer();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
      __nanosleep(20);
    }
    if (globaltimer() - t0 > wait_ns) return false;
  }
}

__device__ __forceinline__ void report_peer_timeout(int* status, int code, int peer, uint32_t call) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = (int)blockIdx.x;
    status[2] = peer;
    status[3] = (int)call;
  }
}

// Sum over all ranks of 8 bf16 at the multicast address (added in the switch, fp32 accumulation).
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const __nv_bfloat16* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
// Store 8 bf16 to the same offset of every rank's buffer.
__device__ __forceinline__ void multimem_st_bf16x8(__nv_bfloat16* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = __uint_as_float(u[j] << 16);
    f[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  return o;
}
__device__ __forceinline__ void load8_cg(const __nv_bfloat16* p, float (&f)[8]) {
  unpack8(__ldcg(reinterpret_cast<const uint4*>(p)), f);
}

// One call of the fused reduce.  `slot_off`: element offset of the slot inside the three buffers.
// Rows [row_lo, row_hi) belong to this rank; one CTA per row, grid-stride.  residual: local bf16
// [rows, H] or null; w: norm scale (bf16 or fp32) or null; want_y = 0 skips the norm (h only).
// ONESHOT: every rank reduces ALL rows itself (one flag exchange, nothing to publish, results written locally);
// otherwise the two-shot scheme above (each rank reduces the rows it owns and publishes them to the group).
template <int THREADS, int VPT, bool MC, bool ONESHOT>
__global__ void __launch_bounds__(THREADS)
tp_reduce_norm_kernel(TpCtx c, long long slot_off, const __nv_bfloat16* __restrict__ residual,
                      const void* __restrict__ w, int wf32, float w_offset, int want_y, int rows, int row_lo,
                      int row_hi, int H, float eps) {
  __shared__ float red[32];
  __shared__ int sh_ok;
  __shared__ int sh_last;
  pdl_wait();  // the GEMM that produced this rank's partial (and everything before it) has completed
  uint32_t* my_flags = c.flags[c.rank];
  // advanced by the last CTA of this kernel (below), which finishes only after every CTA has read it here
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(my_flags + kFlagCall) + 1u;
  pdl_trigger();  // the next kernel of the stream may set itself up; it waits for this one before touching memory
  if (threadIdx.x == 0) sh_ok = 1;
  __syncthreads();
  // ---- 1. partial ready: announce (first CTA) and wait for every peer (every CTA)
  if (threadIdx.x < c.tp && (int)threadIdx.x != c.rank) {
    const int p = threadIdx.x;
    if (blockIdx.x == 0) {
      // the row count travels with the announcement: ranks whose control flow has diverged (different shapes for
      // the same call) are caught here instead of reducing unrelated buffers
      *reinterpret_cast<volatile uint32_t*>(c.flags[p] + kFlagRows + c.rank) = (uint32_t)rows;
      st_release_sys(c.flags[p] + kFlagReady + c.rank, call);
    }
    if (!wait_flag(my_flags + kFlagReady + p, call, c.wait_ns)) {
      report_peer_timeout(c.status, 7, p, call);  // 7: a peer's partial never became ready
      sh_ok = 0;
    } else if (ld_acquire_sys(my_flags + kFlagReady + p) == call &&
               *reinterpret_cast<volatile uint32_t*>(my_flags + kFlagRows + p) != (uint32_t)rows) {
      report_peer_timeout(c.status, 10, p, call);  // 10: the peer is running this call with another row count
      sh_ok = 0;
    }
  }
  __syncthreads();
  const bool ok = sh_ok != 0;
  // ---- 2 + 3. reduce my rows, add the residual, normalise, publish to every rank
  const int nvec = H >> 3;
  if (ok) {
    const int r_first = ONESHOT ? 0 : row_lo, r_end = ONESHOT ? rows : row_hi;
    for (int row = r_first + blockIdx.x; row < r_end; row += gridDim.x) {
      const size_t base = (size_t)row * H;
      float v[VPT][8];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = threadIdx.x + i * THREADS;
        if (vi < nvec) {
          const size_t off = (size_t)slot_off + base + (size_t)vi * 8;
          if constexpr (MC) {
            unpack8(multimem_ld_reduce_bf16x8(c.part_mc + off), v[i]);
          } else {
            uint4 raw[kMaxTp];
#pragma unroll
            for (int r = 0; r < kMaxTp; ++r)
              if (r < c.tp) raw[r] = __ldcg(reinterpret_cast<const uint4*>(c.part[r] + off));
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
#pragma unroll
            for (int r = 0; r < kMaxTp; ++r)   // rank order: the same sum whoever owns the row
              if (r < c.tp) {
                float t[8];
                unpack8(raw[r], t);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i][j] += t[j];
              }
          }
          if (residual != nullptr) {
            float t[8];
            load8_cg(residual + base + (size_t)vi * 8, t);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] += t[j];
          }
          // the stream is kept in bf16: norm statistics are taken on the rounded values
          const uint4 hv = pack8(v[i]);
          unpack8(hv, v[i]);
          if constexpr (ONESHOT) {
            *reinterpret_cast<uint4*>(c.h_out[c.rank] + off) = hv;
          } else if constexpr (MC) {
            multimem_st_bf16x8(c.h_mc + off, hv);
          } else {
#pragma unroll
            for (int r = 0; r < kMaxTp; ++r)
              if (r < c.tp) *reinterpret_cast<uint4*>(c.h_out[r] + off) = hv;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
        }
      }
      if (want_y) {
        ss = warp_sum(ss);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int k = 0; k < THREADS / 32; ++k) tot += red[k];
        const float inv = rsqrtf(tot / (float)H + eps);
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
            const uint4 yv = pack8(o);
            const size_t off = (size_t)slot_off + base + (size_t)vi * 8;
            if constexpr (ONESHOT) {
              *reinterpret_cast<uint4*>(c.y_out[c.rank] + off) = yv;
            } else if constexpr (MC) {
              multimem_st_bf16x8(c.y_mc + off, yv);
            } else {
#pragma unroll
              for (int r = 0; r < kMaxTp; ++r)
                if (r < c.tp) *reinterpret_cast<uint4*>(c.y_out[r] + off) = yv;
            }
          }
        }
      }
    }
  }
  // ---- 4. rows published: the last CTA of this rank tells the peers and waits for theirs
  __syncthreads();
  if (threadIdx.x == 0) {
    if constexpr (!ONESHOT) __threadfence_system();   // this CTA's stores (ordered by the barrier above) before the count
    sh_last = atomicAdd(my_flags + kFlagDone, 1u) == gridDim.x - 1 ? 1 : 0;
  }
  __syncthreads();
  if (!sh_last) return;
  if constexpr (ONESHOT) {
    // nothing was published: the peers only ever read this rank's partial, and they are held off its reuse by the
    // announcement of the next call.  Advance the call counter and leave.
    if (threadIdx.x == 0) {
      my_flags[kFlagDone] = 0;
      my_flags[kFlagCall] = call;
      __threadfence();
    }
    return;
  }
  __threadfence_system();     // the other CTAs' stores are ordered before their counts, which we have seen
  if (threadIdx.x < c.tp && (int)threadIdx.x != c.rank) {
    const int p = threadIdx.x;
    st_release_sys(c.flags[p] + kFlagPublished + c.rank, call);
    // peers that never announced their partial are not waited for a second time
    if (ok && !wait_flag(my_flags + kFlagPublished + p, call, c.wait_ns))
      report_peer_timeout(c.status, 9, p, call);  // 9: a peer never published its rows
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    my_flags[kFlagDone] = 0;
    my_flags[kFlagCall] = call;
    __threadfence();
  }
}

// Rendezvous of the group without data (tests, and teardown ordering): same two flag exchanges.
__global__ void tp_barrier_kernel(TpCtx c) {
  pdl_wait();
  uint32_t* my_flags = c.flags[c.rank];
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(my_flags + kFlagCall) + 1u;
  if (threadIdx.x < c.tp && (int)threadIdx.x != c.rank) {
    const int p = threadIdx.x;
    st_release_sys(c.flags[p] + kFlagReady + c.rank, call);
    if (!wait_flag(my_flags + kFlagReady + p, call, c.wait_ns)) report_peer_timeout(c.status, 7, p, call);
    st_release_sys(c.flags[p] + kFlagPublished + c.rank, call);
  }
  __syncthreads();
  if (threadIdx.x == 0) my_flags[kFlagCall] = call;
}

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
                           unsigned long long wait_ns) {
  __shared__ int sh_ok;
  if (threadIdx.x == 0) sh_ok = 1;
  __syncthreads();
  if (threadIdx.x < c.n) {
    const uint32_t* mine = c.ready[c.rank] + bucket * kMaxTp + threadIdx.x;
    if (!wait_flag(mine, epoch, wait_ns)) {
      if (atomicCAS(c.status, 0, 8) == 0) {  // 8: a peer's gradients never became ready
        c.status[1] = bucket;
        c.status[2] = threadIdx.x;
        c.status[3] = (int)epoch;
      }
      sh_ok = 0;
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

// ------------------------------- legacy symmetric memory (cudaMalloc + CUDA IPC) -----------------
// Used for the gradient buckets (which the caching allocator cannot export) and as the fallback when
// virtual-memory allocations cannot be shared on this machine.
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

// ------------------------------- tensor-parallel fused reduce -------------------------------------
extern "C" long long areno_tp_flags_bytes() { return (long long)kFlagWords * 4; }

// Host description of a TP communicator: arrays of tp pointers in rank order, as mapped on this rank.
struct ArenoTpDesc {
  int tp, rank;
  void* const* flags;
  void* const* part;
  void* const* h_out;
  void* const* y_out;
  void* part_mc;   // multicast addresses or null (all three or none)
  void* h_mc;
  void* y_mc;
  int* status;
  int wait_ms;
};

static int fill_ctx(TpCtx* c, const ArenoTpDesc* d) {
  if (d == nullptr || d->tp < 1 || d->tp > kMaxTp || d->rank < 0 || d->rank >= d->tp) return -3;
  c->tp = d->tp;
  c->rank = d->rank;
  for (int i = 0; i < kMaxTp; ++i) {
    c->flags[i] = i < d->tp ? reinterpret_cast<uint32_t*>(d->flags[i]) : nullptr;
    c->part[i] = i < d->tp && d->part != nullptr ? reinterpret_cast<const __nv_bfloat16*>(d->part[i]) : nullptr;
    c->h_out[i] = i < d->tp && d->h_out != nullptr ? reinterpret_cast<__nv_bfloat16*>(d->h_out[i]) : nullptr;
    c->y_out[i] = i < d->tp && d->y_out != nullptr ? reinterpret_cast<__nv_bfloat16*>(d->y_out[i]) : nullptr;
    if (i < d->tp && c->flags[i] == nullptr) return -3;
  }
  c->part_mc = reinterpret_cast<const __nv_bfloat16*>(d->part_mc);
  c->h_mc = reinterpret_cast<__nv_bfloat16*>(d->h_mc);
  c->y_mc = reinterpret_cast<__nv_bfloat16*>(d->y_mc);
  c->status = d->status;
  int ms = d->wait_ms;
  if (ms < 1) ms = 1;
  if (ms > 20000) ms = 20000;
  c->wait_ns = (unsigned long long)ms * 1000000ull;
  return 0;
}

// Rows of an M-row problem owned by `rank`: contiguous blocks of ceil(M / tp) rows.
static void owned_rows(int M, int tp, int rank, int* lo, int* hi) {
  const int per = (M + tp - 1) / tp;
  *lo = rank * per < M ? rank * per : M;
  *hi = (rank + 1) * per < M ? (rank + 1) * per : M;
}

// Fused all-reduce + residual add + RMSNorm over the group (see the top of this file).  The partial
// of every rank must already be in slot `slot_off` of its `partial` buffer (stream order on each
// rank).  After the kernel, h_out / y_out of this rank hold all `rows` rows at the same offset.
// use_mc: 1 = multimem instructions (needs the multicast addresses), 0 = plain peer loads / stores.
// oneshot: 1 = every rank reduces all rows for itself (one flag exchange; the choice for decode-sized calls and,
// with multimem, for any size: the switch hands each rank the finished sums), 0 = the two-shot scheme.
extern "C" int areno_tp_reduce_norm(const ArenoTpDesc* desc, long long slot_off, const void* residual, const void* w,
                                    int wf32, float w_offset, int want_y, long long rows, int H, float eps,
                                    int use_mc, int oneshot, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H % 8 != 0 || (slot_off & 7) != 0) return -3;
  TpCtx c;
  const int rc = fill_ctx(&c, desc);
  if (rc != 0) return rc;
  if (use_mc && (c.part_mc == nullptr || (!oneshot && (c.h_mc == nullptr || c.y_mc == nullptr)))) return -3;
  if (!use_mc)
    for (int i = 0; i < c.tp; ++i)
      if (c.part[i] == nullptr || c.h_out[i] == nullptr || c.y_out[i] == nullptr) return -3;
  int lo, hi;
  owned_rows((int)rows, c.tp, c.rank, &lo, &hi);
  int grid = oneshot ? (int)rows : hi - lo;
  if (grid > 148 * 4) grid = 148 * 4;
  if (grid < 1) grid = 1;   // a rank without rows still takes part in both flag exchanges
  const int nvec = H >> 3;
  cudaError_t e;
#define TP_ARGS c, slot_off, (const __nv_bfloat16*)residual, w, wf32, w_offset, want_y, (int)rows, lo, hi, H, eps
#define TP_LAUNCH(T, V)                                                                                          \
  do {                                                                                                           \
    if (oneshot)                                                                                                 \
      e = use_mc ? launch_pdl(tp_reduce_norm_kernel<T, V, true, true>, dim3(grid), dim3(T), 0, stream, TP_ARGS)   \
                 : launch_pdl(tp_reduce_norm_kernel<T, V, false, true>, dim3(grid), dim3(T), 0, stream, TP_ARGS); \
    else                                                                                                         \
      e = use_mc ? launch_pdl(tp_reduce_norm_kernel<T, V, true, false>, dim3(grid), dim3(T), 0, stream, TP_ARGS)  \
                 : launch_pdl(tp_reduce_norm_kernel<T, V, false, false>, dim3(grid), dim3(T), 0, stream, TP_ARGS);\
  } while (0)
  if (nvec <= 128) TP_LAUNCH(128, 1);
  else if (nvec <= 256) TP_LAUNCH(256, 1);
  else if (nvec <= 512) TP_LAUNCH(512, 1);
  else if (nvec <= 1024) TP_LAUNCH(512, 2);
  else if (nvec <= 2048) TP_LAUNCH(512, 4);
  else return -2;
#undef TP_ARGS
#undef TP_LAUNCH
  return (int)e;
}

extern "C" int areno_tp_barrier(const ArenoTpDesc* desc, cudaStream_t stream) {
  TpCtx c;
  const int rc = fill_ctx(&c, desc);
  if (rc != 0) return rc;
  return (int)launch_pdl(tp_barrier_kernel, dim3(1), dim3(32), 0, stream, c);
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
  const unsigned long long spin_limit = (unsigned long long)wait_ms * 1000000ull;  // wall time, nanoseconds
  float* o = reinterpret_cast<float*>(out);
  if (n <= 2) grad_reduce_scatter_kernel<8, 2><<<blocks, 256, 0, stream>>>(c, bucket, (uint32_t)epoch, offset, elems, o, spin_limit);
  else if (n <= 4) grad_reduce_scatter_kernel<4, 4><<<blocks, 256, 0, stream>>>(c, bucket, (uint32_t)epoch, offset, elems, o, spin_limit);
  else grad_reduce_scatter_kernel<2, 8><<<blocks, 256, 0, stream>>>(c, bucket, (uint32_t)epoch, offset, elems, o, spin_limit);
  return (int)cudaGetLastError();
}
