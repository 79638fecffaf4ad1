// C ABI of the sm_100a kernel library (libareno_kernels.so).  Every entry point takes raw
// device pointers and a CUDA stream, launches asynchronously and returns 0 or an error code
// (negative: argument / configuration error, positive: CUDA error).  The compute entry points
// allocate no device memory: scratch is passed in by the caller, except for the one variant in
// no_alloc.h that keeps its scratch in a fixed device array of the library.  The only allocating
// calls are the symmetric-memory set-up routines of comm.cu (areno_symm_* / areno_vmm_*), which
// run once at start-up.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace areno {
// Host helper: 2-D bf16 tensor map with 128-byte swizzle (inner box must be 64 elements).
int make_tensor_map_2d_bf16(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer,
                            uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);
}  // namespace areno

extern "C" {

// ---- GEMM (gemm_tcgen05.cu) ----
// D[M,N] = sum_k A(m,k) B(n,k).  a_mn / b_mn: operand stored [K, rows] instead of [rows, K].
// epi: 0 = bf16 store, 1 = bf16 store + bf16 bias[N], 2 = fp32 store, 3 = fp32 accumulate (C += D).
// bn: N-tile (256/128/64/32) or 0 for the built-in heuristic.  status: int[4] device words or NULL.
// workspace: optional fp32 scratch enabling split-K for skinny (M <= 128) problems; see
// areno_gemm_workspace_bytes.  Split partials are summed in a fixed order (deterministic).
int areno_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                    long long ldb, long long ldc, int a_mn, int b_mn, int epi, int bn, void* workspace,
                    long long workspace_bytes, int* status, cudaStream_t stream);
long long areno_gemm_workspace_bytes(int M, int N, int K);

// ---- elementwise.cu ----
int areno_rmsnorm_fwd(const void* x, const void* residual, const void* w, int wf32, float w_offset, void* y,
                      void* h_out, float* inv_rms, long long rows, int H, float eps, cudaStream_t stream);
int areno_rmsnorm_bwd_blocks(long long rows);
int areno_rmsnorm_bwd(const void* dy, const void* h, const void* w, int wf32, float w_offset, const float* inv_rms,
                      const void* dres_in, void* dx, float* dw_partial, float* dw, int dw_accumulate, long long rows,
                      int H, cudaStream_t stream);
int areno_gated_act_fwd(const void* x, void* out, long long rows, int I, int kind, cudaStream_t stream);
int areno_gated_act_bwd(const void* dout, const void* x, void* dx, long long rows, int I, int kind,
                        cudaStream_t stream);
int areno_unary_act(const void* x, const void* dy, void* y, long long n, int kind, int mode, cudaStream_t stream);
int areno_rope(void* x, const int* positions, const float* inv_freq, long long tokens, int heads, int head_dim,
               int rot_dim, long long row_stride, float theta, float sign, int interleaved, cudaStream_t stream);
int areno_embedding_fwd(const long long* ids, const void* table, void* out, long long tokens, int H, long long v0,
                        long long v1, float scale, cudaStream_t stream);
int areno_embedding_bwd(const long long* ids, const void* dout, float* dtable, long long tokens, int H, long long v0,
                        long long v1, float scale, cudaStream_t stream);
int areno_accumulate_bf16(float* acc, const void* g, long long n, cudaStream_t stream);

// ---- attention_fwd.cu / attention_bwd.cu ----
int areno_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_q,
                   const int* cu_k, const int* tile_prefix, int num_seqs, int total_tiles, int hq, int hkv,
                   int head_dim, long long q_stride, long long k_stride, long long v_stride, long long o_stride,
                   float scale, int causal, int window, cudaStream_t stream);
int areno_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                   float* delta, void* dq, void* dk, void* dv, const int* cu_q, const int* cu_k,
                   const int* tile_prefix_q, const int* tile_prefix_k, int num_seqs, int total_q_tiles,
                   int total_k_tiles, long long total_q, int hq, int hkv, int head_dim, long long q_stride,
                   long long k_stride, long long v_stride, long long o_stride, long long do_stride,
                   long long dq_stride, long long dk_stride, long long dv_stride, float scale, int causal,
                   int window, float* dkv_ws, long long total_k, cudaStream_t stream);
}
