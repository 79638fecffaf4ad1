// Device-side bookkeeping of the decode loop (sm_100a): with these kernels one decode step is
// [prepare -> model -> sample -> commit] with no host read-back, so the whole step can be
// replayed from a CUDA graph.  The host only learns about finished sequences by polling the
// `finish_reason` array asynchronously.  Replaces the per-step Python + D2H bookkeeping of the
// reference (areno/engine/inference.py:406-485,561-580).
#include "common.cuh"
#include "launch.h"

namespace areno {

// slot state layout (all arrays indexed by slot):
//   seq_len    int32  tokens whose K/V are in the cache
//   active     int32  1 while the slot is decoding
//   last_token int64  token to feed at the next step
//   gen_count  int32  tokens generated so far
//   max_new    int32  generation budget
//   finish     int32  0 running, 1 stop token, 2 length, 3 cancelled
__global__ void decode_prepare_kernel(const int* __restrict__ seq_len, const int* __restrict__ active,
                                      const long long* __restrict__ last_token, const int* __restrict__ block_table,
                                      int max_pages, int page_size, int batch, long long* __restrict__ input_ids,
                                      int* __restrict__ positions, int* __restrict__ slot_mapping,
                                      int* __restrict__ attn_seq_lens) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch) return;
  if (active[i]) {
    const int pos = seq_len[i];
    positions[i] = pos;
    const int page = block_table[(long long)i * max_pages + pos / page_size];
    slot_mapping[i] = page * page_size + pos % page_size;
    attn_seq_lens[i] = pos + 1;
    input_ids[i] = last_token[i];
  } else {
    positions[i] = 0;
    slot_mapping[i] = -1;
    attn_seq_lens[i] = 0;
    input_ids[i] = 0;
  }
}

__global__ void decode_commit_kernel(const long long* __restrict__ sampled, const float* __restrict__ logprob,
                                     const signed char* __restrict__ cls, int* __restrict__ seq_len,
                                     int* __restrict__ active, long long* __restrict__ last_token,
                                     int* __restrict__ gen_count, const int* __restrict__ max_new,
                                     int* __restrict__ finish, int* __restrict__ out_tokens,
                                     float* __restrict__ out_logprobs, int out_stride, int batch) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch || !active[i]) return;
  const long long tok = sampled[i];
  const int g = gen_count[i];
  if (g < out_stride) {
    out_tokens[(long long)i * out_stride + g] = (int)tok;
    out_logprobs[(long long)i * out_stride + g] = logprob[i];
  }
  gen_count[i] = g + 1;
  seq_len[i] += 1;
  last_token[i] = tok;
  const signed char c = cls != nullptr ? cls[tok] : 0;
  if (c == 2 || c == 3) {
    finish[i] = 1;
    active[i] = 0;
  } else if (g + 1 >= max_new[i]) {
    finish[i] = 2;
    active[i] = 0;
  }
}

// After a prefill step: install the first sampled token of each newly admitted sequence.
// rows[j] = logits row of sequence j, slots[j] = its decode slot, prompt_lens[j] = prompt length.
__global__ void prefill_commit_kernel(const long long* __restrict__ sampled, const float* __restrict__ logprob,
                                      const signed char* __restrict__ cls, const int* __restrict__ slots,
                                      const int* __restrict__ prompt_lens, const int* __restrict__ budgets,
                                      int n, int* __restrict__ seq_len, int* __restrict__ active,
                                      long long* __restrict__ last_token, int* __restrict__ gen_count,
                                      int* __restrict__ max_new, int* __restrict__ finish, int* __restrict__ out_tokens,
                                      float* __restrict__ out_logprobs, int out_stride) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const int s = slots[j];
  const long long tok = sampled[j];
  out_tokens[(long long)s * out_stride] = (int)tok;
  out_logprobs[(long long)s * out_stride] = logprob[j];
  gen_count[s] = 1;
  max_new[s] = budgets[j];
  seq_len[s] = prompt_lens[j];
  last_token[s] = tok;
  const signed char c = cls != nullptr ? cls[tok] : 0;
  if (c == 2 || c == 3) {
    finish[s] = 1;
    active[s] = 0;
  } else if (budgets[j] <= 1) {
    finish[s] = 2;
    active[s] = 0;
  } else {
    finish[s] = 0;
    active[s] = 1;
  }
}

}  // namespace areno

using namespace areno;

extern "C" int areno_decode_prepare(const int* seq_len, const int* active, const long long* last_token,
                                    const int* block_table, int max_pages, int page_size, int batch,
                                    long long* input_ids, int* positions, int* slot_mapping, int* attn_seq_lens,
                                    cudaStream_t stream) {
  if (batch <= 0) return 0;
  decode_prepare_kernel<<<(batch + 127) / 128, 128, 0, stream>>>(seq_len, active, last_token, block_table, max_pages,
                                                                 page_size, batch, input_ids, positions, slot_mapping,
                                                                 attn_seq_lens);
  return (int)cudaGetLastError();
}

extern "C" int areno_decode_commit(const long long* sampled, const float* logprob, const signed char* cls, int* seq_len,
                                   int* active, long long* last_token, int* gen_count, const int* max_new, int* finish,
                                   int* out_tokens, float* out_logprobs, int out_stride, int batch,
                                   cudaStream_t stream) {
  if (batch <= 0) return 0;
  decode_commit_kernel<<<(batch + 127) / 128, 128, 0, stream>>>(sampled, logprob, cls, seq_len, active, last_token,
                                                                gen_count, max_new, finish, out_tokens, out_logprobs,
                                                                out_stride, batch);
  return (int)cudaGetLastError();
}

extern "C" int areno_prefill_commit(const long long* sampled, const float* logprob, const signed char* cls,
                                    const int* slots, const int* prompt_lens, const int* budgets, int n, int* seq_len,
                                    int* active, long long* last_token, int* gen_count, int* max_new, int* finish,
                                    int* out_tokens, float* out_logprobs, int out_stride, cudaStream_t stream) {
  if (n <= 0) return 0;
  prefill_commit_kernel<<<(n + 127) / 128, 128, 0, stream>>>(sampled, logprob, cls, slots, prompt_lens, budgets, n,
                                                             seq_len, active, last_token, gen_count, max_new, finish,
                                                             out_tokens, out_logprobs, out_stride);
  return (int)cudaGetLastError();
}
