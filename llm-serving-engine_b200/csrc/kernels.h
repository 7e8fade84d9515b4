// C launch interface of the engine's CUDA kernels. Every function enqueues work on `stream` and
// returns LSE_OK, or a non-zero code with nothing enqueued when an argument cannot be served.
// dtype codes: 0 = float32, 1 = bfloat16.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "status.h"

#define LSE_F32 0
#define LSE_BF16 1
// Sums that several blocks add to in any order: a 64-bit integer holding value * 2^24. Integer
// addition is associative, so the result has the same bits whatever the order was. A kernel that
// takes such an input converts it to float32 and leaves zeros behind, ready for the next sums.
#define LSE_FIXED64 2

extern "C" {

// out[t, :] = float(table[ids[t], :])                      out float32 [T, H]
int lse_embedding(const int* ids, const void* table, int table_dtype, float* out, int T, int H,
                  cudaStream_t stream);

// Residual add and RMS norm.
//   rows == nullptr: for every row t < T: if residual: x[t] += residual[t] (in place, float32);
//                    out[t] = x[t] * rsqrt(mean(x[t]^2) + eps) * weight
//   rows != nullptr: out[r] = norm(x[rows[r]] (+ residual[rows[r]])) for r < T; x is not written.
// residual_dtype LSE_FIXED64 (rows == nullptr only): residual holds fixed-point sums, which are
// cleared as they are read.
int lse_add_rmsnorm(float* x, const void* residual, int residual_dtype, const float* weight,
                    float eps, void* out, int out_dtype, const int* rows, int T, int H,
                    cudaStream_t stream);

// Rotate the q and k heads of the fused projection and write this step's k and v rows into their
// pages. qkv [T, (nq + 2 nk) D] of in_dtype; the rotated queries go to q_out as `dtype`:
//   in_dtype == dtype: q_out must be qkv itself (rotated in place, row stride (nq + 2 nk) D);
//   in_dtype == LSE_F32 or LSE_FIXED64 (cleared as it is read), dtype == LSE_BF16: q_out is a
//   separate [T, nq D] buffer.
//   cos/sin float32 [max_pos, D/2] or nullptr for no rotation;
//   k_pages/v_pages [pages, nk, page_tokens, D] of `dtype`, or nullptr when this layer only reads.
int lse_rope_kv_write(const void* qkv, int in_dtype, void* q_out, int dtype, int T, int nq, int nk,
                      int D, const int* positions, const int* token_seq, const float* cos,
                      const float* sin, void* k_pages, void* v_pages, const int* block_tables,
                      int table_stride, int page_tokens, cudaStream_t stream);

// out[t, i] = silu(gu[t, i]) * gu[t, I + i]     gu [T, 2I] of in_dtype, out [T, I] of dtype
// (in_dtype == dtype, or float32 / LSE_FIXED64 in and bfloat16 out; a fixed-point input is cleared
// as it is read).
int lse_silu_mul(const void* gu, int in_dtype, void* out, int dtype, int T, int I,
                 cudaStream_t stream);

// True float32 matrix product: out[T, N] = a[T, K] . w[N, K]^T (+ bias[N]). Each output element is
// accumulated over k in ascending order by one thread, so a row's result does not depend on T.
int lse_gemm_f32(const float* a, const float* w, const float* bias, float* out, int T, int N, int K,
                 cudaStream_t stream);

// bfloat16 product for few rows on tcgen05 tensor cores fed by TMA (gemm_bf16_tc.cu):
//   out[T, N] += a[T, K] . w[N, K]^T (+ bias[N]),  T <= lse_gemm_bf16_skinny_max_rows(), K % 8 == 0.
// out is a buffer of 64-bit fixed-point numbers (see LSE_FIXED64). The work is balanced over all
// SMs whatever N is; the sums do not depend on the order of the additions, so they have the same
// bits on every run. error_flag (device-visible int, may be null) receives a non-zero code if a
// bounded wait inside the kernel ran out.
int lse_gemm_bf16_skinny_max_rows(void);
int lse_gemm_bf16_skinny(const void* a, const void* w, const void* bias, void* out, int T, int N,
                         int K, int* error_flag, cudaStream_t stream);

// out[T, N] = value of the fixed-point sums acc[T, N] (+ what out holds, if add != 0); every
// element of acc that is read is set to zero. out float32 or bfloat16 (add needs float32).
int lse_fixed_to_float(void* acc, void* out, int out_dtype, int add, long long n, cudaStream_t stream);

// Sampling. One token per row of logits [R, V] (float32, row stride V).
//   temperature[r] < 1e-5 selects the largest logit (lowest index on ties). Otherwise the row is
//   divided by its temperature, cut to top_k / top_p / min_p, and a token is drawn by the
//   exponential race: argmax p_i / E_i, E_i ~ Exp(1) from a counter-based generator keyed by
//   (seed[r], draw[r], i).
//   scratch: lse_sample_scratch_ints(scratch_rows) ints, zero before the first launch (every
//   launch leaves its counters zero), or null. With it (and scratch_rows >= R), rows that need no
//   cut (and a temperature) are served by several blocks each. which: bit 0 = some row is greedy
//   or has a cut, bit 1 = some row has a temperature and no cut; 3 if the caller does not know.
//   A kernel whose rows are promised absent is not launched.
size_t lse_sample_scratch_ints(int rows);
int lse_sample(const float* logits, int R, int V, const float* temperature, const int* top_k,
               const float* top_p, const float* min_p, const uint64_t* seed, const int* draw,
               int* out_tokens, int* scratch, int scratch_rows, int which,
               cudaStream_t stream);

// out[r] = log(sum_i exp(logits[r, i]))
int lse_logsumexp(const float* logits, int R, int V, float* out, cudaStream_t stream);

// logits[row, token] += / *= per the penalties; entries are unique (row, token) pairs.
int lse_apply_penalties(float* logits, int V, const int* row, const int* token, const int* count,
                        const float* presence, const float* frequency, const float* repetition,
                        int n, cudaStream_t stream);

// logits[row[i], token[i]] = -inf
// Token state of the penalties on the device: state[slots, V] int32, low 30 bits = times
// generated, bit 30 = occurs in the prompt. lse_token_state_add enters n (slot, token) pairs
// (in_prompt[i] != 0: mark as prompt token; else count one more generation).
// lse_apply_penalties_dense applies presence / frequency / repetition (the rule above) to logits
// row row[j] from the state of slot[j], for j < n.
int lse_token_state_add(int* state, int V, const int* slot, const int* token, const int* in_prompt,
                        int n, cudaStream_t stream);
int lse_apply_penalties_dense(float* logits, int V, const int* row, const int* slot,
                              const float* presence, const float* frequency, const float* repetition,
                              const int* state, int n, cudaStream_t stream);
int lse_ban_tokens(float* logits, int V, const int* row, const int* token, int n,
                   cudaStream_t stream);
}
