// Arguments of the paged attention launchers. One library is compiled per head size
// (-DLSE_HEAD_DIM=D) and exports the functions below; the core extension loads it on demand.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

extern "C" {

struct LseAttnArgs {
  int dtype;               // LSE_F32 or LSE_BF16: type of q, out and the pages
  const void* q;           // query rows; head h of token t at q + t*q_row_stride + h*D
  long long q_row_stride;  // in elements
  void* out;               // out + t*out_row_stride + h*D
  long long out_row_stride;
  const void* k_pages;     // [pages, num_kv_heads, page_tokens, D]
  const void* v_pages;
  int num_heads;
  int num_kv_heads;
  int page_tokens;
  int window;              // 0: all earlier keys; w: keys pos-w+1 .. pos
  float scale;
  const int* block_tables; // [sequences, table_stride]
  int table_stride;
  const int* ctx_lens;     // [sequences] tokens in the cache after this step's writes
  const int* cu_q;         // [sequences + 1] offsets of each sequence's rows in the flat batch
  // portions of two or more tokens
  const int* tiles;        // [num_tiles, 2]: sequence, first row of the tile within its portion
  int num_tiles;
  int force_simt;          // run the CUDA-core kernel even where a tensor-core one exists
  // single tokens
  const int* decode_seqs;  // [num_decode] sequence indices with one row each
  int num_decode;
  int num_splits;          // context partitions per (sequence, head)
  float* scratch;          // float32 [num_decode * num_heads * num_splits * (D + 2)] if num_splits > 1
};

int lse_attn_head_dim(void);
// rows per tile that lse_attn_prefill expects in `tiles` for this dtype
int lse_attn_q_tile(int dtype);
size_t lse_attn_decode_scratch_floats(int num_decode, int num_heads, int num_splits);
int lse_attn_prefill(const LseAttnArgs* a, cudaStream_t stream);
int lse_attn_decode(const LseAttnArgs* a, cudaStream_t stream);
}
