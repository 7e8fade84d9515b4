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
  int force_simt;          // 0: fastest kernel that serves the arguments; 1: the CUDA-core kernel;
                           // 2: the mma.sync tensor-core kernel fed by plain loads (no tcgen05, no
                           // TMA); 3: single tokens on the TMA-fed kernel whatever the grid's size
                           // (portions as with 2)
  // single tokens
  const int* decode_seqs;  // [num_decode] sequence indices with one row each
  int num_decode;
  int num_splits;          // context partitions per (sequence, head): 1 to 64
  float* scratch;          // if num_splits > 1: lse_attn_decode_scratch_floats(...) floats; its
                           // first LSE_ATTN_COUNTERS words are counters that must be zero before
                           // a launch (every launch leaves them zero)
  // sizes of the tensors behind q/out and the pages (needed to describe them to TMA)
  long long num_rows;      // rows of q and out
  long long num_pages;     // pages in k_pages / v_pages
  int* error_flag;         // device-visible int that receives a code if a bounded wait ran out, or null
  // Single tokens straight from the fused q|k|v projection (lse_attn_decode only; null: not used).
  // qkv_sums: [rows, (num_heads + 2 num_kv_heads) D] fixed-point sums (LSE_FIXED64) of the projection
  // of this step's rows, every row a single token of its sequence. The kernel then ignores `q`:
  // it makes the queries, and this step's key and value, from the sums (rotated with rope_cos /
  // rope_sin [max_pos, D/2] at position ctx - 1 unless those are null, rounded to the pages'
  // type), writes the key and value into their page, and leaves the sums zero. Served where
  // lse_attn_decode_takes_sums() says so.
  const long long* qkv_sums;
  const float* rope_cos;
  const float* rope_sin;
};

#define LSE_ATTN_COUNTERS 65536  // words at the start of the scratch: one counter per (sequence, head group)

int lse_attn_head_dim(void);
// rows per tile that lse_attn_prefill expects in `tiles` for this dtype
int lse_attn_q_tile(int dtype);
size_t lse_attn_decode_scratch_floats(int num_decode, int num_heads, int num_splits);
// blocks of lse_attn_decode's kernel for these head counts that one SM holds at a time; 0: unknown
int lse_attn_decode_blocks_per_sm(int dtype, int num_heads, int num_kv_heads);
// 1 if lse_attn_decode serves LseAttnArgs::qkv_sums for this type and these head counts
int lse_attn_decode_takes_sums(int dtype, int num_heads, int num_kv_heads);
// The kernels of both launchers are enqueued with programmatic stream serialization and read the
// batch description (`tiles`, `decode_seqs`, `cu_q`, `ctx_lens`) *before* their dependency wait.
// Those four arrays must therefore be complete before the call is enqueued (a host-to-device copy
// or an ordinary kernel earlier in the stream is), and must not be outputs of kernels of this
// package that were launched the same way just before. q, the pages and the block tables are
// read after the wait.
int lse_attn_prefill(const LseAttnArgs* a, cudaStream_t stream);
int lse_attn_decode(const LseAttnArgs* a, cudaStream_t stream);

// ---- Single-token attention for callers that cannot allocate device memory ---------------------
// (This entry point has no counterpart in the reference, whose attention runs on the CPU.)
//
// lse_attn_decode needs a scratch buffer for the partial results of its context partitions, and
// the caller has to allocate it. Some callers cannot: a host program that has given all device
// memory to its own pool and may not call cudaMalloc any more, or a latency-critical serving loop
// that must never meet cudaMalloc's implicit device-wide synchronisation. For them lse_attn_decode_noalloc does the same computation with the scratch in
// a buffer that is part of this library's device image: LSE_ATTN_NOALLOC_MAX_FLOATS floats (4 MiB),
// held on every GPU that loads the library until the process exits. The caller still passes the
// inputs and the output; `a->scratch` is ignored. The function calls no cudaMalloc, cudaFree or
// other allocating routine.
//
//  * Size limit: lse_attn_decode_scratch_floats(num_decode, num_heads, num_splits) must not exceed
//    LSE_ATTN_NOALLOC_MAX_FLOATS when num_splits > 1; otherwise nothing is launched and
//    LSE_TOO_LARGE is returned (lse_attn_decode_noalloc_max_floats() reports the limit).
//  * First call on a device: it looks up the buffer's device address (cudaGetSymbolAddress, with
//    that device current) and remembers it. Make that first call outside any stream capture.
//  * The buffer is shared by every call and keeps the last call's contents. The partial results
//    need no clearing (each launch writes every one it later reads); the completion counters
//    must start at zero, which holds because the buffer is zero when the library is loaded and
//    every launch resets the counters it used. Two calls whose
//    kernels overlap on the GPU (different streams) would race on it; run them one after the other.
//  * The remembered address belongs to the device that is current at the call: `stream` must be
//    a stream of that device. The rule above on `decode_seqs`, `cu_q` and `ctx_lens` holds here too.
#define LSE_ATTN_NOALLOC_MAX_FLOATS (1 << 20)
#define LSE_TOO_LARGE 3
size_t lse_attn_decode_noalloc_max_floats(void);
int lse_attn_decode_noalloc(const LseAttnArgs* a, cudaStream_t stream);
}
