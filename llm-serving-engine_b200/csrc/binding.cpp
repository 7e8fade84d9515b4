// Python binding of the engine's CUDA kernels. Every function checks device, dtype, shape and
// contiguity of what it is given and raises on anything it cannot serve; work is enqueued on
// PyTorch's current CUDA stream. Attention kernels live in one shared library per head size,
// loaded here with dlopen.
#include <ATen/cuda/CUDAContext.h>
#include <dlfcn.h>
#include <torch/extension.h>

#include <map>
#include <optional>
#include <string>

#include "attention_args.h"
#include "kernels.h"

namespace {

using torch::Tensor;
using OptTensor = std::optional<Tensor>;

// Numbers go into messages as strings made here: streaming an integer or a double into an error
// message (operator<< of an ostream) has crashed the interpreter in builds of this extension on
// some hosts, and an error path must never do that.
template <typename N>
std::string num(N v) { return std::to_string(v); }

int dtype_code(const Tensor& t, const char* what) {
  if (t.scalar_type() == torch::kFloat32) return LSE_F32;
  if (t.scalar_type() == torch::kBFloat16) return LSE_BF16;
  if (t.scalar_type() == torch::kInt64) return LSE_FIXED64;  // fixed-point sums of the few-rows product
  TORCH_CHECK(false, what, ": dtype must be float32 or bfloat16, got ", c10::toString(t.scalar_type()));
}

void check_cuda(const Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda(), what, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), what, " must be contiguous");
  // the kernels read and write 16-byte vectors wherever a row holds whole ones
  TORCH_CHECK(t.numel() == 0 || reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, what,
              " must start on a 16-byte boundary");
}

void check_i32(const Tensor& t, const char* what) {
  check_cuda(t, what);
  TORCH_CHECK(t.scalar_type() == torch::kInt32, what, " must be int32");
}

void check_f32(const Tensor& t, const char* what) {
  check_cuda(t, what);
  TORCH_CHECK(t.scalar_type() == torch::kFloat32, what, " must be float32");
}

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void done(int code, const char* what) {
  TORCH_CHECK(code != LSE_BAD_ARGUMENT, what, ": the kernel refused these arguments");
  if (code != LSE_OK) {
    cudaError_t e = cudaGetLastError();
    TORCH_CHECK(false, what, ": launch failed: ", cudaGetErrorString(e));
  }
  // a capture that something has invalidated is reported where it is first seen, not at its end
  cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream(), &status) != cudaSuccess ||
      status == cudaStreamCaptureStatusInvalidated) {
    cudaGetLastError();
    TORCH_CHECK(false, what, ": the stream's graph capture is invalid after this call");
  }
}

void embedding(const Tensor& ids, const Tensor& table, Tensor& out) {
  check_i32(ids, "ids");
  check_cuda(table, "table");
  check_f32(out, "out");
  TORCH_CHECK(table.dim() == 2 && out.dim() == 2 && ids.dim() == 1, "embedding: bad ranks");
  TORCH_CHECK(out.size(0) == ids.size(0) && out.size(1) == table.size(1), "embedding: bad shapes");
  done(lse_embedding(ids.data_ptr<int>(), table.data_ptr(), dtype_code(table, "table"),
                     out.data_ptr<float>(), (int)ids.size(0), (int)table.size(1), stream()),
       "embedding");
}

void add_rmsnorm(Tensor& x, const OptTensor& residual, const Tensor& weight, double eps,
                 Tensor& out, const OptTensor& rows) {
  check_f32(x, "x");
  check_f32(weight, "weight");
  check_cuda(out, "out");
  TORCH_CHECK(x.dim() == 2 && out.dim() == 2 && weight.dim() == 1, "add_rmsnorm: bad ranks");
  const int H = (int)x.size(1);
  TORCH_CHECK(weight.size(0) == H && out.size(1) == H, "add_rmsnorm: widths differ");
  int rcode = LSE_F32;
  const void* rptr = nullptr;
  if (residual) {
    check_cuda(*residual, "residual");
    TORCH_CHECK(residual->sizes() == x.sizes(), "add_rmsnorm: residual shape differs from x");
    rcode = dtype_code(*residual, "residual");
    rptr = residual->data_ptr();
  }
  const int* rows_ptr = nullptr;
  int T = (int)x.size(0);
  if (rows) {
    check_i32(*rows, "rows");
    rows_ptr = rows->data_ptr<int>();
    T = (int)rows->size(0);
  }
  TORCH_CHECK(out.size(0) == T, "add_rmsnorm: out has ", num(out.size(0)), " rows, expected ", num(T));
  done(lse_add_rmsnorm(x.data_ptr<float>(), rptr, rcode, weight.data_ptr<float>(), (float)eps,
                       out.data_ptr(), dtype_code(out, "out"), rows_ptr, T, H, stream()),
       "add_rmsnorm");
}

// Returns the rotated queries: a view of qkv's first nq*D columns when qkv already has the pages'
// dtype, or a new [T, nq*D] tensor of `q_dtype` when qkv holds float32 sums.
Tensor rope_kv_write(Tensor& qkv, int64_t nq, int64_t nk, int64_t D, const Tensor& positions,
                     const Tensor& token_seq, const OptTensor& cos, const OptTensor& sin,
                     const OptTensor& k_pages, const OptTensor& v_pages, const Tensor& block_tables,
                     int64_t page_tokens, bool q_bf16) {
  check_cuda(qkv, "qkv");
  check_i32(positions, "positions");
  check_i32(token_seq, "token_seq");
  check_i32(block_tables, "block_tables");
  TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) == (nq + 2 * nk) * D, "rope_kv_write: qkv width");
  const int T = (int)qkv.size(0);
  TORCH_CHECK(positions.size(0) == T && token_seq.size(0) == T, "rope_kv_write: lengths differ");
  TORCH_CHECK(block_tables.dim() == 2, "rope_kv_write: block_tables must be [sequences, blocks]");
  const int in_code = dtype_code(qkv, "qkv");
  const int out_code = q_bf16 ? LSE_BF16 : LSE_F32;
  TORCH_CHECK(in_code == out_code || in_code == LSE_F32 || (in_code == LSE_FIXED64 && q_bf16),
              "rope_kv_write: this qkv dtype cannot give this q dtype");
  const float *c = nullptr, *s = nullptr;
  if (cos) {
    TORCH_CHECK(sin.has_value(), "rope_kv_write: cos without sin");
    check_f32(*cos, "cos");
    check_f32(*sin, "sin");
    TORCH_CHECK(cos->dim() == 2 && cos->size(1) == D / 2 && sin->sizes() == cos->sizes(),
                "rope_kv_write: tables must be [positions, head_dim/2]");
    c = cos->data_ptr<float>();
    s = sin->data_ptr<float>();
  }
  void *kp = nullptr, *vp = nullptr;
  if (k_pages) {
    TORCH_CHECK(v_pages.has_value(), "rope_kv_write: k_pages without v_pages");
    check_cuda(*k_pages, "k_pages");
    check_cuda(*v_pages, "v_pages");
    TORCH_CHECK(dtype_code(*k_pages, "k_pages") == out_code && dtype_code(*v_pages, "v_pages") == out_code,
                "rope_kv_write: pages and q differ in dtype");
    TORCH_CHECK(k_pages->dim() == 4 && k_pages->size(1) == nk && k_pages->size(2) == page_tokens &&
                    k_pages->size(3) == D && v_pages->sizes() == k_pages->sizes(),
                "rope_kv_write: pages must be [pages, kv_heads, page_tokens, head_dim]");
    kp = k_pages->data_ptr();
    vp = v_pages->data_ptr();
  }
  Tensor q = in_code == out_code
                 ? qkv.narrow(1, 0, nq * D)
                 : torch::empty({T, nq * D}, qkv.options().dtype(torch::kBFloat16));
  done(lse_rope_kv_write(qkv.data_ptr(), in_code, q.data_ptr(), out_code, T, (int)nq, (int)nk, (int)D,
                         positions.data_ptr<int>(), token_seq.data_ptr<int>(), c, s, kp, vp,
                         block_tables.data_ptr<int>(), (int)block_tables.size(1), (int)page_tokens,
                         stream()),
       "rope_kv_write");
  return q;
}

void silu_mul(const Tensor& gu, Tensor& out) {
  check_cuda(gu, "gu");
  check_cuda(out, "out");
  TORCH_CHECK(gu.dim() == 2 && out.dim() == 2 && gu.size(1) == 2 * out.size(1) &&
                  gu.size(0) == out.size(0),
              "silu_mul: gu must be [T, 2I] and out [T, I]");
  done(lse_silu_mul(gu.data_ptr(), dtype_code(gu, "gu"), out.data_ptr(), dtype_code(out, "out"),
                    (int)gu.size(0), (int)out.size(1), stream()),
       "silu_mul");
}

void gemm_f32(const Tensor& a, const Tensor& w, const OptTensor& bias, Tensor& out) {
  check_f32(a, "a");
  check_f32(w, "w");
  check_f32(out, "out");
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && out.dim() == 2 && a.size(1) == w.size(1) &&
                  out.size(0) == a.size(0) && out.size(1) == w.size(0),
              "gemm_f32: need a [T, K], w [N, K], out [T, N]");
  const float* b = nullptr;
  if (bias) {
    check_f32(*bias, "bias");
    TORCH_CHECK(bias->numel() == w.size(0), "gemm_f32: bias length");
    b = bias->data_ptr<float>();
  }
  done(lse_gemm_f32(a.data_ptr<float>(), w.data_ptr<float>(), b, out.data_ptr<float>(),
                    (int)a.size(0), (int)w.size(0), (int)a.size(1), stream()),
       "gemm_f32");
}

// A host-mapped int that kernels set when a bounded wait runs out; the host reads it without a copy.
int* error_flag() {
  static int* flag = nullptr;
  if (!flag) {
    TORCH_CHECK(cudaHostAlloc(&flag, sizeof(int), cudaHostAllocMapped) == cudaSuccess,
                "cannot allocate the kernels' error flag");
    *flag = 0;
  }
  return flag;
}

int64_t kernel_error() { return *error_flag(); }
void clear_kernel_error() { *error_flag() = 0; }

int64_t gemm_bf16_skinny_max_rows() { return lse_gemm_bf16_skinny_max_rows(); }

// out += a w^T (+ bias), out a buffer of fixed-point sums (int64)
void gemm_bf16_skinny(const Tensor& a, const Tensor& w, const OptTensor& bias, Tensor& out) {
  check_cuda(a, "a");
  check_cuda(w, "w");
  check_cuda(out, "out");
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16,
              "gemm_bf16_skinny: a and w must be bfloat16");
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && out.dim() == 2 && a.size(1) == w.size(1) &&
                  out.size(0) == a.size(0) && out.size(1) == w.size(0),
              "gemm_bf16_skinny: need a [T, K], w [N, K], out [T, N]");
  const void* b = nullptr;
  if (bias) {
    check_cuda(*bias, "bias");
    TORCH_CHECK(bias->scalar_type() == torch::kBFloat16 && bias->numel() == w.size(0),
                "gemm_bf16_skinny: bias must be bfloat16 [N]");
    b = bias->data_ptr();
  }
  TORCH_CHECK(out.scalar_type() == torch::kInt64, "gemm_bf16_skinny: out must be int64 (fixed-point sums)");
  done(lse_gemm_bf16_skinny(a.data_ptr(), w.data_ptr(), b, out.data_ptr(),
                            (int)a.size(0), (int)w.size(0), (int)a.size(1), error_flag(), stream()),
       "gemm_bf16_skinny");
}

// out (+)= value of the fixed-point sums in acc; acc is left zero
void fixed_to_float(Tensor& acc, Tensor& out, bool add) {
  check_cuda(acc, "acc");
  check_cuda(out, "out");
  TORCH_CHECK(acc.scalar_type() == torch::kInt64 && acc.numel() == out.numel(),
              "fixed_to_float: acc must be int64 with as many elements as out");
  const int code = dtype_code(out, "out");
  TORCH_CHECK(code != LSE_FIXED64 && (!add || code == LSE_F32), "fixed_to_float: bad out dtype");
  done(lse_fixed_to_float(acc.data_ptr(), out.data_ptr(), code, add ? 1 : 0, (long long)acc.numel(), stream()),
       "fixed_to_float");
}

// ------------------------------------------------------------------ attention libraries
struct AttnLib {
  void* handle;
  int (*head_dim)(void);
  int (*q_tile)(int);
  size_t (*scratch_floats)(int, int, int);
  int (*decode_blocks_per_sm)(int, int, int);
  int (*decode_takes_sums)(int, int, int);
  int (*prefill)(const LseAttnArgs*, cudaStream_t);
  int (*decode)(const LseAttnArgs*, cudaStream_t);
};
std::map<int, AttnLib>& libs() {
  static std::map<int, AttnLib> m;
  return m;
}

void load_attention_library(const std::string& path, int64_t head_dim) {
  if (libs().count((int)head_dim)) return;
  void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  TORCH_CHECK(h, "cannot load attention library ", path, ": ", dlerror());
  AttnLib lib;
  lib.handle = h;
  lib.head_dim = (int (*)(void))dlsym(h, "lse_attn_head_dim");
  lib.q_tile = (int (*)(int))dlsym(h, "lse_attn_q_tile");
  lib.scratch_floats = (size_t(*)(int, int, int))dlsym(h, "lse_attn_decode_scratch_floats");
  lib.decode_blocks_per_sm = (int (*)(int, int, int))dlsym(h, "lse_attn_decode_blocks_per_sm");
  lib.decode_takes_sums = (int (*)(int, int, int))dlsym(h, "lse_attn_decode_takes_sums");
  lib.prefill = (int (*)(const LseAttnArgs*, cudaStream_t))dlsym(h, "lse_attn_prefill");
  lib.decode = (int (*)(const LseAttnArgs*, cudaStream_t))dlsym(h, "lse_attn_decode");
  TORCH_CHECK(lib.head_dim && lib.q_tile && lib.scratch_floats && lib.decode_blocks_per_sm &&
                  lib.decode_takes_sums && lib.prefill && lib.decode,
              "attention library ", path, " lacks an entry point");
  TORCH_CHECK(lib.head_dim() == head_dim, "attention library ", path, " was built for head size ",
              num(lib.head_dim()), ", not ", num(head_dim));
  libs()[(int)head_dim] = lib;
}

const AttnLib& attn_lib(int64_t D) {
  auto it = libs().find((int)D);
  TORCH_CHECK(it != libs().end(), "no attention library loaded for head size ", num(D));
  return it->second;
}

int64_t attention_q_tile(int64_t D, bool bf16, int64_t force_kernel) {
  const AttnLib& lib = attn_lib(D);
  return force_kernel == 1 ? lib.q_tile(LSE_F32) : lib.q_tile(bf16 ? LSE_BF16 : LSE_F32);
}

int64_t attention_scratch_floats(int64_t D, int64_t num_decode, int64_t num_heads, int64_t splits) {
  return (int64_t)attn_lib(D).scratch_floats((int)num_decode, (int)num_heads, (int)splits);
}

int64_t attention_decode_blocks_per_sm(int64_t D, bool bf16, int64_t num_heads, int64_t num_kv_heads) {
  return attn_lib(D).decode_blocks_per_sm(bf16 ? LSE_BF16 : LSE_F32, (int)num_heads, (int)num_kv_heads);
}

// q: the fused projection [T, q_width_total] whose first num_heads*D columns are the queries, or
// any [T, >= num_heads*D] tensor with unit column stride.
void paged_attention(const Tensor& q, Tensor& out, const Tensor& k_pages, const Tensor& v_pages,
                     int64_t num_heads, int64_t num_kv_heads, int64_t D, double scale,
                     int64_t window, const Tensor& block_tables, const Tensor& ctx_lens,
                     const Tensor& cu_q, const OptTensor& tiles, int64_t num_tiles,
                     const OptTensor& decode_seqs, int64_t num_decode, int64_t num_splits,
                     const OptTensor& scratch, int64_t force_kernel) {
  const AttnLib& lib = attn_lib(D);
  TORCH_CHECK(q.is_cuda() && q.dim() == 2 && q.stride(1) == 1 && q.size(1) >= num_heads * D,
              "paged_attention: q must be [T, >= heads*head_dim] with unit column stride");
  check_cuda(out, "out");
  check_cuda(k_pages, "k_pages");
  check_cuda(v_pages, "v_pages");
  check_i32(block_tables, "block_tables");
  check_i32(ctx_lens, "ctx_lens");
  check_i32(cu_q, "cu_q");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == q.size(0) && out.size(1) == num_heads * D,
              "paged_attention: out must be [T, heads*head_dim]");
  TORCH_CHECK(out.scalar_type() == q.scalar_type() && k_pages.scalar_type() == q.scalar_type() &&
                  v_pages.scalar_type() == q.scalar_type(),
              "paged_attention: q, out and pages must share a dtype");
  TORCH_CHECK(k_pages.dim() == 4 && k_pages.size(1) == num_kv_heads && k_pages.size(3) == D &&
                  v_pages.sizes() == k_pages.sizes(),
              "paged_attention: pages must be [pages, kv_heads, page_tokens, head_dim]");
  TORCH_CHECK(block_tables.dim() == 2 && cu_q.size(0) == ctx_lens.size(0) + 1 &&
                  block_tables.size(0) >= ctx_lens.size(0),
              "paged_attention: per-sequence arrays disagree");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(q.data_ptr()) % 16) == 0 &&
                  (q.stride(0) * q.element_size()) % 16 == 0,
              "paged_attention: q rows must be 16-byte aligned");
  LseAttnArgs a{};
  a.dtype = dtype_code(q, "q");
  a.q = q.data_ptr();
  a.q_row_stride = q.stride(0);
  a.out = out.data_ptr();
  a.out_row_stride = out.stride(0);
  a.k_pages = k_pages.data_ptr();
  a.v_pages = v_pages.data_ptr();
  a.num_heads = (int)num_heads;
  a.num_kv_heads = (int)num_kv_heads;
  a.page_tokens = (int)k_pages.size(2);
  a.window = (int)window;
  a.scale = (float)scale;
  a.block_tables = block_tables.data_ptr<int>();
  a.table_stride = (int)block_tables.size(1);
  a.ctx_lens = ctx_lens.data_ptr<int>();
  a.cu_q = cu_q.data_ptr<int>();
  a.force_simt = (int)force_kernel;
  a.num_rows = q.size(0);
  a.num_pages = k_pages.size(0);
  a.error_flag = error_flag();
  if (num_tiles > 0) {
    TORCH_CHECK(tiles.has_value(), "paged_attention: num_tiles > 0 without tiles");
    check_i32(*tiles, "tiles");
    TORCH_CHECK(tiles->numel() >= 2 * num_tiles, "paged_attention: tiles too short");
    a.tiles = tiles->data_ptr<int>();
    a.num_tiles = (int)num_tiles;
    done(lib.prefill(&a, stream()), "paged_attention (portions)");
  }
  if (num_decode > 0) {
    TORCH_CHECK(decode_seqs.has_value(), "paged_attention: num_decode > 0 without decode_seqs");
    check_i32(*decode_seqs, "decode_seqs");
    TORCH_CHECK(decode_seqs->numel() >= num_decode, "paged_attention: decode_seqs too short");
    a.decode_seqs = decode_seqs->data_ptr<int>();
    a.num_decode = (int)num_decode;
    a.num_splits = (int)num_splits;
    if (num_splits > 1) {
      TORCH_CHECK(scratch.has_value(), "paged_attention: num_splits > 1 needs scratch");
      check_f32(*scratch, "scratch");
      TORCH_CHECK((size_t)scratch->numel() >=
                      lib.scratch_floats((int)num_decode, (int)num_heads, (int)num_splits),
                  "paged_attention: scratch too small");
      a.scratch = scratch->data_ptr<float>();
    }
    done(lib.decode(&a, stream()), "paged_attention (single tokens)");
  }
}

bool attention_takes_sums(int64_t D, bool bf16, int64_t num_heads, int64_t num_kv_heads) {
  return attn_lib(D).decode_takes_sums(bf16 ? LSE_BF16 : LSE_F32, (int)num_heads, (int)num_kv_heads) != 0;
}

// Single tokens straight from the fixed-point sums of the fused q|k|v projection: rotation, cache
// write and attention in one launch; the sums are left zero. Every row of `sums` is one sequence's
// single token (row i belongs to sequence decode_seqs[i] through cu_q).
void paged_attention_from_sums(Tensor& sums, Tensor& out, Tensor& k_pages, Tensor& v_pages,
                               int64_t num_heads, int64_t num_kv_heads, int64_t D, double scale,
                               int64_t window, const Tensor& block_tables, const Tensor& ctx_lens,
                               const Tensor& cu_q, const Tensor& decode_seqs, int64_t num_splits,
                               const OptTensor& scratch, const OptTensor& cos, const OptTensor& sin) {
  const AttnLib& lib = attn_lib(D);
  check_cuda(sums, "sums");
  check_cuda(out, "out");
  check_cuda(k_pages, "k_pages");
  check_cuda(v_pages, "v_pages");
  check_i32(block_tables, "block_tables");
  check_i32(ctx_lens, "ctx_lens");
  check_i32(cu_q, "cu_q");
  check_i32(decode_seqs, "decode_seqs");
  const int64_t T = sums.size(0);
  TORCH_CHECK(sums.scalar_type() == torch::kInt64 && sums.dim() == 2 &&
                  sums.size(1) == (num_heads + 2 * num_kv_heads) * D,
              "paged_attention_from_sums: sums must be int64 [T, (heads + 2 kv_heads) * head_dim]");
  TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && k_pages.scalar_type() == torch::kBFloat16 &&
                  v_pages.scalar_type() == torch::kBFloat16,
              "paged_attention_from_sums: out and pages must be bfloat16");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == T && out.size(1) == num_heads * D,
              "paged_attention_from_sums: out must be [T, heads*head_dim]");
  TORCH_CHECK(k_pages.dim() == 4 && k_pages.size(1) == num_kv_heads && k_pages.size(3) == D &&
                  v_pages.sizes() == k_pages.sizes(),
              "paged_attention_from_sums: pages must be [pages, kv_heads, page_tokens, head_dim]");
  TORCH_CHECK(block_tables.dim() == 2 && cu_q.size(0) == ctx_lens.size(0) + 1 &&
                  block_tables.size(0) >= ctx_lens.size(0) && decode_seqs.numel() == T,
              "paged_attention_from_sums: per-sequence arrays disagree, or a row is not a single token");
  TORCH_CHECK(lib.decode_takes_sums(LSE_BF16, (int)num_heads, (int)num_kv_heads),
              "paged_attention_from_sums: not served for these head counts");
  TORCH_CHECK(cos.has_value() == sin.has_value(), "paged_attention_from_sums: cos and sin go together");
  LseAttnArgs a{};
  a.dtype = LSE_BF16;
  a.qkv_sums = reinterpret_cast<const long long*>(sums.data_ptr());
  if (cos) {
    check_f32(*cos, "cos");
    check_f32(*sin, "sin");
    TORCH_CHECK(cos->dim() == 2 && cos->size(1) == D / 2 && sin->sizes() == cos->sizes(),
                "paged_attention_from_sums: cos and sin must be [positions, head_dim / 2]");
    a.rope_cos = cos->data_ptr<float>();
    a.rope_sin = sin->data_ptr<float>();
  }
  a.out = out.data_ptr();
  a.out_row_stride = out.stride(0);
  a.k_pages = k_pages.data_ptr();
  a.v_pages = v_pages.data_ptr();
  a.num_heads = (int)num_heads;
  a.num_kv_heads = (int)num_kv_heads;
  a.page_tokens = (int)k_pages.size(2);
  a.window = (int)window;
  a.scale = (float)scale;
  a.block_tables = block_tables.data_ptr<int>();
  a.table_stride = (int)block_tables.size(1);
  a.ctx_lens = ctx_lens.data_ptr<int>();
  a.cu_q = cu_q.data_ptr<int>();
  a.num_rows = T;
  a.num_pages = k_pages.size(0);
  a.error_flag = error_flag();
  a.decode_seqs = decode_seqs.data_ptr<int>();
  a.num_decode = (int)T;
  a.num_splits = (int)num_splits;
  if (num_splits > 1) {
    TORCH_CHECK(scratch.has_value(), "paged_attention_from_sums: num_splits > 1 needs scratch");
    check_f32(*scratch, "scratch");
    TORCH_CHECK((size_t)scratch->numel() >= lib.scratch_floats((int)T, (int)num_heads, (int)num_splits),
                "paged_attention_from_sums: scratch too small");
    a.scratch = scratch->data_ptr<float>();
  }
  if (T > 0) done(lib.decode(&a, stream()), "paged_attention_from_sums");
}

// ------------------------------------------------------------------ sampling
void sample(const Tensor& logits, const Tensor& temperature, const Tensor& top_k,
            const Tensor& top_p, const Tensor& min_p, const Tensor& seed, const Tensor& draw,
            Tensor& out, const OptTensor& scratch, int64_t which) {
  check_f32(logits, "logits");
  check_f32(temperature, "temperature");
  check_i32(top_k, "top_k");
  check_f32(top_p, "top_p");
  check_f32(min_p, "min_p");
  check_cuda(seed, "seed");
  TORCH_CHECK(seed.scalar_type() == torch::kInt64, "seed must be int64");
  check_i32(draw, "draw");
  check_i32(out, "out");
  const int R = (int)logits.size(0);
  TORCH_CHECK(logits.dim() == 2 && temperature.numel() == R && top_k.numel() == R &&
                  top_p.numel() == R && min_p.numel() == R && seed.numel() == R &&
                  draw.numel() == R && out.numel() == R,
              "sample: one parameter per row of logits is needed");
  int* sc = nullptr;
  int sc_rows = 0;
  if (scratch) {  // several blocks per row for rows without a cut, if it was made for R rows or more
    check_i32(*scratch, "scratch");
    sc = scratch->data_ptr<int>();
    sc_rows = (int)(scratch->numel() / (int64_t)lse_sample_scratch_ints(1));
  }
  done(lse_sample(logits.data_ptr<float>(), R, (int)logits.size(1), temperature.data_ptr<float>(),
                  top_k.data_ptr<int>(), top_p.data_ptr<float>(), min_p.data_ptr<float>(),
                  reinterpret_cast<const uint64_t*>(seed.data_ptr<int64_t>()), draw.data_ptr<int>(),
                  out.data_ptr<int>(), sc, sc_rows, (int)which, stream()),
       "sample");
}

void logsumexp(const Tensor& logits, Tensor& out) {
  check_f32(logits, "logits");
  check_f32(out, "out");
  TORCH_CHECK(logits.dim() == 2 && out.numel() == logits.size(0), "logsumexp: shapes");
  done(lse_logsumexp(logits.data_ptr<float>(), (int)logits.size(0), (int)logits.size(1),
                     out.data_ptr<float>(), stream()),
       "logsumexp");
}

void apply_penalties(Tensor& logits, const Tensor& row, const Tensor& token, const Tensor& count,
                     const Tensor& presence, const Tensor& frequency, const Tensor& repetition) {
  check_f32(logits, "logits");
  check_i32(row, "row");
  check_i32(token, "token");
  check_i32(count, "count");
  check_f32(presence, "presence");
  check_f32(frequency, "frequency");
  check_f32(repetition, "repetition");
  const int n = (int)row.numel();
  TORCH_CHECK(token.numel() == n && count.numel() == n && presence.numel() == n &&
                  frequency.numel() == n && repetition.numel() == n,
              "apply_penalties: lengths differ");
  done(lse_apply_penalties(logits.data_ptr<float>(), (int)logits.size(1), row.data_ptr<int>(),
                           token.data_ptr<int>(), count.data_ptr<int>(), presence.data_ptr<float>(),
                           frequency.data_ptr<float>(), repetition.data_ptr<float>(), n, stream()),
       "apply_penalties");
}

void token_state_add(Tensor& state, const Tensor& slot, const Tensor& token, const Tensor& in_prompt) {
  check_i32(state, "state");
  check_i32(slot, "slot");
  check_i32(token, "token");
  check_i32(in_prompt, "in_prompt");
  TORCH_CHECK(state.dim() == 2, "token_state_add: state must be [slots, vocab]");
  const int n = (int)slot.numel();
  TORCH_CHECK(token.numel() == n && in_prompt.numel() == n, "token_state_add: lengths differ");
  done(lse_token_state_add(state.data_ptr<int>(), (int)state.size(1), slot.data_ptr<int>(),
                           token.data_ptr<int>(), in_prompt.data_ptr<int>(), n, stream()),
       "token_state_add");
}

void apply_penalties_dense(Tensor& logits, const Tensor& row, const Tensor& slot, const Tensor& presence,
                           const Tensor& frequency, const Tensor& repetition, const Tensor& state) {
  check_f32(logits, "logits");
  check_i32(row, "row");
  check_i32(slot, "slot");
  check_f32(presence, "presence");
  check_f32(frequency, "frequency");
  check_f32(repetition, "repetition");
  check_i32(state, "state");
  const int n = (int)row.numel();
  TORCH_CHECK(slot.numel() == n && presence.numel() == n && frequency.numel() == n &&
                  repetition.numel() == n,
              "apply_penalties_dense: lengths differ");
  TORCH_CHECK(logits.dim() == 2 && state.dim() == 2 && state.size(1) == logits.size(1),
              "apply_penalties_dense: state must be [slots, vocab]");
  done(lse_apply_penalties_dense(logits.data_ptr<float>(), (int)logits.size(1), row.data_ptr<int>(),
                                 slot.data_ptr<int>(), presence.data_ptr<float>(),
                                 frequency.data_ptr<float>(), repetition.data_ptr<float>(),
                                 state.data_ptr<int>(), n, stream()),
       "apply_penalties_dense");
}

void ban_tokens(Tensor& logits, const Tensor& row, const Tensor& token) {
  check_f32(logits, "logits");
  check_i32(row, "row");
  check_i32(token, "token");
  TORCH_CHECK(row.numel() == token.numel(), "ban_tokens: lengths differ");
  done(lse_ban_tokens(logits.data_ptr<float>(), (int)logits.size(1), row.data_ptr<int>(),
                      token.data_ptr<int>(), (int)row.numel(), stream()),
       "ban_tokens");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("embedding", &embedding);
  m.def("add_rmsnorm", &add_rmsnorm);
  m.def("rope_kv_write", &rope_kv_write);
  m.def("silu_mul", &silu_mul);
  m.def("gemm_f32", &gemm_f32);
  m.def("gemm_bf16_skinny", &gemm_bf16_skinny);
  m.def("gemm_bf16_skinny_max_rows", &gemm_bf16_skinny_max_rows);
  m.def("fixed_to_float", &fixed_to_float);
  m.def("kernel_error", &kernel_error);
  m.def("clear_kernel_error", &clear_kernel_error);
  m.def("load_attention_library", &load_attention_library);
  m.def("attention_q_tile", &attention_q_tile);
  m.def("attention_scratch_floats", &attention_scratch_floats);
  m.def("attention_decode_blocks_per_sm", &attention_decode_blocks_per_sm);
  m.def("paged_attention", &paged_attention);
  m.def("paged_attention_from_sums", &paged_attention_from_sums);
  m.def("attention_takes_sums", &attention_takes_sums);
  m.def("sample", &sample, py::arg("logits"), py::arg("temperature"), py::arg("top_k"), py::arg("top_p"),
        py::arg("min_p"), py::arg("seed"), py::arg("draw"), py::arg("out"), py::arg("scratch") = py::none(),
        py::arg("which") = 3);
  m.def("sample_scratch_ints", [](int64_t rows) { return (int64_t)lse_sample_scratch_ints((int)rows); });
  m.def("logsumexp", &logsumexp);
  m.def("apply_penalties", &apply_penalties);
  m.def("ban_tokens", &ban_tokens);
  m.def("token_state_add", &token_state_add);
  m.def("apply_penalties_dense", &apply_penalties_dense);
}
