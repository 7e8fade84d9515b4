// Memory-bound kernels around the matrix products: embedding gather, residual add + RMS norm,
// rotary positions + key/value page write, SiLU gate. All arithmetic is float32; values are
// rounded once when they are stored in the compute dtype.
//
// What each computes follows the reference's fused CPU ops
// (src/llmserve/kernels/csrc/fused_ops.cpp:39-125) and src/llmserve/attention.py:221-228.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"

namespace lse {

// ------------------------------------------------------------------------------------ embedding
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int H) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const T* src = table + (size_t)ids[t] * H;
  float* dst = out + (size_t)t * H;
  constexpr int V = Num<T>::kVec;
  if (H % V == 0) {
    for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
      Vec16<T> v = load16(src + i);
#pragma unroll
      for (int j = 0; j < V; j += 4)  // H % V == 0 and 16-byte aligned rows: whole float4 stores
        *reinterpret_cast<float4*>(dst + i + j) =
            make_float4(Num<T>::to_float(v.v[j]), Num<T>::to_float(v.v[j + 1]),
                        Num<T>::to_float(v.v[j + 2]), Num<T>::to_float(v.v[j + 3]));
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = Num<T>::to_float(src[i]);
  }
}

// ------------------------------------------------------------------------------------ rms norm
// One block per output row. The row is visited twice by the same threads at the same indices, so
// the second visit sees this thread's own writes of the first.
template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<bf16>(const bf16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
// Fixed-point sums are taken: read, converted, and zeros left behind for the next sums.
template <>
__device__ __forceinline__ void load4<fixed64>(const fixed64* p, float (&v)[4]) {
  longlong2* q = reinterpret_cast<longlong2*>(const_cast<fixed64*>(p));
  const longlong2 a = q[0], b = q[1];
  q[0] = make_longlong2(0, 0);
  q[1] = make_longlong2(0, 0);
  v[0] = fixed_to_float(a.x); v[1] = fixed_to_float(a.y);
  v[2] = fixed_to_float(b.x); v[3] = fixed_to_float(b.y);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<bf16>(bf16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

// V = 4 or 8 elements at a time (8: two groups of four for float, one 16-byte vector for bfloat16)
template <typename T, int V>
__device__ __forceinline__ void loadv(const T* p, float (&v)[V]) {
  if constexpr (V == 4) {
    load4<T>(p, v);
  } else if constexpr (std::is_same<T, bf16>::value) {
    const Vec16<bf16> t = load16(p);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(t.v[j]);
  } else {
    float lo[4], hi[4];
    load4<T>(p, lo);
    load4<T>(p + 4, hi);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[j] = lo[j];
      v[j + 4] = hi[j];
    }
  }
}
template <typename T, int V>
__device__ __forceinline__ void storev(T* p, const float (&v)[V]) {
  if constexpr (V == 4) {
    store4<T>(p, v);
  } else if constexpr (std::is_same<T, bf16>::value) {
    Vec16<bf16> t;
#pragma unroll
    for (int j = 0; j < 8; ++j) t.v[j] = __float2bfloat16_rn(v[j]);
    store16(p, t);
  } else {
    const float lo[4] = {v[0], v[1], v[2], v[3]}, hi[4] = {v[4], v[5], v[6], v[7]};
    store4<T>(p, lo);
    store4<T>(p + 4, hi);
  }
}

// VEC4: H is a multiple of 4, so rows are read and written four elements at a time.
template <typename TR, typename TO, bool VEC4>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TR* __restrict__ residual,
                                   const float* __restrict__ weight, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows, int H) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src_row = rows ? rows[r] : r;
  float* xr = x + (size_t)src_row * H;
  const TR* rr = residual ? residual + (size_t)src_row * H : nullptr;
  const bool in_place = (rows == nullptr) && (rr != nullptr);
  TO* o = out + (size_t)r * H;
  float ss = 0.f;
  if (VEC4) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float v[4];
      load4<float>(xr + i, v);
      if (rr) {
        float a[4];
        load4<TR>(rr + i, a);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += a[j];
        if (in_place) store4<float>(xr + i, v);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) ss += v[j] * v[j];
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = xr[i];
      if (rr) v += Num<TR>::to_float(rr[i]);
      if (in_place) xr[i] = v;
      ss += v * v;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  if (VEC4) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float v[4], w[4];
      load4<float>(xr + i, v);
      if (rr && !in_place) {
        float a[4];
        load4<TR>(rr + i, a);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += a[j];
      }
      load4<float>(weight + i, w);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = v[j] * inv * w[j];
      store4<TO>(o + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = xr[i];
      if (rr && !in_place) v += Num<TR>::to_float(rr[i]);
      o[i] = Num<TO>::from_float(v * inv * weight[i]);
    }
  }
}

// The same for rows that fit the block's registers (H a multiple of 4, at most blockDim * 4 * NV):
// each thread keeps its NV groups of four elements between the two visits, so a row is read from
// memory once and every load of a row is in flight together.
template <typename TR, typename TO, int NV>
__global__ void add_rmsnorm_regs_kernel(float* __restrict__ x, const TR* __restrict__ residual,
                                        const float* __restrict__ weight, float eps,
                                        TO* __restrict__ out, const int* __restrict__ rows, int H) {
  __shared__ float scratch[32];
  pdl_trigger();
  float w[NV][4];
#pragma unroll
  for (int k = 0; k < NV; ++k) {  // the weights are no result of the kernel before this one
    const int i = (k * blockDim.x + threadIdx.x) * 4;
    if (i < H) load4<float>(weight + i, w[k]);
  }
  pdl_wait();
  const int r = blockIdx.x;
  const int src_row = rows ? rows[r] : r;
  float* xr = x + (size_t)src_row * H;
  const TR* rr = residual ? residual + (size_t)src_row * H : nullptr;
  const bool in_place = (rows == nullptr) && (rr != nullptr);
  TO* o = out + (size_t)r * H;
  float v[NV][4];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (k * blockDim.x + threadIdx.x) * 4;
    if (i < H) load4<float>(xr + i, v[k]);
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (k * blockDim.x + threadIdx.x) * 4;
    if (i < H) {
      if (rr) {
        float a[4];
        load4<TR>(rr + i, a);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[k][j] += a[j];
        if (in_place) store4<float>(xr + i, v[k]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) ss += v[k][j] * v[k][j];
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (k * blockDim.x + threadIdx.x) * 4;
    if (i < H) {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[k][j] = v[k][j] * inv * w[k][j];
      store4<TO>(o + i, v[k]);
    }
  }
}

// ------------------------------------------------------------------------------------ rope + kv write
// One block per token. Work items are (head, pair) with pair < D/2; heads 0..nq-1 are queries,
// nq..nq+nk-1 keys, then values. Queries and keys are rotated:
//   x1' = x1 cos - x2 sin,  x2' = x2 cos + x1 sin   (x1 = first half of the head, x2 = second half)
// (src/llmserve/models/layers.py:82-90). Keys and values go to
// pages[page][kv_head][offset][:] with page = block_table[seq][pos / page_tokens].
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int nq, int nk, int D,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ token_seq,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     const int* __restrict__ block_tables, int table_stride,
                                     int page_tokens, int page_shift) {
  const int t = blockIdx.x;
  const int half = D >> 1;
  const int pos = positions[t];
  T* row = qkv + (size_t)t * (nq + 2 * nk) * D;
  size_t page_base = 0;
  if (k_pages) {
    int pi, off;
    page_of(pos, page_tokens, page_shift, pi, off);
    const int page = block_tables[(size_t)token_seq[t] * table_stride + pi];
    page_base = ((size_t)page * nk * page_tokens + off) * D;  // + kv_head * page_tokens * D
  }
  const float* c = cos_t ? cos_t + (size_t)pos * half : nullptr;
  const float* s = sin_t ? sin_t + (size_t)pos * half : nullptr;
  const int n_rot = (nq + nk) * half;
  const int n_items = n_rot + (k_pages ? nk * half : 0);
  for (int it = threadIdx.x; it < n_items; it += blockDim.x) {
    const int head = it / half, i = it - head * half;
    T* h = row + (size_t)head * D;
    float x1 = Num<T>::to_float(h[i]), x2 = Num<T>::to_float(h[i + half]);
    if (head < nq + nk && c) {
      const float cv = c[i], sv = s[i];
      const float y1 = x1 * cv - x2 * sv;
      const float y2 = x2 * cv + x1 * sv;
      x1 = y1;
      x2 = y2;
    }
    const T o1 = Num<T>::from_float(x1), o2 = Num<T>::from_float(x2);
    if (head < nq) {
      h[i] = o1;
      h[i + half] = o2;
    } else if (k_pages) {
      const bool is_k = head < nq + nk;
      const int kvh = is_k ? head - nq : head - nq - nk;
      T* dst = (is_k ? k_pages : v_pages) + page_base + (size_t)kvh * page_tokens * D;
      dst[i] = o1;
      dst[i + half] = o2;
    }
  }
}

// Same work, 16 bytes at a time: an item is (head, chunk) where the chunk covers kVec elements of
// the first half of the head and the matching kVec elements of the second half. Needs D/2 to be a
// multiple of kVec.
// TIn is the type of the fused projection (T itself, or float when the matrix product left float32
// sums); q_out receives the rotated queries as T (it may alias qkv when TIn == T).
template <typename TIn, typename T>
__global__ void rope_kv_write_vec_kernel(const TIn* qkv, T* q_out,
                                         int nq, int nk, int D,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ token_seq,
                                         const float* __restrict__ cos_t,
                                         const float* __restrict__ sin_t, T* __restrict__ k_pages,
                                         T* __restrict__ v_pages,
                                         const int* __restrict__ block_tables, int table_stride,
                                         int page_tokens, int page_shift) {
  // elements per item and half: a 16-byte vector when both sides are bfloat16 (D is a multiple of
  // 16 there, so a half holds whole vectors), four otherwise
  constexpr int V = (std::is_same<TIn, bf16>::value && std::is_same<T, bf16>::value) ? 8 : 4;
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int half = D >> 1, chunks = half / V;
  const int pos = positions[t];
  const TIn* row = qkv + (size_t)t * (nq + 2 * nk) * D;
  T* qrow = q_out + (size_t)t * (std::is_same<TIn, T>::value ? (nq + 2 * nk) : nq) * D;
  size_t page_base = 0;
  if (k_pages) {
    int pi, off;
    page_of(pos, page_tokens, page_shift, pi, off);
    const int page = block_tables[(size_t)token_seq[t] * table_stride + pi];
    page_base = ((size_t)page * nk * page_tokens + off) * D;
  }
  const float* c = cos_t ? cos_t + (size_t)pos * half : nullptr;
  const float* s = sin_t ? sin_t + (size_t)pos * half : nullptr;
  // fixed-point sums are cleared by reading them, so the value heads are visited even when this
  // layer writes no pages
  const int n_items = ((nq + nk) + ((k_pages || std::is_same<TIn, fixed64>::value) ? nk : 0)) * chunks;
  for (int it = blockIdx.y * blockDim.x + threadIdx.x; it < n_items; it += gridDim.y * blockDim.x) {
    const int head = it / chunks, i = (it - head * chunks) * V;
    const TIn* h = row + (size_t)head * D;
    float a[V], b[V];
    loadv<TIn, V>(h + i, a);
    loadv<TIn, V>(h + i + half, b);
    if (head < nq + nk && c) {
      float cv[V], sv[V];
      loadv<float, V>(c + i, cv);
      loadv<float, V>(s + i, sv);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float x1 = a[e], x2 = b[e];
        a[e] = x1 * cv[e] - x2 * sv[e];
        b[e] = x2 * cv[e] + x1 * sv[e];
      }
    }
    if (head < nq) {
      T* dst = qrow + (size_t)head * D;
      storev<T, V>(dst + i, a);
      storev<T, V>(dst + i + half, b);
    } else if (k_pages) {
      const bool is_k = head < nq + nk;
      const int kvh = is_k ? head - nq : head - nq - nk;
      T* dst = (is_k ? k_pages : v_pages) + page_base + (size_t)kvh * page_tokens * D;
      storev<T, V>(dst + i, a);
      storev<T, V>(dst + i + half, b);
    }
  }
}

// ------------------------------------------------------------------------------------ silu * up
// silu(a) * u. A bfloat16 result keeps 8 bits of mantissa, so the fast exponential and division
// (relative error near 1e-6) give the same stored value as the exact ones; float32 results use
// the exact ones.
template <typename T>
__device__ __forceinline__ float silu_times(float a, float u) {
  if constexpr (std::is_same<T, bf16>::value) return __fdividef(a, 1.f + __expf(-a)) * u;
  else return a / (1.f + expf(-a)) * u;
}
template <typename TIn, typename T>
__global__ void silu_mul_kernel(const TIn* __restrict__ gu, T* __restrict__ out, int I) {
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  const TIn* g = gu + t * 2 * I;
  const TIn* u = g + I;
  T* o = out + t * I;
  if (I % 4 == 0) {
    for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4; i < I; i += gridDim.y * blockDim.x * 4) {
      float gv[4], uv[4];
      load4<TIn>(g + i, gv);
      load4<TIn>(u + i, uv);
#pragma unroll
      for (int j = 0; j < 4; ++j) gv[j] = silu_times<T>(gv[j], uv[j]);
      store4<T>(o + i, gv);
    }
  } else {
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < I; i += gridDim.y * blockDim.x) {
      o[i] = Num<T>::from_float(silu_times<T>(Num<TIn>::to_float(g[i]), Num<TIn>::to_float(u[i])));
    }
  }
}

// The same for input and output of one type and I a multiple of a 16-byte vector: the [T, I]
// outputs are one flat list of vectors, one per thread. (Measured at 2048 x 8192 bfloat16: one
// vector per thread 15.6 us, two 19.0, four 28.8; the bytes alone take 15.1.)
template <typename T>
__global__ void silu_mul_wide_kernel(const T* __restrict__ gu, T* __restrict__ out, int I,
                                     unsigned total) {
  constexpr int V = Num<T>::kVec;
  pdl_trigger();
  pdl_wait();
  const unsigned idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const unsigned per_row = (unsigned)I / V;
  const unsigned t = idx / per_row, c = idx - t * per_row;
  const T* gp = gu + (size_t)t * 2 * I + (size_t)c * V;
  const Vec16<T> g = load16(gp), u = load16(gp + I);
  Vec16<T> o;
#pragma unroll
  for (int j = 0; j < V; ++j)
    o.v[j] = Num<T>::from_float(silu_times<T>(Num<T>::to_float(g.v[j]), Num<T>::to_float(u.v[j])));
  store16(out + (size_t)t * I + (size_t)c * V, o);
}

// ------------------------------------------------------------------------------------ fixed-point sums
// out[i] (+)= value of acc[i]; acc[i] = 0. VEC4: four elements per thread (n a multiple of 4).
template <typename T, bool VEC4>
__global__ void fixed_to_float_kernel(fixed64* __restrict__ acc, T* __restrict__ out, int add, long long n) {
  pdl_trigger();
  pdl_wait();
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * (VEC4 ? 4 : 1);
  if (i >= n) return;
  if (VEC4) {
    float v[4];
    load4<fixed64>(acc + i, v);  // clears what it reads
    if (add) {
      float o[4];
      load4<T>(out + i, o);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] += o[j];
    }
    store4<T>(out + i, v);
  } else {
    float v = fixed_to_float(acc[i]);
    acc[i] = 0;
    if (add) v += Num<T>::to_float(out[i]);
    out[i] = Num<T>::from_float(v);
  }
}

static int shift_of(int n) {
  if (n <= 0 || (n & (n - 1))) return -1;
  int s = 0;
  while ((1 << s) < n) ++s;
  return s;
}

}  // namespace lse

using namespace lse;

#define LSE_CHECK_LAUNCH() (cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED)

extern "C" int lse_embedding(const int* ids, const void* table, int table_dtype, float* out, int T,
                             int H, cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  const int threads = H >= 2048 ? 256 : 128;
  if (table_dtype == LSE_F32)
    launch(embedding_kernel<float>, T, threads, 0, stream, ids, (const float*)table, out, H);
  else if (table_dtype == LSE_BF16)
    launch(embedding_kernel<bf16>, T, threads, 0, stream, ids, (const bf16*)table, out, H);
  else
    return LSE_BAD_ARGUMENT;
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_add_rmsnorm(float* x, const void* residual, int residual_dtype,
                               const float* weight, float eps, void* out, int out_dtype,
                               const int* rows, int T, int H, cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  // Rows of up to 16384 elements: 16 elements per thread, held in registers, so that many rows
  // are resident on an SM together (2048 rows of 2048: 4.3 us; with 8 elements per thread 4.7, with
  // 4 elements 5.8). Longer rows: the kernel that visits the row twice.
  const bool regs = H % 4 == 0 && H <= 16384;
  const int threads = regs ? ((H + 15) / 16 + 31) / 32 * 32 : 1024;
#define LSE_NORM(TR, TO)                                                      \
  do {                                                                        \
    if (regs)                                                                 \
      launch(add_rmsnorm_regs_kernel<TR, TO, 4>, T, threads, 0, stream,       \
             x, (const TR*)residual, weight, eps, (TO*)out, rows, H);         \
    else if (H % 4 == 0)                                                      \
      launch(add_rmsnorm_kernel<TR, TO, true>, T, threads, 0, stream,         \
             x, (const TR*)residual, weight, eps, (TO*)out, rows, H);         \
    else                                                                      \
      launch(add_rmsnorm_kernel<TR, TO, false>, T, threads, 0, stream,        \
             x, (const TR*)residual, weight, eps, (TO*)out, rows, H);         \
  } while (0)
  if (residual_dtype == LSE_F32 && out_dtype == LSE_F32) LSE_NORM(float, float);
  else if (residual_dtype == LSE_F32 && out_dtype == LSE_BF16) LSE_NORM(float, bf16);
  else if (residual_dtype == LSE_BF16 && out_dtype == LSE_BF16) LSE_NORM(bf16, bf16);
  else if (residual_dtype == LSE_BF16 && out_dtype == LSE_F32) LSE_NORM(bf16, float);
  else if (residual_dtype == LSE_FIXED64 && out_dtype == LSE_BF16) {
    // sums that are cleared as they are read: every row once, four elements at a time
    if (!residual || rows || H % 4) return LSE_BAD_ARGUMENT;
    if (regs)
      launch(add_rmsnorm_regs_kernel<fixed64, bf16, 4>, T, threads, 0, stream, x,
             (const fixed64*)residual, weight, eps, (bf16*)out, rows, H);
    else
      launch(add_rmsnorm_kernel<fixed64, bf16, true>, T, threads, 0, stream, x,
             (const fixed64*)residual, weight, eps, (bf16*)out, rows, H);
  }
  else return LSE_BAD_ARGUMENT;
#undef LSE_NORM
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_rope_kv_write(const void* qkv, int in_dtype, void* q_out, int dtype, int T, int nq,
                                 int nk, int D, const int* positions, const int* token_seq,
                                 const float* cos, const float* sin, void* k_pages, void* v_pages,
                                 const int* block_tables, int table_stride, int page_tokens,
                                 cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  if (D % 2 || page_tokens <= 0 || (cos == nullptr) != (sin == nullptr) ||
      (k_pages == nullptr) != (v_pages == nullptr))
    return LSE_BAD_ARGUMENT;
  if (in_dtype != dtype && in_dtype != LSE_F32 && in_dtype != LSE_FIXED64) return LSE_BAD_ARGUMENT;
  if (in_dtype == LSE_FIXED64 && (dtype != LSE_BF16 || (D / 2) % 4)) return LSE_BAD_ARGUMENT;
  if (in_dtype == dtype && q_out != qkv) return LSE_BAD_ARGUMENT;  // same type: rotated in place
  const int ps = shift_of(page_tokens);
  const bool wide = in_dtype == LSE_BF16 && dtype == LSE_BF16 && (D / 2) % 8 == 0;  // the kernel's V = 8
  const bool vec = (D / 2) % 4 == 0 && (wide || !(in_dtype == LSE_BF16 && dtype == LSE_BF16));
#define LSE_ROPE_VEC(TIn, T)                                                                      \
  launch(rope_kv_write_vec_kernel<TIn, T>, vgrid, 128, 0, stream,                                 \
         (const TIn*)qkv, (T*)q_out, nq, nk, D, positions, token_seq, cos, sin, (T*)k_pages,      \
         (T*)v_pages, block_tables, table_stride, page_tokens, ps)
  // one thread per item (head, chunk of V + V elements): every load of a token is in flight at once
  const int items = (nq + 2 * nk) * (D / (wide ? 16 : 8));
  const dim3 vgrid(T, (items + 127) / 128 > 64 ? 64 : (items + 127) / 128);
  if (vec && in_dtype == LSE_F32 && dtype == LSE_F32) LSE_ROPE_VEC(float, float);
  else if (vec && in_dtype == LSE_BF16 && dtype == LSE_BF16) LSE_ROPE_VEC(bf16, bf16);
  else if (vec && in_dtype == LSE_F32 && dtype == LSE_BF16) LSE_ROPE_VEC(float, bf16);
  else if (in_dtype == LSE_FIXED64) LSE_ROPE_VEC(fixed64, bf16);
  else if (in_dtype != dtype) return LSE_BAD_ARGUMENT;
  else if (dtype == LSE_F32)
    rope_kv_write_kernel<float><<<T, 256, 0, stream>>>(
        (float*)q_out, nq, nk, D, positions, token_seq, cos, sin, (float*)k_pages, (float*)v_pages,
        block_tables, table_stride, page_tokens, ps);
  else if (dtype == LSE_BF16)
    rope_kv_write_kernel<bf16><<<T, 256, 0, stream>>>(
        (bf16*)q_out, nq, nk, D, positions, token_seq, cos, sin, (bf16*)k_pages, (bf16*)v_pages,
        block_tables, table_stride, page_tokens, ps);
  else
    return LSE_BAD_ARGUMENT;
#undef LSE_ROPE_VEC
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_silu_mul(const void* gu, int in_dtype, void* out, int dtype, int T, int I,
                            cudaStream_t stream) {
  if (T <= 0 || I <= 0) return LSE_OK;
  const int threads = 256;
  const int vec = in_dtype == LSE_BF16 ? 8 : 4;
  if (in_dtype == dtype && I % vec == 0 && (size_t)T * (I / vec) < (1ull << 31) &&
      (reinterpret_cast<uintptr_t>(gu) % 16) == 0 && (reinterpret_cast<uintptr_t>(out) % 16) == 0) {
    const unsigned total = (unsigned)((size_t)T * (I / vec));
    const unsigned blocks = (total + threads - 1) / threads;
    if (dtype == LSE_F32)
      launch(silu_mul_wide_kernel<float>, blocks, threads, 0, stream, (const float*)gu, (float*)out, I, total);
    else
      launch(silu_mul_wide_kernel<bf16>, blocks, threads, 0, stream, (const bf16*)gu, (bf16*)out, I, total);
    return LSE_CHECK_LAUNCH();
  }
  const int per_block = threads * 4;
  dim3 grid(T, min((I + per_block - 1) / per_block, 65535));
  if (in_dtype == LSE_F32 && dtype == LSE_F32)
    launch(silu_mul_kernel<float, float>, grid, threads, 0, stream, (const float*)gu, (float*)out, I);
  else if (in_dtype == LSE_BF16 && dtype == LSE_BF16)
    launch(silu_mul_kernel<bf16, bf16>, grid, threads, 0, stream, (const bf16*)gu, (bf16*)out, I);
  else if (in_dtype == LSE_F32 && dtype == LSE_BF16)
    launch(silu_mul_kernel<float, bf16>, grid, threads, 0, stream, (const float*)gu, (bf16*)out, I);
  else if (in_dtype == LSE_FIXED64 && dtype == LSE_BF16 && I % 4 == 0)
    launch(silu_mul_kernel<fixed64, bf16>, grid, threads, 0, stream, (const fixed64*)gu, (bf16*)out, I);
  else
    return LSE_BAD_ARGUMENT;
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_fixed_to_float(void* acc, void* out, int out_dtype, int add, long long n,
                                  cudaStream_t stream) {
  if (n <= 0) return LSE_OK;
  if (add && out_dtype != LSE_F32) return LSE_BAD_ARGUMENT;
  const int threads = 128;
  const bool vec = n % 4 == 0 && reinterpret_cast<uintptr_t>(acc) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 16 == 0;
  const long long items = vec ? n / 4 : n;
  const long long blocks = (items + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return LSE_BAD_ARGUMENT;
#define LSE_CONVERT(T, V) \
  launch(fixed_to_float_kernel<T, V>, (unsigned)blocks, threads, 0, stream, (fixed64*)acc, (T*)out, add, n)
  if (out_dtype == LSE_F32) {
    if (vec) LSE_CONVERT(float, true);
    else LSE_CONVERT(float, false);
  } else if (out_dtype == LSE_BF16) {
    if (vec) LSE_CONVERT(bf16, true);
    else LSE_CONVERT(bf16, false);
  } else {
    return LSE_BAD_ARGUMENT;
  }
#undef LSE_CONVERT
  return LSE_CHECK_LAUNCH();
}
