// Memory-bound kernels around the matrix products: embedding gather, residual add + RMS norm,
// rotary positions + key/value page write, SiLU gate. All arithmetic is float32; values are
// rounded once when they are stored in the compute dtype.
//
// What each computes follows the reference's fused CPU ops
// (src/llmserve/kernels/csrc/fused_ops.cpp:39-125) and src/llmserve/attention.py:221-228.
#include "common.cuh"
#include "kernels.h"

namespace lse {

// ------------------------------------------------------------------------------------ embedding
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int H) {
  const int t = blockIdx.x;
  const T* src = table + (size_t)ids[t] * H;
  float* dst = out + (size_t)t * H;
  constexpr int V = Num<T>::kVec;
  if (H % V == 0) {
    for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
      Vec16<T> v = load16(src + i);
#pragma unroll
      for (int j = 0; j < V; ++j) dst[i + j] = Num<T>::to_float(v.v[j]);
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

// VEC4: H is a multiple of 4, so rows are read and written four elements at a time.
template <typename TR, typename TO, bool VEC4>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TR* __restrict__ residual,
                                   const float* __restrict__ weight, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows, int H) {
  __shared__ float scratch[32];
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
template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, int nq, int nk, int D,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ token_seq,
                                         const float* __restrict__ cos_t,
                                         const float* __restrict__ sin_t, T* __restrict__ k_pages,
                                         T* __restrict__ v_pages,
                                         const int* __restrict__ block_tables, int table_stride,
                                         int page_tokens, int page_shift) {
  constexpr int V = Num<T>::kVec;
  const int t = blockIdx.x;
  const int half = D >> 1, chunks = half / V;
  const int pos = positions[t];
  T* row = qkv + (size_t)t * (nq + 2 * nk) * D;
  size_t page_base = 0;
  if (k_pages) {
    int pi, off;
    page_of(pos, page_tokens, page_shift, pi, off);
    const int page = block_tables[(size_t)token_seq[t] * table_stride + pi];
    page_base = ((size_t)page * nk * page_tokens + off) * D;
  }
  const float* c = cos_t ? cos_t + (size_t)pos * half : nullptr;
  const float* s = sin_t ? sin_t + (size_t)pos * half : nullptr;
  const int n_items = ((nq + nk) + (k_pages ? nk : 0)) * chunks;
  for (int it = threadIdx.x; it < n_items; it += blockDim.x) {
    const int head = it / chunks, i = (it - head * chunks) * V;
    T* h = row + (size_t)head * D;
    Vec16<T> a = load16(h + i), b = load16(h + i + half);
    if (head < nq + nk && c) {
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float x1 = Num<T>::to_float(a.v[e]), x2 = Num<T>::to_float(b.v[e]);
        const float cv = c[i + e], sv = s[i + e];
        a.v[e] = Num<T>::from_float(x1 * cv - x2 * sv);
        b.v[e] = Num<T>::from_float(x2 * cv + x1 * sv);
      }
    }
    if (head < nq) {
      store16(h + i, a);
      store16(h + i + half, b);
    } else if (k_pages) {
      const bool is_k = head < nq + nk;
      const int kvh = is_k ? head - nq : head - nq - nk;
      T* dst = (is_k ? k_pages : v_pages) + page_base + (size_t)kvh * page_tokens * D;
      store16(dst + i, a);
      store16(dst + i + half, b);
    }
  }
}

// ------------------------------------------------------------------------------------ silu * up
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I) {
  const size_t t = blockIdx.x;
  const T* g = gu + t * 2 * I;
  const T* u = g + I;
  T* o = out + t * I;
  constexpr int V = Num<T>::kVec;
  if (I % V == 0) {
    for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * V; i < I; i += gridDim.y * blockDim.x * V) {
      Vec16<T> gv = load16(g + i), uv = load16(u + i), ov;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float a = Num<T>::to_float(gv.v[j]);
        ov.v[j] = Num<T>::from_float(a / (1.f + expf(-a)) * Num<T>::to_float(uv.v[j]));
      }
      store16(o + i, ov);
    }
  } else {
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < I; i += gridDim.y * blockDim.x) {
      const float a = Num<T>::to_float(g[i]);
      o[i] = Num<T>::from_float(a / (1.f + expf(-a)) * Num<T>::to_float(u[i]));
    }
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

#define LSE_CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED)

extern "C" int lse_embedding(const int* ids, const void* table, int table_dtype, float* out, int T,
                             int H, cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  const int threads = H >= 2048 ? 256 : 128;
  if (table_dtype == LSE_F32)
    embedding_kernel<float><<<T, threads, 0, stream>>>(ids, (const float*)table, out, H);
  else if (table_dtype == LSE_BF16)
    embedding_kernel<bf16><<<T, threads, 0, stream>>>(ids, (const bf16*)table, out, H);
  else
    return LSE_BAD_ARGUMENT;
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_add_rmsnorm(float* x, const void* residual, int residual_dtype,
                               const float* weight, float eps, void* out, int out_dtype,
                               const int* rows, int T, int H, cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
#define LSE_NORM(TR, TO)                                                      \
  do {                                                                        \
    if (H % 4 == 0)                                                           \
      add_rmsnorm_kernel<TR, TO, true><<<T, threads, 0, stream>>>(            \
          x, (const TR*)residual, weight, eps, (TO*)out, rows, H);            \
    else                                                                      \
      add_rmsnorm_kernel<TR, TO, false><<<T, threads, 0, stream>>>(           \
          x, (const TR*)residual, weight, eps, (TO*)out, rows, H);            \
  } while (0)
  if (residual_dtype == LSE_F32 && out_dtype == LSE_F32) LSE_NORM(float, float);
  else if (residual_dtype == LSE_F32 && out_dtype == LSE_BF16) LSE_NORM(float, bf16);
  else if (residual_dtype == LSE_BF16 && out_dtype == LSE_BF16) LSE_NORM(bf16, bf16);
  else if (residual_dtype == LSE_BF16 && out_dtype == LSE_F32) LSE_NORM(bf16, float);
  else return LSE_BAD_ARGUMENT;
#undef LSE_NORM
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_rope_kv_write(void* qkv, int dtype, int T, int nq, int nk, int D,
                                 const int* positions, const int* token_seq, const float* cos,
                                 const float* sin, void* k_pages, void* v_pages,
                                 const int* block_tables, int table_stride, int page_tokens,
                                 cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  if (D % 2 || page_tokens <= 0 || (cos == nullptr) != (sin == nullptr) ||
      (k_pages == nullptr) != (v_pages == nullptr))
    return LSE_BAD_ARGUMENT;
  const int ps = shift_of(page_tokens);
  const bool vec = (D / 2) % (dtype == LSE_F32 ? 4 : 8) == 0;
  if (vec && dtype == LSE_F32)
    rope_kv_write_vec_kernel<float><<<T, 256, 0, stream>>>(
        (float*)qkv, nq, nk, D, positions, token_seq, cos, sin, (float*)k_pages, (float*)v_pages,
        block_tables, table_stride, page_tokens, ps);
  else if (vec && dtype == LSE_BF16)
    rope_kv_write_vec_kernel<bf16><<<T, 256, 0, stream>>>(
        (bf16*)qkv, nq, nk, D, positions, token_seq, cos, sin, (bf16*)k_pages, (bf16*)v_pages,
        block_tables, table_stride, page_tokens, ps);
  else if (dtype == LSE_F32)
    rope_kv_write_kernel<float><<<T, 256, 0, stream>>>(
        (float*)qkv, nq, nk, D, positions, token_seq, cos, sin, (float*)k_pages, (float*)v_pages,
        block_tables, table_stride, page_tokens, ps);
  else if (dtype == LSE_BF16)
    rope_kv_write_kernel<bf16><<<T, 256, 0, stream>>>(
        (bf16*)qkv, nq, nk, D, positions, token_seq, cos, sin, (bf16*)k_pages, (bf16*)v_pages,
        block_tables, table_stride, page_tokens, ps);
  else
    return LSE_BAD_ARGUMENT;
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_silu_mul(const void* gu, void* out, int dtype, int T, int I,
                            cudaStream_t stream) {
  if (T <= 0 || I <= 0) return LSE_OK;
  const int threads = 256;
  const int per_block = threads * (dtype == LSE_F32 ? 4 : 8);
  dim3 grid(T, min((I + per_block - 1) / per_block, 65535));
  if (dtype == LSE_F32)
    silu_mul_kernel<float><<<grid, threads, 0, stream>>>((const float*)gu, (float*)out, I);
  else if (dtype == LSE_BF16)
    silu_mul_kernel<bf16><<<grid, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, I);
  else
    return LSE_BAD_ARGUMENT;
  return LSE_CHECK_LAUNCH();
}
