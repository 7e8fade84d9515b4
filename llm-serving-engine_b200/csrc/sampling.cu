// Token sampling on the device (src/llmserve/sampling.py:123-190): greedy argmax, or temperature
// -> top-k / top-p / min-p cut -> exponential-race draw. Randomness comes from Philox4x32-10 keyed
// by the request's seed with the counter (vocabulary index / 4, draw number), so a request's
// samples do not depend on what else is in the batch.
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace lse {

constexpr int SAMPLE_THREADS = 1024;

// order-preserving map float -> uint32
__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ ArgMax block_argmax(ArgMax a, ArgMax* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b = {__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
    a = better(a, b);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = a;
  __syncthreads();
  ArgMax r = lane < nw ? scratch[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b = {__shfl_xor_sync(0xffffffffu, r.v, o), __shfl_xor_sync(0xffffffffu, r.i, o)};
    r = better(r, b);
  }
  return r;
}
__device__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  return warp_max(lane < nw ? scratch[lane] : -INFINITY);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const uint64_t* __restrict__ seed,
              const int* __restrict__ draw, int* __restrict__ out) {
  __shared__ float fs[32];
  __shared__ ArgMax as[32];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  const float temp = temperature[r];
  if (temp < 1e-5f) {
    ArgMax a = {-INFINITY, 0x7fffffff};
    if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      // four loads of a thread in flight at once: the row is read once and nothing else hides
      // the latency of memory
      const int step = blockDim.x * 4;
      for (int i0 = threadIdx.x * 4; i0 < V; i0 += 4 * step) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          v[u] = i0 + u * step < V ? *reinterpret_cast<const float4*>(row + i0 + u * step)
                                   : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * step;
          a = better(a, ArgMax{v[u].x, i});
          a = better(a, ArgMax{v[u].y, i + 1});
          a = better(a, ArgMax{v[u].z, i + 2});
          a = better(a, ArgMax{v[u].w, i + 3});
        }
      }
    } else {
      for (int i = threadIdx.x; i < V; i += blockDim.x) a = better(a, ArgMax{row[i], i});
    }
    a = block_argmax(a, as);
    if (threadIdx.x == 0) out[r] = a.i;
    return;
  }
  const float inv_t = 1.f / temp;
  float zmax = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) zmax = fmaxf(zmax, row[i] * inv_t);
  zmax = block_max(zmax, fs);
  const int k = top_k[r];
  const float p = top_p[r], mp = min_p[r];
  uint32_t cut = 0;  // keep elements whose key is >= cut
  if ((k > 0 && k < V) || p < 1.f) {
    float Z = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) Z += expf(row[i] * inv_t - zmax);
    Z = block_sum(Z, fs);
    const float mass_limit = p * Z;
    const int count_limit = (k > 0 && k < V) ? k : V + 1;
    // smallest key u such that a value with key u would be kept:
    //   (number of elements strictly above it) < k  and  (their mass) < top_p
    uint32_t lo = 0, hi = float_key(zmax);  // the maximum is always kept
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1);
      const float val = key_float(mid);
      float mass = 0.f, cnt = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float z = row[i] * inv_t;
        if (z > val) {
          mass += expf(z - zmax);
          cnt += 1.f;
        }
      }
      mass = block_sum(mass, fs);
      cnt = block_sum(cnt, fs);
      if (cnt < (float)count_limit && mass < mass_limit) hi = mid; else lo = mid + 1;
    }
    cut = lo;
  }
  const float min_z = mp > 0.f ? zmax + logf(mp) : -INFINITY;
  const uint64_t sd = seed[r];
  const uint32_t k0 = (uint32_t)sd, k1 = (uint32_t)(sd >> 32);
  const uint32_t dr = (uint32_t)draw[r];
  ArgMax best = {-INFINITY, 0x7fffffff};
  const int quads = (V + 3) >> 2;
  for (int qd = threadIdx.x; qd < quads; qd += blockDim.x) {
    uint32_t c[4] = {(uint32_t)qd, dr, 0u, 0u};
    philox4x32_10(c, k0, k1);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = qd * 4 + e;
      if (i >= V) break;
      const float z = row[i] * inv_t;
      if (float_key(z) < cut || z < min_z) continue;
      const float u = ((float)(c[e] >> 8) + 0.5f) * (1.f / 16777216.f);  // (0, 1)
      // argmax of p_i / E_i with E_i = -log(u): compare log p_i - log E_i
      best = better(best, ArgMax{z - zmax - logf(-logf(u)), i});
    }
  }
  best = block_argmax(best, as);
  if (threadIdx.x == 0) out[r] = best.i;
}

__global__ void logsumexp_kernel(const float* __restrict__ logits, int V, float* __restrict__ out) {
  __shared__ float fs[32];
  const float* row = logits + (size_t)blockIdx.x * V;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
  mx = block_max(mx, fs);
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) s += expf(row[i] - mx);
  s = block_sum(s, fs);
  if (threadIdx.x == 0) out[blockIdx.x] = mx + logf(s);
}

// Penalties of src/llmserve/sampling.py:80-96 on unique (row, token) pairs: count = how often the
// token was generated so far (0 if it only occurs in the prompt).
__global__ void penalties_kernel(float* __restrict__ logits, int V, const int* __restrict__ row,
                                 const int* __restrict__ token, const int* __restrict__ count,
                                 const float* __restrict__ presence,
                                 const float* __restrict__ frequency,
                                 const float* __restrict__ repetition, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float* p = logits + (size_t)row[i] * V + token[i];
  float v = *p;
  const int c = count[i];
  if (c > 0) v -= frequency[i] * (float)c + presence[i];
  const float rp = repetition[i];
  if (rp != 1.f) v = v > 0.f ? v / rp : v * rp;
  *p = v;
}

__global__ void ban_kernel(float* __restrict__ logits, int V, const int* __restrict__ row,
                           const int* __restrict__ token, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) logits[(size_t)row[i] * V + token[i]] = -INFINITY;
}

}  // namespace lse

using namespace lse;

extern "C" int lse_sample(const float* logits, int R, int V, const float* temperature,
                          const int* top_k, const float* top_p, const float* min_p,
                          const uint64_t* seed, const int* draw, int* out_tokens,
                          cudaStream_t stream) {
  if (R <= 0) return LSE_OK;
  if (V <= 0) return LSE_BAD_ARGUMENT;
  launch(sample_kernel, R, SAMPLE_THREADS, 0, stream, logits, V, temperature, top_k, top_p, min_p,
         seed, draw, out_tokens);
  return cudaGetLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}

extern "C" int lse_logsumexp(const float* logits, int R, int V, float* out, cudaStream_t stream) {
  if (R <= 0) return LSE_OK;
  logsumexp_kernel<<<R, 512, 0, stream>>>(logits, V, out);
  return cudaGetLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}

extern "C" int lse_apply_penalties(float* logits, int V, const int* row, const int* token,
                                   const int* count, const float* presence, const float* frequency,
                                   const float* repetition, int n, cudaStream_t stream) {
  if (n <= 0) return LSE_OK;
  penalties_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, V, row, token, count, presence,
                                                        frequency, repetition, n);
  return cudaGetLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}

extern "C" int lse_ban_tokens(float* logits, int V, const int* row, const int* token, int n,
                              cudaStream_t stream) {
  if (n <= 0) return LSE_OK;
  ban_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, V, row, token, n);
  return cudaGetLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}
