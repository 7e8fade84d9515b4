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

// ---- rows without a cut: several blocks per row -----------------------------------------------
// Rows with a temperature but neither top-k, top-p nor min-p need one pass over the row and
// nothing that all of it has to agree on first: the winner is the largest z_i - log(-log u_i),
// and making the random numbers is most of the work. SAMPLE_CHUNKS blocks take a piece of the
// row each; the block that finishes last picks the best of their results (ties: the lowest index,
// as everywhere). Greedy rows stay with one block per row: reading the row once is too little
// work to share (4.5 us alone against 4.9 shared at 8 rows, 4.6 against 7.9 at 64).
constexpr int SAMPLE_CHUNKS = 8;
constexpr int PAR_THREADS = 256;

__device__ __forceinline__ bool row_is_parallel(float temp, int k, float p, float mp, int V) {
  return temp >= 1e-5f && !((k > 0 && k < V) || p < 1.f) && !(mp > 0.f);
}

__global__ void __launch_bounds__(PAR_THREADS)
sample_parallel_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                       const int* __restrict__ top_k, const float* __restrict__ top_p,
                       const float* __restrict__ min_p, const uint64_t* __restrict__ seed,
                       const int* __restrict__ draw, int* __restrict__ out,
                       int* __restrict__ scratch, int scratch_rows) {
  // scratch (made for scratch_rows rows): one counter per row, zero between launches, then per
  // row SAMPLE_CHUNKS (value bits, index) pairs. The counters come first so that launches with
  // different numbers of rows find them in the same place.
  __shared__ ArgMax as[32];
  __shared__ int is_last;
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, c = blockIdx.y;
  const float temp = temperature[r];
  if (!row_is_parallel(temp, top_k[r], top_p[r], min_p[r], V)) return;
  const float* row = logits + (size_t)r * V;
  const int quads = (V + 3) >> 2;
  const int per = (quads + SAMPLE_CHUNKS - 1) / SAMPLE_CHUNKS;  // groups of four entries per block
  const int q_lo = c * per, q_hi = min(quads, q_lo + per);
  const bool vec = (V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  const float inv_t = 1.f / temp;
  const uint64_t sd = seed[r];
  const uint32_t k0 = (uint32_t)sd, k1 = (uint32_t)(sd >> 32), dr = (uint32_t)draw[r];
  ArgMax best = {-INFINITY, 0x7fffffff};
  for (int q0 = q_lo + threadIdx.x; q0 < q_hi; q0 += 2 * PAR_THREADS) {
    float v[2][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {  // two loads of a thread in flight
      const int qd = q0 + u * PAR_THREADS;
#pragma unroll
      for (int e = 0; e < 4; ++e) v[u][e] = -INFINITY;
      if (qd < q_hi) {
        if (vec) {
          const float4 t = *reinterpret_cast<const float4*>(row + 4 * qd);
          v[u][0] = t.x; v[u][1] = t.y; v[u][2] = t.z; v[u][3] = t.w;
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (4 * qd + e < V) v[u][e] = row[4 * qd + e];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int qd = q0 + u * PAR_THREADS;
      if (qd >= q_hi) continue;
      uint32_t cn[4] = {(uint32_t)qd, dr, 0u, 0u};
      philox4x32_10(cn, k0, k1);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (4 * qd + e >= V) continue;
        const float u01 = ((float)(cn[e] >> 8) + 0.5f) * (1.f / 16777216.f);
        best = better(best, ArgMax{v[u][e] * inv_t - logf(-logf(u01)), 4 * qd + e});
      }
    }
  }
  best = block_argmax(best, as);
  int* counter = scratch + r;
  int* pairs = scratch + scratch_rows + ((size_t)r * SAMPLE_CHUNKS + c) * 2;
  if (threadIdx.x == 0) {
    pairs[0] = __float_as_int(best.v);
    pairs[1] = best.i;
    __threadfence();
    is_last = atomicAdd(counter, 1) == SAMPLE_CHUNKS - 1;
  }
  __syncthreads();
  if (!is_last || threadIdx.x != 0) return;
  __threadfence();
  ArgMax win = {-INFINITY, 0x7fffffff};
  const int* all = scratch + scratch_rows + (size_t)r * SAMPLE_CHUNKS * 2;
  for (int j = 0; j < SAMPLE_CHUNKS; ++j)
    win = better(win, ArgMax{__int_as_float(__ldcg(all + 2 * j)), __ldcg(all + 2 * j + 1)});
  out[r] = win.i;
  *counter = 0;
}

// ---- the cut of top-k / top-p --------------------------------------------------------------
// With z = logit / temperature and e = exp(z - max z), element i is kept iff fewer than k elements
// lie strictly above it and their mass (sum of e) is below top_p * (sum of all e). The cut is the
// smallest kept value. It is found without sorting and without a pass per bit:
//   1. one pass puts every element into one of HIST_BINS bins of equal width over
//      [max - HIST_RANGE, max] (count and mass per bin; everything below falls into the last bin)
//      and a scan from the top finds the bin that holds the cut;
//   2. if that bin holds few elements (it usually does) they are listed and ranked against each
//      other: the cut is the smallest of them that is kept. Otherwise
//   3. the same scan inside that bin (HIST_BINS sub-bins), then the elements of the sub-bin are
//      listed and the cut is bisected among their values.
// Masses are summed as 64-bit fixed point (40 fractional bits) with integer atomics, so the result
// does not depend on the order of the additions: the same logits give the same cut on every run.
constexpr int HIST_BINS = 2048;
constexpr float HIST_RANGE = 32.f;
constexpr int LIST_CAP = 2048;  // candidates that fit in the shared-memory list
constexpr int KEPT_CAP = 4096;   // survivors of the cut that fit in the shared-memory list
constexpr int SMALL_LIST = 256;  // up to this many candidates are ranked against each other

__device__ __forceinline__ unsigned long long mass_fix(float z, float zmax) {
  return (unsigned long long)(expf(z - zmax) * 1099511627776.f);  // 2^40; z <= zmax
}
__device__ __forceinline__ int bin1_of(float z, float zmax) {
  const float t = (zmax - z) * ((float)HIST_BINS / HIST_RANGE);
  return t >= (float)(HIST_BINS - 1) ? HIST_BINS - 1 : (int)t;  // also for z = -inf
}
__device__ __forceinline__ int bin2_of(float z, float zmax, int b1) {
  const float t = ((zmax - z) * ((float)HIST_BINS / HIST_RANGE) - (float)b1) * (float)HIST_BINS;
  return t <= 0.f ? 0 : (t >= (float)(HIST_BINS - 1) ? HIST_BINS - 1 : (int)t);
}

// Adds a 64-bit value to a 64-bit sum kept as two 32-bit words (low word first) with 32-bit
// shared-memory atomics: the carry out of the low word is added to the high word. Integer sums do
// not depend on the order of the additions.
__device__ __forceinline__ void add_mass(unsigned long long* sum, unsigned long long x) {
  unsigned int* w = reinterpret_cast<unsigned int*>(sum);
  const unsigned int lo = (unsigned int)x, hi = (unsigned int)(x >> 32);
  const unsigned int old = atomicAdd(&w[0], lo);
  const unsigned int carry = (old + lo < old) ? 1u : 0u;
  if (hi + carry) atomicAdd(&w[1], hi + carry);
}

template <typename V>
__device__ __forceinline__ V warp_add(V v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Over the bins filled by the whole block: the lowest (largest index) non-empty bin whose top
// element is still kept, given what lies above all bins (a_cnt, a_mass). Adds the content of the
// bins above it to a_cnt / a_mass. Called by every thread; warp 0 works; result for all.
__device__ int find_cut_bin(const int* cnt, const unsigned long long* mass, int count_limit,
                            unsigned long long mass_limit, int& a_cnt, unsigned long long& a_mass,
                            int* res) {
  __syncthreads();  // the histogram is complete
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    constexpr int PER = HIST_BINS / 32;
    int c = 0;
    unsigned long long m = 0;
#pragma unroll 16
    for (int b = lane * PER; b < (lane + 1) * PER; ++b) {
      c += cnt[b];
      m += mass[b];
    }
    // what lies above this lane's bins
    int pc = c;
    unsigned long long pm = m;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int c2 = __shfl_up_sync(0xffffffffu, pc, o);
      const unsigned long long m2 = __shfl_up_sync(0xffffffffu, pm, o);
      if (lane >= o) {
        pc += c2;
        pm += m2;
      }
    }
    int rc = a_cnt + pc - c;
    unsigned long long rm = a_mass + pm - m;
    int found = -1, fc = 0;
    unsigned long long fm = 0;
#pragma unroll 8
    for (int b = lane * PER; b < (lane + 1) * PER; ++b) {
      if (cnt[b] > 0 && rc < count_limit && rm < mass_limit) {
        found = b;
        fc = rc;
        fm = rm;
      }
      rc += cnt[b];
      rm += mass[b];
    }
    int best = found;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (best < 0) {  // cannot happen (the maximum is always kept); keep the top bin
      if (lane == 0) {
        res[0] = 0;
        res[1] = a_cnt;
        *reinterpret_cast<unsigned long long*>(res + 2) = a_mass;
      }
    } else if (found == best) {
      res[0] = best;
      res[1] = fc;
      *reinterpret_cast<unsigned long long*>(res + 2) = fm;
    }
  }
  __syncthreads();
  a_cnt = res[1];
  a_mass = *reinterpret_cast<const unsigned long long*>(res + 2);
  return res[0];
}

// CACHE: the scaled row is kept in shared memory after the first read (rows of up to about 50 000
// elements); otherwise every pass reads it from global memory again.
template <bool CACHE>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const uint64_t* __restrict__ seed,
              const int* __restrict__ draw, int* __restrict__ out, int parallel_rows) {
  extern __shared__ __align__(16) unsigned char sample_smem[];
  // histogram (counts, masses), later the candidate list (keys, masses); then the cached row
  int* h_cnt = reinterpret_cast<int*>(sample_smem);
  unsigned long long* h_mass = reinterpret_cast<unsigned long long*>(sample_smem + HIST_BINS * 4);
  float* zrow = reinterpret_cast<float*>(sample_smem + HIST_BINS * 12);
  __shared__ float fs[32];
  __shared__ ArgMax as[32];
  __shared__ __align__(8) int res[4];
  __shared__ int list_n;
  __shared__ unsigned long long z_total;
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  const float temp = temperature[r];
  if (parallel_rows && row_is_parallel(temp, top_k[r], top_p[r], min_p[r], V)) return;
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
  auto Z = [&](int i) -> float { return CACHE ? zrow[i] : row[i] * inv_t; };
  float zmax = -INFINITY;
  {
    const int step = blockDim.x;
    for (int i0 = threadIdx.x; i0 < V; i0 += 4 * step) {
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = i0 + u * step < V ? row[i0 + u * step] * inv_t : -INFINITY;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (CACHE && i0 + u * step < V) zrow[i0 + u * step] = v[u];
        zmax = fmaxf(zmax, v[u]);
      }
    }
  }
  zmax = block_max(zmax, fs);  // its barriers also publish the cached row
  const int k = top_k[r];
  const float p = top_p[r], mp = min_p[r];
  uint32_t cut = 0;  // keep elements whose key is >= cut
  if ((k > 0 && k < V) || p < 1.f) {
    const int count_limit = (k > 0 && k < V) ? k : V + 1;
    // ---- level 1
    for (int b = threadIdx.x; b < HIST_BINS; b += blockDim.x) {
      h_cnt[b] = 0;
      h_mass[b] = 0;
    }
    __syncthreads();
    unsigned long long zsum = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float z = Z(i);
      const unsigned long long e = mass_fix(z, zmax);
      const int b = bin1_of(z, zmax);
      atomicAdd(&h_cnt[b], 1);
      if (e) add_mass(&h_mass[b], e);
      zsum += e;
    }
    zsum = warp_add(zsum);
    if (threadIdx.x == 0) z_total = 0;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) atomicAdd(&z_total, zsum);
    __syncthreads();
    unsigned long long mass_limit =
        p < 1.f ? (unsigned long long)((double)fmaxf(p, 0.f) * (double)z_total) : ~0ull;
    if (mass_limit == 0) mass_limit = 1;  // the maximum is always kept
    int a_cnt = 0;
    unsigned long long a_mass = 0;
    const int b1 = find_cut_bin(h_cnt, h_mass, count_limit, mass_limit, a_cnt, a_mass, res);
    // ---- few elements in bin b1 (the usual case): list them and rank them against each other
    if (h_cnt[b1] <= SMALL_LIST) {
      const int n = h_cnt[b1];
      __syncthreads();  // everyone has read the count before the histogram becomes the list
      uint32_t* s_key = reinterpret_cast<uint32_t*>(h_cnt);
      unsigned long long* s_mass = h_mass;
      if (threadIdx.x == 0) {
        list_n = 0;
        res[0] = (int)0xffffffffu;
      }
      __syncthreads();
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float z = Z(i);
        if (bin1_of(z, zmax) == b1) {
          const int at = atomicAdd(&list_n, 1);
          s_key[at] = float_key(z);
          s_mass[at] = mass_fix(z, zmax);
        }
      }
      __syncthreads();
      if (threadIdx.x < n) {
        const uint32_t mine = s_key[threadIdx.x];
        int c = a_cnt;
        unsigned long long m = a_mass;
        for (int j = 0; j < n; ++j)
          if (s_key[j] > mine) {
            c += 1;
            m += s_mass[j];
          }
        if (c < count_limit && m < mass_limit) atomicMin(reinterpret_cast<unsigned int*>(&res[0]), mine);
      }
      __syncthreads();
      cut = (uint32_t)res[0];
    } else {
    // ---- level 2: inside bin b1
    for (int b = threadIdx.x; b < HIST_BINS; b += blockDim.x) {
      h_cnt[b] = 0;
      h_mass[b] = 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float z = Z(i);
      if (bin1_of(z, zmax) == b1) {
        const int b = bin2_of(z, zmax, b1);
        atomicAdd(&h_cnt[b], 1);
        const unsigned long long e = mass_fix(z, zmax);
        if (e) add_mass(&h_mass[b], e);
      }
    }
    const int b2 = find_cut_bin(h_cnt, h_mass, count_limit, mass_limit, a_cnt, a_mass, res);
    // ---- level 3: the elements of sub-bin (b1, b2); the cut is one of their values
    uint32_t* l_key = reinterpret_cast<uint32_t*>(h_cnt);
    unsigned long long* l_mass = h_mass;
    if (threadIdx.x == 0) list_n = 0;
    __syncthreads();
    uint32_t kmin = 0xffffffffu, kmax = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float z = Z(i);
      if (bin1_of(z, zmax) == b1 && bin2_of(z, zmax, b1) == b2) {
        const uint32_t key = float_key(z);
        kmin = min(kmin, key);
        kmax = max(kmax, key);
        const int at = atomicAdd(&list_n, 1);
        if (at < LIST_CAP) {
          l_key[at] = key;
          l_mass[at] = mass_fix(z, zmax);
        }
      }
    }
    // smallest and largest candidate key of the block (shared-memory atomics on two words)
    if (threadIdx.x == 0) {
      res[0] = (int)0xffffffffu;
      res[1] = 0;
    }
    __syncthreads();
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, o));
      kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
    }
    if ((threadIdx.x & 31) == 0 && kmin <= kmax) {
      atomicMin(reinterpret_cast<unsigned int*>(&res[0]), kmin);
      atomicMax(reinterpret_cast<unsigned int*>(&res[1]), kmax);
    }
    __syncthreads();
    kmin = (uint32_t)res[0];
    kmax = (uint32_t)res[1];
    __syncthreads();
    const int n = list_n;
    // smallest key u in [kmin, kmax] such that fewer than k elements and less than the mass limit
    // lie strictly above u; kmax is kept (its sub-bin was chosen for that)
    uint32_t lo = kmin, hi = kmax;
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1);
      int c = 0;
      unsigned long long m = 0;
      if (n <= LIST_CAP) {
        for (int j = threadIdx.x; j < n; j += blockDim.x)
          if (l_key[j] > mid) {
            c += 1;
            m += l_mass[j];
          }
      } else {  // more equal-looking values than the list holds: scan the row
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
          const float z = Z(i);
          if (bin1_of(z, zmax) == b1 && bin2_of(z, zmax, b1) == b2 && float_key(z) > mid) {
            c += 1;
            m += mass_fix(z, zmax);
          }
        }
      }
      c = warp_add(c);
      m = warp_add(m);
      __syncthreads();
      if (threadIdx.x == 0) {
        res[0] = 0;
        z_total = 0;
      }
      __syncthreads();
      if ((threadIdx.x & 31) == 0 && c) {
        atomicAdd(&res[0], c);
        atomicAdd(&z_total, m);
      }
      __syncthreads();
      if (a_cnt + res[0] < count_limit && a_mass + z_total < mass_limit) hi = mid; else lo = mid + 1;
    }
    cut = lo;
    }
  }
  const float min_z = mp > 0.f ? zmax + logf(mp) : -INFINITY;
  const uint64_t sd = seed[r];
  const uint32_t k0 = (uint32_t)sd, k1 = (uint32_t)(sd >> 32);
  const uint32_t dr = (uint32_t)draw[r];
  ArgMax best = {-INFINITY, 0x7fffffff};
  const int quads = (V + 3) >> 2;
  // The draw adds -log(-log u) to z - zmax, with u a multiple of 2^-24 plus 2^-25 inside (0, 1):
  // that term lies in [-2.86, 17.33]. An element more than 20.2 below the maximum therefore loses
  // to the maximum whatever is drawn, and needs no random number.
  const float floor_z = zmax - 20.5f;
  auto kept = [&](float z) { return float_key(z) >= cut && z >= min_z && z >= floor_z; };
  auto score = [&](int i, float z, uint32_t bits) {
    const float u = ((float)(bits >> 8) + 0.5f) * (1.f / 16777216.f);  // (0, 1)
    // argmax of p_i / E_i with E_i = -log(u): compare log p_i - log E_i; the normaliser of p is
    // the same for every i and left out
    return ArgMax{z - logf(-logf(u)), i};
  };
  bool listed = false;
  if (cut > 0 || mp > 0.f) {
    // Few elements survive a cut. They are listed first, so that the random numbers (made per
    // group of four vocabulary entries, whoever asks) are computed by as many threads as there
    // are survivors instead of by every warp that holds one.
    int* kept_idx = reinterpret_cast<int*>(h_mass);
    __syncthreads();  // the histogram and the candidate list are no longer read
    if (threadIdx.x == 0) list_n = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      if (kept(Z(i))) {
        const int at = atomicAdd(&list_n, 1);
        if (at < KEPT_CAP) kept_idx[at] = i;
      }
    __syncthreads();
    const int n = list_n;
    if (n <= KEPT_CAP) {
      listed = true;
      for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const int i = kept_idx[j];
        uint32_t c[4] = {(uint32_t)(i >> 2), dr, 0u, 0u};
        philox4x32_10(c, k0, k1);
        best = better(best, score(i, Z(i), c[i & 3]));
      }
    }
  }
  if (!listed) {
    for (int qd = threadIdx.x; qd < quads; qd += blockDim.x) {
      float z[4];
      bool keep[4], any = false;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = qd * 4 + e;
        z[e] = i < V ? Z(i) : -INFINITY;
        keep[e] = i < V && kept(z[e]);
        any |= keep[e];
      }
      if (!any) continue;
      uint32_t c[4] = {(uint32_t)qd, dr, 0u, 0u};
      philox4x32_10(c, k0, k1);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (keep[e]) best = better(best, score(qd * 4 + e, z[e], c[e]));
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

// Per-request token state for the penalties, kept on the device: state[slot][v] counts how often
// token v was generated (low 30 bits) and marks tokens of the prompt (bit 30). token_state_add
// enters tokens; penalties_dense applies the rule of penalties_kernel to every marked entry of the
// rows it is given, reading the state instead of a list built on the host.
constexpr int PROMPT_BIT = 1 << 30;

__global__ void token_state_add_kernel(int* __restrict__ state, int V, const int* __restrict__ slot,
                                       const int* __restrict__ token,
                                       const int* __restrict__ in_prompt, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int* p = state + (size_t)slot[i] * V + token[i];
  if (in_prompt[i]) atomicOr(p, PROMPT_BIT);
  else atomicAdd(p, 1);
}

__global__ void penalties_dense_kernel(float* __restrict__ logits, int V, const int* __restrict__ row,
                                       const int* __restrict__ slot,
                                       const float* __restrict__ presence,
                                       const float* __restrict__ frequency,
                                       const float* __restrict__ repetition,
                                       const int* __restrict__ state) {
  const int j = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= V) return;
  const int st = state[(size_t)slot[j] * V + v];
  if (st == 0) return;
  float* p = logits + (size_t)row[j] * V + v;
  float x = *p;
  const int c = st & (PROMPT_BIT - 1);
  if (c > 0) x -= frequency[j] * (float)c + presence[j];
  const float rp = repetition[j];
  if (rp != 1.f) x = x > 0.f ? x / rp : x * rp;
  *p = x;
}

__global__ void ban_kernel(float* __restrict__ logits, int V, const int* __restrict__ row,
                           const int* __restrict__ token, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) logits[(size_t)row[i] * V + token[i]] = -INFINITY;
}

}  // namespace lse

using namespace lse;

extern "C" size_t lse_sample_scratch_ints(int R) { return (size_t)R * (2 * SAMPLE_CHUNKS + 1); }

extern "C" int lse_sample(const float* logits, int R, int V, const float* temperature,
                          const int* top_k, const float* top_p, const float* min_p,
                          const uint64_t* seed, const int* draw, int* out_tokens, int* scratch,
                          int scratch_rows, int which, cudaStream_t stream) {
  if (R <= 0) return LSE_OK;
  if (V <= 0) return LSE_BAD_ARGUMENT;
  // which: bit 0 = some row is greedy or has a cut (one block per row), bit 1 = some row has a
  // temperature and no cut (several blocks per row, needs the scratch); a caller that does not
  // know passes 3. Without scratch the one-block kernel serves every row.
  const int parallel = (scratch != nullptr && scratch_rows >= R && R <= 65535) ? 1 : 0;
  if (parallel && (which & 2))
    launch(sample_parallel_kernel, dim3(R, SAMPLE_CHUNKS), PAR_THREADS, 0, stream, logits, V, temperature,
           top_k, top_p, min_p, seed, draw, out_tokens, scratch, scratch_rows);
  if (parallel && !(which & 1)) return cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
  // histogram / candidate list, and the row itself when it fits beside them
  const size_t base = (size_t)HIST_BINS * 12;
  const size_t cached = base + (size_t)V * 4;
  static int max_smem = -1;
  if (max_smem < 0) {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    max_smem = v;
    if (cudaFuncSetAttribute(sample_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             max_smem - 4096) != cudaSuccess)
      return LSE_LAUNCH_FAILED;
  }
  if (cached <= (size_t)max_smem - 4096)
    launch(sample_kernel<true>, R, SAMPLE_THREADS, cached, stream, logits, V, temperature, top_k, top_p,
           min_p, seed, draw, out_tokens, (parallel && (which & 2)) ? 1 : 0);
  else
    launch(sample_kernel<false>, R, SAMPLE_THREADS, base, stream, logits, V, temperature, top_k, top_p,
           min_p, seed, draw, out_tokens, (parallel && (which & 2)) ? 1 : 0);
  return cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}

extern "C" int lse_logsumexp(const float* logits, int R, int V, float* out, cudaStream_t stream) {
  if (R <= 0) return LSE_OK;
  logsumexp_kernel<<<R, 512, 0, stream>>>(logits, V, out);
  return cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}

extern "C" int lse_apply_penalties(float* logits, int V, const int* row, const int* token,
                                   const int* count, const float* presence, const float* frequency,
                                   const float* repetition, int n, cudaStream_t stream) {
  if (n <= 0) return LSE_OK;
  penalties_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, V, row, token, count, presence,
                                                        frequency, repetition, n);
  return cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}

extern "C" int lse_ban_tokens(float* logits, int V, const int* row, const int* token, int n,
                              cudaStream_t stream) {
  if (n <= 0) return LSE_OK;
  ban_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, V, row, token, n);
  return cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}

extern "C" int lse_token_state_add(int* state, int V, const int* slot, const int* token,
                                   const int* in_prompt, int n, cudaStream_t stream) {
  if (n <= 0) return LSE_OK;
  token_state_add_kernel<<<(n + 255) / 256, 256, 0, stream>>>(state, V, slot, token, in_prompt, n);
  return cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}

extern "C" int lse_apply_penalties_dense(float* logits, int V, const int* row, const int* slot,
                                         const float* presence, const float* frequency,
                                         const float* repetition, const int* state, int n,
                                         cudaStream_t stream) {
  if (n <= 0 || V <= 0) return LSE_OK;
  if (n > 65535) return LSE_BAD_ARGUMENT;
  penalties_dense_kernel<<<dim3((V + 255) / 256, n), 256, 0, stream>>>(logits, V, row, slot, presence,
                                                                       frequency, repetition, state);
  return cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}
