// Causal attention over a paged key/value cache for one head size (compile with -DLSE_HEAD_DIM=D,
// D a multiple of 16, at most 256).
//
// For a query at absolute position p of a sequence, with keys j of the same sequence:
//   s_j = scale * q . k_j   for  max(0, p - window + 1) <= j <= p   (window 0: from 0)
//   o   = sum_j softmax(s)_j * v_j
// Query head h reads key/value head h / (num_heads / num_kv_heads). Scores, the running maximum,
// the normaliser and the weighted sum are float32 (src/llmserve/kernels/csrc/
// paged_attention.cpp:191-243 does the same on the CPU). Keys and values are read from pages
// [page][kv_head][offset][D] through the sequence's block table; nothing at or beyond a sequence's
// context length is ever used (the TMA-fed kernel copies whole tiles of 16 rows and masks or zeroes
// the rows it may not use), so pages that another request used before need no clearing.
//
// Kernels:
//   prefill_simt  portions of >= 2 rows, any dtype: 32 rows per block, 4 threads per row.
//   prefill_tc    (attention_tc.cuh) bfloat16 portions, D = 64, no window: tcgen05 tensor cores with
//                 TMA-fed operands and accumulators in tensor memory.
//   prefill_mma   bfloat16 portions, D <= 128: 128 rows per block (8 warps) on mma.sync tensor
//                 cores; key/value tiles of 64 tokens are double-buffered with cp.async.
//   decode_split  single rows: the context is cut into partitions, one block per (partition,
//                 head group, sequence); partial (max, sum, weighted values) go to scratch and the
//                 block that finishes last for a (sequence, head group) merges them
//                 (src/llmserve/kernels/csrc/paged_attention.cpp:245-346 merges in a second pass).
//                 The scratch starts with LSE_ATTN_COUNTERS int counters (one per (sequence,
//                 head group) is used), then the partial results; the counters must be zero
//                 before a launch and are zero again after it. One dot product per key and
//                 head on the CUDA cores: float32, and head sizes other than 64.
//   decode_mma8 / decode_mma  single rows, bfloat16: the same partitions and merge with mma.sync
//                 tensor-core tiles: keys x heads for up to 8 heads per key/value head (head
//                 sizes 64 and 128), heads x keys for 9 to 16 (head size 64).
//   decode_ring   decode_mma8 with its key/value tiles brought by TMA into swizzled shared memory
//                 (pages of 16 tokens or more): for grids of many waves.
#include <type_traits>

#include "attention_args.h"
#include "common.cuh"
#include "kernels.h"
#include "tma_util.cuh"
#if LSE_HEAD_DIM == 64
#include "attention_tc.cuh"
#endif

#ifndef LSE_HEAD_DIM
#error "compile with -DLSE_HEAD_DIM=<head size>"
#endif

namespace lse {

constexpr int D = LSE_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 up to 256");

template <typename T>
struct Exp;
template <>
struct Exp<float> {
  __device__ __forceinline__ static float f(float x) { return expf(x); }
};
template <>
struct Exp<bf16> {
  __device__ __forceinline__ static float f(float x) { return __expf(x); }
};

__host__ __device__ constexpr int pow2_ceil(int n) {
  int p = 1;
  while (p < n) p <<= 1;
  return p;
}

struct SeqInfo {
  int q_start, q_len, ctx, pos0;
};

__device__ __forceinline__ SeqInfo seq_info(const LseAttnArgs& a, int seq) {
  SeqInfo s;
  s.q_start = a.cu_q[seq];
  s.q_len = a.cu_q[seq + 1] - s.q_start;
  s.ctx = a.ctx_lens[seq];
  s.pos0 = s.ctx - s.q_len;
  return s;
}

// ============================================================================ prefill, CUDA cores
constexpr int SIMT_QT = 32;
constexpr int SIMT_KT = (D <= 128) ? 32 : 16;

template <typename T>
__global__ void __launch_bounds__(128) prefill_simt_kernel(const LseAttnArgs a, int page_shift) {
  constexpr int QT = SIMT_QT, KT = SIMT_KT, DPT = D / 4, VEC = Num<T>::kVec, NCHUNK = D / VEC;
  __shared__ float ks[KT][D];
  __shared__ float vs[KT][D];
  // heads vary fastest over the grid, tiles (longest first) slowest
  const int seq = a.tiles[2 * blockIdx.y], q0 = a.tiles[2 * blockIdx.y + 1];
  const int head = blockIdx.x;
  const int kvh = head / (a.num_heads / a.num_kv_heads);
  const SeqInfo si = seq_info(a, seq);
  const int r = threadIdx.x >> 2, sub = threadIdx.x & 3;
  const int qi = q0 + r;
  const bool row_valid = qi < si.q_len;
  const int qpos = si.pos0 + qi;
  const T* q = (const T*)a.q + (size_t)(si.q_start + (row_valid ? qi : 0)) * a.q_row_stride +
               (size_t)head * D;
  float qreg[DPT], acc[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    qreg[i] = Num<T>::to_float(q[sub + 4 * i]) * a.scale;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int rows_here = min(QT, si.q_len - q0);
  const int k_end = si.pos0 + q0 + rows_here;  // one past the last key any row of the tile reads
  const int k_first = a.window > 0 ? max(0, si.pos0 + q0 - a.window + 1) : 0;
  const int* table = a.block_tables + (size_t)seq * a.table_stride;
  const T* kp = (const T*)a.k_pages;
  const T* vp = (const T*)a.v_pages;

  for (int k0 = (k_first / KT) * KT; k0 < k_end; k0 += KT) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < KT * NCHUNK; idx += blockDim.x) {
      const int jj = idx / NCHUNK, c = idx - jj * NCHUNK;
      const int j = k0 + jj;
      Vec16<T> kv, vv;
      if (j >= k_first && j < k_end) {
        int pi, off;
        page_of(j, a.page_tokens, page_shift, pi, off);
        const size_t base =
            (((size_t)table[pi] * a.num_kv_heads + kvh) * a.page_tokens + off) * D + c * VEC;
        kv = load16(kp + base);
        vv = load16(vp + base);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) kv.v[e] = vv.v[e] = Num<T>::from_float(0.f);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        ks[jj][c * VEC + e] = Num<T>::to_float(kv.v[e]);
        vs[jj][c * VEC + e] = Num<T>::to_float(vv.v[e]);
      }
    }
    __syncthreads();
    float s[KT];
    float tile_max = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < KT; ++jj) {
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) d = fmaf(qreg[i], ks[jj][sub + 4 * i], d);
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      const int j = k0 + jj;
      const bool ok = row_valid && j <= qpos && j >= k_first &&
                      (a.window <= 0 || j > qpos - a.window);
      s[jj] = ok ? d : -INFINITY;
      tile_max = fmaxf(tile_max, s[jj]);
    }
    const float m_new = fmaxf(m, tile_max);
    if (m_new == -INFINITY) continue;  // nothing visible yet for this row (uniform per 4 threads)
    const float corr = Exp<T>::f(m - m_new);  // m = -inf gives 0
    l *= corr;
#pragma unroll
    for (int i = 0; i < DPT; ++i) acc[i] *= corr;
#pragma unroll
    for (int jj = 0; jj < KT; ++jj) {
      const float p = Exp<T>::f(s[jj] - m_new);  // s = -inf gives 0
      l += p;
#pragma unroll
      for (int i = 0; i < DPT; ++i) acc[i] = fmaf(p, vs[jj][sub + 4 * i], acc[i]);
    }
    m = m_new;
  }
  if (row_valid) {
    T* o = (T*)a.out + (size_t)(si.q_start + qi) * a.out_row_stride + (size_t)head * D;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < DPT; ++i) o[sub + 4 * i] = Num<T>::from_float(acc[i] * inv);
  }
}

// ============================================================================ prefill, tensor cores
constexpr int MMA_QT = 128, MMA_KT = 64, MMA_THREADS = 256;  // 8 warps x 16 query rows
constexpr bool kHasMma = (D <= 128);

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(addr), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

#if LSE_HEAD_DIM <= 128
__global__ void __launch_bounds__(MMA_THREADS, (LSE_HEAD_DIM <= 64 ? 2 : 1)) prefill_mma_kernel(const LseAttnArgs a, int page_shift) {
  constexpr int QT = MMA_QT, KT = MMA_KT, LD = D + 8, NCHUNK = D / 8, KS = D / 16, NB = KT / 8,
                DB = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);  // [QT][LD]
  bf16* ks_all = qs + QT * LD;                   // [2][KT][LD]: the next tile loads while one is used
  bf16* vs_all = ks_all + 2 * KT * LD;           // [2][KT][LD]
  // heads vary fastest over the grid, tiles (longest first) slowest
  const int seq = a.tiles[2 * blockIdx.y], q0 = a.tiles[2 * blockIdx.y + 1];
  const int head = blockIdx.x;
  const int kvh = head / (a.num_heads / a.num_kv_heads);
  const SeqInfo si = seq_info(a, seq);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int rows_here = min(QT, si.q_len - q0);
  const int k_end = si.pos0 + q0 + rows_here;
  const int k_first = a.window > 0 ? max(0, si.pos0 + q0 - a.window + 1) : 0;
  const int* table = a.block_tables + (size_t)seq * a.table_stride;
  const bf16* kp = (const bf16*)a.k_pages;
  const bf16* vp = (const bf16*)a.v_pages;

  // queries of this tile -> shared memory (rows past the portion are zero)
  for (int idx = threadIdx.x; idx < QT * NCHUNK; idx += blockDim.x) {
    const int r = idx / NCHUNK, c = idx - r * NCHUNK;
    const bool ok = r < rows_here;
    const bf16* src = (const bf16*)a.q + (size_t)(si.q_start + q0 + (ok ? r : 0)) * a.q_row_stride +
                      (size_t)head * D + c * 8;
    cp_async16(qs + r * LD + c * 8, src, ok);
  }
  asm volatile("cp.async.commit_group;\n" ::);
  asm volatile("cp.async.wait_group 0;\n" ::);
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int kk = 0; kk < KS; ++kk)
    ldmatrix_x4(qf[kk], qs + (warp * 16 + (lane & 15)) * LD + kk * 16 + ((lane >> 4) << 3));

  float o[DB][4];
#pragma unroll
  for (int i = 0; i < DB; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
  const float sl2 = a.scale * 1.4426950408889634f;  // scores in the base-2 domain
  const int qpos_r[2] = {si.pos0 + q0 + warp * 16 + g, si.pos0 + q0 + warp * 16 + g + 8};
  const bool valid_r[2] = {warp * 16 + g < rows_here, warp * 16 + g + 8 < rows_here};
  const int qmin_w = si.pos0 + q0 + warp * 16;  // position of this warp's first query row

  auto load_tile = [&](int buf, int k0) {
    bf16* ks = ks_all + buf * KT * LD;
    bf16* vs = vs_all + buf * KT * LD;
    for (int idx = threadIdx.x; idx < KT * NCHUNK; idx += blockDim.x) {
      const int jj = idx / NCHUNK, c = idx - jj * NCHUNK;
      const int j = k0 + jj;
      const bool ok = j >= k_first && j < k_end;
      size_t base = 0;
      if (ok) {
        int pi, off;
        page_of(j, a.page_tokens, page_shift, pi, off);
        base = (((size_t)table[pi] * a.num_kv_heads + kvh) * a.page_tokens + off) * D + c * 8;
      }
      cp_async16(ks + jj * LD + c * 8, kp + base, ok);
      cp_async16(vs + jj * LD + c * 8, vp + base, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  const int k_start = (k_first / KT) * KT;
  if (k_start < k_end) load_tile(0, k_start);
  int buf = 0;
  for (int k0 = k_start; k0 < k_end; k0 += KT, buf ^= 1) {
    if (k0 + KT < k_end) {
      load_tile(buf ^ 1, k0 + KT);  // that buffer was released by the barrier that ended the last pass
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const bf16* ks = ks_all + buf * KT * LD;
    const bf16* vs = vs_all + buf * KT * LD;

    // S = Q K^T for 16 rows x 64 keys
    float s[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
      for (int nb = 0; nb < NB; nb += 2) {
        uint32_t b[4];
        ldmatrix_x4(b, ks + (nb * 8 + (lane & 7) + ((lane >> 4) << 3)) * LD + kk * 16 +
                           (((lane >> 3) & 1) << 3));
        mma_bf16(s[nb], qf[kk], b[0], b[1]);
        mma_bf16(s[nb + 1], qf[kk], b[2], b[3]);
      }
    }
    // running maximum; only tiles on the diagonal, at a window's edge or at the context's start
    // need the per-element mask (rows past the portion compute garbage that is never stored)
    const bool full_tile = k0 >= k_first && k0 + KT - 1 <= qmin_w &&
                           (a.window <= 0 || qmin_w + 15 - k0 < a.window);
    float tmax[2] = {-INFINITY, -INFINITY};
    if (full_tile) {
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) tmax[e >> 1] = fmaxf(tmax[e >> 1], s[nb][e]);
    } else {
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int rr = e >> 1;
          const int j = k0 + nb * 8 + t4 * 2 + (e & 1);
          const bool ok = valid_r[rr] && j <= qpos_r[rr] && j >= k_first &&
                          (a.window <= 0 || j > qpos_r[rr] - a.window);
          s[nb][e] = ok ? s[nb][e] : -INFINITY;
          tmax[rr] = fmaxf(tmax[rr], s[nb][e]);
        }
      }
    }
    // scores stay unscaled; the scale (times log2 e) is folded into the exponent's multiply-add
    float corr[2], m_use[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 1));
      tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 2));
      const float m_new = fmaxf(m_r[rr], tmax[rr]);
      const float m_fin = (m_new == -INFINITY) ? 0.f : m_new;  // keeps exp2f(-inf - m) = 0, not NaN
      corr[rr] = exp2f((m_r[rr] - m_fin) * sl2);
      m_use[rr] = m_fin * sl2;
      m_r[rr] = m_new;
      l_r[rr] *= corr[rr];
    }
#pragma unroll
    for (int i = 0; i < DB; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
    // P = exp2(S - m), O += P V
#pragma unroll
    for (int kb = 0; kb < KT / 16; ++kb) {
      uint32_t pa[4];
      float p[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p[h][e] = exp2f(fmaf(s[2 * kb + h][e], sl2, -m_use[e >> 1]));
          l_r[e >> 1] += p[h][e];
        }
      pa[0] = pack_bf16(p[0][0], p[0][1]);
      pa[1] = pack_bf16(p[0][2], p[0][3]);
      pa[2] = pack_bf16(p[1][0], p[1][1]);
      pa[3] = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
      for (int db = 0; db < DB; db += 2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vs + (kb * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * LD + db * 8 +
                                 ((lane >> 4) << 3));
        mma_bf16(o[db], pa, b[0], b[1]);
        mma_bf16(o[db + 1], pa, b[2], b[3]);
      }
    }
    __syncthreads();  // all warps are done with this tile's buffers
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    l_r[rr] += __shfl_xor_sync(0xffffffffu, l_r[rr], 1);
    l_r[rr] += __shfl_xor_sync(0xffffffffu, l_r[rr], 2);
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    if (!valid_r[rr]) continue;
    const float inv = l_r[rr] > 0.f ? 1.f / l_r[rr] : 0.f;
    bf16* dst = (bf16*)a.out +
                (size_t)(si.q_start + q0 + warp * 16 + g + rr * 8) * a.out_row_stride +
                (size_t)head * D + t4 * 2;
#pragma unroll
    for (int db = 0; db < DB; ++db)
      *reinterpret_cast<uint32_t*>(dst + db * 8) =
          pack_bf16(o[db][rr * 2] * inv, o[db][rr * 2 + 1] * inv);
  }
}

#endif  // LSE_HEAD_DIM <= 128

// ============================================================================ decode
// Lanes of a warp are arranged as (keys in flight) x (16-byte chunks of a row).
template <typename T>
struct DecodeShape {
  static constexpr int VEC = Num<T>::kVec;
  static constexpr int NCHUNK = D / VEC;
  static constexpr int LPK = pow2_ceil(NCHUNK) < 32 ? pow2_ceil(NCHUNK) : 32;  // lanes per key
  static constexpr int CPL = (NCHUNK + LPK - 1) / LPK;                          // chunks per lane
  static constexpr int KPI = 32 / LPK;                                          // keys per warp pass
};

constexpr int DEC_WARPS = 4;

constexpr int MERGE_SPLITS = 64;  // most context partitions per (sequence, head)

// Merge of the partitions of one (sequence, head group), by the block that finished last. All its
// loads are independent of one another: a warp per head fetches every partition's maximum and sum
// at once and turns them into weights; then a thread per (head, dim) fetches the partitions'
// values eight at a time. Kept out of line so that it does not disturb the register allocation
// and instruction order of the key loop.
template <typename T, int GT>
__device__ __noinline__ void merge_partitions(const float* __restrict__ parts, int num_splits,
                                              int heads_here, T* __restrict__ out) {
  // parts: partition 0 of this block's first head; heads are num_splits * (D + 2) floats apart.
  // out: this token's row at the first head.
  __shared__ float sm_w[GT][MERGE_SPLITS], sm_L[GT];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int gq = warp; gq < heads_here; gq += DEC_WARPS) {
    const float* part = parts + (size_t)gq * num_splits * (D + 2);
    float ms[MERGE_SPLITS / 32], ls[MERGE_SPLITS / 32];
#pragma unroll
    for (int k = 0; k < MERGE_SPLITS / 32; ++k) {
      const int sp = lane + 32 * k;
      ms[k] = sp < num_splits ? __ldcg(part + sp * (D + 2) + D) : -INFINITY;
      ls[k] = sp < num_splits ? __ldcg(part + sp * (D + 2) + D + 1) : 0.f;
    }
    float M = -INFINITY;
#pragma unroll
    for (int k = 0; k < MERGE_SPLITS / 32; ++k) M = fmaxf(M, ms[k]);
    M = warp_max(M);
    float L = 0.f;
#pragma unroll
    for (int k = 0; k < MERGE_SPLITS / 32; ++k) {
      const float wt = (ms[k] == -INFINITY) ? 0.f : Exp<T>::f(ms[k] - M);
      sm_w[gq][lane + 32 * k] = wt;
      L += ls[k] * wt;
    }
    L = warp_sum(L);
    if (lane == 0) sm_L[gq] = L;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < heads_here * D; idx += blockDim.x) {
    const int gq = idx / D, d = idx - gq * D;
    const float* part = parts + (size_t)gq * num_splits * (D + 2) + d;
    float A = 0.f;
#pragma unroll 1
    for (int s0 = 0; s0 < num_splits; s0 += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = s0 + u < num_splits ? __ldcg(part + (s0 + u) * (D + 2)) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) A += v[u] * sm_w[gq][min(s0 + u, MERGE_SPLITS - 1)];
    }
    const float L = sm_L[gq];
    out[idx] = Num<T>::from_float(L > 0.f ? A / L : 0.f);
  }
}

template <typename T, int GT>
__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_split_kernel(const LseAttnArgs a, int page_shift) {
  using S = DecodeShape<T>;
  constexpr int VEC = S::VEC, NCHUNK = S::NCHUNK, LPK = S::LPK, CPL = S::CPL, KPI = S::KPI;
  __shared__ float sm_m[DEC_WARPS][GT], sm_l[DEC_WARPS][GT];
  __shared__ float sm_acc[DEC_WARPS][GT][D];
  pdl_trigger();

  const int split = blockIdx.x, b = blockIdx.z;
  const int G = a.num_heads / a.num_kv_heads;
  const int subs = (G + GT - 1) / GT;
  const int kvh = blockIdx.y / subs, sub = blockIdx.y - kvh * subs;
  const int h0 = kvh * G + sub * GT;
  const int heads_here = min(GT, G - sub * GT);
  const int seq = a.decode_seqs[b];
  const int tok = a.cu_q[seq];
  const int ctx = a.ctx_lens[seq];
  const int k_first = a.window > 0 ? max(0, ctx - a.window) : 0;
  const int span = ctx - k_first;
  const int per = (span + a.num_splits - 1) / a.num_splits;
  const int lo = k_first + split * per;
  const int hi = min(ctx, lo + per);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int li = lane % LPK, slot = lane / LPK;
  const int* table = a.block_tables + (size_t)seq * a.table_stride;
  const T* kp = (const T*)a.k_pages;
  const T* vp = (const T*)a.v_pages;

  // The batch description is an input of the step, not a result of earlier kernels, so the index
  // arithmetic above runs before the dependency wait.
  pdl_wait();  // queries and this step's key/value rows come from the kernel before this one

  float qreg[GT][CPL][VEC], acc[GT][CPL][VEC], m[GT], l[GT];
#pragma unroll
  for (int gq = 0; gq < GT; ++gq) {
    m[gq] = -INFINITY;
    l[gq] = 0.f;
    const T* q = (const T*)a.q + (size_t)tok * a.q_row_stride + (size_t)(h0 + min(gq, heads_here - 1)) * D;
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
      const int ch = li + c * LPK;
      Vec16<T> qv;
      if (ch < NCHUNK) qv = load16(q + ch * VEC);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        qreg[gq][c][e] = ch < NCHUNK ? Num<T>::to_float(qv.v[e]) * a.scale : 0.f;
        acc[gq][c][e] = 0.f;
      }
    }
  }

  // U passes of the warp are in flight together: all their loads are issued before any arithmetic.
  constexpr int U = (GT * CPL <= 2) ? 4 : 2;
  for (int j0 = lo + warp * KPI; j0 < hi; j0 += DEC_WARPS * KPI * U) {
    Vec16<T> kv[U][CPL], vv[U][CPL];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + u * DEC_WARPS * KPI + slot;
      ok[u] = j < hi;
      // a key past the end re-reads the last valid one (its result is dropped): no branch, so
      // every load of the U passes is issued before the first use
      int pi, off;
      page_of(min(j, hi - 1), a.page_tokens, page_shift, pi, off);
      const size_t base = (((size_t)table[pi] * a.num_kv_heads + kvh) * a.page_tokens + off) * D;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const int ch = li + c * LPK;
        if (NCHUNK % LPK == 0 || ch < NCHUNK) {
          kv[u][c] = load16(kp + base + ch * VEC);
          vv[u][c] = load16(vp + base + ch * VEC);
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) kv[u][c].v[e] = vv[u][c].v[e] = Num<T>::from_float(0.f);
        }
      }
    }
    // The U keys of a lane group share one update of the running maximum: one rescaling of the
    // sums for U keys instead of one per key.
#pragma unroll
    for (int gq = 0; gq < GT; ++gq) {
      float d[U];
      float m_new = m[gq];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        d[u] = 0.f;
#pragma unroll
        for (int c = 0; c < CPL; ++c)
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            d[u] = fmaf(qreg[gq][c][e], Num<T>::to_float(kv[u][c].v[e]), d[u]);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) d[u] += __shfl_xor_sync(0xffffffffu, d[u], o);
        if (ok[u]) m_new = fmaxf(m_new, d[u]);  // ok is uniform over the LPK lanes of a key
      }
      const float m_fin = (m_new == -INFINITY) ? 0.f : m_new;  // no key yet: everything stays 0
      const float corr = Exp<T>::f(m[gq] - m_fin);
      float p[U], psum = 0.f;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        p[u] = ok[u] ? Exp<T>::f(d[u] - m_fin) : 0.f;
        psum += p[u];
      }
      l[gq] = l[gq] * corr + psum;
#pragma unroll
      for (int c = 0; c < CPL; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          float t = acc[gq][c][e] * corr;
#pragma unroll
          for (int u = 0; u < U; ++u) t = fmaf(p[u], Num<T>::to_float(vv[u][c].v[e]), t);
          acc[gq][c][e] = t;
        }
      m[gq] = m_new;
    }
  }

  // merge the key slots of a warp (lanes that differ in the bits above LPK)
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
    for (int gq = 0; gq < GT; ++gq) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m[gq], o);
      const float l_o = __shfl_xor_sync(0xffffffffu, l[gq], o);
      const float m_new = fmaxf(m[gq], m_o);
      const float wa = (m[gq] == -INFINITY) ? 0.f : Exp<T>::f(m[gq] - m_new);
      const float wb = (m_o == -INFINITY) ? 0.f : Exp<T>::f(m_o - m_new);
      l[gq] = l[gq] * wa + l_o * wb;
#pragma unroll
      for (int c = 0; c < CPL; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float a_o = __shfl_xor_sync(0xffffffffu, acc[gq][c][e], o);
          acc[gq][c][e] = acc[gq][c][e] * wa + a_o * wb;
        }
      m[gq] = m_new;
    }
  }
  if (slot == 0) {
#pragma unroll
    for (int gq = 0; gq < GT; ++gq) {
      if (li == 0) {
        sm_m[warp][gq] = m[gq];
        sm_l[warp][gq] = l[gq];
      }
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const int ch = li + c * LPK;
        if (ch < NCHUNK)
#pragma unroll
          for (int e = 0; e < VEC; ++e) sm_acc[warp][gq][ch * VEC + e] = acc[gq][c][e];
      }
    }
  }
  __syncthreads();
  // merge the warps; one thread per (head, dim)
  for (int idx = threadIdx.x; idx < heads_here * D; idx += blockDim.x) {
    const int gq = idx / D, d = idx - gq * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_m[w][gq]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float wt = (sm_m[w][gq] == -INFINITY) ? 0.f : Exp<T>::f(sm_m[w][gq] - M);
      L += sm_l[w][gq] * wt;
      A += sm_acc[w][gq][d] * wt;
    }
    const int h = h0 + gq;
    if (a.num_splits == 1) {
      T* o = (T*)a.out + (size_t)tok * a.out_row_stride + (size_t)h * D;
      o[d] = Num<T>::from_float(L > 0.f ? A / L : 0.f);
    } else {
      float* part = a.scratch + LSE_ATTN_COUNTERS +
                    (((size_t)b * a.num_heads + h) * a.num_splits + split) * (D + 2);
      part[d] = A;
      if (d == 0) {
        part[D] = M;
        part[D + 1] = L;
      }
    }
  }
  if (a.num_splits == 1) return;
  // The block that finishes last for this (sequence, head group) merges the partitions. Counters
  // live behind the partial results, start at zero and are reset by the merging block.
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = reinterpret_cast<int*>(a.scratch) + (size_t)b * gridDim.y + blockIdx.y;
    const int done = atomicAdd(counter, 1);
    is_last = (done == a.num_splits - 1);
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  merge_partitions<T, GT>(
      a.scratch + LSE_ATTN_COUNTERS + ((size_t)b * a.num_heads + h0) * a.num_splits * (D + 2),
      a.num_splits, heads_here, (T*)a.out + (size_t)tok * a.out_row_stride + (size_t)h0 * D);
}

#if LSE_HEAD_DIM == 64
// ---------------------------------------------------------------------------- decode, tensor cores
// When several query heads share one key/value head (grouped-query attention) the arithmetic per
// byte of cache grows with the group, and one dot product per (key, head) on the CUDA cores no
// longer keeps up with memory. Here the group's heads are the rows of a tensor-core tile
// (mma.sync m16n8k16, bfloat16, float32 accumulation): per 16 keys a warp computes
// S[heads x 16 keys] = Q K^T and O[heads x 64] += P V, whatever the size of the group (2..16).
// Keys and values come straight from global memory in 16-byte pieces into the operand registers:
//   * K as the "col" operand of Q K^T wants, per thread, pairs of neighbouring head dims of one
//     key: which dims meet in which multiply is free as long as Q is laid out the same way, so
//     thread (g, t) takes the 16-byte pieces t and t + 4 of key g's row;
//   * V as the "col" operand of P V wants pairs of neighbouring *keys* for one dim: thread (g, t)
//     loads piece g of the rows of its four keys (2t, 2t+1, 2t+8, 2t+9) and pairs them up with
//     byte permutes. Column j of output tile g' is then head dim 8 g + j: a fixed permutation that
//     is undone when the result is written.
// Each warp keeps its own running maximum and sums; warps and context partitions are merged as
// in the kernel above.
constexpr int DM_HEADS = 16;

__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_mma_kernel(const LseAttnArgs a, int page_shift) {
  using T = bf16;
  __shared__ float sm_m[DEC_WARPS][DM_HEADS], sm_l[DEC_WARPS][DM_HEADS];
  __shared__ float sm_acc[DEC_WARPS][DM_HEADS][D];
  pdl_trigger();

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = a.num_heads / a.num_kv_heads;
  const int h0 = kvh * G;
  const int seq = a.decode_seqs[b];
  const int tok = a.cu_q[seq];
  const int ctx = a.ctx_lens[seq];
  const int k_first = a.window > 0 ? max(0, ctx - a.window) : 0;
  const int span = ctx - k_first;
  const int per = (span + a.num_splits - 1) / a.num_splits;
  const int lo = k_first + split * per;
  const int hi = min(ctx, lo + per);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int* table = a.block_tables + (size_t)seq * a.table_stride;
  const T* kp = (const T*)a.k_pages;
  const T* vp = (const T*)a.v_pages;
  const bool page_holds_tile = page_shift >= 4;  // pages of 16, 32, ... tokens: a tile of 16 aligned keys lies in one

  pdl_wait();  // queries and this step's key/value rows come from the kernel before this one

  // Q as the row operand: rows g and g + 8 are heads h0 + g and h0 + g + 8 (zero beyond the
  // group). Multiply step s pairs logical k = 2t, 2t+1, 2t+8, 2t+9 with the head dims
  // d0, d0+1, d0+2, d0+3, d0 = 8 (t + 4 (s / 2)) + 4 (s % 2): the same dims that K supplies.
  uint32_t qa[4][4];
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const int d0 = 8 * (t + 4 * (s >> 1)) + 4 * (s & 1);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int head = g + 8 * r;
      uint32_t x0 = 0, x1 = 0;
      if (head < G) {
        const T* q = (const T*)a.q + (size_t)tok * a.q_row_stride + (size_t)(h0 + head) * D + d0;
        x0 = *reinterpret_cast<const uint32_t*>(q);
        x1 = *reinterpret_cast<const uint32_t*>(q + 2);
      }
      qa[s][r] = x0;      // a0 (row g) / a1 (row g + 8)
      qa[s][2 + r] = x1;  // a2 / a3
    }
  }
  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // rows g and g + 8

  auto row_base = [&](int key) -> size_t {  // offset of a key's row for this key/value head
    int pi, off;
    page_of(key, a.page_tokens, page_shift, pi, off);
    return (((size_t)table[pi] * a.num_kv_heads + kvh) * a.page_tokens + off) * D;
  };
  if (hi > lo) {
    const int first_tile = lo >> 4, last_tile = (hi - 1) >> 4;
    for (int tile = first_tile + warp; tile <= last_tile; tile += DEC_WARPS) {
      const int j0 = tile * 16;
      // keys outside [lo, hi) are masked below; their rows are read from a key inside
      auto inside = [&](int key) { return min(max(key, lo), hi - 1); };
      size_t kb[2], vb[4];
      if (page_holds_tile) {
        const size_t page_row =
            ((size_t)table[j0 >> page_shift] * a.num_kv_heads + kvh) * a.page_tokens;
        const int mask = a.page_tokens - 1;
        kb[0] = (page_row + (inside(j0 + g) & mask)) * D;
        kb[1] = (page_row + (inside(j0 + g + 8) & mask)) * D;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          vb[i] = (page_row + (inside(j0 + 2 * t + (i & 1) + 8 * (i >> 1)) & mask)) * D;
      } else {
        kb[0] = row_base(inside(j0 + g));
        kb[1] = row_base(inside(j0 + g + 8));
#pragma unroll
        for (int i = 0; i < 4; ++i) vb[i] = row_base(inside(j0 + 2 * t + (i & 1) + 8 * (i >> 1)));
      }
      uint4 kr[2][2], vr[4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        kr[nt][0] = *reinterpret_cast<const uint4*>(kp + kb[nt] + 8 * t);
        kr[nt][1] = *reinterpret_cast<const uint4*>(kp + kb[nt] + 8 * (t + 4));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) vr[i] = *reinterpret_cast<const uint4*>(vp + vb[i] + 8 * g);

      // S = Q K^T for keys j0 + 8 nt + (2t, 2t+1); rows g and g + 8
      float sc[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          const uint4 c = kr[nt][s >> 1];
          const uint32_t b0 = (s & 1) ? c.z : c.x, b1 = (s & 1) ? c.w : c.y;
          mma_bf16(sc[nt], qa[s], b0, b1);
        }
      }
      float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = j0 + 8 * nt + 2 * t + e;
          const bool ok = key >= lo && key < hi;
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const float v = ok ? sc[nt][2 * r + e] * a.scale : -INFINITY;
            sc[nt][2 * r + e] = v;
            mx[r] = fmaxf(mx[r], v);
          }
        }
      float corr[2];
      uint32_t pa[4];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_fin = (mx[r] == -INFINITY) ? 0.f : mx[r];
        corr[r] = Exp<T>::f(m_run[r] - m_fin);
        m_run[r] = mx[r];
        float p[2][2], sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            p[nt][e] = Exp<T>::f(sc[nt][2 * r + e] - m_fin);
            sum += p[nt][e];
          }
        l_run[r] = l_run[r] * corr[r] + sum;  // this thread's share of the row; joined at the end
        pa[r] = pack_bf16(p[0][0], p[0][1]);      // a0 / a1: keys 2t, 2t+1
        pa[2 + r] = pack_bf16(p[1][0], p[1][1]);  // a2 / a3: keys 2t+8, 2t+9
      }
      // O += P V; column g of output tile j is head dim 8 g + j
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j][0] *= corr[0];
        o[j][1] *= corr[0];
        o[j][2] *= corr[1];
        o[j][3] *= corr[1];
        const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
        const uint32_t v0 = j < 2 ? vr[0].x : j < 4 ? vr[0].y : j < 6 ? vr[0].z : vr[0].w;
        const uint32_t v1 = j < 2 ? vr[1].x : j < 4 ? vr[1].y : j < 6 ? vr[1].z : vr[1].w;
        const uint32_t v2 = j < 2 ? vr[2].x : j < 4 ? vr[2].y : j < 6 ? vr[2].z : vr[2].w;
        const uint32_t v3 = j < 2 ? vr[3].x : j < 4 ? vr[3].y : j < 6 ? vr[3].z : vr[3].w;
        mma_bf16(o[j], pa, __byte_perm(v0, v1, sel), __byte_perm(v2, v3, sel));
      }
    }
  }
  // this warp's result in shared memory, head dims back in their places
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int head = g + 8 * r;
    if (head < G) {
      if (t == 0) {
        sm_m[warp][head] = m_run[r];
        sm_l[warp][head] = l;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        sm_acc[warp][head][8 * (2 * t) + j] = o[j][2 * r];
        sm_acc[warp][head][8 * (2 * t + 1) + j] = o[j][2 * r + 1];
      }
    }
  }
  __syncthreads();
  // merge the warps; one thread per (head, dim)
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int gq = idx / D, d = idx - gq * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_m[w][gq]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float wt = (sm_m[w][gq] == -INFINITY) ? 0.f : Exp<T>::f(sm_m[w][gq] - M);
      L += sm_l[w][gq] * wt;
      A += sm_acc[w][gq][d] * wt;
    }
    const int h = h0 + gq;
    if (a.num_splits == 1) {
      T* op = (T*)a.out + (size_t)tok * a.out_row_stride + (size_t)h * D;
      op[d] = Num<T>::from_float(L > 0.f ? A / L : 0.f);
    } else {
      float* part = a.scratch + LSE_ATTN_COUNTERS +
                    (((size_t)b * a.num_heads + h) * a.num_splits + split) * (D + 2);
      part[d] = A;
      if (d == 0) {
        part[D] = M;
        part[D + 1] = L;
      }
    }
  }
  if (a.num_splits == 1) return;
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = reinterpret_cast<int*>(a.scratch) + (size_t)b * gridDim.y + blockIdx.y;
    const int done = atomicAdd(counter, 1);
    is_last = (done == a.num_splits - 1);
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  merge_partitions<T, DM_HEADS>(
      a.scratch + LSE_ATTN_COUNTERS + ((size_t)b * a.num_heads + h0) * a.num_splits * (D + 2),
      a.num_splits, G, (T*)a.out + (size_t)tok * a.out_row_stride + (size_t)h0 * D);
}
#endif  // LSE_HEAD_DIM == 64

#if LSE_HEAD_DIM == 64 || LSE_HEAD_DIM == 128
constexpr bool kHasDecodeMma8 = true;
// For groups of up to 8 heads (head sizes 64 and 128), with the roles turned: the 16 keys are the rows of the
// tile and the heads its 8 columns, S^T = K Q^T and O^T = V^T P^T. No row of a tile is wasted on
// heads that do not exist, so the accumulators take half the registers and more blocks fit an SM,
// which is what hides the latency of the key/value loads. P^T comes out of S^T's accumulator
// layout by one 8x8 transpose across the warp per eight keys (movmatrix).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

// EARLY: the rows of the warp's first tile are loaded into registers before the dependency wait
// (the registers stay live across it, which costs occupancy: for grids that do not fill the SMs).
// FUSED: the queries, and this step's key and value, are not read from q and the pages but made
// here from the fixed-point sums of the fused q|k|v projection (a.qkv_sums): rotated at position
// ctx - 1 and rounded to bfloat16, exactly what the rotation kernel would have stored. Every thread
// makes the query values of its own multiply operands. In the block whose partition ends at this
// step's token, warp 0 writes the new key and value into their page and adds them to its result
// from shared memory (the tile loop stops one key earlier); the block that finishes last for a
// (sequence, key/value head) clears the sums it stands for. This saves the
// rotation kernel between the projection and the attention of a step of single tokens.
template <bool EARLY, bool FUSED>
__global__ void __launch_bounds__(DEC_WARPS * 32, EARLY ? 4 : ((FUSED && D == 64) ? 7 : 0))  // 0: the compiler's own choice
// (head size 64: 72 registers, 7 blocks per SM; the form that makes its own queries needs the promise to stay there)
decode_mma8_kernel(const LseAttnArgs a, int page_shift) {
  using T = bf16;
  constexpr int HEADS = 8;
  constexpr int KCH = D / 32;  // 16-byte pieces of a key row per thread: pieces t, t + 4, ...
  constexpr int KS = D / 16;   // multiply steps of K Q^T
  constexpr int VCH = D / 64;  // 16-byte pieces of a value row per thread: pieces g, g + 8
  constexpr int MT = D / 16;   // output tiles of 16 head dims
  __shared__ float sm_m[DEC_WARPS][HEADS], sm_l[DEC_WARPS][HEADS];
  __shared__ float sm_acc[DEC_WARPS][HEADS][D];
  __shared__ __align__(16) T sm_new[FUSED ? 2 * D : 8];    // this step's key, then its value (warp 0's)
  pdl_trigger();

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = a.num_heads / a.num_kv_heads;
  const int h0 = kvh * G;
  const int seq = a.decode_seqs[b];
  const int tok = a.cu_q[seq];
  const int ctx = a.ctx_lens[seq];
  const int k_first = a.window > 0 ? max(0, ctx - a.window) : 0;
  const int span = ctx - k_first;
  const int per = (span + a.num_splits - 1) / a.num_splits;
  const int lo = k_first + split * per;
  const int hi_all = min(ctx, lo + per);
  // FUSED: the partition that ends at this step's token takes that key from the sums, not the pages
  const bool owns_new = FUSED && hi_all == ctx && hi_all > lo;
  const int hi = owns_new ? hi_all - 1 : hi_all;  // keys [lo, hi) come from the pages

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int* table = a.block_tables + (size_t)seq * a.table_stride;
  const T* kp = (const T*)a.k_pages;
  const T* vp = (const T*)a.v_pages;
  const bool page_holds_tile = page_shift >= 4;  // pages of 16, 32, ... tokens: a tile of 16 aligned keys lies in one

  // Keys and values of earlier steps do not depend on the kernels before this one in the stream
  // (those write this step's row only), and neither do the block tables. So before the
  // dependency wait the rows of this warp's first tiles are asked for, unless a tile holds this
  // step's key: into L2 (one row of K or V per lane, no registers held across the wait), or, in
  // the EARLY kernel, the first tile straight into the operand registers.
  auto row_base = [&](int key) -> size_t {
    int pi, off;
    page_of(key, a.page_tokens, page_shift, pi, off);
    return (((size_t)table[pi] * a.num_kv_heads + kvh) * a.page_tokens + off) * D;
  };
  auto inside = [&](int key) { return min(max(key, lo), hi - 1); };  // masked keys read a valid row
  uint4 kr[2][KCH], vr[4][VCH];
  auto fetch = [&](int tile) {  // the tile's rows into operand registers
    const int j0 = tile * 16;
    size_t kb[2], vb[4];
    if (page_holds_tile) {
      const size_t page_row = ((size_t)table[j0 >> page_shift] * a.num_kv_heads + kvh) * a.page_tokens;
      const int mask = a.page_tokens - 1;
      kb[0] = (page_row + (inside(j0 + g) & mask)) * D;
      kb[1] = (page_row + (inside(j0 + g + 8) & mask)) * D;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        vb[i] = (page_row + (inside(j0 + 2 * t + (i & 1) + 8 * (i >> 1)) & mask)) * D;
    } else {
      kb[0] = row_base(inside(j0 + g));
      kb[1] = row_base(inside(j0 + g + 8));
#pragma unroll
      for (int i = 0; i < 4; ++i) vb[i] = row_base(inside(j0 + 2 * t + (i & 1) + 8 * (i >> 1)));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int c = 0; c < KCH; ++c)
        kr[r][c] = *reinterpret_cast<const uint4*>(kp + kb[r] + 8 * (t + 4 * c));
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < VCH; ++c)
        vr[i][c] = *reinterpret_cast<const uint4*>(vp + vb[i] + 8 * (g + 8 * c));
  };
  const int first_tile = lo >> 4, last_tile = (hi - 1) >> 4;
  auto older = [&](int tile) { return hi > lo && tile <= last_tile && tile * 16 + 16 <= ctx - 1; };
  bool fetched = false;
  if (EARLY) {
    fetched = older(first_tile + warp);
    if (fetched) fetch(first_tile + warp);
  } else {
#pragma unroll
    for (int ahead = 0; ahead < 2; ++ahead) {
      const int tile = first_tile + warp + ahead * DEC_WARPS;
      if (older(tile)) {
        const T* row = (lane < 16 ? kp : vp) + row_base(inside(tile * 16 + (lane & 15)));
#pragma unroll
        for (int b = 0; b < D * (int)sizeof(T); b += 128)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(row) + b));
      }
    }
  }

  pdl_wait();  // queries and this step's key/value rows come from the kernel before this one

  // Q^T as the column operand: column g is head h0 + g (zero beyond the group); multiply step s
  // pairs logical k = 2t, 2t+1, 2t+8, 2t+9 with head dims d0 .. d0+3, d0 = 8 (t + 4 (s / 2)) +
  // 4 (s % 2), the dims that K's 16-byte pieces t and t + 4 supply.
  uint32_t qb[KS][2];
  if (FUSED) {
    // The thread's dims are the 8-dim pieces t, t + 4, ... of head g: KS/2 pieces, of which the
    // second half are the rotation partners (dim + D/2) of the first half, so every thread
    // rotates what it needs from its own loads, and nothing goes through shared memory.
    constexpr int HALF = D / 2, NPC = KS / 2;
    const long long* row = a.qkv_sums + (size_t)tok * (a.num_heads + 2 * a.num_kv_heads) * D;
    const int pos = ctx - 1;
    const float* c = a.rope_cos ? a.rope_cos + (size_t)pos * HALF : nullptr;
    const float* sn = a.rope_sin ? a.rope_sin + (size_t)pos * HALF : nullptr;
    float x[NPC][8];
#pragma unroll
    for (int pc = 0; pc < NPC; ++pc)
#pragma unroll
      for (int e = 0; e < 8; ++e) x[pc][e] = 0.f;
    if (g < G) {
      const longlong2* src = reinterpret_cast<const longlong2*>(row + (size_t)(h0 + g) * D);
#pragma unroll
      for (int pc = 0; pc < NPC; ++pc) {
        const int piece = t + 4 * pc;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const longlong2 v = __ldcg(src + piece * 4 + e);
          x[pc][2 * e] = fixed_to_float(v.x);
          x[pc][2 * e + 1] = fixed_to_float(v.y);
        }
      }
      if (c) {
#pragma unroll
        for (int pc = 0; pc < NPC / 2; ++pc) {
          const int i0 = 8 * (t + 4 * pc);  // first dim of the piece, below D/2
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float cv = c[i0 + e], sv = sn[i0 + e];
            const float x1 = x[pc][e], x2 = x[pc + NPC / 2][e];
            x[pc][e] = x1 * cv - x2 * sv;
            x[pc + NPC / 2][e] = x2 * cv + x1 * sv;
          }
        }
      }
    }
    // in the block that owns this step's token, warp 0 makes the new key (rotated) and value from
    // the sums, writes them into their page and keeps them for itself (it adds that key after its tiles)
    if (owns_new && warp == 0) {
      int pi, off;
      page_of(pos, a.page_tokens, page_shift, pi, off);
      const size_t page_base = (((size_t)table[pi] * a.num_kv_heads + kvh) * a.page_tokens + off) * D;
      const long long* ksrc = row + (size_t)(a.num_heads + kvh) * D;
      const long long* vsrc = row + (size_t)(a.num_heads + a.num_kv_heads + kvh) * D;
      for (int i = lane; i < HALF; i += 32) {
        float k1 = fixed_to_float(__ldcg(ksrc + i)), k2 = fixed_to_float(__ldcg(ksrc + i + HALF));
        const float v1 = fixed_to_float(__ldcg(vsrc + i)), v2 = fixed_to_float(__ldcg(vsrc + i + HALF));
        if (c) {
          const float cv = c[i], sv = sn[i];
          const float r1 = k1 * cv - k2 * sv, r2 = k2 * cv + k1 * sv;
          k1 = r1;
          k2 = r2;
        }
        const T bk1 = __float2bfloat16(k1), bk2 = __float2bfloat16(k2);
        const T bv1 = __float2bfloat16(v1), bv2 = __float2bfloat16(v2);
        sm_new[i] = bk1;
        sm_new[i + HALF] = bk2;
        sm_new[D + i] = bv1;
        sm_new[D + i + HALF] = bv2;
        T* kd = (T*)a.k_pages + page_base;
        T* vd = (T*)a.v_pages + page_base;
        kd[i] = bk1;
        kd[i + HALF] = bk2;
        vd[i] = bv1;
        vd[i + HALF] = bv2;
      }
      __syncwarp();
    }
#pragma unroll
    for (int s = 0; s < KS; ++s) {
      const int o = 4 * (s & 1);
      qb[s][0] = pack_bf16(x[s >> 1][o], x[s >> 1][o + 1]);
      qb[s][1] = pack_bf16(x[s >> 1][o + 2], x[s >> 1][o + 3]);
    }
  } else {
#pragma unroll
    for (int s = 0; s < KS; ++s) {
      const int d0 = 8 * (t + 4 * (s >> 1)) + 4 * (s & 1);
      qb[s][0] = qb[s][1] = 0;
      if (g < G) {
        const T* q = (const T*)a.q + (size_t)tok * a.q_row_stride + (size_t)(h0 + g) * D + d0;
        qb[s][0] = *reinterpret_cast<const uint32_t*>(q);
        qb[s][1] = *reinterpret_cast<const uint32_t*>(q + 2);
      }
    }
  }
  // O^T: tile i = 4 c + w (piece g + 8 c of the value rows, word w of the piece): rows g and g + 8
  // are head dims 8 (g + 8 c) + 2 w and + 1; columns are heads 2t, 2t+1
  float ot[MT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i) ot[i][0] = ot[i][1] = ot[i][2] = ot[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // heads 2t and 2t + 1

  if (hi > lo) {
    for (int tile = first_tile + warp; tile <= last_tile; tile += DEC_WARPS) {
      const int j0 = tile * 16;
      if (!fetched) fetch(tile);
      fetched = false;

      // S^T[keys g, g + 8][heads 2t, 2t+1]
      float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        const uint4 c0 = kr[0][s >> 1], c1 = kr[1][s >> 1];
        const uint32_t ka[4] = {(s & 1) ? c0.z : c0.x, (s & 1) ? c1.z : c1.x,
                                (s & 1) ? c0.w : c0.y, (s & 1) ? c1.w : c1.y};
        mma_bf16(sc, ka, qb[s][0], qb[s][1]);
      }
      const bool ok0 = j0 + g >= lo && j0 + g < hi, ok1 = j0 + g + 8 >= lo && j0 + g + 8 < hi;
      float corr[2], p[2][2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float s0 = ok0 ? sc[e] * a.scale : -INFINITY;
        const float s1 = ok1 ? sc[2 + e] * a.scale : -INFINITY;
        float mx = fmaxf(m_run[e], fmaxf(s0, s1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        const float m_fin = (mx == -INFINITY) ? 0.f : mx;
        corr[e] = Exp<T>::f(m_run[e] - m_fin);
        m_run[e] = mx;
        p[e][0] = Exp<T>::f(s0 - m_fin);
        p[e][1] = Exp<T>::f(s1 - m_fin);
        l_run[e] = l_run[e] * corr[e] + p[e][0] + p[e][1];  // this thread's share; joined at the end
      }
      // P^T[keys 2t, 2t+1 / 2t+8, 2t+9][head g] from P[key g / g + 8][heads 2t, 2t+1]
      const uint32_t pb0 = movmatrix_trans(pack_bf16(p[0][0], p[1][0]));
      const uint32_t pb1 = movmatrix_trans(pack_bf16(p[0][1], p[1][1]));
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        ot[i][0] *= corr[0];
        ot[i][1] *= corr[1];
        ot[i][2] *= corr[0];
        ot[i][3] *= corr[1];
        const int c = i >> 2, w = i & 3;
        const uint32_t v0 = w == 0 ? vr[0][c].x : w == 1 ? vr[0][c].y : w == 2 ? vr[0][c].z : vr[0][c].w;
        const uint32_t v1 = w == 0 ? vr[1][c].x : w == 1 ? vr[1][c].y : w == 2 ? vr[1][c].z : vr[1][c].w;
        const uint32_t v2 = w == 0 ? vr[2][c].x : w == 1 ? vr[2][c].y : w == 2 ? vr[2][c].z : vr[2][c].w;
        const uint32_t v3 = w == 0 ? vr[3][c].x : w == 1 ? vr[3][c].y : w == 2 ? vr[3][c].z : vr[3][c].w;
        const uint32_t va[4] = {__byte_perm(v0, v1, 0x5410u), __byte_perm(v0, v1, 0x7632u),
                                __byte_perm(v2, v3, 0x5410u), __byte_perm(v2, v3, 0x7632u)};
        mma_bf16(ot[i], va, pb0, pb1);
      }
    }
  }
  if (FUSED && owns_new && warp == 0) {
    // this step's own key, from shared memory: its scores for heads 2t and 2t + 1 (dims shared
    // out over g), then one more step of the running softmax and of O^T
    // q . k for head g over this thread's dims (its query registers), joined over t; heads 2t and
    // 2t + 1, whose softmax state this thread keeps, are fetched from the lanes that hold them
    float dot = 0.f;
#pragma unroll
    for (int s = 0; s < KS; ++s) {
      const int d0 = 8 * (t + 4 * (s >> 1)) + 4 * (s & 1);
      const __nv_bfloat162 q01 = *reinterpret_cast<const __nv_bfloat162*>(&qb[s][0]);
      const __nv_bfloat162 q23 = *reinterpret_cast<const __nv_bfloat162*>(&qb[s][1]);
      dot += __low2float(q01) * __bfloat162float(sm_new[d0]) + __high2float(q01) * __bfloat162float(sm_new[d0 + 1]) +
             __low2float(q23) * __bfloat162float(sm_new[d0 + 2]) + __high2float(q23) * __bfloat162float(sm_new[d0 + 3]);
    }
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
    float corr[2], pn[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int head = 2 * t + e;
      const float of_head = __shfl_sync(0xffffffffu, dot, 4 * head);
      const float sc_new = head < G ? of_head * a.scale : -INFINITY;
      const float mx = fmaxf(m_run[e], sc_new);
      const float m_fin = (mx == -INFINITY) ? 0.f : mx;
      corr[e] = Exp<T>::f(m_run[e] - m_fin);
      const float p = Exp<T>::f(sc_new - m_fin);
      m_run[e] = mx;
      l_run[e] = l_run[e] * corr[e] + (g == 0 ? p : 0.f);  // the warp's sum is joined over g below
      pn[e] = __bfloat162float(__float2bfloat16(p));     // weights meet values as bfloat16, as in the tiles
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      const int dim = 8 * (g + 8 * (i >> 2)) + 2 * (i & 3);
      const float v0 = __bfloat162float(sm_new[D + dim]), v1 = __bfloat162float(sm_new[D + dim + 1]);
      ot[i][0] = ot[i][0] * corr[0] + pn[0] * v0;
      ot[i][1] = ot[i][1] * corr[1] + pn[1] * v0;
      ot[i][2] = ot[i][2] * corr[0] + pn[0] * v1;
      ot[i][3] = ot[i][3] * corr[1] + pn[1] * v1;
    }
  }
  // this warp's result in shared memory, head dims back in their places
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    float l = l_run[e];
    l += __shfl_xor_sync(0xffffffffu, l, 4);
    l += __shfl_xor_sync(0xffffffffu, l, 8);
    l += __shfl_xor_sync(0xffffffffu, l, 16);
    const int head = 2 * t + e;
    if (head < G) {
      if (g == 0) {
        sm_m[warp][head] = m_run[e];
        sm_l[warp][head] = l;
      }
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const int dim = 8 * (g + 8 * (i >> 2)) + 2 * (i & 3);
        sm_acc[warp][head][dim] = ot[i][e];
        sm_acc[warp][head][dim + 1] = ot[i][2 + e];
      }
    }
  }
  __syncthreads();
  // merge the warps; one thread per (head, dim)
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int gq = idx / D, d = idx - gq * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_m[w][gq]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float wt = (sm_m[w][gq] == -INFINITY) ? 0.f : Exp<T>::f(sm_m[w][gq] - M);
      L += sm_l[w][gq] * wt;
      A += sm_acc[w][gq][d] * wt;
    }
    const int h = h0 + gq;
    if (a.num_splits == 1) {
      T* op = (T*)a.out + (size_t)tok * a.out_row_stride + (size_t)h * D;
      op[d] = Num<T>::from_float(L > 0.f ? A / L : 0.f);
    } else {
      float* part = a.scratch + LSE_ATTN_COUNTERS +
                    (((size_t)b * a.num_heads + h) * a.num_splits + split) * (D + 2);
      part[d] = A;
      if (d == 0) {
        part[D] = M;
        part[D + 1] = L;
      }
    }
  }
  // FUSED: the sums that this (sequence, key/value head) stands for are cleared by the block after
  // which no block reads them: the only one, or the one that finishes last (every other block
  // read them before it counted itself done).
  auto clear_sums = [&]() {
    long long* row = const_cast<long long*>(a.qkv_sums) + (size_t)tok * (a.num_heads + 2 * a.num_kv_heads) * D;
    for (int idx = threadIdx.x; idx < (G + 2) * D; idx += blockDim.x) {
      const int part = idx / D, d = idx - part * D;
      const size_t col = part < G ? (size_t)(h0 + part) * D
                                  : (size_t)(a.num_heads + (part - G) * a.num_kv_heads + kvh) * D;
      row[col + d] = 0;
    }
  };
  if (a.num_splits == 1) {
    if (FUSED) clear_sums();
    return;
  }
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = reinterpret_cast<int*>(a.scratch) + (size_t)b * gridDim.y + blockIdx.y;
    const int done = atomicAdd(counter, 1);
    is_last = (done == a.num_splits - 1);
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (FUSED) clear_sums();
  merge_partitions<T, HEADS>(
      a.scratch + LSE_ATTN_COUNTERS + ((size_t)b * a.num_heads + h0) * a.num_splits * (D + 2),
      a.num_splits, G, (T*)a.out + (size_t)tok * a.out_row_stride + (size_t)h0 * D);
}

// The same computation fed by TMA: every warp has PER slots of 128-byte-swizzled shared memory, each
// for one key/value tile (16 keys), and asks for its next tile as soon as a slot's contents are in
// its registers (ldmatrix), so a tile's load runs while the tile before it is worked on. Tiles of
// earlier steps are asked for before the dependency wait. A tile is 16 consecutive rows of one
// page, so this kernel needs pages of at least 16 tokens; a tile's rows outside the partition
// (other partitions' keys, or rows of the page that were never written) are masked out of the
// scores and zeroed as values before they are used. (A separate producer warp with a ring of 8 or
// 12 tiles per block was slower: 178 us against 159 at batch 64, 37.7 against 30.5 at batch 8; the
// hand-over between warps costs more than the deeper ring gains.)
namespace ring {
using namespace tma;
constexpr int BOXES = D / 64;             // TMA boxes of 64 head dims per row
constexpr int TILE_BYTES = 16 * D * 2;    // keys or values of one tile

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// byte offset of 16-byte piece `c` (8 head dims) of row `r` inside a tile: box c / 8 holds pieces
// 8 (c / 8) .. + 7 of all 16 rows, rows of 128 bytes, pieces permuted by the 128-byte swizzle
__device__ __forceinline__ uint32_t piece(int r, int c) {
  return (uint32_t)((c >> 3) * 2048 + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}
}  // namespace ring

// PER: tiles in flight per warp. Every warp is its own producer: lane 0 asks for the warp's tile
// k + PER into the slot that tile k has just been read from, so no warp waits for another.
template <int PER>
__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_ring_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const LseAttnArgs a, int page_shift) {
  using T = bf16;
  using namespace ring;
  constexpr int HEADS = 8;
  constexpr int KS = D / 16;   // multiply steps of K Q^T
  constexpr int MT = D / 16;   // output tiles of 16 head dims
  constexpr int SLOTS = PER * DEC_WARPS;
  extern __shared__ __align__(1024) unsigned char ring_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(ring_raw) + 1023) & ~(uintptr_t)1023);  // [SLOTS][K tile, V tile]
  __shared__ __align__(8) uint64_t full[SLOTS];
  __shared__ float sm_m[DEC_WARPS][HEADS], sm_l[DEC_WARPS][HEADS];
  __shared__ float sm_acc[DEC_WARPS][HEADS][D];
  __shared__ volatile int failed;
  pdl_trigger();

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = a.num_heads / a.num_kv_heads;
  const int h0 = kvh * G;
  const int seq = a.decode_seqs[b];
  const int tok = a.cu_q[seq];
  const int ctx = a.ctx_lens[seq];
  const int k_first = a.window > 0 ? max(0, ctx - a.window) : 0;
  const int span = ctx - k_first;
  const int per = (span + a.num_splits - 1) / a.num_splits;
  const int lo = k_first + split * per;
  const int hi = min(ctx, lo + per);
  const int first_tile = lo >> 4;
  const int n_tiles = hi > lo ? ((hi - 1) >> 4) - first_tile + 1 : 0;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_mine = n_tiles > warp ? (n_tiles - warp + DEC_WARPS - 1) / DEC_WARPS : 0;  // tiles warp, warp + 4, ...
  if (threadIdx.x == 0) {
    failed = 0;
    for (int s = 0; s < SLOTS; ++s) mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  __syncthreads();

  const int* table = a.block_tables + (size_t)seq * a.table_stride;
  const int mask = a.page_tokens - 1;
  // rows of the warp's tiles base .. base + 31 (of its own count), one per lane: one dependent
  // load for 32 tiles instead of one per tile
  int rows_base = 0, my_row = 0;
  auto look_up = [&](int base) {
    rows_base = base;
    my_row = 0;
    if (base + lane < n_mine) {
      const int j0 = (first_tile + warp + (base + lane) * DEC_WARPS) * 16;
      my_row = (int)(((long long)table[j0 >> page_shift] * a.num_kv_heads + kvh) * a.page_tokens + (j0 & mask));
    }
  };
  auto ask = [&](int k) {  // all lanes call; lane 0 asks
    if (k >= rows_base + 32) look_up(k);
    const int row = __shfl_sync(0xffffffffu, my_row, k - rows_base);
    if (lane == 0) {
      const int s = warp * PER + k % PER;
      unsigned char* kt = tiles + (size_t)s * 2 * TILE_BYTES;
      mbar_expect_tx(&full[s], 2 * TILE_BYTES);
#pragma unroll
      for (int x = 0; x < BOXES; ++x) {
        tma_load_2d(kt + x * 2048, &map_k, &full[s], x * 64, row);
        tma_load_2d(kt + TILE_BYTES + x * 2048, &map_v, &full[s], x * 64, row);
      }
    }
  };
  // Keys and values of earlier steps depend on no kernel before this one in the stream (those
  // write this step's row only), and neither do the block tables: tiles of earlier steps are
  // asked for before the dependency wait.
  look_up(0);
  int asked = 0;
  for (; asked < n_mine && asked < PER && (first_tile + warp + asked * DEC_WARPS) * 16 + 16 <= ctx - 1; ++asked)
    ask(asked);
  pdl_wait();  // queries and this step's key/value row come from the kernels before this one
  for (; asked < n_mine && asked < PER; ++asked) ask(asked);

  // Q^T as the column operand of step s: heads g, head dims 16 s + 2t, +1 and + 8, + 9
  uint32_t qb[KS][2];
#pragma unroll
  for (int s = 0; s < KS; ++s) {
    qb[s][0] = qb[s][1] = 0;
    if (g < G) {
      const T* q = (const T*)a.q + (size_t)tok * a.q_row_stride + (size_t)(h0 + g) * D + 16 * s + 2 * t;
      qb[s][0] = *reinterpret_cast<const uint32_t*>(q);
      qb[s][1] = *reinterpret_cast<const uint32_t*>(q + 8);
    }
  }
  float ot[MT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i) ot[i][0] = ot[i][1] = ot[i][2] = ot[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // heads 2t and 2t + 1

  const int mat = lane >> 3, r8 = lane & 7;
  int k = 0;
  for (; k < n_mine; ++k) {
    const int s = warp * PER + k % PER, j0 = (first_tile + warp + k * DEC_WARPS) * 16;
    if (!mbar_wait(&full[s], (k / PER) & 1)) {
      failed = 2;
      break;
    }
    unsigned char* kt = tiles + (size_t)s * 2 * TILE_BYTES;
    unsigned char* vt = kt + TILE_BYTES;
    if (j0 < lo || j0 + 16 > hi) {
      // rows outside the partition may hold anything (also NaN bits in rows never written):
      // zero them as values, so that their weight of zero gives zero
      const int r = lane >> 1;
      if (j0 + r < lo || j0 + r >= hi) {
#pragma unroll
        for (int x = 0; x < BOXES; ++x) {
          uint4* row = reinterpret_cast<uint4*>(vt + x * 2048 + r * 128 + (lane & 1) * 64);
          row[0] = row[1] = row[2] = row[3] = make_uint4(0, 0, 0, 0);
        }
      }
      __syncwarp();
    }
    const uint32_t kaddr = smem_u32(kt), vaddr = smem_u32(vt);
    // S^T[keys g, g + 8][heads 2t, 2t+1]
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t ka[4];  // keys 0-7 / 8-15 (mat & 1), pieces 2 ks / 2 ks + 1 (mat >> 1)
      ldmatrix_x4(ka, kaddr + piece((mat & 1) * 8 + r8, 2 * ks + (mat >> 1)));
      mma_bf16(sc, ka, qb[ks][0], qb[ks][1]);
    }
    uint32_t va[MT][4];  // V^T: head dims 16 m .. + 7 / + 8 .. + 15 (mat & 1), keys 0-7 / 8-15 (mat >> 1)
#pragma unroll
    for (int m = 0; m < MT; ++m) ldmatrix_x4_trans(va[m], vaddr + piece((mat >> 1) * 8 + r8, 2 * m + (mat & 1)));
    // the tile is in registers: its slot can take the warp's tile k + PER
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (k + PER < n_mine) ask(k + PER);

    const bool ok0 = j0 + g >= lo && j0 + g < hi, ok1 = j0 + g + 8 >= lo && j0 + g + 8 < hi;
    float corr[2], p[2][2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float s0 = ok0 ? sc[e] * a.scale : -INFINITY;
      const float s1 = ok1 ? sc[2 + e] * a.scale : -INFINITY;
      float mx = fmaxf(m_run[e], fmaxf(s0, s1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_fin = (mx == -INFINITY) ? 0.f : mx;
      corr[e] = Exp<T>::f(m_run[e] - m_fin);
      m_run[e] = mx;
      p[e][0] = Exp<T>::f(s0 - m_fin);
      p[e][1] = Exp<T>::f(s1 - m_fin);
      l_run[e] = l_run[e] * corr[e] + p[e][0] + p[e][1];  // this thread's share; joined at the end
    }
    // P^T[keys 2t, 2t+1 / 2t+8, 2t+9][head g] from P[key g / g + 8][heads 2t, 2t+1]
    const uint32_t pb0 = movmatrix_trans(pack_bf16(p[0][0], p[1][0]));
    const uint32_t pb1 = movmatrix_trans(pack_bf16(p[0][1], p[1][1]));
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      ot[m][0] *= corr[0];
      ot[m][1] *= corr[1];
      ot[m][2] *= corr[0];
      ot[m][3] *= corr[1];
      mma_bf16(ot[m], va[m], pb0, pb1);
    }
  }
  if (k < n_mine) {
    // a wait ran out: the tiles still asked for must land before the block's memory is given up
    for (int c = k; c < n_mine && c < k + PER; ++c)
      if (!mbar_wait(&full[warp * PER + c % PER], (c / PER) & 1)) break;
  }
  // this warp's result in shared memory
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    float l = l_run[e];
    l += __shfl_xor_sync(0xffffffffu, l, 4);
    l += __shfl_xor_sync(0xffffffffu, l, 8);
    l += __shfl_xor_sync(0xffffffffu, l, 16);
    const int head = 2 * t + e;
    if (head < G) {
      if (g == 0) {
        sm_m[warp][head] = m_run[e];
        sm_l[warp][head] = l;
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        sm_acc[warp][head][16 * m + g] = ot[m][e];
        sm_acc[warp][head][16 * m + g + 8] = ot[m][2 + e];
      }
    }
  }
  __syncthreads();
  if (failed && threadIdx.x == 0 && a.error_flag) atomicExch(a.error_flag, 200 + failed);
  // merge the warps; one thread per (head, dim)
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int gq = idx / D, d = idx - gq * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_m[w][gq]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float wt = (sm_m[w][gq] == -INFINITY) ? 0.f : Exp<T>::f(sm_m[w][gq] - M);
      L += sm_l[w][gq] * wt;
      A += sm_acc[w][gq][d] * wt;
    }
    const int h = h0 + gq;
    if (a.num_splits == 1) {
      T* op = (T*)a.out + (size_t)tok * a.out_row_stride + (size_t)h * D;
      op[d] = Num<T>::from_float(L > 0.f ? A / L : 0.f);
    } else {
      float* part = a.scratch + LSE_ATTN_COUNTERS +
                    (((size_t)b * a.num_heads + h) * a.num_splits + split) * (D + 2);
      part[d] = A;
      if (d == 0) {
        part[D] = M;
        part[D + 1] = L;
      }
    }
  }
  if (a.num_splits == 1) return;
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = reinterpret_cast<int*>(a.scratch) + (size_t)b * gridDim.y + blockIdx.y;
    const int done = atomicAdd(counter, 1);
    is_last = (done == a.num_splits - 1);
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  merge_partitions<T, HEADS>(
      a.scratch + LSE_ATTN_COUNTERS + ((size_t)b * a.num_heads + h0) * a.num_splits * (D + 2),
      a.num_splits, G, (T*)a.out + (size_t)tok * a.out_row_stride + (size_t)h0 * D);
}
#else
constexpr bool kHasDecodeMma8 = false;
#endif  // LSE_HEAD_DIM == 64 || LSE_HEAD_DIM == 128

static int shift_of(int n) {
  if (n <= 0 || (n & (n - 1))) return -1;
  int s = 0;
  while ((1 << s) < n) ++s;
  return s;
}

static bool args_ok(const LseAttnArgs* a) {
  return a && (a->dtype == LSE_F32 || a->dtype == LSE_BF16) && a->num_heads > 0 &&
         a->num_kv_heads > 0 && a->num_heads % a->num_kv_heads == 0 && a->page_tokens > 0 &&
         a->window >= 0 && (a->q || a->qkv_sums) && a->out && a->k_pages && a->v_pages && a->block_tables &&
         a->ctx_lens && a->cu_q;
}

template <typename T>
static int launch_decode(const LseAttnArgs* a, cudaStream_t stream) {
  const int G = a->num_heads / a->num_kv_heads;
  const int ps = shift_of(a->page_tokens);
#if LSE_HEAD_DIM == 64 || LSE_HEAD_DIM == 128
  // On the tensor cores: one block per (partition, key/value head, sequence). Also for a single
  // head per key/value head: seven of the tile's eight columns are idle then, but the kernel
  // still issues fewer instructions per key than a dot product on the CUDA cores (head size 64,
  // batch 8, 2176 keys: 27.1 us against 30.6; batch 64: 168 against 176).
  constexpr int kMmaHeads = LSE_HEAD_DIM == 64 ? 16 : 8;  // 9..16 heads: head size 64 only
  if (std::is_same<T, bf16>::value && G <= kMmaHeads && a->force_simt != 1) {
    dim3 mgrid(a->num_splits, a->num_kv_heads, a->num_decode);
    if (mgrid.y > 65535 || mgrid.z > 65535) return LSE_BAD_ARGUMENT;
    if (a->num_splits > 1 && (size_t)mgrid.y * mgrid.z > (size_t)LSE_ATTN_COUNTERS) return LSE_BAD_ARGUMENT;
    if (a->num_splits > MERGE_SPLITS) return LSE_BAD_ARGUMENT;
    static int sms = 0;
    if (!sms) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const long long blocks = (long long)mgrid.x * mgrid.y * mgrid.z;
    const long long pool_rows = a->num_pages * a->num_kv_heads * a->page_tokens;
    // The TMA-fed kernel needs pages that hold whole tiles of 16 keys and the pool's size. It is
    // the faster one where a block walks a whole context and the grid is several waves (head size
    // 64, 32 heads, alone: 64 sequences of 2118 keys 160.8 us against 164.5, of 600 keys 51.0
    // against 51.5; in the whole step batch 64 gains 2.7 %). A block's start costs more than the
    // register-fed kernel's (barriers, descriptor fetch), so with partitions (shorter walks: 48
    // sequences in 2 partitions 137 us against 130) and with grids of about one wave (batch 8 in 4
    // partitions: 30.6 against 27.3) the other one is taken.
    const bool ring_can = G <= 8 && ps >= 4 && pool_rows > 0 && pool_rows < (1LL << 31);
    if (a->qkv_sums && G > 8) return LSE_BAD_ARGUMENT;  // only the kernel for groups of up to 8 makes its own queries
    if (ring_can && !a->qkv_sums && (a->force_simt == 3 ||
                     (a->force_simt == 0 && a->num_splits == 1 && blocks >= 10LL * sms))) {
      constexpr int PER = 1;
      constexpr int smem = PER * DEC_WARPS * 2 * ring::TILE_BYTES + 1024;
      static bool configured = false;
      if (!configured) {
        if (cudaFuncSetAttribute(decode_ring_kernel<PER>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem) != cudaSuccess)
          return LSE_LAUNCH_FAILED;
        configured = true;
      }
      CUtensorMap mk, mv;
      if (!tma::make_map_bf16(&mk, a->k_pages, pool_rows, D, D, 16) ||
          !tma::make_map_bf16(&mv, a->v_pages, pool_rows, D, D, 16))
        return LSE_LAUNCH_FAILED;
      launch(decode_ring_kernel<PER>, mgrid, DEC_WARPS * 32, smem, stream, mk, mv, *a, ps);
      return cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
    }
    if (G <= 8) {
      // a grid that leaves the SMs part empty can afford the registers of an early first tile
      const bool small = blocks <= 4LL * sms;
      if (a->qkv_sums) {
        if (small) launch(decode_mma8_kernel<true, true>, mgrid, DEC_WARPS * 32, 0, stream, *a, ps);
        else launch(decode_mma8_kernel<false, true>, mgrid, DEC_WARPS * 32, 0, stream, *a, ps);
      } else {
        if (small) launch(decode_mma8_kernel<true, false>, mgrid, DEC_WARPS * 32, 0, stream, *a, ps);
        else launch(decode_mma8_kernel<false, false>, mgrid, DEC_WARPS * 32, 0, stream, *a, ps);
      }
    }
#if LSE_HEAD_DIM == 64
    else launch(decode_mma_kernel, mgrid, DEC_WARPS * 32, 0, stream, *a, ps);
#endif
    return cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
  }
#endif
  if (a->qkv_sums) return LSE_BAD_ARGUMENT;  // the kernels below read their queries from q
  const int gt = G == 1 ? 1 : (G == 2 ? 2 : 4);
  dim3 grid(a->num_splits, a->num_kv_heads * ((G + gt - 1) / gt), a->num_decode);
  if (grid.y > 65535 || grid.z > 65535) return LSE_BAD_ARGUMENT;
  if (a->num_splits > 1 && (size_t)grid.y * grid.z > (size_t)LSE_ATTN_COUNTERS) return LSE_BAD_ARGUMENT;
  if (a->num_splits > MERGE_SPLITS) return LSE_BAD_ARGUMENT;
  if (gt == 1) launch(decode_split_kernel<T, 1>, grid, DEC_WARPS * 32, 0, stream, *a, ps);
  else if (gt == 2) launch(decode_split_kernel<T, 2>, grid, DEC_WARPS * 32, 0, stream, *a, ps);
  else launch(decode_split_kernel<T, 4>, grid, DEC_WARPS * 32, 0, stream, *a, ps);
  return cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}

}  // namespace lse

using namespace lse;

extern "C" int lse_attn_head_dim(void) { return D; }

extern "C" int lse_attn_q_tile(int dtype) {
  return (dtype == LSE_BF16 && kHasMma) ? MMA_QT : SIMT_QT;
}

extern "C" size_t lse_attn_decode_scratch_floats(int num_decode, int num_heads, int num_splits) {
  // a fixed region of completion counters, then the partial results
  return num_splits > 1 ? (size_t)LSE_ATTN_COUNTERS + (size_t)num_decode * num_heads * num_splits * (D + 2)
                        : 0;
}

// Blocks of the single-token kernel for these head counts that one SM holds at a time (0 if it
// cannot be asked): what the choice of the number of context partitions rests on.
template <typename K>
static int blocks_per_sm(K kernel) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, DEC_WARPS * 32, 0) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}
extern "C" int lse_attn_decode_blocks_per_sm(int dtype, int num_heads, int num_kv_heads) {
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads) return 0;
  const int G = num_heads / num_kv_heads;
#if LSE_HEAD_DIM == 64 || LSE_HEAD_DIM == 128
  if (dtype == LSE_BF16 && G <= 8) return blocks_per_sm(decode_mma8_kernel<false, false>);
#endif
#if LSE_HEAD_DIM == 64
  if (dtype == LSE_BF16 && G <= 16) return blocks_per_sm(decode_mma_kernel);
#endif
  const int gt = G == 1 ? 1 : (G == 2 ? 2 : 4);
  if (dtype == LSE_BF16)
    return gt == 1 ? blocks_per_sm(decode_split_kernel<bf16, 1>)
                   : gt == 2 ? blocks_per_sm(decode_split_kernel<bf16, 2>) : blocks_per_sm(decode_split_kernel<bf16, 4>);
  return gt == 1 ? blocks_per_sm(decode_split_kernel<float, 1>)
                 : gt == 2 ? blocks_per_sm(decode_split_kernel<float, 2>) : blocks_per_sm(decode_split_kernel<float, 4>);
}

extern "C" int lse_attn_decode_takes_sums(int dtype, int num_heads, int num_kv_heads) {
#if LSE_HEAD_DIM == 64 || LSE_HEAD_DIM == 128
  return dtype == LSE_BF16 && num_kv_heads > 0 && num_heads % num_kv_heads == 0 && num_heads / num_kv_heads <= 8;
#else
  return 0;
#endif
}

extern "C" int lse_attn_prefill(const LseAttnArgs* a, cudaStream_t stream) {
  if (!args_ok(a) || !a->q || (a->num_tiles > 0 && !a->tiles)) return LSE_BAD_ARGUMENT;
  if (a->num_tiles <= 0) return LSE_OK;
  if (a->num_tiles > 65535) return LSE_BAD_ARGUMENT;
  const int ps = shift_of(a->page_tokens);
  dim3 grid(a->num_heads, a->num_tiles);
  if (a->dtype == LSE_F32) {
    prefill_simt_kernel<float><<<grid, 128, 0, stream>>>(*a, ps);
#if LSE_HEAD_DIM == 64
  } else if (a->force_simt == 0 && a->num_rows > 0 && a->num_pages > 0 && atc::supported(a)) {
    // 128-row tiles, like the mma.sync kernel
    return atc::launch_prefill(a, a->num_rows, a->num_pages * a->num_kv_heads * a->page_tokens,
                               a->error_flag, stream);
#endif
  } else if (!kHasMma || a->force_simt == 1) {
    // the caller built tiles of SIMT_QT rows in this case
    prefill_simt_kernel<bf16><<<grid, 128, 0, stream>>>(*a, ps);
  } else {
#if LSE_HEAD_DIM <= 128
    constexpr int smem = (MMA_QT + 4 * MMA_KT) * (D + 8) * (int)sizeof(bf16);
    static bool configured = false;
    if (!configured) {
      if (cudaFuncSetAttribute(prefill_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               smem) != cudaSuccess)
        return LSE_LAUNCH_FAILED;
      configured = true;
    }
    prefill_mma_kernel<<<grid, MMA_THREADS, smem, stream>>>(*a, ps);
#endif
  }
  return cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}

// ---- no-allocation variant: scratch inside the library's device image ---------------------------
// In host code the array's name is only a handle for the runtime, not a device address; the
// address each device gives it is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_scratch[LSE_ATTN_NOALLOC_MAX_FLOATS];

static float* noalloc_scratch_address() {
  constexpr int kMaxDevices = 64;
  static float* address[kMaxDevices] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (!address[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess) {
      cudaGetLastError();  // leave no sticky error behind
      return nullptr;
    }
    address[dev] = static_cast<float*>(p);
  }
  return address[dev];
}

extern "C" size_t lse_attn_decode_noalloc_max_floats(void) { return LSE_ATTN_NOALLOC_MAX_FLOATS; }

extern "C" int lse_attn_decode_noalloc(const LseAttnArgs* a, cudaStream_t stream) {
  if (!args_ok(a) || (a->num_decode > 0 && !a->decode_seqs)) return LSE_BAD_ARGUMENT;
  if (a->num_decode <= 0) return LSE_OK;
  if (a->num_splits < 1) return LSE_BAD_ARGUMENT;
  if (lse_attn_decode_scratch_floats(a->num_decode, a->num_heads, a->num_splits) >
      (size_t)LSE_ATTN_NOALLOC_MAX_FLOATS)
    return LSE_TOO_LARGE;
  LseAttnArgs b = *a;
  b.scratch = noalloc_scratch_address();
  if (!b.scratch) return LSE_LAUNCH_FAILED;
  return b.dtype == LSE_F32 ? launch_decode<float>(&b, stream) : launch_decode<bf16>(&b, stream);
}

extern "C" int lse_attn_decode(const LseAttnArgs* a, cudaStream_t stream) {
  if (!args_ok(a) || (a->num_decode > 0 && !a->decode_seqs)) return LSE_BAD_ARGUMENT;
  if (a->num_decode <= 0) return LSE_OK;
  if (a->num_splits < 1 || (a->num_splits > 1 && !a->scratch)) return LSE_BAD_ARGUMENT;
  return a->dtype == LSE_F32 ? launch_decode<float>(a, stream) : launch_decode<bf16>(a, stream);
}
