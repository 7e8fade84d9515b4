// Flash-style causal attention for portions of prompts on the 5th-generation tensor cores
// (head size 64, bfloat16, no window, page size a power of two >= 8).
//
// One block = 128 query rows of one head. Per tile of 64 keys:
//   S = Q K^T        tcgen05.mma, A = Q tile and B = K tile in shared memory (both K-major, TMA with
//                    128-byte swizzle, K tiles fetched page by page through the block table),
//                    accumulator S [128 x 64] float32 in tensor memory;
//   softmax          128 threads, one query row each: tcgen05.ld of the row, running maximum and
//                    sum in float32 (base-2 exponent, scale folded into the multiply-add), P rounded
//                    to bfloat16 and written back to tensor memory with tcgen05.st;
//   O += P V         tcgen05.mma with A = P from tensor memory and B = V tile in shared memory
//                    (N-major: rows are keys), accumulator O [128 x 64] float32 in tensor memory.
// When a row's maximum grows, O is rescaled in tensor memory (tcgen05.ld / st) before the next
// P V; warps whose maxima did not change skip that. Warps 0-3 do the softmax, one lane of warp 4
// runs the TMA pipeline, one lane of warp 5 issues the MMAs. Every barrier wait is bounded.
#pragma once

#include "attention_args.h"
#include "tma_util.cuh"

namespace lse {
namespace atc {

using namespace tma;

constexpr int HD = 64;           // head size served by this kernel
constexpr int QT = 128;          // query rows per block
constexpr int KT = 64;           // keys per tile
constexpr int STAGES = 3;        // key/value tiles in flight
constexpr int THREADS = 192;
constexpr uint32_t Q_BYTES = QT * HD * 2, KV_BYTES = KT * HD * 2;
// Tensor-memory columns. S is double-buffered so that Q K^T of the next tile runs while the
// softmax threads work on this one. P (32 packed columns) is written over the first half of the S
// buffer it came from once the row is in registers; MMAs of one thread run in issue order, so a
// later Q K^T into that buffer cannot overtake the P V that still reads P.
constexpr uint32_t COL_S = 0, S_COLS = 64, COL_O = 128, TMEM_COLS = 256;

__device__ __forceinline__ void umma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
      "%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
        "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
        "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
        "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,"
      "%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
        "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
        "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]),
        "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]),
        "r"(v[31])
      : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct Params {
  LseAttnArgs a;
  int page_shift;   // log2(page_tokens)
  int box_rows;     // rows per key/value TMA box: min(page_tokens, KT)
  int* error_flag;
};

__global__ void __launch_bounds__(THREADS, 2)
prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const Params p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_tile = base;
  unsigned char* k_tiles = q_tile + Q_BYTES;
  unsigned char* v_tiles = k_tiles + STAGES * KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_tiles + STAGES * KV_BYTES);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* kv_full = bars + 1;            // [STAGES]
  uint64_t* kv_empty = kv_full + STAGES;   // [STAGES]
  uint64_t* s_full = kv_empty + STAGES;    // [2] S of a tile is in tensor memory (buffer tile & 1)
  uint64_t* p_full = s_full + 2;           // P is written (and O rescaled): 4 arrivals
  uint64_t* pv_done = p_full + 1;          // O += P V of this tile has finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 1);
  __shared__ volatile int failed;
  __shared__ volatile int issued;  // key/value tiles the producer has requested

  const LseAttnArgs& a = p.a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heads vary fastest over the grid, tiles (longest first) slowest: every head's long tiles start early
  const int seq = a.tiles[2 * blockIdx.y], q0 = a.tiles[2 * blockIdx.y + 1];
  const int head = blockIdx.x;
  const int kvh = head / (a.num_heads / a.num_kv_heads);
  const int q_start = a.cu_q[seq];
  const int q_len = a.cu_q[seq + 1] - q_start;
  const int ctx = a.ctx_lens[seq];
  const int pos0 = ctx - q_len;
  const int rows_here = min(QT, q_len - q0);
  const int k_end = pos0 + q0 + rows_here;  // one past the last key any row of the tile reads
  const int n_tiles = (k_end + KT - 1) / KT;

  pdl_trigger();
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    failed = 0;
    issued = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  pdl_wait();  // queries, keys and values were written by the kernel before this one

  if (warp == 4) {
    if (lane == 0) {
      // ---- TMA producer
      mbar_expect_tx(q_full, Q_BYTES);
      tma_load_2d(q_tile, &map_q, q_full, head * HD, q_start + q0);
      const int* table = a.block_tables + (size_t)seq * a.table_stride;
      const int last_page_idx = (k_end - 1) >> p.page_shift;
      const int boxes = KT / p.box_rows;
      for (int it = 0; it < n_tiles && !failed; ++it) {
        const int s = it % STAGES;
        if (it >= STAGES && !mbar_wait(&kv_empty[s], ((it / STAGES) - 1) & 1)) {
          failed = 1;
          break;
        }
        mbar_expect_tx(&kv_full[s], 2 * KV_BYTES);
        for (int b = 0; b < boxes; ++b) {
          const int j = it * KT + b * p.box_rows;
          // a box past the context re-reads the last valid page: its keys are masked anyway,
          // and what it brings is finite
          const int pi = min(j >> p.page_shift, last_page_idx);
          const int off = (j >> p.page_shift) <= last_page_idx ? (j & (a.page_tokens - 1)) : 0;
          const int row = (table[pi] * a.num_kv_heads + kvh) * a.page_tokens + off;
          tma_load_2d(k_tiles + s * KV_BYTES + b * p.box_rows * HD * 2, &map_k, &kv_full[s], 0, row);
          tma_load_2d(v_tiles + s * KV_BYTES + b * p.box_rows * HD * 2, &map_v, &kv_full[s], 0, row);
        }
        issued = it + 1;
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    if (lane == 0) {
      // ---- MMA issuer
      constexpr uint32_t idesc_qk = instr_desc_bf16(QT, KT, 0);   // K tile K-major
      constexpr uint32_t idesc_pv = instr_desc_bf16(QT, HD, 1);   // V tile N-major (rows are keys)
      bool ok = mbar_wait(q_full, 0);
      const uint64_t dq = smem_desc_sw128(smem_u32(q_tile));
      auto issue_qk = [&](int t) -> bool {  // S[t & 1] = Q K_t^T once tile t has landed
        const int s = t % STAGES;
        if (!mbar_wait(&kv_full[s], (t / STAGES) & 1)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t dk = smem_desc_sw128(smem_u32(k_tiles + s * KV_BYTES));
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)  // 16 head dims = 32 bytes along the swizzled row
          umma_ss(tmem + COL_S + (t & 1) * S_COLS, dq + 2 * kk, dk + 2 * kk, idesc_qk, kk > 0 ? 1u : 0u);
        umma_commit(&s_full[t & 1]);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_qk(0);
      for (int it = 0; it < n_tiles && ok && !failed; ++it) {
        const int s = it % STAGES;
        if (it + 1 < n_tiles) {  // the next tile's scores are computed while this tile's softmax runs
          ok = issue_qk(it + 1);
          if (!ok) break;
        }
        ok = mbar_wait(p_full, it & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t dv = smem_desc_sw128(smem_u32(v_tiles + s * KV_BYTES));
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk)  // 16 keys = 16 rows of 128 bytes = 8 packed columns of P
          umma_ts(tmem + COL_O, tmem + COL_S + (it & 1) * S_COLS + 8 * kk, dv + (2048 >> 4) * kk,
                  idesc_pv, (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&kv_empty[s]);
        umma_commit(pv_done);
      }
      if (!ok) failed = 2;
    }
    __syncwarp();
  } else {
    // ---- softmax: thread r of warps 0..3 owns query row r (tensor-memory lane r)
    const int r = threadIdx.x;
    const int qpos = pos0 + q0 + r;
    const bool row_valid = r < rows_here;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    const float sl2 = a.scale * 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int it = 0; it < n_tiles && !failed; ++it) {
      ok = mbar_wait(&s_full[it & 1], (it >> 1) & 1);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t s_buf = lane_base + COL_S + (it & 1) * S_COLS;
      uint32_t sv[2][32];
      tmem_ld32(s_buf, sv[0]);
      tmem_ld32(s_buf + 32, sv[1]);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const int k0 = it * KT;
      // four independent chains for the maximum and for the sum: a single chain of 64 dependent
      // operations would leave the warp waiting on its own results
      float mx4[4] = {m_run, -INFINITY, -INFINITY, -INFINITY};
      if (k0 + KT - 1 > pos0 + q0) {  // a tile that reaches the diagonal: mask per element
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float v = (k0 + h * 32 + j <= qpos) ? __uint_as_float(sv[h][j]) : -INFINITY;
            sv[h][j] = __float_as_uint(v);
            mx4[j & 3] = fmaxf(mx4[j & 3], v);
          }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int j = 0; j < 32; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(sv[h][j]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_fin = (mx == -INFINITY) ? 0.f : mx;
      const float corr = ex2((m_run - m_fin) * sl2);  // m_run = -inf gives 0
      const float ms = m_fin * sl2;
      m_run = mx;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int h = j >> 4, c = (j & 15) * 2;
        const float p0 = ex2(fmaf(__uint_as_float(sv[h][c]), sl2, -ms));
        const float p1 = ex2(fmaf(__uint_as_float(sv[h][c + 1]), sl2, -ms));
        sum4[j & 3] += p0 + p1;
        pk[j] = pack2(p0, p1);  // element 2j in the low half, 2j+1 in the high half
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l_run = l_run * corr + sum;
      if (it > 0) {
        // O of the tiles so far must be complete (and P of the last tile consumed) before either
        // is overwritten
        ok = mbar_wait(pv_done, (it - 1) & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (!__all_sync(0xffffffffu, corr == 1.f)) {
          uint32_t ov[32];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            tmem_ld32(lane_base + COL_O + 32 * h, ov);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * corr);
            tmem_st32(lane_base + COL_O + 32 * h, ov);
          }
        }
      }
      tmem_st32(s_buf, pk);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (!ok) failed = 3;
    // ---- epilogue: O / l -> out
    if (ok && !failed && n_tiles > 0) {
      ok = mbar_wait(pv_done, (n_tiles - 1) & 1);
      if (!ok) failed = 4;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && !failed) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      bf16* dst = (bf16*)a.out + (size_t)(q_start + q0 + r) * a.out_row_stride + (size_t)head * HD;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t ov[32];
        tmem_ld32(lane_base + COL_O + 32 * h, ov);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row_valid) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 w;
            w.x = pack2(__uint_as_float(ov[j]) * inv, __uint_as_float(ov[j + 1]) * inv);
            w.y = pack2(__uint_as_float(ov[j + 2]) * inv, __uint_as_float(ov[j + 3]) * inv);
            w.z = pack2(__uint_as_float(ov[j + 4]) * inv, __uint_as_float(ov[j + 5]) * inv);
            w.w = pack2(__uint_as_float(ov[j + 6]) * inv, __uint_as_float(ov[j + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + h * 32 + j) = w;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && failed != 0) {
    if (p.error_flag) atomicExch(p.error_flag, 200 + failed);
    // copies that were requested must land before the block's shared memory is given up
    mbar_wait(q_full, 0);
    for (int c = max(0, issued - STAGES); c < issued; ++c)
      if (!mbar_wait(&kv_full[c % STAGES], (c / STAGES) & 1)) break;
  }
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS)
                 : "memory");
  }
}

inline bool supported(const LseAttnArgs* a) {
  const int pt = a->page_tokens;
  return a->dtype == LSE_BF16 && a->window == 0 && pt >= 8 && (pt & (pt - 1)) == 0 &&
         (a->q_row_stride % 8) == 0 && (a->out_row_stride % 8) == 0;
}

// total_rows: rows of the query tensor; pool_rows: pages * kv_heads * page_tokens.
inline int launch_prefill(const LseAttnArgs* a, long long total_rows, long long pool_rows,
                          int* error_flag, cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  const int box_rows = a->page_tokens < KT ? a->page_tokens : KT;
  if (!make_map_bf16(&mq, a->q, total_rows, (long long)a->num_heads * HD, a->q_row_stride, QT) ||
      !make_map_bf16(&mk, a->k_pages, pool_rows, HD, HD, box_rows) ||
      !make_map_bf16(&mv, a->v_pages, pool_rows, HD, HD, box_rows))
    return LSE_LAUNCH_FAILED;
  Params p;
  p.a = *a;
  p.box_rows = box_rows;
  p.page_shift = 0;
  while ((1 << p.page_shift) < a->page_tokens) ++p.page_shift;
  p.error_flag = error_flag;
  constexpr int smem = Q_BYTES + 2 * STAGES * KV_BYTES + (2 * STAGES + 5) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess)
      return LSE_LAUNCH_FAILED;
    configured = true;
  }
  dim3 grid(a->num_heads, a->num_tiles);
  return lse::launch(prefill_tc_kernel, grid, THREADS, smem, stream, mq, mk, mv, p) == cudaSuccess
             ? LSE_OK
             : LSE_LAUNCH_FAILED;
}

}  // namespace atc
}  // namespace lse
