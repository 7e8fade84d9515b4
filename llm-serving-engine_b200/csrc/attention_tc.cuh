// Flash-style causal attention for portions of prompts on the 5th-generation tensor cores
// (head size 64, bfloat16, no window, page size a power of two >= 8).
//
// One block = 128 query rows of one head. Per tile of 64 keys:
//   S = Q K^T        tcgen05.mma, A = Q tile and B = K tile in shared memory (both K-major, TMA with
//                    128-byte swizzle, K tiles fetched page by page through the block table),
//                    accumulator S [128 x 64] float32 in tensor memory;
//   softmax          256 threads, two per query row: the keys of every tile are dealt to two
//                    *streams* (keys 0-31 and 32-63 of the tile), and each stream is a complete
//                    online softmax of its own: tcgen05.ld of its 32 scores, running maximum and sum
//                    in float32 (base-2 exponent, scale folded into the multiply-add), P rounded to
//                    bfloat16 and written back to tensor memory with tcgen05.st. The two threads of
//                    a row never talk to each other until the end, so twice as many independent
//                    instruction chains hide the latencies of tensor memory and of the exp unit;
//   O_s += P_s V_s   per stream s: tcgen05.mma with A = P from tensor memory and B = the stream's 32
//                    rows of the V tile in shared memory (N-major: rows are keys), accumulator
//                    O_s [128 x 64] float32 in tensor memory;
//   end              O = (O_0 w_0 + O_1 w_1) / (l_0 w_0 + l_1 w_1), w_s = 2^(m_s - max m): each thread
//                    of a row writes half of the head dims.
// A stream's reference maximum moves only when a row of the warp outgrows it by 2^8; only then is
// its O rescaled in tensor memory (tcgen05.ld / st) before its next P V. Warps 0-3 are stream 0 and warps 4-7
// stream 1 (warp w owns tensor-memory lanes 32 (w mod 4) ..), one lane of warp 8 runs the TMA
// pipeline, one lane of warp 9 issues the MMAs. Every barrier wait is bounded.
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
constexpr int SOFTMAX_WARPS = 8;  // two streams of four warps
constexpr int THREADS = (SOFTMAX_WARPS + 2) * 32;
constexpr uint32_t Q_BYTES = QT * HD * 2, KV_BYTES = KT * HD * 2;
// Tensor-memory columns. S is double-buffered so that Q K^T of the next tile runs while the
// softmax threads work on this one. A stream's P (16 packed columns) is written over the start of
// that stream's own 32 columns of the S buffer once they are in registers; MMAs of one thread run
// in issue order, so a later Q K^T into that buffer cannot overtake the P V that still reads P.
constexpr uint32_t COL_S = 0, S_COLS = 64, COL_O = 128, O_COLS = 64, TMEM_COLS = 256;

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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
        "=r"(v[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
        "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
        "r"(v[15])
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
  uint64_t* p_full = s_full + 2;           // [stream][tile & 1] the stream's P is written (and its O
                                           // rescaled): 4 arrivals
  uint64_t* pv_done = p_full + 4;          // [2] O_s += P_s V_s of this tile has finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  __shared__ float pair_m[2][QT], pair_l[2][QT];  // the streams' final maxima and sums
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
    for (int b = 0; b < 4; ++b) mbar_init(&p_full[b], 4);
    mbar_init(&pv_done[0], 1);
    mbar_init(&pv_done[1], 1);
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
  // Dependents may become resident only now that this block holds its tensor memory: a dependent
  // that allocated columns first and then sat in its dependency wait could keep this block
  // waiting in tcgen05.alloc for ever.
  pdl_trigger();
  pdl_wait();  // queries, keys and values were written by the kernel before this one

  if (warp == SOFTMAX_WARPS) {
    // ---- TMA producer. The whole warp looks up block-table entries, one box of a key/value tile
    // per lane and 32 boxes at a time, so that the lookups of several tiles are one round trip
    // to memory; lane 0 then waits for free stages and issues the copies, with the rows handed
    // over by shuffles. The other lanes rest at the warp barrier meanwhile.
    if (lane == 0) {
      mbar_expect_tx(q_full, Q_BYTES);
      tma_load_2d(q_tile, &map_q, q_full, head * HD, q_start + q0);
    }
    const int* table = a.block_tables + (size_t)seq * a.table_stride;
    const int last_page_idx = (k_end - 1) >> p.page_shift;
    const int boxes = KT / p.box_rows;  // 1, 2, 4 or 8
    const int group = 32 / boxes;       // tiles looked up together
    int ok = 1;
    for (int g0 = 0; g0 < n_tiles && ok; g0 += group) {
      const int t_l = g0 + lane / boxes, b_l = lane % boxes;
      int row_l = 0;
      if (t_l < n_tiles) {
        const int j = t_l * KT + b_l * p.box_rows;
        // a box past the context re-reads the last valid page: its keys are masked anyway,
        // and what it brings is finite
        const int pi = min(j >> p.page_shift, last_page_idx);
        const int off = (j >> p.page_shift) <= last_page_idx ? (j & (a.page_tokens - 1)) : 0;
        row_l = (table[pi] * a.num_kv_heads + kvh) * a.page_tokens + off;
      }
      const int g_end = min(g0 + group, n_tiles);
      for (int t = g0; t < g_end && ok; ++t) {
        int rows[8];
#pragma unroll
        for (int b = 0; b < 8; ++b) rows[b] = __shfl_sync(0xffffffffu, row_l, ((t - g0) * boxes + b) & 31);
        if (lane == 0) {
          const int s = t % STAGES;
          if (failed || (t >= STAGES && !mbar_wait(&kv_empty[s], ((t / STAGES) - 1) & 1))) {
            failed = 1;
            ok = 0;
          } else {
            mbar_expect_tx(&kv_full[s], 2 * KV_BYTES);
#pragma unroll
            for (int b = 0; b < 8; ++b) {
              if (b < boxes) {
                tma_load_2d(k_tiles + s * KV_BYTES + b * p.box_rows * HD * 2, &map_k, &kv_full[s], 0, rows[b]);
                tma_load_2d(v_tiles + s * KV_BYTES + b * p.box_rows * HD * 2, &map_v, &kv_full[s], 0, rows[b]);
              }
            }
            issued = t + 1;
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
      }
    }
  } else if (warp == SOFTMAX_WARPS + 1) {
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
        const uint64_t dv = smem_desc_sw128(smem_u32(v_tiles + s * KV_BYTES));
#pragma unroll
        for (int st = 0; st < 2; ++st) {
          ok = mbar_wait(&p_full[2 * st + (it & 1)], (it >> 1) & 1);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int kk = 0; kk < 2; ++kk)  // 16 keys = 16 rows of 128 bytes = 8 packed columns of P
            umma_ts(tmem + COL_O + st * O_COLS, tmem + COL_S + (it & 1) * S_COLS + 32 * st + 8 * kk,
                    dv + (2048 >> 4) * (2 * st + kk), idesc_pv, (it > 0 || kk > 0) ? 1u : 0u);
          if (st == 1) umma_commit(&kv_empty[s]);
          umma_commit(&pv_done[st]);
        }
        if (!ok) break;
      }
      if (!ok) failed = 2;
    }
    __syncwarp();
  } else {
    // ---- softmax: threads r and 128 + r own query row r (tensor-memory lane r); the first is
    // stream 0 (keys 0-31 of every tile), the second stream 1 (keys 32-63)
    const int st = warp >> 2, wq = warp & 3;
    const int r = wq * 32 + lane;
    const int qpos = pos0 + q0 + r;
    const bool row_valid = r < rows_here;
    const uint32_t lane_base = tmem + ((uint32_t)(wq * 32) << 16);
    const uint32_t o_col = lane_base + COL_O + st * O_COLS;
    const float sl2 = a.scale * 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int it = 0; it < n_tiles && !failed; ++it) {
      ok = mbar_wait(&s_full[it & 1], (it >> 1) & 1);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t s_buf = lane_base + COL_S + (it & 1) * S_COLS + 32 * st;
      uint32_t sv[32];
      tmem_ld32(s_buf, sv);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const int k0 = it * KT + 32 * st;
      // four independent chains for the maximum and for the sum: a single chain of dependent
      // operations would leave the warp waiting on its own results
      float mx4[4] = {m_run, -INFINITY, -INFINITY, -INFINITY};
      if (k0 + 31 > pos0 + q0) {  // keys that reach the diagonal: mask per element
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float v = (k0 + j <= qpos) ? __uint_as_float(sv[j]) : -INFINITY;
          sv[j] = __float_as_uint(v);
          mx4[j & 3] = fmaxf(mx4[j & 3], v);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(sv[j]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // The reference maximum of the exponent moves only when some row of the warp has outgrown
      // it by a factor 2^8: until then P may reach 256 (exact enough in bfloat16, sums are
      // float32) and O needs no rescaling, so most tiles neither touch O nor wait for the P V
      // before them. (-inf) - (-inf) is NaN and compares false: a row without keys asks for nothing.
      const bool grow = __any_sync(0xffffffffu, (mx - m_run) * sl2 > 8.f);
      const float m_new = grow ? mx : m_run;
      const float m_fin = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = grow ? ex2((m_run - m_fin) * sl2) : 1.f;  // m_run = -inf gives 0
      const float ms = m_fin * sl2;
      m_run = m_new;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float p0 = ex2(fmaf(__uint_as_float(sv[2 * j]), sl2, -ms));
        const float p1 = ex2(fmaf(__uint_as_float(sv[2 * j + 1]), sl2, -ms));
        sum4[j & 3] += p0 + p1;
        pk[j] = pack2(p0, p1);  // element 2j in the low half, 2j+1 in the high half
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l_run = l_run * corr + sum;
      if (it > 0 && grow) {
        // this stream's O of the tiles so far must be complete before it is rescaled
        ok = mbar_wait(&pv_done[st], (it - 1) & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t ov[16];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          tmem_ld16(o_col + 16 * h, ov);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 16; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * corr);
          tmem_st16(o_col + 16 * h, ov);
        }
      }
      tmem_st16(s_buf, pk);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      // Even and odd tiles arrive on different barriers. A warp that does not wait for the P V
      // of the tile before may be a tile ahead of the other warps of its stream, and of the MMA
      // thread; it can be two tiles ahead of neither, because S of tile it + 2 is computed only
      // after the MMA thread has seen every arrival of tile it. So an arrival is never counted
      // for a phase that is still collecting an earlier tile, and the MMA thread never finds a
      // barrier two phases on.
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[2 * st + (it & 1)]);
    }
    if (!ok) failed = 3;
    // ---- epilogue: the two streams of a row are merged; each of its threads writes 32 head dims
    pair_m[st][r] = m_run;
    pair_l[st][r] = l_run;
    if (ok && !failed && n_tiles > 0) {
      ok = mbar_wait(&pv_done[0], (n_tiles - 1) & 1) && mbar_wait(&pv_done[1], (n_tiles - 1) & 1);
      if (!ok) failed = 4;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");  // the softmax warps only
    if (ok && !failed) {
      const float m0 = pair_m[0][r], m1 = pair_m[1][r];
      const float mm = fmaxf(m0, m1);
      const float w0 = (m0 == -INFINITY) ? 0.f : ex2((m0 - mm) * sl2);
      const float w1 = (m1 == -INFINITY) ? 0.f : ex2((m1 - mm) * sl2);
      const float l = pair_l[0][r] * w0 + pair_l[1][r] * w1;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const float f0 = w0 * inv, f1 = w1 * inv;
      bf16* dst = (bf16*)a.out + (size_t)(q_start + q0 + r) * a.out_row_stride + (size_t)head * HD + 32 * st;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t oa[16], ob[16];
        tmem_ld16(lane_base + COL_O + 32 * st + 16 * h, oa);
        tmem_ld16(lane_base + COL_O + O_COLS + 32 * st + 16 * h, ob);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row_valid) {
#pragma unroll
          for (int j = 0; j < 16; j += 8) {
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              o[e] = __uint_as_float(oa[j + e]) * f0 + __uint_as_float(ob[j + e]) * f1;
            uint4 w;
            w.x = pack2(o[0], o[1]);
            w.y = pack2(o[2], o[3]);
            w.z = pack2(o[4], o[5]);
            w.w = pack2(o[6], o[7]);
            *reinterpret_cast<uint4*>(dst + 16 * h + j) = w;
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
  constexpr int smem = Q_BYTES + 2 * STAGES * KV_BYTES + (2 * STAGES + 9) * 8 + 16 + 1024;
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
