// bfloat16 matrix product for few rows (decode), on the 5th-generation tensor cores:
//   out[T, N] += a[T, K] . w[N, K]^T        T <= 32, float32 accumulation in the tensor cores
//
// With few rows the product is bound by streaming the weights once from HBM, so the operands are
// swapped: the *weights* are the 128-row operand of tcgen05.mma (M = 128 output features per
// block) and the tokens are its N dimension (16 or 32). Both operands are K-major in global memory
// already, so TMA brings [rows, 64] tiles straight into 128-byte-swizzled shared memory. One
// elected thread issues tcgen05.mma (cta_group::1, kind::f16) with the accumulator [128 x T] in
// tensor memory; another thread runs the TMA pipeline; all four warps read the accumulator back
// with tcgen05.ld and write out[t, n] with n across lanes (coalesced).
//
// The kernel is persistent: blocks walk contiguous ranges of (tile, k stage) units, balanced over
// all blocks whatever N is, so a tile's K may be shared by several blocks. The output is a buffer
// of 64-bit fixed-point numbers (LSE_FIXED64) to which every block *adds* its partial sums with
// integer atomics: value * 2^24, rounded to an integer. Integer addition is associative, so the
// order in which the blocks arrive does not matter: the same inputs give the same bits on every
// run, and a row's sum does not depend on the other rows of the batch (a float32 atomic sum would
// depend on the order). The kernel that consumes the buffer converts back and clears it.
//
// Every wait on an mbarrier is bounded: on expiry the block records an error code in *error_flag
// and leaves through the normal teardown (tensor memory is released).
#include "kernels.h"
#include "tma_util.cuh"

namespace lse {
namespace tc {

constexpr int BM = 128;        // output features per block (MMA M)
constexpr int BK = 64;         // k elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;

using namespace tma;

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc,
                                     uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct Params {
  int T, N, K;
  int tiles, chunks;      // output tiles of 128 features; k stages of 64 per tile
  unsigned long long* out;  // [T, N] fixed-point sums
  const bf16* bias;       // [N] or nullptr (added with the first k stage of a tile)
  int* error_flag;
};

// Work of one block: units [u_begin, u_end) of the sequence (tile 0 stage 0, tile 0 stage 1, ...).
__device__ __forceinline__ void block_range(const Params& p, long long& u_begin, long long& u_end) {
  const long long G = gridDim.x, g = blockIdx.x;
  const long long U = (long long)p.tiles * p.chunks;
  u_begin = g * U / G;
  u_end = (g + 1) * U / G;
}

// Persistent, warp-specialised kernel. 192 threads: warp 0 runs the TMA pipeline, warp 1 issues the
// MMAs, warps 2..5 read accumulators back and write the output. A block walks a contiguous range
// of (tile, k stage) units; each maximal run of units of one tile is a *segment* with its own
// accumulator in tensor memory. Two accumulators alternate, so the epilogue of one segment overlaps
// the loads and MMAs of the next.
// NT: tokens per block, padded (MMA N): 16 or 32. STAGES: pipeline depth.
template <int NT, int STAGES>
__global__ void __launch_bounds__(192)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                   const Params p) {
  constexpr uint32_t W_BYTES = BM * BK * 2, A_BYTES = NT * BK * 2;
  constexpr uint32_t ACC_COLS = NT < 16 ? 16 : NT;
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // 1024-byte alignment of the tiles is required by the swizzled descriptors
  unsigned char* base = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* w_tiles = base;
  unsigned char* a_tiles = base + STAGES * W_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(a_tiles + STAGES * A_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  __shared__ volatile int failed;
  __shared__ volatile int issued;  // stages the producer has requested from TMA

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long u_begin, u_end;
  block_range(p, u_begin, u_end);
  const int my_units = (int)(u_end - u_begin);
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    failed = 0;
    issued = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {  // one warp allocates tensor memory for the block
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  // Dependents may become resident only now that this block holds its tensor memory: one that
  // allocated columns first and then sat in its dependency wait could block this allocation.
  pdl_trigger();

  // Lanes 1..31 of the two role warps wait at __syncwarp, not on a barrier: a lane that spins in
  // try_wait would take turns with the role lane of its own warp and stall the pipeline.
  if (my_units > 0 && warp == 0) {
    if (lane == 0) {
      // ---- TMA producer: one (weights, activations) stage per unit. The weights depend on no
      // earlier kernel, so the first STAGES weight tiles are requested before pdl_wait(); the
      // activations (written by the kernel before this one) only after it.
      const int early = min(my_units, STAGES);
      for (int it = 0; it < early; ++it) {
        const long long u = u_begin + it;
        const int tile = (int)(u / p.chunks), kc = (int)(u - (long long)tile * p.chunks);
        mbar_expect_tx(&full[it], W_BYTES + A_BYTES);
        tma_load_2d(w_tiles + it * W_BYTES, &map_w, &full[it], kc * BK, tile * BM);
        issued = it + 1;
      }
      pdl_wait();
      for (int it = 0; it < my_units && !failed; ++it) {
        const int s = it % STAGES;
        const long long u = u_begin + it;
        const int tile = (int)(u / p.chunks), kc = (int)(u - (long long)tile * p.chunks);
        if (it >= STAGES) {
          if (!mbar_wait(&empty[s], ((it / STAGES) - 1) & 1)) {
            failed = 1;
            break;
          }
          mbar_expect_tx(&full[s], W_BYTES + A_BYTES);
          tma_load_2d(w_tiles + s * W_BYTES, &map_w, &full[s], kc * BK, tile * BM);
        }
        tma_load_2d(a_tiles + s * A_BYTES, &map_a, &full[s], kc * BK, 0);
        issued = it + 1;
      }
    }
    __syncwarp();
  } else if (my_units > 0 && warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer
      constexpr uint32_t idesc = instr_desc_bf16(BM, NT);
      int it = 0, seg = 0;
      while (it < my_units && !failed) {
        const long long u0 = u_begin + it;
        const int tile = (int)(u0 / p.chunks);
        const int seg_units = (int)min((long long)my_units - it, (long long)(tile + 1) * p.chunks - u0);
        const int b = seg & 1;
        if (seg >= 2 && !mbar_wait(&acc_empty[b], ((seg >> 1) - 1) & 1)) {
          failed = 2;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + b * ACC_COLS;
        bool ok = true;
        for (int j = 0; j < seg_units; ++j, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&full[s], (it / STAGES) & 1);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t da = smem_desc_sw128(smem_u32(w_tiles + s * W_BYTES));
          const uint64_t db = smem_desc_sw128(smem_u32(a_tiles + s * A_BYTES));
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // 16 k-elements = 32 bytes further along the swizzled row: +2 in the address field
            umma(tmem_d, da + 2 * kk, db + 2 * kk, idesc, (j > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);  // arrives when the MMAs that read this stage are done
        }
        if (!ok) {
          failed = 3;
          break;
        }
        umma_commit(&acc_full[b]);
        ++seg;
      }
    }
    __syncwarp();
  } else if (my_units > 0 && warp >= 2) {
    // ---- epilogue: warp w may read TMEM lanes 32*(w%4) .. +31, i.e. accumulator rows of that quarter
    const int quarter = warp & 3;
    pdl_wait();  // the output may still be read or written by the kernels before this one
    int it = 0, seg = 0;
    while (it < my_units && !failed) {
      const long long u0 = u_begin + it;
      const int tile = (int)(u0 / p.chunks), kc0 = (int)(u0 - (long long)tile * p.chunks);
      const int seg_units = (int)min((long long)my_units - it, (long long)(tile + 1) * p.chunks - u0);
      const int b = seg & 1;
      if (!mbar_wait(&acc_full[b], (seg >> 1) & 1)) {
        failed = 4;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int n = tile * BM + quarter * 32 + lane;
      const float bias = (p.bias && kc0 == 0 && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll 1
      for (int t0 = 0; t0 < NT && t0 < p.T; t0 += 16) {
        uint32_t v[16];
        const uint32_t taddr = tmem_base + b * ACC_COLS + ((uint32_t)(quarter * 32) << 16) + (uint32_t)t0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,"
            "%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
              "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
              "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + j;
            if (t >= p.T) break;
            const float val = __uint_as_float(v[j]) + bias;
            const size_t o = (size_t)t * p.N + n;
            atomicAdd(p.out + o, (unsigned long long)__float2ll_rn(val * kFixedScale));
          }
        }
      }
      // this accumulator may be overwritten once all four epilogue warps have read it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0)
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[b])) : "memory");
      it += seg_units;
      ++seg;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();  // every role is done; `failed` is final
  if (threadIdx.x == 0 && failed != 0) {
    if (p.error_flag) atomicExch(p.error_flag, 100 + failed);
    // copies that were requested must land before the block's shared memory is given up
    for (int c = max(0, issued - STAGES); c < issued; ++c)
      if (!mbar_wait(&full[c % STAGES], (c / STAGES) & 1)) break;
  }
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------- host side
template <int NT, int STAGES>
static int launch(const CUtensorMap& mw, const CUtensorMap& ma, const Params& p, int grid,
                  cudaStream_t stream) {
  constexpr int smem = STAGES * (BM * BK * 2 + NT * BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(skinny_gemm_kernel<NT, STAGES>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return LSE_LAUNCH_FAILED;
    configured = true;
  }
  return lse::launch(skinny_gemm_kernel<NT, STAGES>, grid, 192, smem, stream, mw, ma, p) == cudaSuccess
             ? LSE_OK
             : LSE_LAUNCH_FAILED;
}

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 1;
  }
  return n;
}

}  // namespace tc
}  // namespace lse

using namespace lse;

extern "C" int lse_gemm_bf16_skinny_max_rows(void) { return 32; }

extern "C" int lse_gemm_bf16_skinny(const void* a, const void* w, const void* bias, void* out,
                                    int T, int N, int K, int* error_flag, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return LSE_OK;
  if (T > 32 || K <= 0 || K % 8) return LSE_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) return LSE_BAD_ARGUMENT;
  if (!out || (reinterpret_cast<uintptr_t>(out) & 7)) return LSE_BAD_ARGUMENT;
  const int nt = T <= 16 ? 16 : 32;
  CUtensorMap mw, ma;
  if (!tma::make_map_bf16(&mw, w, N, K, K, tc::BM) || !tma::make_map_bf16(&ma, a, T, K, K, nt)) return LSE_LAUNCH_FAILED;
  tc::Params p;
  p.T = T; p.N = N; p.K = K;
  p.tiles = (N + tc::BM - 1) / tc::BM;
  p.chunks = (K + tc::BK - 1) / tc::BK;
  p.out = reinterpret_cast<unsigned long long*>(out);
  p.bias = reinterpret_cast<const bf16*>(bias); p.error_flag = error_flag;
  const long long units = (long long)p.tiles * p.chunks;
  // Shallow pipelines and many blocks. Measured in whole decode steps (SmolLM2-1.7B sizes): up to 16
  // rows, four blocks per SM of two stages each (37 KB) give 1.62 ms at batch 8 and 859 tok/s at
  // batch 1, where two blocks of five stages (94 KB each) gave 1.71 ms and 768 tok/s: the blocks
  // of the next product fit beside the running ones and ask for their first weights early, and the
  // attention blocks between two products are not kept off the SM. 17 to 32 rows: two blocks of
  // three stages (3.38 ms at batch 32; four of two 3.95, two of five 3.86).
  const int per_sm = nt == 16 ? 4 : 2;
  int grid = tc::sm_count() * per_sm;
  if (units < grid) grid = (int)units;
  return nt == 16 ? tc::launch<16, 2>(mw, ma, p, grid, stream) : tc::launch<32, 3>(mw, ma, p, grid, stream);
}
