// True float32 matrix product on the CUDA cores (no tensor-core mode, no reduced precision):
//   out[T, N] = a[T, K] . w[N, K]^T (+ bias[N])
// Every output element is accumulated by one thread over k = 0 .. K-1 in ascending order with
// fused multiply-adds, so the value of a row does not depend on how many other rows are in the
// batch or on where the row sits in it.
#include "common.cuh"
#include "kernels.h"

namespace lse {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ a, const float* __restrict__ w,
                const float* __restrict__ bias, float* __restrict__ out, int T, int N, int K) {
  __shared__ float as[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * TM, tn = (tid % 16) * TN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // each thread loads 4 consecutive k of one row of each tile
  const int lr = tid / 4, lk = (tid % 4) * 4;
  const bool vec_ok = (K % 4 == 0);
  for (int k0 = 0; k0 < K; k0 += BK) {
    float av[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
    const int gm = m0 + lr, gn = n0 + lr, gk = k0 + lk;
    if (gm < T) {
      if (vec_ok && gk + 3 < K) {
        const float4 v = *reinterpret_cast<const float4*>(a + (size_t)gm * K + gk);
        av[0] = v.x; av[1] = v.y; av[2] = v.z; av[3] = v.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) if (gk + j < K) av[j] = a[(size_t)gm * K + gk + j];
      }
    }
    if (gn < N) {
      if (vec_ok && gk + 3 < K) {
        const float4 v = *reinterpret_cast<const float4*>(w + (size_t)gn * K + gk);
        wv[0] = v.x; wv[1] = v.y; wv[2] = v.z; wv[3] = v.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) if (gk + j < K) wv[j] = w[(size_t)gn * K + gk + j];
      }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      as[lk + j][lr] = av[j];
      ws[lk + j][lr] = wv[j];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float ar[TM], wr[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) ar[i] = as[kk][tm + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) wr[j] = ws[kk][tn + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + tm + i;
    if (gm >= T) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tn + j;
      if (gn < N) out[(size_t)gm * N + gn] = acc[i][j] + (bias ? bias[gn] : 0.f);
    }
  }
}

}  // namespace lse

extern "C" int lse_gemm_f32(const float* a, const float* w, const float* bias, float* out, int T,
                            int N, int K, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return LSE_OK;
  if (K <= 0) return LSE_BAD_ARGUMENT;
  dim3 grid((N + lse::BN - 1) / lse::BN, (T + lse::BM - 1) / lse::BM);
  if (grid.y > 65535) return LSE_BAD_ARGUMENT;
  lse::gemm_f32_kernel<<<grid, 256, 0, stream>>>(a, w, bias, out, T, N, K);
  return cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED;
}
