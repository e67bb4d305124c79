// True 32-bit matrix product for the float32 path: C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]),
// plain FMA on the CUDA cores, no tensor-core mode of reduced precision.
// (The reference's float32 mode is cublasGemmEx with CUBLAS_COMPUTE_32F,
// kernels/cuda/kernels.cu:752-767.)
//
// Each output element is accumulated over k = 0..K-1 in that order by one thread, so a
// row's result does not depend on how many other rows the batch holds or where it stands.
#include <stdio.h>

#include "common.cuh"

namespace sllm {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                float* __restrict__ C, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  pdl_wait();
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // each thread loads 4 consecutive k of one row of A and of W per tile
  const int lr = tid / 4;            // 0..63 row within the tile
  const int lk = (tid % 4) * 4;      // 0,4,8,12
  const bool vec = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(W) & 15) == 0);

  for (int k0 = 0; k0 < K; k0 += BK) {
    float a[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
    const int gm = m0 + lr, gn = n0 + lr, gk = k0 + lk;
    if (gm < M) {
      if (vec && gk + 3 < K) {
        const float4 v = *reinterpret_cast<const float4*>(A + (size_t)gm * K + gk);
        a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) if (gk + i < K) a[i] = A[(size_t)gm * K + gk + i];
      }
    }
    if (gn < N) {
      if (vec && gk + 3 < K) {
        const float4 v = *reinterpret_cast<const float4*>(W + (size_t)gn * K + gk);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) if (gk + i < K) w[i] = W[(size_t)gn * K + gk + i];
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) { As[lk + i][lr] = a[i]; Ws[lk + i][lr] = w[i]; }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float av[TM], wv[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) av[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) wv[j] = Ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[(size_t)m * N + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K,
                              cudaStream_t stream) {
  SLLM_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
  if (M == 0) return SLLM_OK;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  SLLM_REQUIRE(grid.y <= 65535, "gemm_f32: M=%d is too large for one launch", M);
  launch_kernel(gemm_f32_kernel, grid, 256, 0, stream, A, W, bias, C, M, N, K);
  return launch_status("gemm_f32");
}
