// out[M, N] = x[M, K] @ w[N, K]^T (+ bias[N]) in plain FFMA code with 32-bit
// accumulation: the matrix product of the true 32-bit path (tensor cores have no
// full-precision 32-bit mode), also instantiated for bfloat16 storage as the path
// for shapes the tensor-core kernels refuse.
//
// Every output element adds its K products in the same order (k ascending,
// one accumulator), whatever M and N are, so a row's result does not depend on
// which other rows are in the batch.
#include "common.cuh"

namespace li {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ out,
                 int M, int N, int K) {
  __shared__ float xs[BK][BM + 1];
  __shared__ float ws[BK][BN + 1];
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int lr = threadIdx.x / 4;         // 0..63: tile row this thread loads
  const int lk = (threadIdx.x % 4) * 4;   // 0,4,8,12: first of its four k
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      const int m = m0 + lr, n = n0 + lr;
      xs[lk + i][lr] = (m < M && k < K) ? to_float(x[(size_t)m * K + k]) : 0.f;
      ws[lk + i][lr] = (n < N && k < K) ? to_float(w[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += to_float(bias[n]);
      out[(size_t)m * N + n] = from_float<T>(v);
    }
  }
}

}  // namespace li

using namespace li;

LI_EXPORT int li_gemm_simt(int dtype, const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                           cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return LI_ERR_UNSUPPORTED;
  if (dtype == kFloat32)
    gemm_simt_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (const float*)w, (const float*)bias,
                                                      (float*)out, M, N, K);
  else
    gemm_simt_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)x, (const bf16*)w, (const bf16*)bias, (bf16*)out, M,
                                                     N, K);
  LI_LAUNCH_CHECK();
}
