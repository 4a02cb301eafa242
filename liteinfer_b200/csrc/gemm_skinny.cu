// out[M, N] = x[M, K] @ w[N, K]^T (+ bias) for bfloat16 and a handful of rows
// (M <= 64): the matrix product of a decode step, where every weight is read
// once and the time is the time to stream w from HBM.
//
// The weights are the 16-row operand of mma.sync m16n8k16 and the few rows of x
// are its 8-wide operand, so no tensor-core work is wasted on padding M.  Each
// thread reads its weights straight from global memory as 16-byte vectors in
// fragment order (the k index inside a 32-wide block is permuted the same way
// for both operands, which a sum over k does not notice), with many loads in
// flight and no shared-memory staging; x comes through L1/L2.  A block owns 16
// rows of w; its warps take interleaved 32-wide k blocks and add their partial
// sums through shared memory in a fixed order (32-bit).
#include "common.cuh"

namespace li {

constexpr int kSkinnyWarps = 8;
constexpr int kUnroll = 4;

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                          unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT>   // NT tiles of 8 rows of x
__global__ void __launch_bounds__(kSkinnyWarps * 32)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ bias,
                   bf16* __restrict__ out, int M, int N, int K) {
  __shared__ float partial[kSkinnyWarps][16][NT * 8 + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 16;
  // Rows past N read the last row again; their results are not stored.
  const bf16* w_lo = w + (size_t)min(row0 + g, N - 1) * K;
  const bf16* w_hi = w + (size_t)min(row0 + g + 8, N - 1) * K;
  const bf16* xr[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) xr[j] = x + (size_t)min(j * 8 + g, M - 1) * K;

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

  const int kblocks = (K + 31) / 32;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int kb0 = warp; kb0 < kblocks; kb0 += kSkinnyWarps * kUnroll) {
    uint4 wl[kUnroll], wh[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int k = (kb0 + u * kSkinnyWarps) * 32 + 8 * t;
      const bool in = k < K;
      wl[u] = in ? ldg_stream(w_lo + k) : zero;
      wh[u] = in ? ldg_stream(w_hi + k) : zero;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int k = (kb0 + u * kSkinnyWarps) * 32 + 8 * t;
      const bool in = k < K;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const uint4 xv = (in && j * 8 + g < M) ? *reinterpret_cast<const uint4*>(xr[j] + k) : zero;
        mma_16816(acc[j], wl[u].x, wh[u].x, wl[u].y, wh[u].y, xv.x, xv.y);
        mma_16816(acc[j], wl[u].z, wh[u].z, wl[u].w, wh[u].w, xv.z, xv.w);
      }
    }
  }

  // acc[j]: c0,c1 = (w row g, x rows j*8 + 2t, +1); c2,c3 = (w row g+8, same x rows).
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    partial[warp][g][j * 8 + 2 * t] = acc[j][0];
    partial[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
    partial[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
    partial[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 16 * NT * 8; e += kSkinnyWarps * 32) {
    const int r = e % 16, m = e / 16;     // consecutive threads write consecutive output columns
    const int n = row0 + r;
    if (m >= M || n >= N) continue;
    float sum = 0.f;
#pragma unroll
    for (int wv = 0; wv < kSkinnyWarps; ++wv) sum += partial[wv][r][m];
    if (bias) sum += __bfloat162float(bias[n]);
    out[(size_t)m * N + n] = __float2bfloat16_rn(sum);
  }
}

template <int NT>
int launch_skinny(const void* x, const void* w, const void* bias, void* out, int M, int N, int K, cudaStream_t s) {
  gemm_skinny_kernel<NT><<<(N + 15) / 16, kSkinnyWarps * 32, 0, s>>>((const bf16*)x, (const bf16*)w,
                                                                   (const bf16*)bias, (bf16*)out, M, N, K);
  LI_LAUNCH_CHECK();
}

}  // namespace li

using namespace li;

// bfloat16 only; 1 <= M <= 64; K a multiple of 8 and 16-byte aligned rows.
LI_EXPORT int li_gemm_skinny(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                             cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M > 64 || K < 8 || (K % 8)) return LI_ERR_UNSUPPORTED;
  if (!aligned16(x) || !aligned16(w)) return LI_ERR_ALIGNMENT;
  if (M <= 8) return launch_skinny<1>(x, w, bias, out, M, N, K, stream);
  if (M <= 16) return launch_skinny<2>(x, w, bias, out, M, N, K, stream);
  if (M <= 32) return launch_skinny<4>(x, w, bias, out, M, N, K, stream);
  return launch_skinny<8>(x, w, bias, out, M, N, K, stream);
}
