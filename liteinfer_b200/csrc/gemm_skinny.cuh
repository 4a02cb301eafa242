// The weight-streaming kernel of gemm_skinny.cu, shared with gemm_skinny_static.cu (same kernel, other
// scratch).  See gemm_skinny.cu for what it computes and how.
#pragma once
#include "common.cuh"

namespace li {

constexpr int kSkinnyWarps = 4;                                   // warps of the usual block; others have 2, 8 or 16
constexpr int kBlocksPerWarp = 8;                                  // 32-wide k blocks per warp and pass
constexpr int kMaxSlices = 16;
constexpr int kStatsFloats = 2048;                                  // parts x rows of statistics a block keeps in shared memory

// Copies `bytes` (4 or 16) from global to shared memory without passing through registers; the thread goes on.
__device__ __forceinline__ void copy_async_4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void copy_async_16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void copy_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

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

__device__ __forceinline__ float gated(float gate, float up, int act) {
  float a;
  switch (act) {
    case 0: a = gate / (1.0f + expf(-gate)); break;
    case 1: a = 0.5f * gate * (1.0f + erff(gate * 0.70710678118654752440f)); break;
    case 2: a = 0.5f * gate * (1.0f + tanhf(0.79788456080286535588f * (gate + 0.044715f * gate * gate * gate))); break;
    default: a = fmaxf(gate, 0.f);
  }
  return __bfloat162float(__float2bfloat16_rn(a)) * up;   // the activation is rounded before the multiply
}

struct SkinnyParams {
  const bf16* x;
  const bf16* w;
  const bf16* bias;
  bf16* out;
  int M, N, K;
  int slice_k;        // k per slice, a multiple of 32
  int num_slices;
  int gated_act;      // -1: plain product
  float* scratch;     // [tiles][num_slices][16][NT*8] partial tiles, when num_slices > 1
  unsigned* counters; // [tiles], zero between launches
  // A root-mean-square norm of x fused in (kernels built with kNorm): x holds unnormalised rows, norm_weight [K]
  // multiplies them on their way into the product, and the rows' inverse root mean squares multiply the sums at
  // the end.  The sums of squares come in parts (what the product before this one left: one part per 16 columns
  // it wrote), in_sumsq[part * in_stride + row], added here in a fixed order.
  const bf16* norm_weight = nullptr;
  const float* in_sumsq = nullptr;
  int in_parts = 0;
  int in_stride = 0;
  float eps = 0.f;
  const int* x_rows = nullptr;   // optional: row m of x is x[x_rows[m]] (and its statistics those of that row)
  // The residual sum fused in: out [M, N] is the residual stream; it becomes round(out + round(product)), and
  // out_sumsq[tile * out_stride + m] receives the sum of the squares of the tile's 16 new values of row m.
  float* out_sumsq = nullptr;
  int out_stride = 0;
};

// a * b for two pairs of bfloat16, each product rounded to bfloat16 (exact product, one rounding).
__device__ __forceinline__ unsigned mul_bf16x2(unsigned a, unsigned b) {
  unsigned d;
  asm("mul.rn.bf16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Starts the copy of the statistics' parts (if they fit) into the block's shared memory.
__device__ __forceinline__ void request_stats(const SkinnyParams& p, float* stats) {
  const int total = p.in_parts * p.in_stride;
  if (total > kStatsFloats) return;
  if ((total & 3) == 0 && aligned16(p.in_sumsq)) {
    for (int i = threadIdx.x * 4; i < total; i += blockDim.x * 4) copy_async_16(stats + i, p.in_sumsq + i);
  } else {
    for (int i = threadIdx.x; i < total; i += blockDim.x) copy_async_4(stats + i, p.in_sumsq + i);
  }
}

// NT tiles of 8 rows of x; kWarps warps share a slice's k blocks; kNorm: x is normalised on its way in.
template <int NT, int kWarps = kSkinnyWarps, bool kNorm = false>
__global__ void __launch_bounds__(kWarps * 32)
gemm_skinny_kernel(const SkinnyParams p) {
  constexpr int kCols = NT * 8;
  constexpr int kSlicePass = kWarps * kBlocksPerWarp * 32;   // k per pass of the block
  __shared__ float partial[4][16][kCols + 1];   // four warps' tiles at a time; [0] ends up holding the block's sum
  __shared__ float inv_rms[kNorm ? kCols : 1];
  __shared__ __align__(16) float stats[kNorm ? kStatsFloats : 4];   // the parts of the rows' sums of squares
  __shared__ bool is_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int tile = blockIdx.x, slice = blockIdx.y;
  const int row0 = tile * 16;
  const int K = p.K, M = p.M, N = p.N;
  // Rows past N read the last row again; their results are not stored.
  const bf16* w_lo = p.w + (size_t)min(row0 + g, N - 1) * K;
  const bf16* w_hi = p.w + (size_t)min(row0 + g + 8, N - 1) * K;
  const bf16* xr[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) xr[j] = p.x + (size_t)min(j * 8 + g, M - 1) * K;   // (gathered rows: set after the wait)

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

  const int k_begin = slice * p.slice_k, k_end = min(K, k_begin + p.slice_k);
  const uint4 zero = make_uint4(0, 0, 0, 0);
  bool waited = false;
  for (int pass = k_begin; pass < k_end; pass += kSlicePass) {
    uint4 wl[kBlocksPerWarp], wh[kBlocksPerWarp];
#pragma unroll
    for (int u = 0; u < kBlocksPerWarp; ++u) {
      const int k = pass + (u * kWarps + warp) * 32 + 8 * t;
      const bool in = k < k_end;
      wl[u] = in ? ldg_stream(w_lo + k) : zero;
      wh[u] = in ? ldg_stream(w_hi + k) : zero;
    }
    // The weights above depend on no earlier kernel and are already on their way; x does.
    if (!waited) {
      grid_dependency_wait();
      waited = true;
      if (kNorm) {
        if (p.x_rows) {
#pragma unroll
          for (int j = 0; j < NT; ++j) xr[j] = p.x + (size_t)p.x_rows[min(j * 8 + g, M - 1)] * K;
        }
        // The parts of the rows' sums of squares start on their way to shared memory; they are added up at
        // the very end, when they have long arrived.
        request_stats(p, stats);
      }
    }
#pragma unroll
    for (int u = 0; u < kBlocksPerWarp; ++u) {
      const int k = pass + (u * kWarps + warp) * 32 + 8 * t;
      const bool in = k < k_end;
      uint4 nw = zero;
      if (kNorm && in) nw = *reinterpret_cast<const uint4*>(p.norm_weight + k);
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        uint4 xv = (in && j * 8 + g < M) ? *reinterpret_cast<const uint4*>(xr[j] + k) : zero;
        if (kNorm) {
          xv.x = mul_bf16x2(xv.x, nw.x);
          xv.y = mul_bf16x2(xv.y, nw.y);
          xv.z = mul_bf16x2(xv.z, nw.z);
          xv.w = mul_bf16x2(xv.w, nw.w);
        }
        mma_16816(acc[j], wl[u].x, wh[u].x, wl[u].y, wh[u].y, xv.x, xv.y);
        mma_16816(acc[j], wl[u].z, wh[u].z, wl[u].w, wh[u].w, xv.z, xv.w);
      }
    }
  }

  if (!waited) {
    grid_dependency_wait();
    if (kNorm) request_stats(p, stats);
  }
  if (kNorm) {
    // One warp per row of x adds the parts of its sum of squares: lane by lane, then across the lanes, an order
    // that depends on nothing but the number of parts.  Read at the very end, behind block barriers.
    copy_async_wait_all();
    __syncthreads();
    const bool local = p.in_parts * p.in_stride <= kStatsFloats;
    for (int m = warp; m < M; m += kWarps) {
      const int src = p.x_rows ? p.x_rows[m] : m;
      float ss = 0.f;
      for (int i = lane; i < p.in_parts; i += 32)
        ss += local ? stats[i * p.in_stride + src] : __ldcg(p.in_sumsq + (size_t)i * p.in_stride + src);
      ss = warp_sum(ss);
      if (lane == 0) inv_rms[m] = 1.0f / sqrtf(ss / (float)K + p.eps);
    }
  }
  grid_launch_dependents();
  // acc[j]: c0,c1 = (w row g, x rows j*8 + 2t, +1); c2,c3 = (w row g+8, same x rows).
  // The warps' tiles are added in warp order, four warps per round through shared memory; every element of
  // the tile belongs to one thread, which keeps its running sum in a register.
  constexpr int kThreads = kWarps * 32;
  constexpr int kOwned = (16 * kCols + kThreads - 1) / kThreads;
  float running[kOwned];
#pragma unroll
  for (int i = 0; i < kOwned; ++i) running[i] = 0.f;
#pragma unroll
  for (int round = 0; round < (kWarps + 3) / 4; ++round) {
    if (warp / 4 == round) {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        partial[warp % 4][g][j * 8 + 2 * t] = acc[j][0];
        partial[warp % 4][g][j * 8 + 2 * t + 1] = acc[j][1];
        partial[warp % 4][g + 8][j * 8 + 2 * t] = acc[j][2];
        partial[warp % 4][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kOwned; ++i) {
      const int e = threadIdx.x + i * kThreads;
      if (e < 16 * kCols) {
        const int r = e % 16, m = e / 16;
#pragma unroll
        for (int wv = 0; wv < (kWarps < 4 ? kWarps : 4); ++wv) running[i] += partial[wv][r][m];
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < kOwned; ++i) {
    const int e = threadIdx.x + i * kThreads;
    if (e < 16 * kCols) partial[0][e % 16][e / 16] = running[i];   // read below by this thread only, or after a barrier
  }

  if (p.num_slices > 1) {
    float* mine = p.scratch + ((size_t)tile * p.num_slices + slice) * (16 * kCols);
    for (int e = threadIdx.x; e < 16 * kCols; e += kWarps * 32) mine[e] = partial[0][e % 16][e / 16];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned arrived = atomicAdd(&p.counters[tile], 1u);
      is_last = arrived == (unsigned)p.num_slices - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float* all = p.scratch + (size_t)tile * p.num_slices * (16 * kCols);
    for (int e = threadIdx.x; e < 16 * kCols; e += kWarps * 32) {
      // Every slice's value is requested before the first is added: one trip to L2, not one per slice.
      float v[kMaxSlices];
#pragma unroll
      for (int s = 0; s < kMaxSlices; ++s)
        if (s < p.num_slices) v[s] = __ldcg(all + (size_t)s * (16 * kCols) + e);
      float sum = 0.f;
#pragma unroll
      for (int s = 0; s < kMaxSlices; ++s)
        if (s < p.num_slices) sum += v[s];
      partial[0][e % 16][e / 16] = sum;
    }
    if (threadIdx.x == 0) p.counters[tile] = 0;   // ready for the next launch
  }
  __syncthreads();

  if (p.gated_act < 0 && p.out_sumsq) {
    // The residual sum: out = round(out + round(product)), and the squares of the tile's new values per row
    // (sixteen neighbouring lanes hold one row's sixteen columns).
    for (int e = threadIdx.x; e < 16 * kCols; e += kWarps * 32) {
      const int r = e % 16, m = e / 16;
      const int n = row0 + r;
      float sq = 0.f;
      if (m < M && n < N) {
        float sum = partial[0][r][m];
        if (kNorm) sum *= inv_rms[m];
        if (p.bias) sum += __bfloat162float(p.bias[n]);
        bf16* at = p.out + (size_t)m * N + n;
        const float h = __bfloat162float(__float2bfloat16_rn(__bfloat162float(*at) + __bfloat162float(__float2bfloat16_rn(sum))));
        *at = __float2bfloat16_rn(h);
        sq = h * h;
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (r == 0 && m < M) p.out_sumsq[(size_t)tile * p.out_stride + m] = sq;
    }
  } else if (p.gated_act < 0) {
    for (int e = threadIdx.x; e < 16 * kCols; e += kWarps * 32) {
      const int r = e % 16, m = e / 16;     // consecutive threads write consecutive output columns
      const int n = row0 + r;
      if (m >= M || n >= N) continue;
      float sum = partial[0][r][m];
      if (kNorm) sum *= inv_rms[m];
      if (p.bias) sum += __bfloat162float(p.bias[n]);
      p.out[(size_t)m * N + n] = __float2bfloat16_rn(sum);
    }
  } else {
    const int half = N / 2;                 // rows [0, 8) of the tile are gate rows, [8, 16) their up rows
    for (int e = threadIdx.x; e < 8 * kCols; e += kWarps * 32) {
      const int r = e % 8, m = e / 8;
      const int n = tile * 8 + r;
      if (m >= M || n >= half) continue;
      float gate = partial[0][r][m], up = partial[0][r + 8][m];
      if (kNorm) {
        gate *= inv_rms[m];
        up *= inv_rms[m];
      }
      if (p.bias) {
        gate += __bfloat162float(p.bias[row0 + r]);
        up += __bfloat162float(p.bias[row0 + r + 8]);
      }
      // The products are rounded to bfloat16 before the activation, as a separate kernel would see them.
      gate = __bfloat162float(__float2bfloat16_rn(gate));
      up = __bfloat162float(__float2bfloat16_rn(up));
      p.out[(size_t)m * half + n] = __float2bfloat16_rn(gated(gate, up, p.gated_act));
    }
  }
}

// How narrow blocks (four warps) cut k for a weight of [N, K]: (slices, k per slice).  Slices are at least 512
// wide and are used only while there are too few 16-row tiles to occupy the GPU.
inline int skinny_slices(int N, int K, int* slice_k) {
  const int tiles = (N + 15) / 16;
  int slices = 1024 / tiles;
  const int most = K / 512;
  if (slices > most) slices = most;
  if (slices > kMaxSlices) slices = kMaxSlices;
  if (slices < 1) slices = 1;
  int per = (K + slices - 1) / slices;
  per = (per + 31) / 32 * 32;
  slices = (K + per - 1) / per;
  if (slice_k) *slice_k = per;
  return slices;
}

// The plan for at most eight rows of x: warps per block (4, 8 or 16) and slices of k.  A weight with few
// 16-row tiles is better served by wider blocks, whose warps add up through shared memory, than by slices,
// which add up through scratch memory and a counter.  Measured on B200 at 8 rows: 3072 x 2048 with 8 warps
// uncut 4.3 us (4 warps in 4 slices: 7.4 us); 2048 x 2048 likewise 3.7 us (5.5 us); 2048 x 8192 with 16
// warps uncut 9.2 us (4 warps in 8 slices: 12.1 us); 16384 x 2048 with 2 warps 13.8 us (4 warps: 15.3 us: its
// 1,024 blocks came to a wave and a third).
// The aim is some 2,400 warps in all with at least one full pass (256 k) each; k is cut only if wide blocks
// still leave the GPU half empty and the slices stay long.
inline int skinny_plan(int N, int K, int* warps_out, int* slice_k) {
  const int tiles = (N + 15) / 16;
  int warps = tiles > 5 * 148 ? 2 : 4;   // more tiles than blocks of four warps fit at once: blocks of two, twice as many at once
  while (warps >= 4 && warps < 16 && tiles * warps < 2400 && K / (2 * warps) >= 256) warps *= 2;
  int slices = 1;
  while (slices < kMaxSlices && tiles * warps * (slices + 1) <= 1200 && K / (slices + 1) >= warps * 512) ++slices;
  int per = (K + slices - 1) / slices;
  per = (per + 31) / 32 * 32;
  slices = (K + per - 1) / per;
  if (warps_out) *warps_out = warps;
  if (slice_k) *slice_k = per;
  return slices;
}

}  // namespace li
