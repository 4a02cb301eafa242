// out[M, N] = x[M, K] @ w[N, K]^T (+ bias) for bfloat16 and at most 16 rows of x: the product of a decode step as
// a stream of TMA copies.
//
// The time of such a product is the time to read w once.  A block here stays on its SM and walks over 16-row
// tiles of w; each of its warps owns a ring of shared-memory stages and keeps it full by itself: one lane asks
// the TMA unit for the next 16 rows x 128 k of the warp's share of the tile (two boxes of 16 x 64 with the
// 128-byte swizzle, 4 KB behind one mbarrier), the warp waits for the oldest stage, multiplies it
// (mma.sync m16n8k16 with the weights as the 16-row operand and the rows of x as the 8-wide one; both operands are
// read 16 bytes per lane with k permuted alike on both sides, which a sum over k does not notice) and hands the
// stage back.  Nothing passes through registers on its way in, so what is in flight is bounded by shared memory,
// not by registers: eight warps x three stages = 96 KB a block, of which 64 KB are on their way at any time.
//
// Because w depends on no earlier kernel, a block fills its rings before it waits for the kernel ahead of it
// (programmatic dependent launch), and it lets the kernel behind it start at once: with at most one block of 97 KB
// per SM, two such kernels fit on an SM side by side, so the next product's first 14 MB are on their way while
// this one still runs, and a chain of products reads memory without the pause that a launch otherwise costs.
//
// The warps of a block split a tile's k among them (chunk c goes to warp c mod 8) and add their partial tiles
// through shared memory in warp order at the end of each tile; the order of every sum is fixed by the shapes.
// Epilogues: bias; act(gate) * up on weights whose rows are interleaved in eights; or the residual sum
// (out += product) with the new rows' sums of squares per tile.
//
// Every wait is bounded: a wait that runs out raises the error flag, lets the copies still on their way land (a
// bounded wait again) and ends the block's work.
#include <map>
#include <mutex>
#include <tuple>

#include "gemm_skinny.cuh"
#include "tcgen05.cuh"

namespace li {

constexpr int kChunkK = 128;                         // k per stage
constexpr unsigned kStageBytes = 16 * kChunkK * 2;   // 4 KB: two boxes of 16 rows x 64 k

struct StreamParams {
  const bf16* x;
  const bf16* bias;
  bf16* out;
  int M, N, K;
  int gated_act;      // -1: plain product
  float* out_sumsq;   // not null: out is added to, and [tiles][out_stride] receives the new rows' sums of squares
  int out_stride;
  int* error_flag;
};

__device__ __forceinline__ uint4 lds128(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// The end of a tile: bias, then the plain store, act(gate) * up, or the residual sum with its sums of squares.
// `sum(r, m)` gives column r of the tile for row m of x; the threads e = first, first + step, ... share the tile's
// elements so that 16 neighbouring threads hold the 16 columns of one row.
template <int kCols, typename Sum>
__device__ __forceinline__ void finish_tile(const StreamParams& p, int tile, int first, int step, Sum sum) {
  const int M = p.M, N = p.N, row0 = tile * 16;
  if (p.gated_act < 0) {
    for (int e = first; e < 16 * kCols; e += step) {
      const int r = e % 16, m = e / 16;
      const int col = row0 + r;
      float v = sum(r, m);
      const bool live = m < M && col < N;
      if (live && p.bias) v += __bfloat162float(p.bias[col]);
      if (p.out_sumsq) {
        float sq = 0.f;
        if (live) {
          bf16* at = p.out + (size_t)m * N + col;
          const float h = __bfloat162float(__float2bfloat16_rn(__bfloat162float(*at) + __bfloat162float(__float2bfloat16_rn(v))));
          *at = __float2bfloat16_rn(h);
          sq = h * h;
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (r == 0 && m < M) p.out_sumsq[(size_t)tile * p.out_stride + m] = sq;
      } else if (live) {
        p.out[(size_t)m * N + col] = __float2bfloat16_rn(v);
      }
    }
  } else {
    const int half = N / 2;                 // rows [0, 8) of the tile are gate rows, [8, 16) their up rows
    for (int e = first; e < 8 * kCols; e += step) {
      const int r = e % 8, m = e / 8;
      const int col = tile * 8 + r;
      if (m >= M || col >= half) continue;
      float gate = sum(r, m), up = sum(r + 8, m);
      if (p.bias) {
        gate += __bfloat162float(p.bias[row0 + r]);
        up += __bfloat162float(p.bias[row0 + r + 8]);
      }
      // The products are rounded to bfloat16 before the activation, as a separate kernel would see them.
      gate = __bfloat162float(__float2bfloat16_rn(gate));
      up = __bfloat162float(__float2bfloat16_rn(up));
      p.out[(size_t)m * half + col] = __float2bfloat16_rn(gated(gate, up, p.gated_act));
    }
  }
}

// kWarps warps with a ring of kRing stages each.  kWarpTiles: every warp multiplies whole tiles by itself (weights
// of many tiles: nothing is added up across warps and the block never meets at a barrier); otherwise the warps
// of a block split each tile's k (weights of few tiles).
// kCache > 0 (one tile of x's rows, warps that split k): a warp multiplies the same at most kCache chunks of k in every
// tile, so it reads its share of x once and keeps it in registers.
template <int NT, int kWarps, int kRing, bool kWarpTiles, int kCache = 0>
__global__ void __launch_bounds__(kWarps * 32, kWarps * kRing <= 24 ? 2 : 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const StreamParams p) {
  constexpr int kCols = NT * 8;
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  __shared__ float partial[kWarps][16][kCols + 1];
  __shared__ __align__(8) unsigned long long ring_bars[kWarps * kRing];
  __shared__ int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int M = p.M, K = p.K;
  const int tiles = (p.N + 15) / 16;
  const int chunks = (K + kChunkK - 1) / kChunkK;
  // The tiles of this warp are first_tile, first_tile + tile_step, ...; of each it multiplies `per_tile` chunks,
  // chunk_first, chunk_first + chunk_step, ...
  const int first_tile = kWarpTiles ? blockIdx.x * kWarps + warp : blockIdx.x;
  const int tile_step = kWarpTiles ? gridDim.x * kWarps : gridDim.x;
  const int chunk_first = kWarpTiles ? 0 : warp, chunk_step = kWarpTiles ? 1 : kWarps;
  const int per_tile = chunk_first < chunks ? (chunks - chunk_first + chunk_step - 1) / chunk_step : 0;
  const int my_tiles = first_tile < tiles ? (tiles - first_tile + tile_step - 1) / tile_step : 0;
  const int items = my_tiles * per_tile;
  const unsigned ring = base + (unsigned)warp * kRing * kStageBytes;
  const unsigned bars = smem_addr(ring_bars) + (unsigned)warp * kRing * 8;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kWarps * kRing; ++i) mbar_init(smem_addr(ring_bars) + 8u * i, 1);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto request = [&](int n) {
    if (lane != 0 || n >= items) return;
    const int tile = first_tile + (n / per_tile) * tile_step;
    const int k0 = (chunk_first + (n % per_tile) * chunk_step) * kChunkK;
    const unsigned slot = ring + (unsigned)(n % kRing) * kStageBytes, bar = bars + 8u * (n % kRing);
    mbar_expect_tx(bar, kStageBytes);
    tma_load_2d(slot, &map_w, bar, k0, tile * 16);
    tma_load_2d(slot + kStageBytes / 2, &map_w, bar, k0 + 64, tile * 16);
  };
  // The weights wait for nobody: the rings fill while the kernel ahead still runs, and the kernel behind may start.
  for (int n = 0; n < kRing - 1; ++n) request(n);
  grid_launch_dependents();
  grid_dependency_wait();

  const bf16* xr[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) xr[j] = p.x + (size_t)min(j * 8 + g, M - 1) * K;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  const unsigned row_lo = (unsigned)g * 128u, row_hi = (unsigned)(g + 8) * 128u;
  const unsigned swz = (unsigned)(g & 7);

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

  uint4 xq[kCache > 0 ? kCache : 1][4];
  if (kCache > 0) {
#pragma unroll
    for (int c = 0; c < kCache; ++c)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int k = (chunk_first + c * chunk_step) * kChunkK + (q >> 1) * 64 + (2 * t + (q & 1)) * 8;
        xq[c][q] = (c < per_tile && k < K && g < M) ? *reinterpret_cast<const uint4*>(xr[0] + k) : zero;
      }
  }

  // Without that, the warp's share of x for the chunk after the one it multiplies is asked for one chunk ahead, so
  // that its way from the second-level cache overlaps the wait for the chunk's weights.
  uint4 xn[4][NT];
  auto ask_x = [&](int c) {
    const int k0 = (chunk_first + c * chunk_step) * kChunkK;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int k = k0 + (q >> 1) * 64 + (2 * t + (q & 1)) * 8;
#pragma unroll
      for (int j = 0; j < NT; ++j)
        xn[q][j] = (k < K && j * 8 + g < M) ? *reinterpret_cast<const uint4*>(xr[j] + k) : zero;
    }
  };
  if (kCache == 0 && per_tile > 0) ask_x(0);

  int n = 0;
  bool gave_up = false;
  // Waits for item n and multiplies it; `cached` says where the warp keeps its x for this chunk, if it does.
  auto multiply = [&](int c, const uint4* cached) -> bool {
    request(n + kRing - 1);
    if (!mbar_wait(bars + 8u * (n % kRing), (unsigned)(n / kRing) & 1, p.error_flag, 31)) {
      // Gave up: the copies still on their way get one more bounded chance to land before the memory is let go.
      for (int r = n + 1; r < items && r < n + kRing; ++r)
        mbar_wait(bars + 8u * (r % kRing), (unsigned)(r / kRing) & 1, nullptr, 0);
      gave_up = true;
      failed = 1;
      return false;
    }
    const unsigned slot = ring + (unsigned)(n % kRing) * kStageBytes;
    uint4 xc[4][NT];
    if (kCache == 0) {
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int j = 0; j < NT; ++j) xc[q][j] = xn[q][j];
      ask_x(c + 1 < per_tile ? c + 1 : 0);      // (every tile meets the same x: after a tile's last chunk comes the first)
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        // Piece 2t + h of the box's 128-byte rows: the lanes of a quarter warp then hit eight different banks.
        const unsigned piece = (unsigned)(2 * t + h);
        const unsigned at = slot + (unsigned)b * (kStageBytes / 2) + ((piece ^ swz) << 4);
        const uint4 wl = lds128(at + row_lo), wh = lds128(at + row_hi);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const uint4 xv = kCache > 0 ? cached[b * 2 + h] : xc[b * 2 + h][j];
          mma_16816(acc[j], wl.x, wh.x, wl.y, wh.y, xv.x, xv.y);
          mma_16816(acc[j], wl.z, wh.z, wl.w, wh.w, xv.z, xv.w);
        }
      }
    }
    __syncwarp();     // every lane has read the stage before lane 0 asks for new contents
    ++n;
    return true;
  };
  // (With tiles split among the warps every warp walks the same tiles, so the block's barriers below are met by all.)
  const int rounds = kWarpTiles ? my_tiles : (blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0);
  for (int ti = 0; ti < rounds; ++ti) {
    const int tile = first_tile + ti * tile_step;
    if (kCache > 0) {
#pragma unroll
      for (int c = 0; c < kCache; ++c)
        if (c < per_tile && !gave_up) multiply(c, xq[c]);
    } else {
      for (int c = 0; c < per_tile && !gave_up; ++c)
        if (!multiply(c, nullptr)) break;
    }
    if (kWarpTiles && gave_up) break;
    // The tile's sum goes through shared memory: to meet the other warps' shares (added in warp order), or, for a
    // warp with a tile of its own, to turn its fragments into rows.
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      partial[warp][g][j * 8 + 2 * t] = acc[j][0];
      partial[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
      partial[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
      partial[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
    }
    if (kWarpTiles) {
      __syncwarp();
      finish_tile<kCols>(p, tile, lane, 32, [&](int r, int m) { return partial[warp][r][m]; });
      __syncwarp();
    } else {
      __syncthreads();
      if (failed) break;      // (uniform: read after the barrier)
      finish_tile<kCols>(p, tile, threadIdx.x, kWarps * 32, [&](int r, int m) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) v += partial[w][r][m];
        return v;
      });
      __syncthreads();        // the partial tiles are free again
    }
  }
  if (gave_up || failed) {
    // Copies that were asked for and never multiplied: a bounded wait for each, so that none lands after the
    // block's shared memory has gone to another block.
    for (int r = n; r < items && r < n + kRing - 1; ++r)
      mbar_wait(bars + 8u * (r % kRing), (unsigned)(r / kRing) & 1, nullptr, 0);
  }
}

template <int kWarps, int kRing> constexpr size_t stream_gemm_smem() { return (size_t)kWarps * kRing * kStageBytes + 1024; }

// w [N, K] as a 2-D map with boxes of 16 rows x 64 k, 128-byte swizzle; what lies beyond N or K reads as zero.
static bool make_weight_map(CUtensorMap* map, const void* w, int N, int K) {
  static std::map<std::tuple<const void*, int, int>, CUtensorMap> cache;
  static std::mutex guard;
  std::lock_guard<std::mutex> lock(guard);
  const auto key = std::make_tuple(w, N, K);
  const auto found = cache.find(key);
  if (found != cache.end()) {
    *map = found->second;
    return true;
  }
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {64, 16};
  const cuuint32_t elem[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *map);
  return true;
}

static int stream_sms() {
  static int sms = 0;
  if (!sms) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms < 1)
      sms = 148;
  }
  return sms;
}

template <int NT, int kWarps, int kRing, bool kWarpTiles, int kCache = 0>
static int launch_stream_gemm(const CUtensorMap& map, const StreamParams& p, int grid, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<NT, kWarps, kRing, kWarpTiles, kCache>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)stream_gemm_smem<kWarps, kRing>());
    if (e != cudaSuccess) return (int)e;
    // Two blocks of six warps leave the SM a level-one cache that holds x (measured: gate_up at 8 rows 14.3 us with
    // 72 % of the SM's memory as shared memory, 16.0 us when all of it is).
    static const char* carve = getenv("LITEINFER_STREAM_CARVEOUT");
    const int percent = carve ? atoi(carve) : (kWarps * kRing <= 18 ? 72 : -1);
    if (percent >= 0) cudaFuncSetAttribute(gemm_stream_kernel<NT, kWarps, kRing, kWarpTiles, kCache>,
                                           cudaFuncAttributePreferredSharedMemoryCarveout, percent);
    configured = true;
  }
  return (int)launch_maybe_early(pdl_mode() >= 1, gemm_stream_kernel<NT, kWarps, kRing, kWarpTiles, kCache>, dim3(grid),
                                 dim3(kWarps * 32), stream_gemm_smem<kWarps, kRing>(), stream, map, p);
}

// A weight of few tiles (at most two for every SM: the projections around the attention, the down projection) gives
// every tile a block of eight warps that split k.  A weight of more tiles gets two blocks of six warps per SM, which
// walk over the tiles; the smaller blocks leave a level-one cache that holds x.  Measured on B200 at 8 rows
// (register-loading kernel in brackets): qkv 3.7 us (4.5), o 2.9 (4.0), down 8.8 (9.7), gate_up with its activation
// 14.3 (15.2), the head 82.8 (91.2).  LITEINFER_STREAM_PLAN=b|c|a|d forces one plan for every weight (b: eight warps
// split k; c: six warps split k, two blocks per SM; a, d: every warp takes whole tiles, which measured slower).
template <int NT>
static int plan_and_launch(const CUtensorMap& map, const StreamParams& p, cudaStream_t stream) {
  const int tiles = (p.N + 15) / 16;
  const int sms = stream_sms();
  static const char* forced = getenv("LITEINFER_STREAM_PLAN");
  const char plan = forced ? forced[0] : (tiles <= 2 * sms ? 'b' : 'c');
  switch (plan) {
    case 'a': return launch_stream_gemm<NT, 7, 4, true>(map, p, min(sms, (tiles + 6) / 7), stream);
    case 'e': return launch_stream_gemm<NT, 8, 5, false>(map, p, tiles <= 2 * sms ? tiles : sms, stream);
    case 'f': return launch_stream_gemm<NT, 12, 3, false>(map, p, tiles <= 2 * sms ? tiles : sms, stream);
    case 'd': return launch_stream_gemm<NT, 6, 3, true>(map, p, min(2 * sms, (tiles + 5) / 6), stream);
    case 'c':
      // (with at most three chunks of k a warp and one tile of rows, a warp keeps its share of x in registers)
      if (NT == 1 && (p.K + kChunkK - 1) / kChunkK <= 18 && !getenv("LITEINFER_STREAM_NO_X_CACHE"))
        return launch_stream_gemm<1, 6, 3, false, 3>(map, p, min(tiles, 2 * sms), stream);
      return launch_stream_gemm<NT, 6, 3, false>(map, p, min(tiles, 2 * sms), stream);
    default: return launch_stream_gemm<NT, 8, 3, false>(map, p, tiles <= 2 * sms ? tiles : sms, stream);
  }
}

}  // namespace li

using namespace li;

// Whether li_gemm_stream takes these sizes: at most 16 rows of x, k a multiple of 8 (rows of w start on 16 bytes).
LI_EXPORT int li_gemm_stream_supports(int M, int N, int K) { return M >= 1 && M <= 16 && N >= 1 && K >= 8 && K % 8 == 0; }

// bfloat16.  gated_act as li_gemm_skinny's.  out_sumsq (may be null; plain product only): out [M, N] is added to,
// out = round(out + round(product + bias)), and out_sumsq [ceil(N/16)][out_stride] receives the new rows' sums of
// squares, one part per 16 columns.  error_flag (device int, may be null): set to 31 if a wait for weights gave up.
LI_EXPORT int li_gemm_stream(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                             int gated_act, float* out_sumsq, int out_stride, int* error_flag, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (!li_gemm_stream_supports(M, N, K)) return LI_ERR_UNSUPPORTED;
  if (gated_act > 3 || (gated_act >= 0 && (N % 16))) return LI_ERR_UNSUPPORTED;
  if (out_sumsq && (gated_act >= 0 || out_stride < M)) return LI_ERR_UNSUPPORTED;
  if (!aligned16(x) || !aligned16(w)) return LI_ERR_ALIGNMENT;
  CUtensorMap map;
  if (!make_weight_map(&map, w, N, K)) return LI_ERR_UNSUPPORTED;
  StreamParams p{(const bf16*)x, (const bf16*)bias, (bf16*)out, M, N, K, gated_act, out_sumsq, out_stride, error_flag};
  return M <= 8 ? plan_and_launch<1>(map, p, stream) : plan_and_launch<2>(map, p, stream);
}
