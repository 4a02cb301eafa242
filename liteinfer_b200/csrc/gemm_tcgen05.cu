// out[M, N] = x[M, K] @ w[N, K]^T (+ bias) in bfloat16 on the fifth-generation tensor cores:
// the matrix product of prefill, where M is in the hundreds or thousands.
//
// One persistent block per SM walks 128 x BN output tiles.  Inside a block the work is split
// by warp: warp 0 moves tiles of x and w from global to shared memory with TMA
// (cp.async.bulk.tensor, 128-byte swizzle) through a ring of stages guarded by mbarriers; one
// thread of warp 1 issues tcgen05.mma (M 128, N BN, K 16 per instruction, operands straight
// from shared memory through matrix descriptors) accumulating in tensor memory, and commits
// each stage back to the loader; warps 2-5 drain a finished accumulator from tensor memory
// with tcgen05.ld, round it to bfloat16 and store it, while the next tile's products already
// run into the second accumulator (2 x BN of the 512 TMEM columns).
//
// Optional epilogue for a gated feed-forward (`gated_act >= 0`): the rows of w are interleaved in
// eights (eight gate rows, then their eight up rows); the block then writes act(gate) * up,
// N/2 columns wide, with the same rounding points as the separate kernels (products rounded to
// bfloat16, activation rounded, then the multiply).
//
// Every wait on an mbarrier is bounded: a wait that runs out records where it gave up in
// `error_flag` and the block winds down (tensor memory is freed on every path), so a fault in
// the choreography shows up as an error code, not as a hang.
#include <map>
#include <mutex>
#include <tuple>

#include "tcgen05.cuh"

namespace li {

constexpr int kTileM = 128;
constexpr int kTileK = 64;                 // 64 bf16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;          // loader, issuer, four epilogue warps
constexpr int kPairThreads = 320;          // the kernel for pairs of CTAs: loader, issuer, eight epilogue warps
__device__ __forceinline__ float gated_value(float gate, float up, int act) {
  gate = __bfloat162float(__float2bfloat16_rn(gate));
  up = __bfloat162float(__float2bfloat16_rn(up));
  float a;
  switch (act) {
    case 0: a = gate / (1.0f + expf(-gate)); break;
    case 1: a = 0.5f * gate * (1.0f + erff(gate * 0.70710678118654752440f)); break;
    case 2: a = 0.5f * gate * (1.0f + tanhf(0.79788456080286535588f * (gate + 0.044715f * gate * gate * gate))); break;
    default: a = fmaxf(gate, 0.f);
  }
  return __bfloat162float(__float2bfloat16_rn(a)) * up;
}

// Tiles are walked in bands of eight tile rows, column by column inside a band, so that the blocks running at
// the same time share a few tiles of x and a few of w (which then come from L2, not from HBM).
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int kBand = 8;
  const int per_band = kBand * tiles_n;
  const int band = tile / per_band, in_band = tile - band * per_band;
  const int rows = min(kBand, tiles_m - band * kBand);
  tn = in_band / rows;
  tm = band * kBand + in_band % rows;
}

struct GemmParams {
  bf16* out;
  const bf16* bias;
  int M, N, K;
  int gated_act;
  int* error_flag;
};

// 32 consecutive columns of one output row, from the accumulator's registers to global memory: rounded to
// bfloat16 (with the bias), or for a gated feed-forward two groups of (eight gate, eight up) columns turned into
// 16 outputs.  The caller has checked m < M and n0 < N.
__device__ __forceinline__ void store_chunk(const GemmParams& p, const unsigned (&r)[32], int m, int n0) {
  if (p.gated_act < 0) {
    bf16* dst = p.out + (size_t)m * p.N + n0;
    if (n0 + 32 <= p.N && (p.N % 8) == 0) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        uint4 pack;
        unsigned* w = reinterpret_cast<unsigned*>(&pack);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float lo = __uint_as_float(r[v * 8 + 2 * j]), hi = __uint_as_float(r[v * 8 + 2 * j + 1]);
          if (p.bias) {
            lo += __bfloat162float(p.bias[n0 + v * 8 + 2 * j]);
            hi += __bfloat162float(p.bias[n0 + v * 8 + 2 * j + 1]);
          }
          __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
          w[j] = *reinterpret_cast<unsigned*>(&h);
        }
        *reinterpret_cast<uint4*>(dst + v * 8) = pack;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (n0 + j < p.N) {
          float v = __uint_as_float(r[j]);
          if (p.bias) v += __bfloat162float(p.bias[n0 + j]);
          dst[j] = __float2bfloat16_rn(v);
        }
      }
    }
  } else {
    // 32 columns = two groups of (eight gate, eight up) -> 16 outputs at column n0 / 2.
    const int half = p.N / 2;
    bf16* dst = p.out + (size_t)m * half + n0 / 2;
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
      if (n0 + grp * 16 >= p.N) break;
      uint4 pack;
      unsigned* w = reinterpret_cast<unsigned*>(&pack);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = grp * 16 + 2 * j + e;
          float gate = __uint_as_float(r[col]), up = __uint_as_float(r[col + 8]);
          if (p.bias) {
            gate += __bfloat162float(p.bias[n0 + col]);
            up += __bfloat162float(p.bias[n0 + col + 8]);
          }
          v[e] = gated_value(gate, up, p.gated_act);
        }
        __nv_bfloat162 h = __floats2bfloat162_rn(v[0], v[1]);
        w[j] = *reinterpret_cast<unsigned*>(&h);
      }
      *reinterpret_cast<uint4*>(dst + grp * 8) = pack;
    }
  }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  // Tiles must start on 1024-byte boundaries for the 128-byte swizzle.
  const unsigned base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  constexpr unsigned kBytesA = kTileM * kTileK * 2, kBytesB = BN * kTileK * 2, kStageBytes = kBytesA + kBytesB;
  const unsigned bars = base + STAGES * kStageBytes;       // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
  const unsigned tmem_slot = bars + 8u * (2 * STAGES + 4);
  __shared__ unsigned tmem_base_shared;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + kTileM - 1) / kTileM, tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + kTileK - 1) / kTileK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 4);     // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // the issuing warp owns tensor memory: 2 accumulators of BN columns, all 512 columns asked for
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  if (threadIdx.x == 0) {
    unsigned v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(tmem_slot));
    tmem_base_shared = v;
  }
  __syncthreads();
  const unsigned tmem_base = tmem_base_shared;
  grid_dependency_wait();   // x comes from the kernel before (a no-op under an ordinary launch)

  if (warp == 0) {
    // ------------------------------------------------------------------ loader
    if (lane == 0) {
      int stage = 0;
      unsigned phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, p.error_flag, 1)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), kStageBytes);
          const unsigned a = base + stage * kStageBytes;
          tma_load_2d(a, &map_x, full_bar(stage), kb * kTileK, tm * kTileM);
          tma_load_2d(a + kBytesA, &map_w, full_bar(stage), kb * kTileK, tn * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer
    if (lane == 0) {
      // Instruction descriptor: f32 accumulate, bf16 x bf16, both operands K-major, N = BN, M = 128.
      constexpr unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) |
                                 ((unsigned)(kTileM >> 4) << 24);
      int stage = 0;
      unsigned phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        const unsigned use = (unsigned)(local >> 1);
        if (!mbar_wait(acc_empty_bar(buf), (use & 1) ^ 1, p.error_flag, 2)) { ok = false; break; }
        tcgen05_fence_after();
        const unsigned acc = tmem_base + (unsigned)(buf * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.error_flag, 3)) { ok = false; break; }
          tcgen05_fence_after();
          const unsigned a = base + stage * kStageBytes, b = a + kBytesA;
#pragma unroll
          for (int k = 0; k < kTileK / kUmmaK; ++k)
            umma_bf16(acc, umma_desc(a + k * kUmmaK * 2), umma_desc(b + k * kUmmaK * 2), idesc, kb > 0 || k > 0);
          umma_commit(empty_bar(stage));          // the stage is free once these products have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(acc_full_bar(buf));   // the accumulator is complete once all products are done
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;                 // the TMEM lanes this warp may read: 32 * (warp % 4) ...
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      const int buf = local & 1;
      const unsigned use = (unsigned)(local >> 1);
      if (!mbar_wait(acc_full_bar(buf), use & 1, p.error_flag, 4)) { ok = false; break; }
      tcgen05_fence_after();
      const int m = tm * kTileM + quarter * 32 + lane;
      const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        unsigned r[32];
        __syncwarp();                       // the load below is a warp-wide instruction
        tmem_load32(taddr + c * 32, r);
        tmem_load_wait();
        const int n0 = tn * BN + c * 32;
        if (m >= p.M || n0 >= p.N) continue;
        store_chunk(p, r, m, n0);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(buf));
    }
  }

  // ------------------------------------------------------------------ teardown (every path comes here)
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}


// The same product by pairs of CTAs (a cluster of two, cta_group::2): a pair owns a 256 x 256 tile, each CTA
// loading its 128 rows of x and its 128 of the tile's 256 rows of w, 32 KB a stage instead of 48, so that six
// stages fit and the loads run further ahead of the products (with one CTA per tile the tensor cores waited a
// third of the time for the next stage).  The leader's issuer multiplies for both; every CTA drains its own
// half of the accumulator.
template <int STAGES>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  constexpr int BN = 256;                        // columns of the pair's tile; each CTA loads BN / 2 rows of w
  const unsigned base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  constexpr unsigned kBytesA = kTileM * kTileK * 2, kBytesB = (BN / 2) * kTileK * 2, kStageBytes = kBytesA + kBytesB;
  const unsigned bars = base + STAGES * kStageBytes;       // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
  auto full_bar = [&](int s) { return bars + 8u * s; };                       // waited on in the leader only
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };           // signalled in both CTAs
  auto acc_full_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };    // signalled in both CTAs
  auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };   // the leader's: 16 epilogue warps arrive
  const unsigned tmem_slot = bars + 8u * (2 * STAGES + 4);
  __shared__ unsigned tmem_base_shared;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_cta_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int tiles_m = (p.M + 2 * kTileM - 1) / (2 * kTileM), tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + kTileK - 1) / kTileK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 16);    // one arrival per epilogue warp of either CTA
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // the same warp in both CTAs: the allocation is made for the pair
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  if (threadIdx.x == 0) {
    unsigned v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(tmem_slot));
    tmem_base_shared = v;
  }
  cluster_sync_all();       // both CTAs' barriers exist before either signals the other
  const unsigned tmem_base = tmem_base_shared;
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ loader (one per CTA)
    if (lane == 0) {
      int stage = 0;
      unsigned phase = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < num_tiles; tile += pairs) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, p.error_flag, 1)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * kStageBytes);   // the bytes of both CTAs
          const unsigned a = base + stage * kStageBytes;
          tma_load_2d_pair(a, &map_x, full_bar(stage), kb * kTileK, tm * 2 * kTileM + (int)rank * kTileM);
          tma_load_2d_pair(a + kBytesA, &map_w, full_bar(stage), kb * kTileK, tn * BN + (int)rank * (BN / 2));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer (the leader's only)
    if (lane == 0 && rank == 0) {
      // Instruction descriptor: f32 accumulate, bf16 x bf16, both operands K-major, N = 256, M = 256 over the pair.
      constexpr unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) |
                                 ((unsigned)((2 * kTileM) >> 4) << 24);
      int stage = 0;
      unsigned phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < num_tiles; tile += pairs, ++local) {
        const int buf = local & 1;
        const unsigned use = (unsigned)(local >> 1);
        if (!mbar_wait(acc_empty_bar(buf), (use & 1) ^ 1, p.error_flag, 2)) { ok = false; break; }
        tcgen05_fence_after();
        const unsigned acc = tmem_base + (unsigned)(buf * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.error_flag, 3)) { ok = false; break; }
          tcgen05_fence_after();
          const unsigned a = base + stage * kStageBytes, b = a + kBytesA;
#pragma unroll
          for (int k = 0; k < kTileK / kUmmaK; ++k)
            umma_bf16_pair(acc, umma_desc(a + k * kUmmaK * 2), umma_desc(b + k * kUmmaK * 2), idesc, kb > 0 || k > 0);
          umma_commit_pair(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(acc_full_bar(buf));
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (eight warps per CTA)
    // A warp may read the 32 lanes of tensor memory that its number modulo four names; two warps share each
    // quarter and take half of the tile's columns each.
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    int local = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < num_tiles; tile += pairs, ++local) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      const int buf = local & 1;
      const unsigned use = (unsigned)(local >> 1);
      if (!mbar_wait(acc_full_bar(buf), use & 1, p.error_flag, 4)) { ok = false; break; }
      tcgen05_fence_after();
      const int m = tm * 2 * kTileM + (int)rank * kTileM + quarter * 32 + lane;
      const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BN);
#pragma unroll 1
      for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
        unsigned r[32];
        __syncwarp();
        tmem_load32(taddr + c * 32, r);
        tmem_load_wait();
        const int n0 = tn * BN + c * 32;
        if (m >= p.M || n0 >= p.N) continue;
        store_chunk(p, r, m, n0);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(acc_empty_bar(buf));
    }
  }

  // ------------------------------------------------------------------ teardown (every path comes here)
  tcgen05_fence_before();
  cluster_sync_all();        // neither CTA leaves, nor frees tensor memory, while the other may still use it
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// A [rows, K] bfloat16 row-major matrix as a 2-D tensor map with boxes of 64 x box_rows and 128-byte swizzle;
// elements outside the matrix read as zero.
static bool make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
  // Encoding is pure host arithmetic on (pointer, sizes): the same matrix gives the same map, so maps are kept.
  static std::map<std::tuple<const void*, int, int, int>, CUtensorMap> cache;
  static std::mutex guard;                 // several host threads may launch (an asyncio engine beside its caller)
  std::lock_guard<std::mutex> lock(guard);
  const auto key = std::make_tuple(ptr, rows, K, box_rows);
  const auto found = cache.find(key);
  if (found != cache.end()) {
    *map = found->second;
    return true;
  }
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *map);
  return true;
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& mx, const CUtensorMap& mw, const GemmParams& p, int sms, cudaStream_t s) {
  constexpr size_t smem = (size_t)STAGES * (kTileM + BN) * kTileK * 2 + 8 * (2 * STAGES + 4) + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((p.M + kTileM - 1) / kTileM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  gemm_tcgen05_kernel<BN, STAGES><<<grid, kGemmThreads, smem, s>>>(mx, mw, p);
  return (int)cudaGetLastError();
}


template <int STAGES>
static int launch_gemm_pair(const CUtensorMap& mx, const CUtensorMap& mw, const GemmParams& p, int sms, cudaStream_t s) {
  constexpr size_t smem = (size_t)STAGES * (kTileM + 128) * kTileK * 2 + 8 * (2 * STAGES + 4) + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((p.M + 2 * kTileM - 1) / (2 * kTileM)) * ((p.N + 255) / 256);
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(2 * pairs);
  config.blockDim = dim3(kPairThreads);
  config.dynamicSmemBytes = smem;
  config.stream = s;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = 2;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // barriers and tensor memory are set up early
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl_enabled(0) ? 2 : 1;
  return (int)cudaLaunchKernelEx(&config, gemm_tcgen05_pair_kernel<STAGES>, mx, mw, p);
}

}  // namespace li

using namespace li;

// bfloat16; K a multiple of 8; x and w 16-byte aligned.  gated_act: -1 plain; 0..3 act(gate) * up on rows of w
// interleaved in eights (N a multiple of 16; out is [M, N/2]).  error_flag (device int, zero): set to the number
// of the wait that gave up if the kernel's choreography ever stalls (1 loader, 2 accumulator free, 3 stage full,
// 4 accumulator full); the output is then not to be trusted.
LI_EXPORT int li_gemm_tcgen05(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                              int gated_act, int* error_flag, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (K < 8 || (K % 8) || gated_act > 3 || (gated_act >= 0 && (N % 16))) return LI_ERR_UNSUPPORTED;
  if (!aligned16(x) || !aligned16(w) || !aligned16(out)) return LI_ERR_ALIGNMENT;
  static int sms = 0;
  if (!sms) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (sms <= 0) sms = 148;
  }
  // Large products go to pairs of CTAs on 256 x 256 tiles (LITEINFER_TCGEN05_PAIR=0 keeps them on single CTAs).
  static int pair_mode = -1;
  if (pair_mode < 0) {
    const char* e = getenv("LITEINFER_TCGEN05_PAIR");
    pair_mode = e ? atoi(e) : 1;
  }
  if (pair_mode && M >= 256 && N >= 256) {
    CUtensorMap px, pw;
    if (!make_map(&px, x, M, K, kTileM) || !make_map(&pw, w, N, K, 128)) return LI_ERR_UNSUPPORTED;
    GemmParams pp{(bf16*)out, (const bf16*)bias, M, N, K, gated_act, error_flag};
    return launch_gemm_pair<6>(px, pw, pp, sms, stream);
  }
  // Tile width: whichever of 256 and 128 needs less time in whole waves of blocks (ties go to the wide tile,
  // which reads less per product).
  const int tiles_m = (M + kTileM - 1) / kTileM;
  const long cost_wide = (long)((tiles_m * ((N + 255) / 256) + sms - 1) / sms) * 256;
  const long cost_narrow = (long)((tiles_m * ((N + 127) / 128) + sms - 1) / sms) * 128;
  const bool wide = N > 128 && 2 * cost_wide <= 3 * cost_narrow;
  CUtensorMap mx, mw;
  if (!make_map(&mx, x, M, K, kTileM) || !make_map(&mw, w, N, K, wide ? 256 : 128)) return LI_ERR_UNSUPPORTED;
  GemmParams p{(bf16*)out, (const bf16*)bias, M, N, K, gated_act, error_flag};
  return wide ? launch_gemm<256, 4>(mx, mw, p, sms, stream) : launch_gemm<128, 6>(mx, mw, p, sms, stream);
}
