// Paged attention for prompts and portions of prompts on the fifth-generation tensor cores
// (bfloat16, head sizes 64 and 128, pages of 16, 32 or 64 tokens).
//
// Rule as in attention_generic.cu (liteinfer/models/attention.py:24-27,69-84).  A block owns one tile of 128
// rows for one KV head (two tiles at head size 128, see KvStages below), a row being (query token, head of the
// group), and walks the visible keys in tiles of 64.  Per tile of rows:
//
//   loader  (warp 0)    TMA: each page of a tile's keys and values is one box of the pool's tensor map per 64
//                       dimensions, landing in 128-byte-swizzled shared memory, five tiles ahead at most;
//                       lane b requests page b of a tile, and one barrier per stage counts keys and values
//                       (one loader for the block, whatever its number of query tiles).  The block table's entries are in the warp's registers, 32 at a time, the
//                       next 32 on their way.
//   issuer  (warp 1)    tcgen05.mma: S = Q K^T (128 x 64, K = head size) into one of two score buffers in
//                       tensor memory, then O += P V (128 x 64 per 64 dimensions, K 64 keys, P from tensor
//                       memory) into the output accumulator; S of the next tile is issued before P V of this
//                       one, so the tensor cores work while the softmax of this tile is computed.  The thread
//                       waits twice per tile (the next stage has landed; this tile's probabilities are
//                       written): what else must hold follows from those two and from the order in which
//                       products run (the one in which they were issued).
//   softmax (warps 2-5) one thread per row: tcgen05.ld brings the row's 64 scores into registers, so
//                       maximum and sum need no exchange between threads; the probabilities go back as
//                       bfloat16 over the first 32 columns of those scores (tcgen05.st), where P V reads its
//                       first operand; the accumulator in tensor memory is rescaled (ld, multiply, st) only
//                       when a row's maximum has outgrown the reference of its exponentials by 2^8, so the
//                       softmax of one tile does not wait for P V of the tile before it.
//
// Blocks are handed out longest first (the query tile is the slowest index of the grid); two fit an SM at head
// size 64.  What sets the pace (cycle counters written by one block of a prompt of 8,192 tokens, B200): a tile
// takes a block about 1,450 cycles, and both single-thread chains are that long.  The softmax warp: 220 for a wait
// that is already satisfied, 85 for the scores to arrive, 900 for maxima, exponentials and packing (two warps of
// two blocks share a scheduler's special-function unit), 115 for the store to tensor memory, 110 for fence and
// arrival.  The issuer: 200 for each of its two waits, about 100 for every product and commit it issues (four for
// S, four for P V, three commits).  With the exponentials, or three quarters of the products, or the stores of
// the probabilities taken out, the prompt takes 416, 414 and 420 us instead of 429: no single unit is the bound.
// Tried on this ground and not kept (all correct, none faster): 256 rows per block with 128-key tiles (432 us;
// 597 with the probabilities in tensor memory, where softmax and products of one query tile form one chain),
// two softmax threads per row with accumulators of their own (423 us; the issuer then issues twice as many
// products).  Kept: the probabilities in tensor memory and the deeper ring that their shared memory pays for (413),
// the block table in registers (405).  Head size 128 has twice the products per tile and had one block of four
// softmax warps per SM (its shared memory): there two query tiles per block, each with an issuing thread of its own,
// took a prompt of 8,192 tokens from 898 to 554 us (612 to 992 TFLOP/s, 0.61 of the burst peak) and one of 2,048 from
// 82 to 52 us; the same at head size 64, where two blocks per SM already give every SM two issuers: 472 against 407.
// A second issuing thread per tile (one for S, one for P V, ordered by a barrier where the order of issue used to
// do) changed nothing for the better: 579 against 554 us at head size 128, 425 against 407 at 64.
//
// Scores, maximum, sum and accumulator are 32-bit; probabilities are rounded to bfloat16 for P V
// (liteinfer/models/paged_kernels.py:282-284).  Keys outside the visible range are masked to -inf and
// their value rows are zeroed in shared memory, so an unwritten slot of a page cannot leak.
// Every mbarrier wait is bounded (see tcgen05.cuh); a wait that runs out sets `error_flag`.
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "tcgen05.cuh"

namespace li {

constexpr int kRows = 128;       // rows (query token x head in group) per block
constexpr int kKeys = 64;        // keys per tile
constexpr float kLog2eF = 1.4426950408889634f;
constexpr float kLazyLog2 = 8.f;   // how far (in powers of two) a row's maximum may outgrow the reference of its exponentials

struct TcAttnParams {
  const bf16* q;
  int q_row_stride;
  bf16* out;
  int out_row_stride;
  const int* block_table;
  int table_stride;
  const int* query_start_loc;
  const int* context_lens;
  const int* seq_index;
  int heads, kv_heads, page_size, page_shift, num_pages;
  float scale_log2;
  int window;
  int* error_flag;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Three-input maximum and two-wide 32-bit arithmetic: fewer instructions for the softmax threads, whose
// instruction stream is what a tile's time is made of.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

// Shared memory holds everything in sub-tiles of 64 columns (128 bytes, one swizzle row): Q is D/64 sub-tiles of
// 128 rows, a K or V stage D/64 sub-tiles of 64 keys.  The probabilities do not pass through it: a softmax thread
// writes its row of them as bfloat16 over the first 32 columns of the scores it has read, and P V takes its first
// operand from tensor memory.  What that saves goes to the ring of keys and values: the kernel's time is how long a
// tile takes to arrive divided by how many are on their way.
//
// X query tiles of 128 rows per block (X = 2 at head size 128, where one tile's block would be alone on its SM with
// four softmax warps and an issuing thread that sets the pace: 612 TFLOP/s for a prompt of 8,192 tokens).  Every tile
// has an issuing thread, four softmax warps, score buffers, accumulator and barriers of its own and runs as if it
// were alone; the tiles share the loader and the ring, so a tile of keys and values is fetched once for all of them,
// and a stage is free when every tile's P V has read it.
template <int D, int X>
struct KvStages { static constexpr int value = D == 64 ? 5 : (X == 1 ? 6 : 5); };

template <int X> constexpr int attn_threads() { return 32 + 32 * X + 128 * X; }   // loader, X issuers, X x 4 softmax warps

template <int D, int X>
__global__ void __launch_bounds__(attn_threads<X>(), (D == 64 && X == 1) ? 2 : 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         const TcAttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  constexpr int kSub = D / 64;                                      // sub-tiles of 64 dimensions
  constexpr unsigned kKeySubBytes = kKeys * 64 * 2;                 // 8 KB: 64 keys x 64 dimensions
  constexpr unsigned kRowSubBytes = kRows * 64 * 2;                 // 16 KB: 128 rows x 64 columns
  constexpr unsigned kTileBytes = kSub * kKeySubBytes;              // one K or V tile
  constexpr int kKvStages = KvStages<D, X>::value;
  const unsigned q_smem = base;                                     // X tiles
  const unsigned k_smem = q_smem + X * kSub * kRowSubBytes;         // kKvStages
  const unsigned v_smem = k_smem + kKvStages * kTileBytes;          // kKvStages
  const unsigned bars = v_smem + kKvStages * kTileBytes;
  auto kv_full = [&](int s) { return bars + 8u * s; };                    // keys and values of a stage have landed
  auto kv_empty = [&](int s) { return bars + 8u * (2 * kKvStages + s); };
  // (tile x's own barriers: x is the warp's tile, fixed below)
  auto tile_bar = [&](int x, int which, int b) { return bars + 8u * (3 * kKvStages + x * 6 + which * 2 + b); };
  const unsigned tmem_slot = bars + 8u * (3 * kKvStages + 6 * X);
  __shared__ unsigned tmem_base_shared;
  unsigned char* generic_base = smem_raw + (base - smem_addr(smem_raw));   // the same place as a generic pointer

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = p.seq_index ? p.seq_index[blockIdx.y] : blockIdx.y;
  if (seq < 0) return;        // a place of padding in the list of sequences
  const int kvh = blockIdx.x;
  const int q_begin = p.query_start_loc[seq], q_len = p.query_start_loc[seq + 1] - q_begin;
  const int groups = p.heads / p.kv_heads;
  const int tq = kRows / groups;
  // The last query tiles see the most keys: they are handed out first, across all heads and sequences (the query
  // tile is the slowest index of the grid), so that the long blocks do not end up alone at the end of the launch.
  const int block_q0 = (int)(gridDim.z - 1 - blockIdx.z) * X * tq;
  if (block_q0 >= q_len) return;
  const int ctx = p.context_lens[seq];
  const int block_q = min(X * tq, q_len - block_q0);         // query tokens of the block: its tiles walk the same keys
  const int* table = p.block_table + (size_t)seq * p.table_stride;
  const int hi = ctx - q_len + block_q0 + block_q;
  const int lo = (p.window > 0 && ctx - q_len + block_q0 - p.window + 1 > 0) ? ctx - q_len + block_q0 - p.window + 1 : 0;
  // The warp's own tile (issuer x is warp 1 + x, its softmax warps are 1 + X + 4 x ...): its queries and positions.
  const int x = X == 1 ? 0 : (warp <= X ? max(warp - 1, 0) : (warp - 1 - X) >> 2);
  const int q0 = block_q0 + x * tq;
  const int tile_q = max(0, min(tq, q_len - q0));
  const int rows_used = tile_q * groups;
  const int first_qpos = ctx - q_len + q0, last_qpos = first_qpos + max(tile_q, 1) - 1;
  auto s_full = [&](int b) { return tile_bar(x, 0, b); };
  auto p_full = [&](int b) { return tile_bar(x, 1, b); };
  auto pv_done = [&](int b) { return tile_bar(x, 2, b); };
  const int tile_lo = lo / kKeys, tile_hi = (hi + kKeys - 1) / kKeys;
  const int ntiles = tile_hi - tile_lo;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), X);          // every tile's issuer says when its P V has read the stage
    }
    for (int t = 0; t < X; ++t)
      for (int b = 0; b < 2; ++b) {
        mbar_init(tile_bar(t, 0, b), 1);
        mbar_init(tile_bar(t, 1, b), 4);
        mbar_init(tile_bar(t, 2, b), 1);
      }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Per tile two score buffers of 64 columns and an accumulator of D: a power of two of columns is asked for.
  constexpr unsigned kTmemCols = X * (128 + D) <= 256 ? 256u : 512u;
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  grid_dependency_wait();   // q and the newest keys and values come from the kernel before; what is above waits for nobody
  // The loader's warp: lane b looks up page b of tile t and asks for its boxes (keys and values, per 64 dimensions),
  // so that the lookups and the requests of a tile's pages run side by side.  Returns false if a wait gave up.
  const int boxes = kKeys / p.page_size;
  const unsigned box_bytes = (unsigned)p.page_size * 64 * 2;
  // The warp keeps 32 entries of the block table in registers (lane i the i-th of the chunk) and has the next 32
  // on their way: a lookup in memory for every tile would set the pace of the whole block (its latency under load
  // is about what a tile's softmax takes).  A tile's pages lie in one chunk: their number divides 32 and the first
  // is a multiple of it.
  int chunk = -1, entries = -1, entries_ahead = -1;
  auto table_chunk = [&](int c) { return c * 32 + lane < p.table_stride ? table[c * 32 + lane] : -1; };
  auto load_tile = [&](int t, bool stage_is_new) -> bool {
    const int stage = t % kKvStages;
    const unsigned phase = (unsigned)(t / kKvStages) & 1;
    const int kpos = (tile_lo + t) * kKeys + lane * p.page_size;
    const int first_page = ((tile_lo + t) * kKeys) >> p.page_shift;
    if ((first_page >> 5) != chunk) {
      entries = (first_page >> 5) == chunk + 1 && chunk >= 0 ? entries_ahead : table_chunk(first_page >> 5);
      chunk = first_page >> 5;
      entries_ahead = table_chunk(chunk + 1);
    }
    const int page = __shfl_sync(0xffffffffu, entries, (first_page + lane) & 31);
    int row = -1;
    if (lane < boxes && kpos < hi && kpos + p.page_size > lo && page >= 0 && page < p.num_pages)
      row = (page * p.kv_heads + kvh) * p.page_size;
    const int valid = __popc(__ballot_sync(0xffffffffu, row >= 0));
    bool fine = true;
    if (lane == 0) {
      if (!stage_is_new) fine = mbar_wait(kv_empty(stage), phase ^ 1, p.error_flag, 11);
      if (fine) mbar_expect_tx(kv_full(stage), 2 * valid * kSub * box_bytes);
    }
    fine = __shfl_sync(0xffffffffu, fine, 0);
    if (!fine) return false;
    if (row >= 0) {
#pragma unroll
      for (int sub = 0; sub < kSub; ++sub) {
        tma_load_2d(k_smem + stage * kTileBytes + sub * kKeySubBytes + lane * box_bytes, &map_k, kv_full(stage), sub * 64, row);
        tma_load_2d(v_smem + stage * kTileBytes + sub * kKeySubBytes + lane * box_bytes, &map_v, kv_full(stage), sub * 64, row);
      }
    }
    return true;
  };
  // The first tiles set out while Q is copied and tensor memory is handed round (the barriers were made by lane 0
  // of this same warp, above).
  const int tiles_ahead = min(kKvStages, ntiles);
  if (warp == 0) {
    __syncwarp();
    for (int t = 0; t < tiles_ahead; ++t) load_tile(t, true);
  }
  // Q: each softmax thread copies its row (128 bytes) into the swizzled tile; rows of padding are zero.
  if (warp > X) {
    const int row = (warp & 3) * 32 + lane;
#pragma unroll
    for (int sub = 0; sub < kSub; ++sub) {
      uint4 v[8];
      if (row < rows_used) {
        const int qi = q0 + row / groups, head = kvh * groups + row % groups;
        const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t)(q_begin + qi) * p.q_row_stride + (size_t)head * D + sub * 64);
#pragma unroll
        for (int c = 0; c < 8; ++c) v[c] = src[c];
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) v[c] = make_uint4(0, 0, 0, 0);
      }
      unsigned char* dst = generic_base + (q_smem - base) + (x * kSub + sub) * kRowSubBytes + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(dst + ((c ^ (row & 7)) << 4)) = v[c];
    }
    fence_async_shared();
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
  const unsigned tmem_s[2] = {tmem_base + x * 128u, tmem_base + x * 128u + 64u};
  const unsigned tmem_o = tmem_base + X * 128u + x * D;

  if (warp == 0) {
    // ------------------------------------------------------------------ loader
    for (int t = tiles_ahead; t < ntiles; ++t)
      if (!load_tile(t, false)) break;
  } else if (warp <= X) {
    // ------------------------------------------------------------------ issuer
    if (lane == 0) {
      // f32 accumulate, bf16 x bf16, M 128, N 64; for P V the second operand (values) is N-major.
      constexpr unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(kKeys >> 3) << 17) | ((unsigned)(kRows >> 4) << 24);
      constexpr unsigned idesc_pv = idesc_qk | (1u << 16);
      // A descriptor's low bits are its address in units of 16 bytes, so the descriptor of a place further on in
      // shared memory is the first one plus the distance: one addition per product instead of the whole encoding.
      const unsigned long long desc_q = umma_desc(q_smem + x * kSub * kRowSubBytes), desc_k = umma_desc(k_smem),
                               desc_v = umma_desc(v_smem);
      // S of tile t may overwrite its buffer: the softmax threads read tile t-2 out of it before they announced its
      // probabilities (which lie in the same columns), that announcement was waited for before P V of tile t-2 was
      // issued, and products run in the order they were issued.
      auto issue_qk = [&](int t) -> bool {
        const int stage = t % kKvStages, buf = t & 1;
        if (!mbar_wait(kv_full(stage), (unsigned)(t / kKvStages) & 1, p.error_flag, 13)) return false;
        tcgen05_fence_after();
        const unsigned long long dk = desc_k + (unsigned long long)((stage * kTileBytes) >> 4);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem_s[buf], desc_q + (unsigned long long)(((k / 4) * kRowSubBytes + (k % 4) * 32) >> 4),
                    dk + (unsigned long long)(((k / 4) * kKeySubBytes + (k % 4) * 32) >> 4), idesc_qk, k > 0);
        umma_commit(s_full(buf));
        return true;
      };
      bool ok = ntiles > 0 && issue_qk(0);
      for (int t = 0; ok && t < ntiles; ++t) {
        if (t + 1 < ntiles && !issue_qk(t + 1)) { ok = false; break; }
        const int stage = t % kKvStages, buf = t & 1;
        // The stage's values landed with its keys, which S = Q K^T of this tile waited for.
        if (!mbar_wait(p_full(buf), (unsigned)(t >> 1) & 1, p.error_flag, 15)) { ok = false; break; }
        tcgen05_fence_after();
        const unsigned long long dv = desc_v + (unsigned long long)((stage * kTileBytes) >> 4);
        // One product per 16 keys covers all D dimensions: the values' sub-tiles of 64 dimensions lie kKeySubBytes
        // apart, which the descriptor's leading offset says (it is unused where D is 64).
        constexpr unsigned idesc_pv_all = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(D >> 3) << 17) |
                                          ((unsigned)(kRows >> 4) << 24);
        const unsigned long long dv_all = (dv & ~(0x3fffULL << 16)) | ((unsigned long long)((kKeySubBytes >> 4) & 0x3fff) << 16);
#pragma unroll
        for (int k = 0; k < kKeys / 16; ++k)
          umma_bf16_ts(tmem_o, tmem_s[buf] + k * 8u, (kSub == 1 ? dv : dv_all) + (unsigned long long)((k * 16 * 128) >> 4),
                       kSub == 1 ? idesc_pv : idesc_pv_all, t > 0 || k > 0);
        umma_commit(kv_empty(stage));
        umma_commit(pv_done(buf));
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const unsigned lane_field = (unsigned)(quarter * 32) << 16;
    const int qpos = row < rows_used ? first_qpos + row / groups : -1;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int t = 0; ok && t < ntiles; ++t) {
      const int buf = t & 1, stage = t % kKvStages;
      const int key0 = (tile_lo + t) * kKeys;
      if (!mbar_wait(s_full(buf), (unsigned)(t >> 1) & 1, p.error_flag, 16)) { ok = false; break; }
      tcgen05_fence_after();
      unsigned sa[32], sb[32];
      __syncwarp();
      tmem_load32(tmem_s[buf] + lane_field, sa);
      tmem_load32(tmem_s[buf] + lane_field + 32, sb);
      tmem_load_wait();

      const bool all_visible = key0 + kKeys - 1 <= first_qpos && (p.window <= 0 || key0 > last_qpos - p.window);
      float mx = m;
      if (all_visible && qpos >= 0) {
        float part[4] = {m, m, m, m};      // four chains, so that the maxima do not wait for one another
#pragma unroll
        for (int j = 0; j < 32; ++j) part[j & 3] = max3(part[j & 3], __uint_as_float(sa[j]), __uint_as_float(sb[j]));
        mx = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int ka = key0 + j, kb = key0 + 32 + j;
          const bool va = ka <= qpos && (p.window <= 0 || ka > qpos - p.window);
          const bool vb = kb <= qpos && (p.window <= 0 || kb > qpos - p.window);
          if (!va) sa[j] = __float_as_uint(-INFINITY);
          if (!vb) sb[j] = __float_as_uint(-INFINITY);
          mx = fmaxf(mx, fmaxf(__uint_as_float(sa[j]), __uint_as_float(sb[j])));
        }
      }
      // Exponentials are taken against m, which follows the row's maximum lazily: it moves only when the maximum
      // has outgrown it by more than 2^kLazyLog2, so that the accumulator is rarely rescaled.  Numerator and
      // denominator share m, so the result is the same up to rounding; values stay below 2^kLazyLog2.
      float m_new = m, alpha = 1.f;
      if ((mx - m) * p.scale_log2 > kLazyLog2) {     // also when m is still -inf and a score is not
        m_new = mx;
        alpha = ex2((m - mx) * p.scale_log2);
      }
      const bool rescale = alpha != 1.f && m != -INFINITY;   // a row that has seen no key yet holds zeros
      const float neg = m_new == -INFINITY ? 0.f : -m_new * p.scale_log2;
      // Column c of the probabilities holds keys 2c and 2c + 1 of the tile; they go where the scores were.
      float2 sums[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), neg2 = make_float2(neg, neg);
      unsigned packed[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int j = 2 * c;
        const float2 x = make_float2(__uint_as_float(j < 32 ? sa[j] : sb[j - 32]),
                                     __uint_as_float(j + 1 < 32 ? sa[j + 1] : sb[j + 1 - 32]));
        const float2 y = fma2(x, scale2, neg2);
        const float2 ev = make_float2(ex2(y.x), ex2(y.y));
        sums[c & 3] = add2(sums[c & 3], ev);
        __nv_bfloat162 h = __floats2bfloat162_rn(ev.x, ev.y);
        packed[c] = *reinterpret_cast<unsigned*>(&h);
      }
      tmem_store32(tmem_s[buf] + lane_field, packed);
      const float2 total = add2(add2(sums[0], sums[1]), add2(sums[2], sums[3]));
      const float sum = total.x + total.y;
      // The accumulator may be rescaled only between P V of tile t-1 and P V of this tile; the latter waits for
      // this warp's arrival below.  The softmax of this tile has not waited for P V of the last one otherwise.
      if (t >= 1 && __any_sync(0xffffffffu, rescale)) {
        if (!mbar_wait(pv_done((t - 1) & 1), (unsigned)((t - 1) >> 1) & 1, p.error_flag, 20)) { ok = false; break; }
        tcgen05_fence_after();
        unsigned o[32];
#pragma unroll
        for (int part = 0; part < D / 32; ++part) {
          tmem_load32(tmem_o + lane_field + part * 32, o);
          tmem_load_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_store32(tmem_o + lane_field + part * 32, o);
        }
      }
      tmem_store_wait();
      m = m_new;
      l = l * alpha + sum;
      // Value rows of keys outside [lo, hi) may hold anything (an unwritten slot): zero them before P V reads them.
      if (key0 < lo || key0 + kKeys > hi) {
        if (!mbar_wait(kv_full(stage), (unsigned)(t / kKvStages) & 1, p.error_flag, 18)) { ok = false; break; }
        unsigned char* vt = generic_base + (v_smem - base) + stage * kTileBytes;
        for (int e = threadIdx.x - 32 * (1 + X) - 128 * x; e < kSub * kKeys * 8; e += 128) {
          const int sub = e / (kKeys * 8), key = (e >> 3) % kKeys;
          const int kpos = key0 + key;
          if (kpos < lo || kpos >= hi)
            *reinterpret_cast<uint4*>(vt + sub * kKeySubBytes + key * 128 + ((e & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        fence_async_shared();
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(buf));
    }
    // Output: wait for the last P V, read the row, divide by the row's sum, store.
    if (ok && ntiles > 0 && mbar_wait(pv_done((ntiles - 1) & 1), (unsigned)((ntiles - 1) >> 1) & 1, p.error_flag, 19)) {
      tcgen05_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int qi = q0 + row / groups, head = kvh * groups + row % groups;
      bf16* dst = p.out + (size_t)(q_begin + qi) * p.out_row_stride + (size_t)head * D;
#pragma unroll
      for (int half = 0; half < D / 32; ++half) {
        unsigned o[32];
        __syncwarp();
        tmem_load32(tmem_o + lane_field + half * 32, o);
        tmem_load_wait();
        if (row < rows_used) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            unsigned w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[v * 8 + 2 * e]) * inv,
                                                       __uint_as_float(o[v * 8 + 2 * e + 1]) * inv);
              w[e] = *reinterpret_cast<unsigned*>(&h);
            }
            *reinterpret_cast<uint4*>(dst + half * 32 + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// The pool [pages, kv_heads, page_size, head_dim] as a 2-D map of rows of head_dim; a box is 64 dimensions of one
// page of one head.
static bool make_pool_map(CUtensorMap* map, const void* pool, long rows, int page_size, int head_dim) {
  static std::map<std::tuple<const void*, long, int, int>, CUtensorMap> cache;
  static std::mutex guard;                 // several host threads may launch (an asyncio engine beside its caller)
  std::lock_guard<std::mutex> lock(guard);
  const auto key = std::make_tuple(pool, rows, page_size, head_dim);
  const auto found = cache.find(key);
  if (found != cache.end()) {
    *map = found->second;
    return true;
  }
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
  const cuuint32_t elem[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *map);
  return true;
}

template <int D, int X>
static int launch_tc_attention(const CUtensorMap& mk, const CUtensorMap& mv, const TcAttnParams& p, dim3 grid,
                               cudaStream_t stream) {
  constexpr int kKvStages = KvStages<D, X>::value;
  constexpr size_t smem = (size_t)X * (D / 64) * kRows * 64 * 2 + 2 * kKvStages * (size_t)kKeys * D * 2 +
                          8 * (3 * kKvStages + 6 * X + 2) + 16 + 1024;
  static_assert(smem <= 232448, "more shared memory than a block may have");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel<D, X>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)launch_pdl(0, attention_tcgen05_kernel<D, X>, grid, dim3(attn_threads<X>()), smem, stream, mk, mv, p);
}

}  // namespace li

using namespace li;

// Whether li_paged_attention_tcgen05 takes these sizes.
LI_EXPORT int li_paged_attention_tcgen05_supports(int heads, int kv_heads, int head_dim, int page_size) {
  if (kv_heads < 1 || heads % kv_heads || (head_dim != 64 && head_dim != 128)) return 0;
  const int groups = heads / kv_heads;
  if (groups > kRows) return 0;      // a block's 128 rows hold 128 / groups query tokens (the rest is padding)
  return page_size == 16 || page_size == 32 || page_size == 64;
}

// bfloat16; head_dim 64 or 128; page_size 16, 32 or 64; groups of at most 128 heads.  Sequences may bring any number of queries
// (the kernel is meant for those that bring many).  error_flag (device int, zero): set if a wait inside gave up.
LI_EXPORT int li_paged_attention_tcgen05(const void* q, int q_row_stride, void* out, int out_row_stride,
                                         const void* k_pool, const void* v_pool, const int* block_table,
                                         int table_stride, const int* query_start_loc, const int* context_lens,
                                         const int* seq_index, int num_seqs, int max_q_len, int heads, int kv_heads,
                                         int head_dim, int page_size, int num_pages, float scale, int window,
                                         int* error_flag, cudaStream_t stream) {
  if (num_seqs == 0 || max_q_len == 0) return 0;
  if (!li_paged_attention_tcgen05_supports(heads, kv_heads, head_dim, page_size)) return LI_ERR_UNSUPPORTED;
  if (num_seqs > 65535 || (max_q_len + 0L) * heads / kv_heads / kRows >= 65535) return LI_ERR_UNSUPPORTED;
  if ((q_row_stride % 8) || (out_row_stride % 8) || !aligned16(q) || !aligned16(out) || !aligned16(k_pool) ||
      !aligned16(v_pool))
    return LI_ERR_ALIGNMENT;
  CUtensorMap mk, mv;
  const long rows = (long)num_pages * kv_heads * page_size;
  if (!make_pool_map(&mk, k_pool, rows, page_size, head_dim) || !make_pool_map(&mv, v_pool, rows, page_size, head_dim))
    return LI_ERR_UNSUPPORTED;
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  TcAttnParams p{(const bf16*)q, q_row_stride, (bf16*)out, out_row_stride, block_table, table_stride,
                 query_start_loc, context_lens, seq_index, heads, kv_heads, page_size, shift, num_pages,
                 scale * kLog2eF, window, error_flag};
  const int groups = heads / kv_heads;
  const int tq = kRows / groups;
  // Two query tiles per block at head size 128 where some sequence brings enough queries for two
  // (LITEINFER_TCGEN05_ATTN_TILES=1 keeps one).
  static const bool one_tile = [] { const char* e = getenv("LITEINFER_TCGEN05_ATTN_TILES"); return e && atoi(e) == 1; }();
  if (head_dim == 128 && max_q_len > tq && !one_tile)
    return launch_tc_attention<128, 2>(mk, mv, p, dim3(kv_heads, num_seqs, (max_q_len + 2 * tq - 1) / (2 * tq)), stream);
  const dim3 grid(kv_heads, num_seqs, (max_q_len + tq - 1) / tq);
  return head_dim == 64 ? launch_tc_attention<64, 1>(mk, mv, p, grid, stream)
                        : launch_tc_attention<128, 1>(mk, mv, p, grid, stream);
}
