// Paged attention for single decoded tokens with one TMA pipeline per warp
// (bfloat16, head sizes 64 and 128, groups of at most 16 heads, pages of a multiple of 16 tokens).
//
// Rule and split scheme as in attention_mma.cu: a block owns one (sequence, KV head, split of the keys), its
// rows are the heads of the group; with several splits the last block to arrive merges them.  What differs
// is the data path.  Each of the four warps walks its own 16 keys of every 64-key tile and never meets the
// others before the end.  A group of 16 keys lies in one page (hence pages of a multiple of 16 tokens), so its
// keys are one box of the pool's tensor map and its values another (two each for head size 128): one lane asks
// for them with cp.async.bulk.tensor into the warp's own ring of shared-memory slots, several groups ahead,
// and an mbarrier per slot tells the warp when a group has landed.  No thread computes an address per row, and
// no block barrier sits in the loop.  Every wait is bounded; one that runs out sets `error_flag`.
//
// Fragments come out of the 128-byte-swizzled slots with 16-byte loads in the order mma.sync wants:
//
//   S = Q K^T   B operand = K.  Thread (g, t) of a warp (g = lane / 4, t = lane % 4) reads pieces t, t+4, ...
//               of key g.  The eight values of a piece serve two k steps (values 0-3, then 4-7), and the
//               same pieces of Q's row are the A operand, so both sides meet the dimensions in the same
//               (permuted) order, which a sum over dimensions does not notice.
//   O += P V    B operand = V.  Thread (g, t) reads, of keys 2t, 2t+1, 2t+8, 2t+9, the piece(s) that hold
//               dimensions g*D/8 ...; byte permutes pair the two keys of each k slot.  Output tile j of
//               the product then holds dimension g*D/8 + j in column g, so a thread ends up with D/4
//               consecutive dimensions of rows g and g+8.
//
// The splits of one (sequence, KV head) merge without a trip to global memory where the launch can make them one
// thread-block cluster (up to 16 splits, the partial results fitting beside the warps' states): every block leaves
// its combined result in its own shared memory, the cluster meets at a barrier, the first block reads the others'
// results through distributed shared memory, merges and writes the output, and a second barrier keeps the others
// resident until it has read them.  Otherwise the last block to arrive at a counter merges partial results that
// went through global memory (merge_splits), which costs every block a fence and an atomic and the last one three
// more trips to L2.
//
// With the rotary encoding fused in (see li_paged_attention_mma) the owner of the newest position writes the
// rotated key and the value to their page and, for its own use, takes them from shared memory.
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "attention_mma.cuh"
#include "tcgen05.cuh"

#ifndef RING64
#define RING64 2
#endif

namespace li {

constexpr int kMaxRing = 4;
constexpr int kGroupKeys = 16;

__device__ __forceinline__ uint4 lds16(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 ldg16(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ unsigned low_halves(unsigned a, unsigned b) { return __byte_perm(a, b, 0x5410); }
__device__ __forceinline__ unsigned high_halves(unsigned a, unsigned b) { return __byte_perm(a, b, 0x7632); }
__device__ __forceinline__ unsigned word(const uint4& v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }

// Piece `piece` (16 bytes: dimensions 8*piece ...) of row `row` of a slot half (K or V): boxes of 16 rows x 64
// dimensions, 2 KB each, rows of 128 bytes whose 16-byte pieces are swizzled by the row's low three bits.
__device__ __forceinline__ unsigned piece_addr(unsigned half_base, int row, int piece) {
  return half_base + (unsigned)((piece >> 3) * 2048 + row * 128 + (((piece & 7) ^ (row & 7)) << 4));
}

// The end of a block whose (sequence, KV head) is one cluster of splits (rank = split): see the head of the file.
// A function of its own, so that its registers are not the loop's.
template <int D>
__device__ __noinline__ void merge_in_cluster(const AttnParams& p, const float* os, const float* ms, float* ls, int groups,
                                              int q_begin, int kvh, int split) {
  // ---- the splits are one cluster (rank = split).  This block's result: mine [groups][D], normalised, and its
  // log-sum-exp per row, behind the warps' states in this block's own shared memory.
  float* mine = ls + kWarps * 16;                        // [16][D]
  float* mine_lse = mine + 16 * D;                       // [16]
  float* weights = mine_lse + 16;                        // [16][17], the first block only
  for (int e = threadIdx.x; e < groups * D; e += kWarps * 32) {
    const int row = e / D, d = e % D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, ms[w * 16 + row]);
    float denom = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = ms[w * 16 + row];
      const float wgt = mw == -INFINITY ? 0.f : exp2f(mw - mx);
      denom += wgt * ls[w * 16 + row];
      acc += wgt * os[((size_t)w * 16 + row) * D + d];
    }
    mine[row * D + d] = denom > 0.f ? acc / denom : 0.f;
    if (d == 0) mine_lse[row] = denom > 0.f ? mx + log2f(denom) : -INFINITY;
  }
  cluster_sync_all();                                    // every block's result is in place (release / acquire)
  if (split == 0) {
    const int S = p.num_splits;
    auto remote = [&](const float* local, int rank) {    // the same place in the shared memory of block `rank`
      unsigned addr;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(smem_addr(local)), "r"(rank));
      return addr;
    };
    for (int e = threadIdx.x; e < groups * S; e += kWarps * 32) {
      const int row = e / S, s = e % S;
      float v;
      asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote(mine_lse + row, s)));
      weights[row * 17 + s] = v;
    }
    __syncthreads();
    if (threadIdx.x < groups) {
      float* w = weights + threadIdx.x * 17;
      float mx = -INFINITY;
      for (int s = 0; s < S; ++s) mx = fmaxf(mx, w[s]);
      float denom = 0.f;
      for (int s = 0; s < S; ++s) {
        const float e = w[s] == -INFINITY ? 0.f : exp2f(w[s] - mx);
        w[s] = e;
        denom += e;
      }
      const float inv = denom > 0.f ? 1.f / denom : 0.f;
      for (int s = 0; s < S; ++s) w[s] *= inv;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < groups * (D / 4); e += kWarps * 32) {
      const int row = e / (D / 4), d4 = e % (D / 4);
      const float* w = weights + row * 17;
      float4 v[16];
#pragma unroll
      for (int s = 0; s < 16; ++s)
        if (s < S)
          asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(v[s].x), "=f"(v[s].y), "=f"(v[s].z), "=f"(v[s].w) : "r"(remote(mine + row * D + d4 * 4, s)));
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int s = 0; s < 16; ++s)
        if (s < S) {
          acc.x += w[s] * v[s].x; acc.y += w[s] * v[s].y; acc.z += w[s] * v[s].z; acc.w += w[s] * v[s].w;
        }
      bf16* dst = p.out + (size_t)q_begin * p.out_row_stride + (size_t)(kvh * groups + row) * D + d4 * 4;
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    }
  }
  cluster_sync_all();                                    // nobody leaves while the first block reads
}

// kRing: slots per warp; up to kRing - 1 groups are on their way while one is multiplied.
template <int D, int kRing, bool kCluster>
__global__ void __launch_bounds__(kWarps * 32, D == 64 ? 5 : 2)   // blocks per SM that the rings leave room for
attention_stream_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const AttnParams p) {
  constexpr unsigned kHalfBytes = kGroupKeys * D * 2;      // K or V of one group
  constexpr unsigned kSlotBytes = 2 * kHalfBytes;
  constexpr int kBoxes = D / 64;                           // boxes of 64 dimensions per row
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  unsigned char* generic_base = smem_raw + (base - smem_addr(smem_raw));
  __shared__ bool is_last;
  __shared__ float rope_cos[D / 2], rope_sin[D / 2];
  __shared__ __align__(16) bf16 newest[2 * D];             // the rotated key and the value of the newest token
  __shared__ __align__(8) unsigned long long ring_bars[kWarps * kMaxRing];
  __shared__ int slot_filled[kWarps * kMaxRing];           // whether the slot's current group was fetched at all

  const int seq = p.seq_index ? p.seq_index[blockIdx.z] : blockIdx.z;
  if (seq < 0) return;        // a place of padding in the list of sequences
  const int kvh = blockIdx.y, split = blockIdx.x;
  const int q_begin = p.query_start_loc[seq];
  const int groups = p.heads / p.kv_heads;
  const int ctx = p.context_lens[seq];
  const int* table = p.block_table + (size_t)seq * p.table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int qpos = ctx - 1, hi = ctx;
  const int lo = (p.window > 0 && qpos - p.window + 1 > 0) ? qpos - p.window + 1 : 0;
  const int tile_lo = lo / kBlockN, tile_hi = (hi + kBlockN - 1) / kBlockN;
  const int per_split = (tile_hi - tile_lo + p.num_splits - 1) / p.num_splits;
  const int my_lo = tile_lo + split * per_split, my_hi = min(tile_hi, my_lo + per_split);
  const int my_groups = max(0, my_hi - my_lo);             // groups of this warp: one per tile of the block
  const bool fused = p.rope_inv_freq != nullptr;
  const bool owns_newest = fused && p.store_new && qpos / kBlockN >= my_lo && qpos / kBlockN < my_hi;
  const unsigned ring = base + (unsigned)warp * kRing * kSlotBytes;
  const unsigned bars = smem_addr(ring_bars) + (unsigned)warp * kRing * 8;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kWarps * kRing; ++i) mbar_init(smem_addr(ring_bars) + 8u * i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (fused)
    for (int i = threadIdx.x; i < D / 2; i += kWarps * 32) {
      const float angle = __fmul_rn((float)qpos, p.rope_inv_freq[i]);
      rope_cos[i] = cosf(angle);
      rope_sin[i] = sinf(angle);
    }
  __syncthreads();

  // First row (in the pool seen as rows of D) of the group this warp takes from tile `my_lo + i`, or -1 when
  // none of its keys is visible (or its page was given back: then all of them lie before the window).
  auto group_row = [&](int i) -> long {
    const int kpos0 = (my_lo + i) * kBlockN + warp * kGroupKeys;
    if (i >= my_groups || kpos0 >= hi || kpos0 + kGroupKeys <= lo) return -1;
    const int block = p.page_shift >= 0 ? kpos0 >> p.page_shift : kpos0 / p.page_size;
    const int page = table[block];
    if (page < 0 || page >= p.num_pages) return -1;
    return ((long)page * p.kv_heads + kvh) * p.page_size + (kpos0 - block * p.page_size);
  };
  // One lane asks for group i's boxes, or just arrives where there is nothing to fetch (the slot's phase moves on
  // either way).  The slot's last reader has finished: the warp synchronised after reading it.
  auto request = [&](int i) {
    if (lane != 0 || i >= my_groups) return;
    const unsigned slot = ring + (unsigned)(i % kRing) * kSlotBytes, bar = bars + 8u * (i % kRing);
    const long row = group_row(i);
    slot_filled[warp * kMaxRing + i % kRing] = row >= 0;      // read by the warp after its wait on the barrier below
    if (row < 0) {
      mbar_arrive(bar);
      return;
    }
    mbar_expect_tx(bar, kSlotBytes);
#pragma unroll
    for (int b = 0; b < kBoxes; ++b) {
      tma_load_2d(slot + b * 2048, &map_k, bar, b * 64, (int)row);
      tma_load_2d(slot + kHalfBytes + b * 2048, &map_v, bar, b * 64, (int)row);
    }
  };
  // The pages hold nothing that the kernel before this one wrote when the cache write is fused in here; otherwise
  // the newest key and value come from it, and the first requests wait for it too.
  if (fused)
    for (int i = 0; i < kRing - 1; ++i) request(i);
  grid_dependency_wait();
  if (!fused)
    for (int i = 0; i < kRing - 1; ++i) request(i);

  const size_t token = (size_t)q_begin * p.q_row_stride;
  // Q: rows g and g+8 of the group (zero beyond it), pieces t, t+4, ...  Asked for before the newest key and value
  // below, so that both trips to L2 run side by side.
  uint4 qa[2][D / 32];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = g + 8 * h;
    const bf16* src = p.q + token + (size_t)(kvh * groups + row) * D;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) qa[h][c] = row < groups ? ldg16(src + (t + 4 * c) * 8) : make_uint4(0, 0, 0, 0);
  }
  if (owns_newest) {
    // The rotated key and the value of the newest token: to their page for the steps to come, and to shared
    // memory for this one (the copy on its way from the page may be older than the store).
    const int block = p.page_shift >= 0 ? qpos >> p.page_shift : qpos / p.page_size;
    const int page = table[block];
    const bool store = page >= 0 && page < p.num_pages;
    const size_t dst = (((size_t)(store ? page : 0) * p.kv_heads + kvh) * p.page_size + (qpos - block * p.page_size)) * D;
    bf16* k_pool = const_cast<bf16*>(p.k_pool);
    bf16* v_pool = const_cast<bf16*>(p.v_pool);
    for (int w = threadIdx.x; w < D / 16 + D / 8; w += kWarps * 32) {
      if (w < D / 16) {
        const int j = w * 8;
        const bf16* src = p.k_new + token + (size_t)kvh * D + j;
        Vec16<bf16> low, high;
        rotate_eight(load16(src), load16(src + D / 2), rope_cos + j, rope_sin + j, low, high);
        store16(newest + j, low);
        store16(newest + j + D / 2, high);
        if (store) {
          store16(k_pool + dst + j, low);
          store16(k_pool + dst + j + D / 2, high);
        }
      } else {
        const int j = (w - D / 16) * 8;
        const Vec16<bf16> v = load16(p.v_new + token + (size_t)kvh * D + j);
        store16(newest + D + j, v);
        if (store) store16(v_pool + dst + j, v);
      }
    }
    __syncthreads();
  }

  // Q is rotated here when the rotation is fused in (pieces t+4c and t+4c+D/16 hold the two halves of the same pairs).
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = g + 8 * h;
    if (fused && row < groups) {
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        Vec16<bf16> a, b, low, high;
        a.raw = qa[h][c];
        b.raw = qa[h][c + D / 64];
        const int j = (t + 4 * c) * 8;
        rotate_eight(a, b, rope_cos + j, rope_sin + j, low, high);
        qa[h][c] = low.raw;
        qa[h][c + D / 64] = high.raw;
      }
    }
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

  // Where this thread's pieces lie inside a slot (the swizzle depends on the row only): K pieces t, t+4, ... of
  // keys g and g+8; V pieces g*D/64 ... of keys 2t, 2t+1, 2t+8, 2t+9.
  unsigned k_at[2][D / 32], v_at[4][D / 64];
#pragma unroll
  for (int half = 0; half < 2; ++half)
#pragma unroll
    for (int c = 0; c < D / 32; ++c) k_at[half][c] = piece_addr(0, half * 8 + g, t + 4 * c);
#pragma unroll
  for (int q = 0; q < 4; ++q)
#pragma unroll
    for (int c = 0; c < D / 64; ++c)
      v_at[q][c] = kHalfBytes + piece_addr(0, 2 * t + (q & 1) + (q >> 1) * 8, g * (D / 64) + c);

  for (int i = 0; i < my_groups; ++i) {
    request(i + kRing - 1);
    const int kpos0 = (my_lo + i) * kBlockN + warp * kGroupKeys;
    if (kpos0 < hi && kpos0 + kGroupKeys > lo) {
      if (!mbar_wait(bars + 8u * (i % kRing), (unsigned)(i / kRing) & 1, p.error_flag, 21)) {
        // Gave up: before the ring's memory is used for anything else, give the copies still on their way one
        // more (bounded) chance to land.
        for (int r = i + 1; r < my_groups && r < i + kRing - 1; ++r)
          mbar_wait(bars + 8u * (r % kRing), (unsigned)(r / kRing) & 1, nullptr, 0);
        break;
      }
      const unsigned slot = ring + (unsigned)(i % kRing) * kSlotBytes;
      const bool filled = slot_filled[warp * kMaxRing + i % kRing] != 0;
      if (owns_newest && qpos >= kpos0 && qpos < kpos0 + kGroupKeys) {
        // This group holds the newest token: its row of the slot is replaced by what this kernel computed.
        const int row = qpos - kpos0;
        if (lane < 2 * (D / 8)) {
          const int piece = lane % (D / 8);
          const bool is_v = lane >= D / 8;
          unsigned char* dst = generic_base + (slot - base) + (is_v ? kHalfBytes : 0) +
                               (piece >> 3) * 2048 + row * 128 + (((piece & 7) ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(newest + (is_v ? D : 0) + piece * 8);
        }
        __syncwarp();
      }
      if (filled) {
        // S = Q K^T: two tiles of eight keys.
        float s[2][4];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int j = 0; j < 4; ++j) s[half][j] = 0.f;
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            const uint4 k = lds16(slot + k_at[half][c]);
            const unsigned a_lo[4] = {qa[0][c].x, qa[1][c].x, qa[0][c].y, qa[1][c].y};
            const unsigned a_hi[4] = {qa[0][c].z, qa[1][c].z, qa[0][c].w, qa[1][c].w};
            mma_bf16(s[half], a_lo, k.x, k.y);
            mma_bf16(s[half], a_hi, k.z, k.w);
          }
        }
        uint4 v[4][D / 64];
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int c = 0; c < D / 64; ++c) v[q][c] = lds16(slot + v_at[q][c]);
        // Scale and mask (only a group at the end of the context or at the window's start needs the mask; values
        // of keys that are not visible become zero there, since an unwritten slot of a page may hold anything).
        float group_max[2] = {-INFINITY, -INFINITY};
        if (kpos0 >= lo && kpos0 + kGroupKeys <= hi) {
#pragma unroll
          for (int half = 0; half < 2; ++half)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              s[half][j] *= p.scale_log2;
              group_max[j >> 1] = fmaxf(group_max[j >> 1], s[half][j]);
            }
        } else {
#pragma unroll
          for (int half = 0; half < 2; ++half)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int kpos = kpos0 + half * 8 + 2 * t + (j & 1);
              s[half][j] = (kpos >= lo && kpos < hi) ? s[half][j] * p.scale_log2 : -INFINITY;
              group_max[j >> 1] = fmaxf(group_max[j >> 1], s[half][j]);
            }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int kpos = kpos0 + 2 * t + (q & 1) + (q >> 1) * 8;
            if (kpos < lo || kpos >= hi)
#pragma unroll
              for (int c = 0; c < D / 64; ++c) v[q][c] = make_uint4(0, 0, 0, 0);
          }
        }
        // Online softmax.
        float alpha[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          group_max[h] = fmaxf(group_max[h], __shfl_xor_sync(0xffffffffu, group_max[h], 1));
          group_max[h] = fmaxf(group_max[h], __shfl_xor_sync(0xffffffffu, group_max[h], 2));
          const float m_new = fmaxf(m[h], group_max[h]);
          m_use[h] = m_new == -INFINITY ? 0.f : m_new;
          alpha[h] = fast_exp2(m[h] - m_use[h]);   // m = -inf gives 0
          m[h] = m_new;
        }
        float row_sum[2] = {0.f, 0.f};
        unsigned pa[4];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float e[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            e[j] = fast_exp2(s[half][j] - m_use[j >> 1]);
            row_sum[j >> 1] += e[j];
          }
          pa[half * 2] = pack_bf16(e[0], e[1]);        // row g, keys 2t, 2t+1 of this half
          pa[half * 2 + 1] = pack_bf16(e[2], e[3]);    // row g+8
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) l[h] = l[h] * alpha[h] + row_sum[h];
        if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
          for (int j = 0; j < D / 8; ++j) {
            o[j][0] *= alpha[0]; o[j][1] *= alpha[0];
            o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
          }
        }
        // O += P V: output tile j of the product is dimension g*D/8 + j in column g.
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
          const int c = j / 8, w = (j % 8) / 2;
          const unsigned b0 = (j & 1) ? high_halves(word(v[0][c], w), word(v[1][c], w))
                                      : low_halves(word(v[0][c], w), word(v[1][c], w));
          const unsigned b1 = (j & 1) ? high_halves(word(v[2][c], w), word(v[3][c], w))
                                      : low_halves(word(v[2][c], w), word(v[3][c], w));
          mma_bf16(o[j], pa, b0, b1);
        }
      }
    }
    __syncwarp();     // every lane is done with this slot before lane 0 asks for new contents
  }
  grid_launch_dependents();

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  // The warps' states through shared memory (the rings are no longer needed once every warp is here).  Thread
  // (g, t) holds, of rows g and g+8, the dimensions (2t)*D/8 + j and (2t+1)*D/8 + j for j < D/8.
  __syncthreads();
  float* os = reinterpret_cast<float*>(generic_base);    // [4 warps][16 rows][D]
  float* ms = os + kWarps * 16 * D;                      // [4][16]
  float* ls = ms + kWarps * 16;                          // [4][16]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = g + 8 * h;
    if (row >= groups) continue;          // rows of padding are never read
    float4* dst = reinterpret_cast<float4*>(os + ((size_t)warp * 16 + row) * D + (2 * t) * (D / 8));
#pragma unroll
    for (int j = 0; j < D / 8; j += 4) {
      dst[j / 4] = make_float4(o[j][2 * h], o[j + 1][2 * h], o[j + 2][2 * h], o[j + 3][2 * h]);
      dst[(D / 8 + j) / 4] = make_float4(o[j][2 * h + 1], o[j + 1][2 * h + 1], o[j + 2][2 * h + 1], o[j + 3][2 * h + 1]);
    }
    if (t == 0) {
      ms[warp * 16 + row] = m[h];
      ls[warp * 16 + row] = l[h];
    }
  }
  __syncthreads();
  if (!kCluster) {
    combine_warps<D>(p, os, ms, ls, groups, groups, q_begin, 0, kvh, split);
    if (p.num_splits == 1) return;
    merge_splits<D>(p, generic_base, &is_last, groups, groups, q_begin, 0, kvh, 0);
    return;
  }
  merge_in_cluster<D>(p, os, ms, ls, groups, q_begin, kvh, split);
}

// The rings, which at the end hold the warps' states ([4][16][D] floats and two of [4][16]) and, with a cluster's
// merge, the block's own result ([16][D], [16]) and the first block's weights ([16][17]).
template <int D, int kRing> constexpr size_t stream_smem() {
  constexpr size_t rings = (size_t)kWarps * kRing * 2 * kGroupKeys * D * 2;
  constexpr size_t states = ((size_t)kWarps * 16 * D + 2 * kWarps * 16 + 16 * D + 16 + 16 * 17) * sizeof(float);
  return (rings > states ? rings : states) + 1024;
}

// The pool [pages, kv_heads, page_size, D] as a 2-D map of rows of D with boxes of 16 rows x 64 dimensions.
static bool make_group_map(CUtensorMap* map, const void* pool, long rows, int head_dim) {
  static std::map<std::tuple<const void*, long, int>, CUtensorMap> cache;
  static std::mutex guard;                 // several host threads may launch (an asyncio engine beside its caller)
  std::lock_guard<std::mutex> lock(guard);
  const auto key = std::make_tuple(pool, rows, head_dim);
  const auto found = cache.find(key);
  if (found != cache.end()) {
    *map = found->second;
    return true;
  }
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)kGroupKeys};
  const cuuint32_t elem[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *map);
  return true;
}

template <int D, int kRing>
int launch_stream(const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p, int num_seqs, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_stream_kernel<D, kRing, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)stream_smem<D, kRing>());
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_stream_kernel<D, kRing, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)stream_smem<D, kRing>());
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const dim3 grid(p.num_splits, p.kv_heads, num_seqs);
  if (!p.cluster_merge)
    return (int)launch_pdl(num_seqs, attention_stream_kernel<D, kRing, false>, grid, dim3(kWarps * 32), stream_smem<D, kRing>(), stream, mk, mv, p);
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = dim3(kWarps * 32);
  config.dynamicSmemBytes = stream_smem<D, kRing>();
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = p.num_splits;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = pdl_enabled(num_seqs) ? 2 : 1;
  return (int)cudaLaunchKernelEx(&config, attention_stream_kernel<D, kRing, true>, mk, mv, p);
}

// How many clusters of `splits` blocks of the kernel the device holds at once (0: such a cluster cannot be launched).
template <int D, int kRing>
int stream_cluster_capacity(int splits) {
  static int cached[17] = {0};
  static bool known[17] = {false};
  if (splits < 2 || splits > 16) return 0;
  if (known[splits]) return cached[splits];
  int clusters = 0;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(splits, 148, 16);
  config.blockDim = dim3(kWarps * 32);
  config.dynamicSmemBytes = stream_smem<D, kRing>();
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = splits;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  if (cudaFuncSetAttribute(attention_stream_kernel<D, kRing, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)stream_smem<D, kRing>()) != cudaSuccess ||
      (splits > 8 && cudaFuncSetAttribute(attention_stream_kernel<D, kRing, true>,
                                          cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) ||
      cudaOccupancyMaxActiveClusters(&clusters, attention_stream_kernel<D, kRing, true>, &config) != cudaSuccess) {
    cudaGetLastError();
    clusters = 0;
  }
  cached[splits] = clusters;
  known[splits] = true;
  return clusters;
}

// Blocks of the kernel that the current device holds at once; 0 if the query fails.
template <int D, int kRing>
int stream_capacity() {
  static int capacity = -1;
  if (capacity >= 0) return capacity;
  int device = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
      cudaFuncSetAttribute(attention_stream_kernel<D, kRing, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)stream_smem<D, kRing>()) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_stream_kernel<D, kRing, false>, kWarps * 32,
                                                    stream_smem<D, kRing>()) != cudaSuccess)
    return 0;
  capacity = per_sm * sms;
  return capacity;
}

// Slots per warp: a slot is 4 KB at head size 64 and 8 KB at 128; with these, three blocks fit on an SM.
constexpr int kRing64 = RING64, kRing128 = 2;

}  // namespace li

using namespace li;

LI_EXPORT int li_paged_attention_stream_supports(int heads, int kv_heads, int head_dim, int page_size) {
  if (kv_heads < 1 || heads % kv_heads || heads / kv_heads > 16) return 0;
  if (head_dim != 64 && head_dim != 128) return 0;
  return page_size >= 16 && page_size % 16 == 0;
}

// Clusters of `splits` blocks that the device holds at once; 0 where the splits cannot be one cluster.
LI_EXPORT int li_paged_attention_stream_cluster_capacity(int head_dim, int splits) {
  return head_dim == 64 ? stream_cluster_capacity<64, kRing64>(splits)
                        : (head_dim == 128 ? stream_cluster_capacity<128, kRing128>(splits) : 0);
}

LI_EXPORT int li_paged_attention_stream_capacity(int head_dim) {
  return head_dim == 64 ? stream_capacity<64, kRing64>() : (head_dim == 128 ? stream_capacity<128, kRing128>() : 0);
}

// Every launched sequence brings exactly one token.  Arguments as li_paged_attention_mma (its counters export
// says how many counters a split launch needs); sizes as li_paged_attention_stream_supports allows.
// error_flag (device int, zero; may be null): set to 21 if a wait for a group of keys ever gave up.
LI_EXPORT int li_paged_attention_stream(const void* q, int q_row_stride, void* out, int out_row_stride,
                                        const void* k_pool, const void* v_pool, const int* block_table,
                                        int table_stride, const int* query_start_loc, const int* context_lens,
                                        const int* seq_index, int num_seqs, int heads, int kv_heads, int head_dim,
                                        int page_size, int num_pages, float scale, int window, int num_splits,
                                        float* partial_out, float* partial_lse, unsigned* counters,
                                        const float* rope_inv_freq, const void* k_new, const void* v_new,
                                        int store_new, int* error_flag, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (!li_paged_attention_stream_supports(heads, kv_heads, head_dim, page_size)) return LI_ERR_UNSUPPORTED;
  if (kv_heads > 65535 || num_seqs > 65535 || num_splits < 1 || num_splits > 32) return LI_ERR_UNSUPPORTED;
  if (num_splits > 1 && (out_row_stride % 4)) return LI_ERR_ALIGNMENT;
  if (num_splits > 1 && (!partial_out || !partial_lse || !counters)) return LI_ERR_UNSUPPORTED;
  if ((q_row_stride % 8) || (out_row_stride % 2) || !aligned16(q) || !aligned16(k_pool) || !aligned16(v_pool))
    return LI_ERR_ALIGNMENT;
  if (rope_inv_freq && (!k_new || !v_new || !aligned16(k_new) || !aligned16(v_new))) return LI_ERR_UNSUPPORTED;
  const long rows = (long)num_pages * kv_heads * page_size;
  if (rows > 0x7fffffffL) return LI_ERR_UNSUPPORTED;
  CUtensorMap mk, mv;
  if (!make_group_map(&mk, k_pool, rows, head_dim) || !make_group_map(&mv, v_pool, rows, head_dim))
    return LI_ERR_UNSUPPORTED;
  AttnParams p{(const bf16*)q, q_row_stride, (bf16*)out, out_row_stride, (const bf16*)k_pool, (const bf16*)v_pool,
               block_table, table_stride, query_start_loc, context_lens, seq_index, heads, kv_heads, page_size,
               num_pages, -1, scale * kLog2e, window, num_splits, partial_out, partial_lse, counters,
               rope_inv_freq, (const bf16*)k_new, (const bf16*)v_new, store_new, error_flag, 0};
  // LITEINFER_ATTN_CLUSTER_MERGE=1 (read at every call) merges the splits as clusters where all the launch's
  // clusters are resident at once.  Off by default: measured on B200 the launch alone gains (batch 8 at 4,096
  // tokens: 17.5 against 18.6 us; batch 1: 8.6 against 10.7), but inside the decode step, where every kernel starts
  // while the one before it drains (programmatic dependent launch), a launch of clusters starts later than a
  // launch of single blocks does, and the step loses more than the merge gains (1.065 against 0.948 ms).
  const char* cluster_env = getenv("LITEINFER_ATTN_CLUSTER_MERGE");
  if (cluster_env && atoi(cluster_env) == 1 && num_splits >= 2 && num_splits <= 16 &&
      li_paged_attention_stream_cluster_capacity(head_dim, num_splits) >= kv_heads * num_seqs)
    p.cluster_merge = 1;
  if ((page_size & (page_size - 1)) == 0)
    for (int s = 0; s < 31; ++s)
      if ((1 << s) == page_size) p.page_shift = s;
  return head_dim == 64 ? launch_stream<64, kRing64>(mk, mv, p, num_seqs, stream)
                        : launch_stream<128, kRing128>(mk, mv, p, num_seqs, stream);
}
