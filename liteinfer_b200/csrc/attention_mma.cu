// Paged attention on tensor cores for bfloat16, head sizes 64 and 128: whole
// prompts, portions of prompts and single decoded tokens, with the keys of one
// sequence optionally split over several blocks (decode at small batch), plus the
// kernel that merges the splits.
//
// Rule as in attention_generic.cu (liteinfer/models/attention.py:24-27,69-84): a
// sequence's queries are the last q_len positions of its context; query head h
// reads KV head h / groups.  A block owns a tile of 64 rows for one KV head, a
// row being (query token, head of the group): grouped heads share every K/V
// tile that is loaded (liteinfer/models/paged_kernels.py:291-371 packs the group
// into its query rows the same way).  Scores, running maximum and sum, the
// accumulator, split partials and their log-sum-exp are 32-bit; probabilities
// are rounded to bfloat16 for P.V (paged_kernels.py:282-284).
//
// Two shapes of block.  With several query tokens per sequence each of the four
// warps owns 16 of the tile's 64 rows and walks all 64 keys of a K/V tile.  With
// one token per sequence (decode) the rows of a tile are just the heads of one
// group (at most 16), so all four warps share those rows and each takes 16 of
// the tile's 64 keys; their four running softmax states are merged through
// shared memory at the end.  When the keys are split over several blocks, each
// block leaves its partial result in scratch memory and bumps a counter; the
// block that arrives last merges the splits (in split order) and resets the
// counter, so no second launch and no waiting is needed.
//
// Data path: K and V tiles of 64 keys are gathered page by page with cp.async
// into swizzled shared memory, double buffered; fragments come from ldmatrix;
// the products are mma.sync m16n8k16 (bf16 in, f32 out).  Keys outside the
// visible range are zero-filled in shared memory and masked to -inf, so an
// unwritten page cannot leak.
#include "attention_mma.cuh"

namespace li {

// One K tile and one V tile of 64 keys -> shared memory.  A thread always copies the same 16-byte chunk
// of a row and walks the keys in steps of (threads / chunks per row), so the index arithmetic of a tile
// is a few instructions per copy; a page size that is a power of two is divided by shifting.
template <int D>
__device__ __forceinline__ void load_kv_tile(bf16* ks, bf16* vs, const AttnParams& p, const int* table, int kvh,
                                             int tile_start, int lo, int hi) {
  constexpr int kChunks = D / 8;
  constexpr int kKeysPerPass = kWarps * 32 / kChunks;
  const int chunk = threadIdx.x % kChunks, key0 = threadIdx.x / kChunks;
#pragma unroll
  for (int pass = 0; pass < kBlockN / kKeysPerPass; ++pass) {
    const int key = key0 + pass * kKeysPerPass;
    const int kpos = tile_start + key;
    bool valid = kpos >= lo && kpos < hi;
    size_t off = 0;
    if (valid) {
      const int block = p.page_shift >= 0 ? kpos >> p.page_shift : kpos / p.page_size;
      const int slot = p.page_shift >= 0 ? kpos & (p.page_size - 1) : kpos - block * p.page_size;
      const int page = table[block];
      valid = page >= 0 && page < p.num_pages;
      if (valid) off = (((size_t)page * p.kv_heads + kvh) * p.page_size + slot) * D + chunk * 8;
    }
    cp_async16(tile_ptr<D>(ks, key, chunk), p.k_pool + off, valid);
    cp_async16(tile_ptr<D>(vs, key, chunk), p.v_pool + off, valid);
  }
}

// kDecode: every launched sequence brings one token and the group has at most 16 heads.
template <int D, bool kDecode, int kStages>   // kStages: K/V tiles in flight per block
__global__ void __launch_bounds__(kWarps * 32)   // forcing a sixth block per SM (80 registers) measured slower in a step
attention_mma_kernel(const AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int kQRows = kDecode ? 16 : kBlockM;
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);           // [kQRows][D]
  bf16* kbuf = qs + kQRows * D;                           // kStages x [64][D]
  bf16* vbuf = kbuf + kStages * kBlockN * D;              // kStages x [64][D]
  __shared__ bool is_last;
  __shared__ float rope_cos[D / 2], rope_sin[D / 2];
  __shared__ __align__(16) bf16 newest[2 * D];   // the rotated key and the value of the newest token

  // Tables and lengths are inputs of the step; what an earlier kernel wrote is read after the wait below.
  const int seq = p.seq_index ? p.seq_index[blockIdx.z] : blockIdx.z;
  if (seq < 0) return;        // a place of padding in the list of sequences
  const int kvh = blockIdx.y;
  // The last query tiles see the most keys: they are handed out first.
  const int split = blockIdx.x % p.num_splits, qtile = (int)(gridDim.x / p.num_splits) - 1 - (int)(blockIdx.x / p.num_splits);
  const int q_begin = p.query_start_loc[seq], q_len = p.query_start_loc[seq + 1] - q_begin;
  const int groups = p.heads / p.kv_heads;
  const int tq = (kDecode ? 16 : kBlockM) / groups;       // query tokens per tile
  const int q0 = qtile * tq;
  if (q0 >= q_len) return;
  const int ctx = p.context_lens[seq];
  const int tile_q = min(tq, q_len - q0);
  const int rows_used = tile_q * groups;
  const int* table = p.block_table + (size_t)seq * p.table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  constexpr int kChunks = D / 8;
  constexpr int kGroupsPerWarp = kDecode ? 1 : kBlockN / 16;   // 16-key groups of a tile that a warp walks
  const int row_base = kDecode ? 0 : warp * 16;               // first tile row of this warp
  const int key_group0 = kDecode ? warp : 0;                  // first 16-key group of this warp

  // Visible keys of this tile: [lo, hi).
  const int first_qpos = ctx - q_len + q0, last_qpos = first_qpos + tile_q - 1;
  const int hi = last_qpos + 1;
  const int lo = (p.window > 0 && first_qpos - p.window + 1 > 0) ? first_qpos - p.window + 1 : 0;
  const int tile_lo = lo / kBlockN, tile_hi = (hi + kBlockN - 1) / kBlockN;   // key tiles [tile_lo, tile_hi)
  const int ntiles = tile_hi - tile_lo;
  const int per_split = (ntiles + p.num_splits - 1) / p.num_splits;
  const int my_lo = tile_lo + split * per_split, my_hi = min(tile_hi, my_lo + per_split);

  const bool fused = kDecode && p.rope_inv_freq != nullptr;
  const int newest_pos = ctx - 1;
  // With the rotary encoding fused in, the block whose keys include the newest position rotates that key,
  // stores it and the value into their page, and uses them from shared memory.
  const bool owns_newest = fused && p.store_new && newest_pos / kBlockN >= my_lo && newest_pos / kBlockN < my_hi;
  if (kDecode && fused) {
    for (int i = threadIdx.x; i < D / 2; i += kWarps * 32) {
      const float angle = __fmul_rn((float)newest_pos, p.rope_inv_freq[i]);
      rope_cos[i] = cosf(angle);
      rope_sin[i] = sinf(angle);
    }
    // The pages hold nothing that the kernel before this one wrote (the newest token is stored here, not
    // there), so the first K/V tiles are requested before that kernel is waited for.
#pragma unroll
    for (int st = 0; st < kStages - 1; ++st) {
      if (my_lo + st < my_hi)
        load_kv_tile<D>(kbuf + st * kBlockN * D, vbuf + st * kBlockN * D, p, table, kvh, (my_lo + st) * kBlockN, lo, hi);
      cp_async_commit();
    }
  }
  grid_dependency_wait();   // q, and without the fused rotation the newest keys and values, come from the kernels before
  if (kDecode && fused) {
    __syncthreads();
    constexpr int kItems = D / 16;                   // work items of eight pairs (j, j + D/2) per head
    const size_t token = (size_t)(q_begin + q0) * p.q_row_stride;
    for (int w = threadIdx.x; w < kQRows * kItems; w += kWarps * 32) {
      const int row = w / kItems, j = (w % kItems) * 8;
      Vec16<bf16> lo, hi;
      if (row < rows_used) {
        const bf16* src = p.q + token + (size_t)(kvh * groups + row) * D + j;
        rotate_eight(load16(src), load16(src + D / 2), rope_cos + j, rope_sin + j, lo, hi);
      } else {
        lo.raw = hi.raw = make_uint4(0, 0, 0, 0);
      }
      store16(tile_ptr<D>(qs, row, j / 8), lo);
      store16(tile_ptr<D>(qs, row, (j + D / 2) / 8), hi);
    }
    if (owns_newest) {
      const int page = table[p.page_shift >= 0 ? newest_pos >> p.page_shift : newest_pos / p.page_size];
      const int slot = newest_pos - (p.page_shift >= 0 ? (newest_pos >> p.page_shift) << p.page_shift
                                                       : newest_pos / p.page_size * p.page_size);
      const bool store = page >= 0 && page < p.num_pages;
      const size_t dst = (((size_t)(store ? page : 0) * p.kv_heads + kvh) * p.page_size + slot) * D;
      bf16* k_pool = const_cast<bf16*>(p.k_pool);
      bf16* v_pool = const_cast<bf16*>(p.v_pool);
      for (int w = threadIdx.x; w < kItems + D / 8; w += kWarps * 32) {
        if (w < kItems) {
          const int j = w * 8;
          const bf16* src = p.k_new + token + (size_t)kvh * D + j;
          Vec16<bf16> lo, hi;
          rotate_eight(load16(src), load16(src + D / 2), rope_cos + j, rope_sin + j, lo, hi);
          store16(newest + j, lo);
          store16(newest + j + D / 2, hi);
          if (store) {
            store16(k_pool + dst + j, lo);
            store16(k_pool + dst + j + D / 2, hi);
          }
        } else {
          const int j = (w - kItems) * 8;
          const Vec16<bf16> v = load16(p.v_new + token + (size_t)kvh * D + j);
          store16(newest + D + j, v);
          if (store) store16(v_pool + dst + j, v);
        }
      }
    }
  } else {
    // ---- Q tile -> shared (zero rows beyond rows_used), then A fragments in registers.
    for (int c = threadIdx.x; c < kQRows * kChunks; c += kWarps * 32) {
      const int row = c / kChunks, chunk = c % kChunks;
      const bool valid = row < rows_used;
      const int qi = q0 + row / groups, head = kvh * groups + row % groups;
      const bf16* src = p.q + (valid ? (size_t)(q_begin + qi) * p.q_row_stride + (size_t)head * D + chunk * 8 : 0);
      cp_async16(tile_ptr<D>(qs, row, chunk), src, valid);
    }
  }
  if (!fused) {
    cp_async_commit();
    // The first kStages-1 tiles are requested at once; a group is committed per tile even when it is empty.
#pragma unroll
    for (int st = 0; st < kStages - 1; ++st) {
      if (my_lo + st < my_hi)
        load_kv_tile<D>(kbuf + st * kBlockN * D, vbuf + st * kBlockN * D, p, table, kvh, (my_lo + st) * kBlockN, lo, hi);
      cp_async_commit();
    }
    cp_async_wait<kStages - 1>();   // the Q tile has landed
  }
  __syncthreads();

  unsigned qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk)
    ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3],
                tile_ptr<D>(qs, row_base + (lane & 15), kk * 2 + (lane >> 4)));

  // Rows of this thread: row_base + g and + 8.
  int qpos[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = row_base + g + 8 * h;
    qpos[h] = row < rows_used ? first_qpos + row / groups : -1;   // -1: a padding row sees nothing
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

  for (int tile = my_lo; tile < my_hi; ++tile) {
    const int buf = (tile - my_lo) % kStages;
    bf16* ks = kbuf + buf * kBlockN * D;
    bf16* vs = vbuf + buf * kBlockN * D;
    {
      const int ahead = tile + kStages - 1, abuf = (ahead - my_lo) % kStages;
      if (ahead < my_hi)
        load_kv_tile<D>(kbuf + abuf * kBlockN * D, vbuf + abuf * kBlockN * D, p, table, kvh, ahead * kBlockN, lo, hi);
    }
    cp_async_commit();
    cp_async_wait<kStages - 1>();   // all but the newest kStages-1 groups are complete: this tile is here
    __syncthreads();
    if (kDecode && owns_newest && tile == newest_pos / kBlockN) {
      // The page's copy of the newest token may be older than the store above: take it from shared memory.
      const int key = newest_pos - tile * kBlockN;
      if (threadIdx.x < 2 * kChunks) {
        const int c = threadIdx.x % kChunks;
        bf16* dst = tile_ptr<D>(threadIdx.x < kChunks ? ks : vs, key, c);
        store16(dst, load16(newest + (threadIdx.x < kChunks ? 0 : D) + c * 8));
      }
      __syncthreads();
    }

    // S = Q K^T for 16 rows x (16 keys per group).
    float s[kGroupsPerWarp * 2][4];
#pragma unroll
    for (int i = 0; i < kGroupsPerWarp * 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int nn = 0; nn < kGroupsPerWarp; ++nn) {
        unsigned b0, b1, b2, b3;
        const int mtx = lane >> 3;
        ldmatrix_x4(b0, b1, b2, b3,
                    tile_ptr<D>(ks, (key_group0 + nn) * 16 + (mtx >> 1) * 8 + (lane & 7), kk * 2 + (mtx & 1)));
        mma_bf16(s[nn * 2], qf[kk], b0, b1);
        mma_bf16(s[nn * 2 + 1], qf[kk], b2, b3);
      }
    }

    // Scale, mask, online softmax.
    const int key0 = tile * kBlockN + key_group0 * 16;
    float tile_max[2] = {-INFINITY, -INFINITY};
    // A tile needs the mask only where it meets the diagonal or the window's start.  (Rows of padding hold
    // zero queries: their scores are finite, and they are never stored.)
    const bool all_visible = (tile + 1) * kBlockN - 1 <= first_qpos &&
                             (p.window <= 0 || tile * kBlockN > last_qpos - p.window);
    if (all_visible) {
#pragma unroll
      for (int i = 0; i < kGroupsPerWarp * 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          s[i][j] *= p.scale_log2;
          tile_max[j >> 1] = fmaxf(tile_max[j >> 1], s[i][j]);
        }
    } else {
#pragma unroll
      for (int i = 0; i < kGroupsPerWarp * 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kpos = key0 + i * 8 + 2 * t + (j & 1);
          const int qp = qpos[j >> 1];
          const bool visible = kpos <= qp && (p.window <= 0 || kpos > qp - p.window);
          s[i][j] = visible ? s[i][j] * p.scale_log2 : -INFINITY;
          tile_max[j >> 1] = fmaxf(tile_max[j >> 1], s[i][j]);
        }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
      const float m_new = fmaxf(m[h], tile_max[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;
      alpha[h] = fast_exp2(m[h] - m_use[h]);   // m = -inf gives 0
      m[h] = m_new;
    }
    float row_sum[2] = {0.f, 0.f};
    unsigned pf[kGroupsPerWarp][4];
#pragma unroll
    for (int i = 0; i < kGroupsPerWarp * 2; ++i) {
      float e[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        e[j] = fast_exp2(s[i][j] - m_use[j >> 1]);
        row_sum[j >> 1] += e[j];
      }
      pf[i >> 1][(i & 1) * 2] = pack_bf16(e[0], e[1]);
      pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(e[2], e[3]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) l[h] = l[h] * alpha[h] + row_sum[h];
    // The accumulator is rescaled only when some row of the warp saw a new maximum.
    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
        o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
      }
    }

    // O += P V.
#pragma unroll
    for (int kb = 0; kb < kGroupsPerWarp; ++kb) {
#pragma unroll
      for (int dd = 0; dd < D / 16; ++dd) {
        unsigned b0, b1, b2, b3;
        const int mtx = lane >> 3;
        ldmatrix_x4_trans(b0, b1, b2, b3,
                          tile_ptr<D>(vs, (key_group0 + kb) * 16 + (mtx & 1) * 8 + (lane & 7), dd * 2 + (mtx >> 1)));
        mma_bf16(o[dd * 2], pf[kb], b0, b1);
        mma_bf16(o[dd * 2 + 1], pf[kb], b2, b3);
      }
    }
    __syncthreads();   // this buffer is overwritten by the load issued in the next iteration
  }
  cp_async_wait<0>();
  grid_launch_dependents();

  // Row sums across the quad.
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }

  if (kDecode) {
    // ---- merge the four warps' states (each saw a quarter of the keys) through shared memory.
    __syncthreads();
    float* os = reinterpret_cast<float*>(kbuf);            // [4 warps][16 rows][D]
    float* ms = os + kWarps * 16 * D;                      // [4][16]
    float* ls = ms + kWarps * 16;                          // [4][16]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = g + 8 * h;
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<float2*>(os + ((size_t)warp * 16 + row) * D + i * 8 + 2 * t) =
            make_float2(o[i][2 * h], o[i][2 * h + 1]);
      if (t == 0) {
        ms[warp * 16 + row] = m[h];
        ls[warp * 16 + row] = l[h];
      }
    }
    __syncthreads();
    combine_warps<D>(p, os, ms, ls, rows_used, groups, q_begin, q0, kvh, split);
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = row_base + g + 8 * h;
      if (row >= rows_used) continue;
      const int qi = q0 + row / groups, head = kvh * groups + row % groups;
      const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
      if (p.num_splits == 1) {
        bf16* dst = p.out + (size_t)(q_begin + qi) * p.out_row_stride + (size_t)head * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
          *reinterpret_cast<unsigned*>(dst + i * 8 + 2 * t) = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
      } else {
        const size_t slot = ((size_t)(q_begin + qi) * p.heads + head) * p.num_splits + split;
        float* dst = p.partial_out + slot * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
          *reinterpret_cast<float2*>(dst + i * 8 + 2 * t) = make_float2(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
        // log-sum-exp in base 2 of the scaled scores; -inf marks a split that saw no key
        if (t == 0) p.partial_lse[slot] = l[h] > 0.f ? m[h] + log2f(l[h]) : -INFINITY;
      }
    }
  }
  if (p.num_splits == 1) return;

  merge_splits<D>(p, smem_raw, &is_last, rows_used, groups, q_begin, q0, kvh, qtile);
}

template <int D, bool kDecode, int kStages>
int launch_attention(const AttnParams& p, int num_seqs, int max_q_len, cudaStream_t stream) {
  const int groups = p.heads / p.kv_heads;
  const int tq = (kDecode ? 16 : kBlockM) / groups;
  const size_t smem = (size_t)((kDecode ? 16 : kBlockM) + 2 * kStages * kBlockN) * D * sizeof(bf16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<D, kDecode, kStages>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const dim3 grid(((max_q_len + tq - 1) / tq) * p.num_splits, p.kv_heads, num_seqs);
  return (int)launch_pdl((long)num_seqs * max_q_len, attention_mma_kernel<D, kDecode, kStages>, grid, dim3(kWarps * 32), smem, stream, p);
}

// Blocks of the decode kernel with kStages K/V tiles per block that the current device holds at once
// (asked of the occupancy calculator the first time); 0 if the query fails.
template <int D, int kStages>
int decode_capacity() {
  static int capacity = -1;
  if (capacity >= 0) return capacity;
  int device = 0, sms = 0, per_sm = 0;
  const size_t smem = (size_t)(16 + 2 * kStages * kBlockN) * D * sizeof(bf16);
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
      cudaFuncSetAttribute(attention_mma_kernel<D, true, kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_mma_kernel<D, true, kStages>, kWarps * 32,
                                                    smem) != cudaSuccess)
    return 0;
  capacity = per_sm * sms;
  return capacity;
}

}  // namespace li

using namespace li;

// Counters the launch needs when num_splits > 1 (unsigned, all zero before the first launch).
LI_EXPORT int li_paged_attention_mma_counters(int num_seqs, int max_q_len, int heads, int kv_heads) {
  const int groups = heads / kv_heads;
  const bool decode = max_q_len == 1 && groups <= 16;
  const int tq = (decode ? 16 : kBlockM) / groups;
  return num_seqs * kv_heads * ((max_q_len + tq - 1) / tq);
}

// How many blocks of the decode launch (the variant with two K/V tiles per block) the device holds at once:
// a launch of up to this many blocks runs as one wave.  0 if the head size has no kernel or the query fails.
LI_EXPORT int li_paged_attention_mma_decode_capacity(int head_dim) {
  return head_dim == 64 ? decode_capacity<64, 2>() : (head_dim == 128 ? decode_capacity<128, 2>() : 0);
}

// Tensor-core paged attention (bfloat16; head_dim 64 or 128; groups of at most 64 heads).
// seq_index (optional, [num_seqs]): the batch rows to run, so that a mixed step can send its
// single-token sequences through a split launch and the others through an unsplit one.
// num_splits > 1 needs scratch: partial_out [tokens*heads*splits, head_dim] and partial_lse
// [tokens*heads*splits] (float32, tokens = rows of q), and `counters`
// (li_paged_attention_mma_counters(...) unsigned values, zero; the kernel leaves them zero).
// rope_inv_freq (optional, [head_dim / 2] float32; only with max_q_len 1 and groups of at most 16): the rotary
// encoding and the cache write are done here instead of by li_rope_kv_write.  q, k_new and v_new then point at
// the unrotated projections of the tokens (same row stride); every sequence brings exactly one token, at position
// context_len - 1.  q is rotated on its way into shared memory (the buffer keeps the unrotated values); the key
// is rotated and, with store_new, written to its page together with the value.  Without store_new the pages
// already hold the newest token.
LI_EXPORT int li_paged_attention_mma(const void* q, int q_row_stride, void* out, int out_row_stride,
                                     const void* k_pool, const void* v_pool, const int* block_table,
                                     int table_stride, const int* query_start_loc, const int* context_lens,
                                     const int* seq_index, int num_seqs, int max_q_len, int heads, int kv_heads,
                                     int head_dim, int page_size, int num_pages, float scale, int window,
                                     int num_splits, float* partial_out, float* partial_lse, unsigned* counters,
                                     const float* rope_inv_freq, const void* k_new, const void* v_new, int store_new,
                                     cudaStream_t stream) {
  if (num_seqs == 0 || max_q_len == 0) return 0;
  if (kv_heads < 1 || heads % kv_heads) return LI_ERR_UNSUPPORTED;
  const int groups = heads / kv_heads;
  if (groups > kBlockM || (head_dim != 64 && head_dim != 128)) return LI_ERR_UNSUPPORTED;
  if (kv_heads > 65535 || num_seqs > 65535 || num_splits < 1 || num_splits > 32) return LI_ERR_UNSUPPORTED;
  if (num_splits > 1 && (out_row_stride % 4)) return LI_ERR_ALIGNMENT;
  if (num_splits > 1 && (!partial_out || !partial_lse || !counters)) return LI_ERR_UNSUPPORTED;
  if ((q_row_stride % 8) || (out_row_stride % 2) || !aligned16(q) || !aligned16(k_pool) || !aligned16(v_pool))
    return LI_ERR_ALIGNMENT;
  AttnParams p{(const bf16*)q, q_row_stride, (bf16*)out, out_row_stride, (const bf16*)k_pool, (const bf16*)v_pool,
               block_table, table_stride, query_start_loc, context_lens, seq_index, heads, kv_heads, page_size,
               num_pages, -1, scale * kLog2e, window, num_splits, partial_out, partial_lse, counters,
               rope_inv_freq, (const bf16*)k_new, (const bf16*)v_new, store_new};
  if ((page_size & (page_size - 1)) == 0)
    for (int s = 0; s < 31; ++s)
      if ((1 << s) == page_size) p.page_shift = s;
  const bool decode = max_q_len == 1 && groups <= 16;
  if (rope_inv_freq && (!decode || !k_new || !v_new || !aligned16(k_new) || !aligned16(v_new))) return LI_ERR_UNSUPPORTED;
  if (!decode)
    return head_dim == 64 ? launch_attention<64, false, 2>(p, num_seqs, max_q_len, stream)
                          : launch_attention<128, false, 2>(p, num_seqs, max_q_len, stream);
  // As many K/V tiles in flight per block as still lets all blocks of the launch run at once: few blocks (a
  // narrow batch) go deep, many blocks get more of themselves per SM instead.
  static int stages_override = -1;
  if (stages_override < 0) {
    const char* e = getenv("LITEINFER_DECODE_STAGES");
    stages_override = e ? atoi(e) : 0;
  }
  const long blocks = (long)num_seqs * kv_heads * num_splits;
  if (head_dim == 64) {
    int stages = blocks <= decode_capacity<64, 4>() ? 4 : (blocks <= decode_capacity<64, 3>() ? 3 : 2);
    if (stages_override) stages = stages_override;
    if (stages >= 4) return launch_attention<64, true, 4>(p, num_seqs, max_q_len, stream);
    if (stages == 3) return launch_attention<64, true, 3>(p, num_seqs, max_q_len, stream);
    return launch_attention<64, true, 2>(p, num_seqs, max_q_len, stream);
  }
  int stages = blocks <= decode_capacity<128, 3>() ? 3 : 2;
  if (stages_override) stages = stages_override;
  return stages >= 3 ? launch_attention<128, true, 3>(p, num_seqs, max_q_len, stream)
                     : launch_attention<128, true, 2>(p, num_seqs, max_q_len, stream);
}
