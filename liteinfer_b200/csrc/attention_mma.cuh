// What the tensor-core attention kernels share: parameters, fragment helpers, and the two merges of a split
// decode (the warps of a block, then the blocks of a sequence).
#pragma once
#include "common.cuh"

namespace li {

constexpr int kBlockM = 64;   // rows (query token x head in group) per block
constexpr int kBlockN = 64;   // keys per tile
constexpr int kWarps = 4;
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
  const bf16* q;
  int q_row_stride;
  bf16* out;
  int out_row_stride;
  const bf16* k_pool;
  const bf16* v_pool;
  const int* block_table;
  int table_stride;
  const int* query_start_loc;
  const int* context_lens;
  const int* seq_index;   // optional: batch row of each launched sequence
  int heads, kv_heads, page_size, num_pages;
  int page_shift;         // log2(page_size) when it is a power of two, else -1
  float scale_log2;       // scale * log2(e)
  int window;
  int num_splits;
  float* partial_out;     // [tokens * heads * splits, D] when num_splits > 1
  float* partial_lse;     // [tokens * heads * splits]
  unsigned* counters;     // [grid.z * kv_heads * query tiles], zero between launches, when num_splits > 1
  // Decode with the rotary encoding and the cache write fused in (see li_paged_attention_mma): q, k_new and
  // v_new are the unrotated projections of each sequence's newest token, all with q_row_stride.
  const float* rope_inv_freq;   // [D / 2], or null: q is already rotated and the newest key is in its page
  const bf16* k_new;
  const bf16* v_new;
  int store_new;                // 0: this layer reads pages that another layer writes
  int* error_flag;              // kernels with bounded waits record here where one gave up (may be null)
  int cluster_merge;            // the splits of a (sequence, KV head) are one thread-block cluster and merge through
                                // distributed shared memory (attention_stream.cu only)
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;   // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x for x <= 0 (and -inf -> 0) in one instruction; the argument is a score minus the running maximum.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Tile [rows][D] of bf16 in shared memory; the 16-byte chunk c of row r lives at chunk c ^ (r & 7).
template <int D> __device__ __forceinline__ bf16* tile_ptr(bf16* base, int row, int chunk) {
  return base + row * D + ((chunk ^ (row & 7)) << 3);
}

// Decode: the four warps of a block each saw a quarter of the keys and left (accumulator, maximum, sum) in
// shared memory (os [4][16][D], ms and ls [4][16]); their combination is the block's result: the output itself,
// or with several splits this split's partial result and its log-sum-exp.
template <int D>
__device__ __forceinline__ void combine_warps(const AttnParams& p, const float* os, const float* ms, const float* ls,
                                              int rows_used, int groups, int q_begin, int q0, int kvh, int split) {
  for (int e = threadIdx.x; e < rows_used * D; e += kWarps * 32) {
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
    const int qi = q0 + row / groups, head = kvh * groups + row % groups;
    const float value = denom > 0.f ? acc / denom : 0.f;
    if (p.num_splits == 1) {
      p.out[(size_t)(q_begin + qi) * p.out_row_stride + (size_t)head * D + d] = __float2bfloat16_rn(value);
    } else {
      const size_t slot = ((size_t)(q_begin + qi) * p.heads + head) * p.num_splits + split;
      p.partial_out[slot * D + d] = value;
      if (d == 0) p.partial_lse[slot] = denom > 0.f ? mx + log2f(denom) : -INFINITY;
    }
  }
}

// The block that arrives last at the counter of its (sequence, KV head, query tile) merges the splits' partial
// results (in split order, eight at a time) into the output and leaves the counter at zero.  Called by all threads
// of every block of a split launch, after the block's partial result is written (`smem_raw` is not used any more).
template <int D>
__device__ __forceinline__ void merge_splits(const AttnParams& p, unsigned char* smem_raw, bool* is_last_flag,
                                             int rows_used, int groups, int q_begin, int q0, int kvh, int qtile) {
  // ---- the block that arrives last merges the splits of this (sequence, KV head, query tile).
  __threadfence();
  __syncthreads();
  const unsigned counter_index = ((unsigned)blockIdx.z * gridDim.y + blockIdx.y) * (gridDim.x / p.num_splits) + qtile;
  if (threadIdx.x == 0) {
    const unsigned arrived = atomicAdd(&p.counters[counter_index], 1u);
    *is_last_flag = arrived == (unsigned)p.num_splits - 1;
  }
  __syncthreads();
  if (!*is_last_flag) return;
  __threadfence();
  // A thread merges four dimensions of one row, eight splits at a time: the eight log-sum-exps and the eight partial
  // rows are asked for together (one trip to L2 per eight splits), and the running result is rescaled to the largest
  // log-sum-exp seen so far, as a softmax over blocks of keys would be.  Where the block has more threads than such
  // items, P neighbouring lanes share an item (lane j takes the splits j, j + P, ...) and merge their running
  // results by shuffles at the end.  No shared memory, no barrier.
  const int S = p.num_splits;
  const int items = rows_used * (D / 4);
  const int P = items * 4 <= kWarps * 32 ? 4 : (items * 2 <= kWarps * 32 ? 2 : 1);
  for (int e0 = 0; e0 < items * P; e0 += kWarps * 32) {
    const int e = e0 + threadIdx.x;
    const bool live = e < items * P;             // (whole warps are live or not where P > 1: items * P is a multiple of 32 then, or the loop runs once)
    const int item = live ? e / P : 0, part = e % P;
    const int row = item / (D / 4), d4 = item % (D / 4);
    const int qi = q0 + row / groups, head = kvh * groups + row % groups;
    const size_t first = ((size_t)(q_begin + qi) * p.heads + head) * S;
    const float* lse = p.partial_lse + first;
    const float4* src = reinterpret_cast<const float4*>(p.partial_out + first * D) + d4;
    float mx = -INFINITY, denom = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = part; live && s0 < S; s0 += 8 * P) {
      float w[8];
      float4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j * P < S) {
          w[j] = __ldcg(lse + s0 + j * P);
          v[j] = __ldcg(src + (size_t)(s0 + j * P) * (D / 4));
        }
      float top = mx;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j * P < S) top = fmaxf(top, w[j]);
      if (top == -INFINITY) continue;            // nothing seen yet in any of these splits
      const float keep = mx == -INFINITY ? 0.f : exp2f(mx - top);
      denom *= keep;
      acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
      mx = top;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j * P < S) {
          const float wj = w[j] == -INFINITY ? 0.f : exp2f(w[j] - top);
          denom += wj;
          acc.x += wj * v[j].x; acc.y += wj * v[j].y; acc.z += wj * v[j].z; acc.w += wj * v[j].w;
        }
    }
    // The lanes of an item meet: each pair's results are scaled to the larger maximum and added.
    for (int o = 1; o < P; o <<= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, mx, o), dn = __shfl_xor_sync(0xffffffffu, denom, o);
      const float ax = __shfl_xor_sync(0xffffffffu, acc.x, o), ay = __shfl_xor_sync(0xffffffffu, acc.y, o);
      const float az = __shfl_xor_sync(0xffffffffu, acc.z, o), aw = __shfl_xor_sync(0xffffffffu, acc.w, o);
      const float top = fmaxf(mx, mo);
      const float mine = mx == -INFINITY ? 0.f : exp2f(mx - top), theirs = mo == -INFINITY ? 0.f : exp2f(mo - top);
      denom = denom * mine + dn * theirs;
      acc.x = acc.x * mine + ax * theirs; acc.y = acc.y * mine + ay * theirs;
      acc.z = acc.z * mine + az * theirs; acc.w = acc.w * mine + aw * theirs;
      mx = top;
    }
    if (live && part == 0) {
      const float inv = denom > 0.f ? 1.f / denom : 0.f;
      bf16* dst = p.out + (size_t)(q_begin + qi) * p.out_row_stride + (size_t)head * D + d4 * 4;
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
    }
  }
  if (threadIdx.x == 0) p.counters[counter_index] = 0;   // ready for the next launch
}

}  // namespace li
