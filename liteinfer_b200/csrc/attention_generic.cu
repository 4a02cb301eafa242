// Paged attention for any batch of (sequence, its newest queries), in plain SIMT
// code: the true 32-bit path, and the path for head sizes and types the tensor-core
// kernels refuse.  One kernel serves whole prompts, portions of prompts and single
// decoded tokens in the same launch.
//
// Rule (liteinfer/models/attention.py:24-27,81-84): a sequence's queries are the
// last `q_len` positions of its context of `ctx` tokens, so query j has position
// ctx - q_len + j and sees keys 0..position (with a window w: the newest w of
// them).  Query head h reads KV head h / groups (attention.py:69-78).  Scores,
// running maximum, sum and the output accumulator are 32-bit; the softmax is
// the online form (liteinfer/models/paged_kernels.py:216-288).
//
// Work split: block = (query tile, KV head, sequence); its warps take the rows
// (query, head-in-group) of the tile in turn, one row per warp at a time.  A row
// walks its keys 32 at a time from the first visible one rounded down to a
// multiple of 32, so the order of every sum depends on the row's position only,
// never on how the batch was cut.  Masked keys are not read at all: a page that
// was never written, or holds another request's tokens, cannot leak through a
// NaN or a stale value.
#include "common.cuh"

namespace li {

constexpr int kMaxHeadDim = 256;
constexpr int kQueriesPerBlock = 8;

template <typename T>
__global__ void __launch_bounds__(256)
paged_attention_generic_kernel(const T* __restrict__ q, int q_row_stride, T* __restrict__ out, int out_row_stride,
                               const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                               const int* __restrict__ block_table, int table_stride,
                               const int* __restrict__ query_start_loc, const int* __restrict__ context_lens,
                               int heads, int kv_heads, int head_dim, int page_size, int num_pages, float scale,
                               int window) {
  extern __shared__ float q_smem[];  // [warps][head_dim]
  const int seq = blockIdx.z, kvh = blockIdx.y;
  const int q_begin = query_start_loc[seq], q_len = query_start_loc[seq + 1] - q_begin;
  const int tile_start = blockIdx.x * kQueriesPerBlock;
  if (tile_start >= q_len) return;
  const int ctx = context_lens[seq];
  const int groups = heads / kv_heads;
  const int tile_q = min(kQueriesPerBlock, q_len - tile_start);
  const int rows = tile_q * groups;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  float* qs = q_smem + warp * head_dim;
  const int* table = block_table + (size_t)seq * table_stride;
  constexpr int kDimsPerLane = kMaxHeadDim / 32;

  for (int row = warp; row < rows; row += nwarps) {
    const int qi = tile_start + row / groups;          // query index within the sequence's queries
    const int head = kvh * groups + row % groups;
    const int qpos = ctx - q_len + qi;                 // absolute position of this query
    const T* qrow = q + (size_t)(q_begin + qi) * q_row_stride + (size_t)head * head_dim;
    __syncwarp();
    for (int d = lane; d < head_dim; d += 32) qs[d] = to_float(qrow[d]);
    __syncwarp();

    int first = 0;
    if (window > 0 && qpos - window + 1 > 0) first = qpos - window + 1;
    float m = -INFINITY, l = 0.f;
    float acc[kDimsPerLane];
#pragma unroll
    for (int i = 0; i < kDimsPerLane; ++i) acc[i] = 0.f;

    for (int base = (first / 32) * 32; base <= qpos; base += 32) {
      const int kpos = base + lane;
      const bool valid = kpos >= first && kpos <= qpos;
      int krow = -1;  // row index of this lane's key inside the pool: (page * kv_heads + kvh) * page_size + slot
      float s = -INFINITY;
      if (valid) {
        const int page = table[kpos / page_size];
        if (page >= 0 && page < num_pages) {
          krow = (page * kv_heads + kvh) * page_size + kpos % page_size;
          const T* kp = k_pool + (size_t)krow * head_dim;
          float dot = 0.f;
          for (int d = 0; d < head_dim; ++d) dot += qs[d] * to_float(kp[d]);
          s = dot * scale;
        }
      }
      const float m_new = fmaxf(m, warp_max(s));
      if (m_new == -INFINITY) continue;  // nothing visible in this chunk (cannot happen for a valid row)
      const float p = krow >= 0 ? expf(s - m_new) : 0.f;
      const float alpha = expf(m - m_new);  // m = -inf on the first chunk gives 0
      l = l * alpha + warp_sum(p);
#pragma unroll
      for (int i = 0; i < kDimsPerLane; ++i) acc[i] *= alpha;
      // The probability is rounded to the value type before P.V (paged_kernels.py:282-284).
      const float p_store = round_to<T>(p);
      unsigned live = __ballot_sync(0xffffffffu, krow >= 0);
      while (live) {
        const int j = __ffs(live) - 1;
        live &= live - 1;
        const float pj = __shfl_sync(0xffffffffu, p_store, j);
        const int vr = __shfl_sync(0xffffffffu, krow, j);
        const T* vp = v_pool + (size_t)vr * head_dim;
#pragma unroll
        for (int i = 0; i < kDimsPerLane; ++i) {
          const int d = lane + 32 * i;
          if (d < head_dim) acc[i] += pj * to_float(vp[d]);
        }
      }
      m = m_new;
    }
    T* orow = out + (size_t)(q_begin + qi) * out_row_stride + (size_t)head * head_dim;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < kDimsPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < head_dim) orow[d] = from_float<T>(acc[i] * inv);
    }
  }
}

}  // namespace li

using namespace li;

// q: [tokens, q_row_stride] with head h of a token at columns [h*head_dim, (h+1)*head_dim).
// out: [tokens, out_row_stride] likewise.  k_pool / v_pool: [num_pages, kv_heads, page_size, head_dim].
// window <= 0: every earlier key is visible.
LI_EXPORT int li_paged_attention_generic(int dtype, const void* q, int q_row_stride, void* out, int out_row_stride,
                                         const void* k_pool, const void* v_pool, const int* block_table,
                                         int table_stride, const int* query_start_loc, const int* context_lens,
                                         int num_seqs, int max_q_len, int heads, int kv_heads, int head_dim,
                                         int page_size, int num_pages, float scale, int window,
                                         cudaStream_t stream) {
  if (num_seqs == 0 || max_q_len == 0) return 0;
  if (head_dim < 1 || head_dim > kMaxHeadDim || kv_heads < 1 || heads % kv_heads) return LI_ERR_UNSUPPORTED;
  if (kv_heads > 65535 || num_seqs > 65535) return LI_ERR_UNSUPPORTED;
  const int threads = 256;
  const dim3 grid((max_q_len + kQueriesPerBlock - 1) / kQueriesPerBlock, kv_heads, num_seqs);
  const size_t smem = (size_t)(threads / 32) * head_dim * sizeof(float);
  if (dtype == kFloat32)
    paged_attention_generic_kernel<float><<<grid, threads, smem, stream>>>(
        (const float*)q, q_row_stride, (float*)out, out_row_stride, (const float*)k_pool, (const float*)v_pool,
        block_table, table_stride, query_start_loc, context_lens, heads, kv_heads, head_dim, page_size, num_pages,
        scale, window);
  else
    paged_attention_generic_kernel<bf16><<<grid, threads, smem, stream>>>(
        (const bf16*)q, q_row_stride, (bf16*)out, out_row_stride, (const bf16*)k_pool, (const bf16*)v_pool,
        block_table, table_stride, query_start_loc, context_lens, heads, kv_heads, head_dim, page_size, num_pages,
        scale, window);
  LI_LAUNCH_CHECK();
}
