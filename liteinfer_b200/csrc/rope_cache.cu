// Rotary position encoding of q and k, fused with the write of k and v into the
// paged cache.
//
// q, k, v of a token lie side by side in one row of the fused projection's
// output: [q heads | k heads | v heads], each head `head_dim` wide.  q is rotated
// in place; k is rotated and v copied into this layer's pages.  Angles are
// position * inv_freq in 32-bit, cos and sin in 32-bit (liteinfer/models/llama.py:
// 78-86 computes them in float32 too, then rounds the tables to the model type;
// here the tables are never rounded, only the rotated result is).  Pairing is
// half-split: dimension j pairs with j + rotary_dim/2 (llama.py:89-102).
// Dimensions from rotary_dim on pass through unrotated.
//
// A page holds `page_size` tokens of every KV head: pool[page][kv_head][slot][dim].
// The page of a token is block_table[seq][position / page_size]; a negative entry
// (a page already given back) skips the write.
#include "common.cuh"

namespace li {

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                     int table_stride, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                     const float* __restrict__ inv_freq, int heads, int kv_heads, int head_dim,
                                     int rotary_dim, int page_size, int num_pages) {
  extern __shared__ float cs[];  // cos[half], sin[half]
  const int t = blockIdx.x;
  grid_launch_dependents();
  const int pos = positions[t];   // positions, tables and inv_freq are inputs of the step, not of a kernel
  const int half = rotary_dim / 2;
  float* cosv = cs;
  float* sinv = cs + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float angle = __fmul_rn((float)pos, inv_freq[i]);
    cosv[i] = cosf(angle);
    sinv[i] = sinf(angle);
  }
  const int seq = seq_of_token[t];
  const int page = seq < 0 ? -1 : block_table[(size_t)seq * table_stride + pos / page_size];   // a row of padding belongs to no sequence
  grid_dependency_wait();           // q, k and v come from the projection before this kernel
  __syncthreads();

  const int row_width = (heads + 2 * kv_heads) * head_dim;
  T* row = qkv + (size_t)t * row_width;

  // q: rotate in place.  Work item = (head, pair index or pass-through dim).
  const int pass = head_dim - rotary_dim;
  const int per_head = half;  // rotated pairs per head; pass-through dims stay as they are
  for (int w = threadIdx.x; w < heads * per_head; w += blockDim.x) {
    const int h = w / per_head, i = w - h * per_head;
    T* p = row + h * head_dim;
    const float a = to_float(p[i]), b = to_float(p[i + half]);
    p[i] = from_float<T>(rotate_lo(a, b, cosv[i], sinv[i]));
    p[i + half] = from_float<T>(rotate_hi(a, b, cosv[i], sinv[i]));
  }
  (void)pass;

  if (page < 0 || page >= num_pages) return;
  const int slot = pos % page_size;

  const T* krow = row + heads * head_dim;
  const T* vrow = krow + kv_heads * head_dim;
  for (int w = threadIdx.x; w < kv_heads * head_dim; w += blockDim.x) {
    const int h = w / head_dim, j = w - h * head_dim;
    const size_t dst = (((size_t)page * kv_heads + h) * page_size + slot) * head_dim + j;
    float kv;
    if (j < half) {
      kv = rotate_lo(to_float(krow[w]), to_float(krow[w + half]), cosv[j], sinv[j]);
    } else if (j < rotary_dim) {
      kv = rotate_hi(to_float(krow[w - half]), to_float(krow[w]), cosv[j - half], sinv[j - half]);
    } else {
      kv = to_float(krow[w]);
    }
    k_pool[dst] = from_float<T>(kv);
    v_pool[dst] = vrow[w];
  }
}

// The same with 16-byte accesses, for bfloat16 with every dimension rotated and halves that are multiples of
// eight: one work item is eight pairs (j, j + half) of one head, or eight values of v.
__global__ void rope_kv_write_vec_kernel(bf16* __restrict__ qkv, const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                         int table_stride, bf16* __restrict__ k_pool, bf16* __restrict__ v_pool,
                                         const float* __restrict__ inv_freq, int heads, int kv_heads, int head_dim,
                                         int page_size, int num_pages) {
  extern __shared__ float cs[];  // cos[half], sin[half]
  const int t = blockIdx.x;
  grid_launch_dependents();
  const int pos = positions[t];
  const int half = head_dim / 2;
  float* cosv = cs;
  float* sinv = cs + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float angle = __fmul_rn((float)pos, inv_freq[i]);
    cosv[i] = cosf(angle);
    sinv[i] = sinf(angle);
  }
  const int seq = seq_of_token[t];
  const int page = seq < 0 ? -1 : block_table[(size_t)seq * table_stride + pos / page_size];   // a row of padding belongs to no sequence
  grid_dependency_wait();
  __syncthreads();

  bf16* row = qkv + (size_t)t * (heads + 2 * kv_heads) * head_dim;
  const bool store = page >= 0 && page < num_pages;
  const int slot = pos % page_size;
  const int per_head = half / 8;                       // work items per rotated head
  const int rotated = (heads + kv_heads) * per_head;   // q heads, then k heads
  const int copies = kv_heads * (head_dim / 8);        // v
  for (int w = threadIdx.x; w < rotated + copies; w += blockDim.x) {
    if (w < rotated) {
      const int h = w / per_head, j = (w - h * per_head) * 8;
      bf16* p = row + h * head_dim + j;
      const Vec16<bf16> a = load16(p), b = load16(p + half);
      Vec16<bf16> lo, hi;
      rotate_eight(a, b, cosv + j, sinv + j, lo, hi);
      if (h < heads) {
        store16(p, lo);
        store16(p + half, hi);
      } else if (store) {
        bf16* dst = k_pool + (((size_t)page * kv_heads + (h - heads)) * page_size + slot) * head_dim + j;
        store16(dst, lo);
        store16(dst + half, hi);
      }
    } else if (store) {
      const int c = w - rotated;
      const int h = c / (head_dim / 8), j = (c % (head_dim / 8)) * 8;
      const bf16* src = row + (heads + kv_heads + h) * head_dim + j;
      store16(v_pool + (((size_t)page * kv_heads + h) * page_size + slot) * head_dim + j, load16(src));
    }
  }
}

}  // namespace li

using namespace li;

// inv_freq may be null with rotary_dim 0: nothing is rotated, k and v are only stored.
LI_EXPORT int li_rope_kv_write(int dtype, void* qkv, const int* positions, const int* seq_of_token,
                               const int* block_table, int table_stride, void* k_pool, void* v_pool,
                               const float* inv_freq, int tokens, int heads, int kv_heads, int head_dim,
                               int rotary_dim, int page_size, int num_pages, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return LI_ERR_UNSUPPORTED;
  if (rotary_dim > 0 && inv_freq == nullptr) return LI_ERR_UNSUPPORTED;
  const size_t smem = (size_t)rotary_dim * sizeof(float);
  if (smem > 48 * 1024) return LI_ERR_UNSUPPORTED;
  const int block = 256;
  if (dtype == kBFloat16 && rotary_dim == head_dim && head_dim % 16 == 0 && aligned16(qkv) && aligned16(k_pool) &&
      aligned16(v_pool))
    return (int)launch_pdl(tokens, rope_kv_write_vec_kernel, dim3(tokens), dim3(block), smem, stream, (bf16*)qkv,
                           positions, seq_of_token, block_table, table_stride, (bf16*)k_pool, (bf16*)v_pool, inv_freq,
                           heads, kv_heads, head_dim, page_size, num_pages);
  if (dtype == kFloat32)
    return (int)launch_pdl(tokens, rope_kv_write_kernel<float>, dim3(tokens), dim3(block), smem, stream, (float*)qkv,
                           positions, seq_of_token, block_table, table_stride, (float*)k_pool, (float*)v_pool,
                           inv_freq, heads, kv_heads, head_dim, rotary_dim, page_size, num_pages);
  return (int)launch_pdl(tokens, rope_kv_write_kernel<bf16>, dim3(tokens), dim3(block), smem, stream, (bf16*)qkv, positions,
                         seq_of_token, block_table, table_stride, (bf16*)k_pool, (bf16*)v_pool, inv_freq, heads,
                         kv_heads, head_dim, rotary_dim, page_size, num_pages);
}
