// Sampling: one block per row of logits.
//
// Order of operations as liteinfer/sampling/sampler.py:50-63: logits / temperature
// -> top-k (exactly k survive; ties at the boundary do not widen it, :76-83)
// -> softmax -> top-p on those probabilities (an entry is dropped when the mass
// before it, in descending order, exceeds p: the entry that crosses p is kept,
// :86-97) -> one draw.  temperature == 0 or top_k == 1 is the arg-max (:36).
//
// The draw takes a uniform number in [0, 1) that the host supplies per row, so a
// request's stream of draws does not depend on what else is in the batch.  All
// arithmetic is 32-bit; the selections use exact integer sums (counts, and
// probabilities in 2^-32 fixed point), so a given row always gives the same
// token.  Among equal values the lower index comes first.
#include "common.cuh"

namespace li {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t ordered_key(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ ArgMax block_argmax(ArgMax mine, ArgMax* scratch /* 32 */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, mine.v, o), __shfl_xor_sync(0xffffffffu, mine.i, o)};
    mine = better(mine, other);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = mine;
  __syncthreads();
  ArgMax r = scratch[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) r = better(r, scratch[w]);
  return r;
}

// Exclusive prefix of `v` over the block's threads in thread order, and the total.
__device__ unsigned long long block_exclusive_scan(unsigned long long v, unsigned long long* scratch /* 33 */,
                                                   unsigned long long* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  unsigned long long incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long run = 0;
    for (int w = 0; w < nwarps; ++w) {
      const unsigned long long t = scratch[w];
      scratch[w] = run;
      run += t;
    }
    scratch[32] = run;
  }
  __syncthreads();
  *total = scratch[32];
  return scratch[warp] + incl - v;
}

struct Keep {        // the surviving set: key > beta, or key == beta and index <= tie_cut
  uint32_t beta;
  int tie_cut;
  __device__ __forceinline__ bool has(uint32_t key, int i) const { return key > beta || (key == beta && i <= tie_cut); }
};

struct SelectSmem {
  unsigned long long mass[256];
  unsigned int count[256];
  unsigned long long scan[33];
  unsigned long long above;
  uint32_t prefix;
  int found;
  int tie_cut;
  unsigned long long n_tie;
};

// Among the elements of `within`, in descending order of value (equal values by
// ascending index), keeps each element whose preceding weight sum is <= limit.
// `unit` weights count elements (top-k with limit k-1); otherwise the weight is
// exp(x - row_max) in 2^-32 fixed point (top-p with limit p * total).
template <typename T, bool unit>
__device__ Keep select_prefix(const T* __restrict__ row, int n, float temp, float row_max, Keep within,
                              unsigned long long limit, SelectSmem& sm) {
  if (threadIdx.x == 0) {
    sm.prefix = 0;
    sm.above = 0;
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int b = threadIdx.x; b < 256; b += blockDim.x) {
      sm.mass[b] = 0;
      sm.count[b] = 0;
    }
    __syncthreads();
    const uint32_t prefix = sm.prefix;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float x = to_float(row[i]) / temp;
      const uint32_t key = ordered_key(x);
      if (!within.has(key, i)) continue;
      if (pass > 0 && (key >> (shift + 8)) != prefix) continue;
      const int bin = (key >> shift) & 255;
      const unsigned long long w = unit ? 1ull : (unsigned long long)(expf(x - row_max) * 4294967296.0f);
      atomicAdd(&sm.mass[bin], w);
      atomicAdd(&sm.count[bin], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      // The boundary lies in the lowest non-empty bin whose preceding mass is still <= limit.
      unsigned long long above = sm.above, chosen_above = sm.above;
      int chosen = -1;
      for (int b = 255; b >= 0; --b) {
        if (above > limit) break;
        if (sm.count[b]) {
          chosen = b;
          chosen_above = above;
        }
        above += sm.mass[b];
      }
      if (chosen < 0) {  // even the largest element's predecessors exceed the limit: keep the top bin
        for (int b = 255; b >= 0; --b)
          if (sm.count[b]) { chosen = b; break; }
        if (chosen < 0) chosen = 0;
      }
      sm.prefix = (prefix << 8) | (uint32_t)chosen;
      sm.above = chosen_above;
      if (pass == 3) {
        const unsigned long long w_each = sm.count[chosen] ? sm.mass[chosen] / sm.count[chosen] : 0;
        unsigned long long keep = sm.count[chosen];
        if (limit >= chosen_above && w_each > 0) {
          const unsigned long long fit = (limit - chosen_above) / w_each + 1;
          if (fit < keep) keep = fit;
        } else if (limit < chosen_above) {
          keep = 1;
        }
        if (keep < 1) keep = 1;
        sm.n_tie = keep;
        sm.tie_cut = n;
        sm.found = (int)sm.count[chosen];
      }
    }
    __syncthreads();
  }
  Keep out{sm.prefix, n};
  const unsigned long long n_tie = sm.n_tie;
  if (n_tie < (unsigned long long)sm.found) {
    // Not every element equal to beta survives: find the index of the n_tie-th one.
    const int seg = (n + blockDim.x - 1) / blockDim.x;
    const int lo = min(n, (int)threadIdx.x * seg), hi = min(n, lo + seg);
    unsigned long long mine = 0;
    for (int i = lo; i < hi; ++i) {
      const uint32_t key = ordered_key(to_float(row[i]) / temp);
      mine += (key == out.beta && within.has(key, i)) ? 1 : 0;
    }
    unsigned long long total;
    const unsigned long long before = block_exclusive_scan(mine, sm.scan, &total);
    if (before < n_tie && before + mine >= n_tie) {
      unsigned long long c = before;
      for (int i = lo; i < hi; ++i) {
        const uint32_t key = ordered_key(to_float(row[i]) / temp);
        if (key == out.beta && within.has(key, i) && ++c == n_tie) {
          sm.tie_cut = i;
          break;
        }
      }
    }
    __syncthreads();
    out.tie_cut = sm.tie_cut;
  }
  __syncthreads();
  return out;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
sample_kernel(const T* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out) {
  __shared__ ArgMax am_scratch[32];
  __shared__ SelectSmem sm;
  __shared__ int result;
  const int r = blockIdx.x;
  const T* row = logits + (size_t)r * vocab;

  ArgMax mine{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) mine = better(mine, ArgMax{to_float(row[i]), i});
  const ArgMax top = block_argmax(mine, am_scratch);
  const float temp = temperature ? temperature[r] : 0.f;
  const int k = top_k ? top_k[r] : -1;
  if (!(temp > 0.f) || k == 1) {
    if (threadIdx.x == 0) out[r] = top.i;
    return;
  }
  const float row_max = top.v / temp;

  Keep keep{0u, vocab};  // every finite value has a key > 0
  if (k > 0 && k < vocab)
    keep = select_prefix<T, true>(row, vocab, temp, row_max, keep, (unsigned long long)(k - 1), sm);

  const float p = top_p ? top_p[r] : 1.f;
  const int seg = (vocab + blockDim.x - 1) / blockDim.x;
  const int lo = min(vocab, (int)threadIdx.x * seg), hi = min(vocab, lo + seg);
  if (p > 0.f && p < 1.f) {
    unsigned long long part = 0;
    for (int i = lo; i < hi; ++i) {
      const float x = to_float(row[i]) / temp;
      if (keep.has(ordered_key(x), i)) part += (unsigned long long)(expf(x - row_max) * 4294967296.0f);
    }
    unsigned long long total;
    block_exclusive_scan(part, sm.scan, &total);
    const unsigned long long limit = (unsigned long long)((double)p * (double)total);
    keep = select_prefix<T, false>(row, vocab, temp, row_max, keep, limit, sm);
  }

  // Draw: the first index (ascending) at which the running weight passes uniform * total.
  unsigned long long part = 0;
  for (int i = lo; i < hi; ++i) {
    const float x = to_float(row[i]) / temp;
    if (keep.has(ordered_key(x), i)) part += (unsigned long long)(expf(x - row_max) * 4294967296.0f);
  }
  unsigned long long total;
  const unsigned long long before = block_exclusive_scan(part, sm.scan, &total);
  double u = uniform ? (double)uniform[r] : 0.5;
  u = u < 0.0 ? 0.0 : (u >= 1.0 ? 0.99999994 : u);
  unsigned long long target = (unsigned long long)(u * (double)total);
  if (target >= total) target = total ? total - 1 : 0;
  if (threadIdx.x == 0) result = top.i;  // total == 0 cannot happen (the maximum weighs 2^32); stay safe
  __syncthreads();
  if (part > 0 && before <= target && target < before + part) {
    unsigned long long c = before;
    for (int i = lo; i < hi; ++i) {
      const float x = to_float(row[i]) / temp;
      if (!keep.has(ordered_key(x), i)) continue;
      c += (unsigned long long)(expf(x - row_max) * 4294967296.0f);
      if (c > target) {
        result = i;
        break;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = result;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
argmax_kernel(const T* __restrict__ logits, int vocab, int* __restrict__ out) {
  __shared__ ArgMax scratch[32];
  const T* row = logits + (size_t)blockIdx.x * vocab;
  ArgMax mine{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) mine = better(mine, ArgMax{to_float(row[i]), i});
  const ArgMax top = block_argmax(mine, scratch);
  if (threadIdx.x == 0) out[blockIdx.x] = top.i;
}

// A row split over gridDim.y blocks: each finds the best of its chunk and leaves it in scratch; the block
// that arrives last (a counter per row, reset by that block) picks the best of the chunks.
constexpr int kArgmaxThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kArgmaxThreads)
argmax_split_kernel(const T* __restrict__ logits, int vocab, int chunk, float* __restrict__ part_value,
                    int* __restrict__ part_index, unsigned* __restrict__ counters, int* __restrict__ out) {
  __shared__ ArgMax scratch[32];
  __shared__ bool is_last;
  const int r = blockIdx.x, c = blockIdx.y, chunks = gridDim.y;
  grid_launch_dependents();
  grid_dependency_wait();
  const T* row = logits + (size_t)r * vocab;
  const int lo = c * chunk, hi = min(vocab, lo + chunk);
  ArgMax mine{-INFINITY, 0x7fffffff};
  constexpr int N = Vec16<T>::N;
  if ((((size_t)r * vocab + lo) * sizeof(T)) % 16 == 0 && aligned16(logits)) {
    const int vec_hi = lo + (hi - lo) / N * N;
    for (int i = lo + threadIdx.x * N; i < vec_hi; i += kArgmaxThreads * N) {
      const Vec16<T> v = load16(row + i);
#pragma unroll
      for (int k = 0; k < N; ++k) mine = better(mine, ArgMax{v.get(k), i + k});
    }
    for (int i = vec_hi + threadIdx.x; i < hi; i += kArgmaxThreads) mine = better(mine, ArgMax{to_float(row[i]), i});
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += kArgmaxThreads) mine = better(mine, ArgMax{to_float(row[i]), i});
  }
  const ArgMax top = block_argmax(mine, scratch);
  if (threadIdx.x == 0) {
    part_value[(size_t)r * chunks + c] = top.v;
    part_index[(size_t)r * chunks + c] = top.i;
    __threadfence();
    is_last = atomicAdd(&counters[r], 1u) == (unsigned)chunks - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (threadIdx.x == 0) {
    ArgMax best{-INFINITY, 0x7fffffff};
    for (int k = 0; k < chunks; ++k)
      best = better(best, ArgMax{__ldcg(part_value + (size_t)r * chunks + k), __ldcg(part_index + (size_t)r * chunks + k)});
    out[r] = best.i;
    counters[r] = 0;
  }
}

}  // namespace li

using namespace li;

// out[r] = index of the largest logit of row r (the lowest index among equals).
// With scratch (part_value/part_index of rows*32 entries, counters of `rows` zeros) a row is split over
// several blocks; without, one block scans a row.
LI_EXPORT int li_argmax(int dtype, const void* logits, int rows, int vocab, int* out, float* part_value,
                        int* part_index, unsigned* counters, int scratch_rows, cudaStream_t stream) {
  if (rows == 0) return 0;
  int chunks = (vocab + 4095) / 4096;
  if (chunks > 32) chunks = 32;
  if (chunks > 1 && part_value && part_index && counters && rows <= scratch_rows && rows <= 65535) {
    const int chunk = ((vocab + chunks - 1) / chunks + 7) / 8 * 8;
    const dim3 grid(rows, (vocab + chunk - 1) / chunk);
    if (dtype == kFloat32)
      return (int)launch_pdl(rows, argmax_split_kernel<float>, grid, dim3(kArgmaxThreads), 0, stream,
                             (const float*)logits, vocab, chunk, part_value, part_index, counters, out);
    return (int)launch_pdl(rows, argmax_split_kernel<bf16>, grid, dim3(kArgmaxThreads), 0, stream, (const bf16*)logits,
                           vocab, chunk, part_value, part_index, counters, out);
  }
  if (dtype == kFloat32)
    argmax_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)logits, vocab, out);
  else
    argmax_kernel<bf16><<<rows, kThreads, 0, stream>>>((const bf16*)logits, vocab, out);
  LI_LAUNCH_CHECK();
}

// Per row: temperature (<= 0: arg-max), top_k (<= 0 or >= vocab: off), top_p (>= 1: off), uniform in [0, 1).
LI_EXPORT int li_sample(int dtype, const void* logits, int rows, int vocab, const float* temperature,
                        const int* top_k, const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (dtype == kFloat32)
    sample_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)logits, vocab, temperature, top_k, top_p,
                                                        uniform, out);
  else
    sample_kernel<bf16><<<rows, kThreads, 0, stream>>>((const bf16*)logits, vocab, temperature, top_k, top_p, uniform,
                                                       out);
  LI_LAUNCH_CHECK();
}
