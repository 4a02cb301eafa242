// Row-wise kernels: embedding gather, RMSNorm (alone, fused with the residual
// add, fused with the gather of the rows whose logits are wanted), gated
// activation, bias add.  Statistics, the residual sum and the activation are
// computed in 32-bit whatever the storage type.
//
// Rounding points follow liteinfer/models/llama.py:43-48 (the normalised value is
// rounded to the storage type, then multiplied by the weight), :114 (the
// activation is rounded, then multiplied by `up`) and :187,192 (the residual
// sum is rounded to the storage type).
#include "common.cuh"

namespace li {

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                 int width, int vocab, int* __restrict__ error_flag) {
  const int t = blockIdx.x;
  grid_launch_dependents();
  grid_dependency_wait();
  int id = ids[t];
  if (id < 0 || id >= vocab) {  // a token id outside the table: record it, write zeros, read nothing
    if (threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)t * width + i] = from_float<T>(0.f);
    return;
  }
  const T* src = table + (size_t)id * width;
  T* dst = out + (size_t)t * width;
  constexpr int N = Vec16<T>::N;
  if (width % N == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0) {
    for (int i = threadIdx.x * N; i < width; i += blockDim.x * N) store16(dst + i, load16(src + i));
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
  }
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row.  `rows` (optional) picks the input row of each output
// row; `delta` (optional) is added to the input row first, and when
// `write_residual` the sum is stored back to the input row (in place).
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ x, const T* __restrict__ delta, const T* __restrict__ weight,
                               T* __restrict__ out, const int* __restrict__ rows, int width, float eps,
                               int write_residual) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t src_row = rows ? (size_t)rows[r] : (size_t)r;
  T* xr = x + src_row * width;
  const T* dr = delta ? delta + src_row * width : nullptr;
  T* outr = out + (size_t)r * width;

  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = to_float(xr[i]);
    if (dr) {
      v = round_to<T>(v + to_float(dr[i]));
      if (write_residual) xr[i] = from_float<T>(v);
    }
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = to_float(xr[i]);
    if (dr && !write_residual) v = round_to<T>(v + to_float(dr[i]));
    const float normed = round_to<T>(v * inv);
    outr[i] = from_float<T>(to_float(weight[i]) * normed);
  }
}

// The same, with the row held in registers between the two passes: VPT 16-byte vectors per thread.
template <typename T, int VPT>
__global__ void __launch_bounds__(256)
rmsnorm_reg_kernel(T* __restrict__ x, const T* __restrict__ delta, const T* __restrict__ weight, T* __restrict__ out,
                   const int* __restrict__ rows, int width, float eps, int write_residual) {
  constexpr int N = Vec16<T>::N;
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int vectors = width / N;
  grid_launch_dependents();
  Vec16<T> w[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < vectors) w[i] = load16(weight + v * N);      // the weight waits for nobody
  }
  grid_dependency_wait();
  const size_t src_row = rows ? (size_t)rows[r] : (size_t)r;
  T* xr = x + src_row * width;
  const T* dr = delta ? delta + src_row * width : nullptr;
  float vals[VPT][N];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < vectors) {
      Vec16<T> xv = load16(xr + v * N);
      if (dr) {
        const Vec16<T> dv = load16(dr + v * N);
#pragma unroll
        for (int k = 0; k < N; ++k) xv.set(k, xv.get(k) + dv.get(k));    // rounded to T by set()
        if (write_residual) store16(xr + v * N, xv);
      }
#pragma unroll
      for (int k = 0; k < N; ++k) {
        vals[i][k] = xv.get(k);
        ss += vals[i][k] * vals[i][k];
      }
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  T* outr = out + (size_t)r * width;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < vectors) {
      Vec16<T> o;
#pragma unroll
      for (int k = 0; k < N; ++k) o.set(k, w[i].get(k) * round_to<T>(vals[i][k] * inv));
      store16(outr + v * N, o);
    }
  }
}

// residual += delta (no norm): used where a block ends without a following norm.
template <typename T>
__global__ void add_kernel(T* __restrict__ x, const T* __restrict__ delta, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) x[i] = from_float<T>(to_float(x[i]) + to_float(delta[i]));
}

// out[r, c] += bias[c]
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ out, const T* __restrict__ bias, size_t rows, int width) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t n = rows * (size_t)width, stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = from_float<T>(to_float(out[i]) + to_float(bias[i % width]));
}

// --------------------------------------------------------- gated activation
constexpr int kSilu = 0, kGelu = 1, kGeluTanh = 2, kRelu = 3;

__device__ __forceinline__ float activate(float x, int act) {
  switch (act) {
    case kSilu: return x / (1.0f + expf(-x));
    case kGelu: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
    case kGeluTanh: {
      const float inner = 0.79788456080286535588f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + tanhf(inner));
    }
    default: return fmaxf(x, 0.f);
  }
}

// gate_up [rows, 2*width]: gate in the first `width` columns, up in the rest.
template <typename T>
__global__ void act_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, size_t rows, int width, int act) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t n = rows * (size_t)width, stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const size_t r = i / width;
    const int c = (int)(i - r * width);
    const float g = to_float(gate_up[r * 2 * width + c]);
    const float u = to_float(gate_up[r * 2 * width + width + c]);
    out[i] = from_float<T>(round_to<T>(activate(g, act)) * u);
  }
}

template <typename T>
__global__ void act_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, size_t rows, int width, int act) {
  constexpr int N = Vec16<T>::N;
  const int vec_per_row = width / N;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t n = rows * (size_t)vec_per_row, stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const size_t r = i / vec_per_row;
    const int c = (int)(i - r * vec_per_row) * N;
    const Vec16<T> g = load16(gate_up + r * 2 * width + c);
    const Vec16<T> u = load16(gate_up + r * 2 * width + width + c);
    Vec16<T> o;
#pragma unroll
    for (int k = 0; k < N; ++k) o.set(k, round_to<T>(activate(g.get(k), act)) * u.get(k));
    store16(out + r * width + c, o);
  }
}

// gate_up [rows, 2*width] with columns interleaved in eights: columns [16b, 16b+8) are gate columns
// [8b, 8b+8), columns [16b+8, 16b+16) the matching up columns (the layout of the fused product's weights).
template <typename T>
__global__ void act_mul_interleaved_kernel(const T* __restrict__ gate_up, T* __restrict__ out, size_t rows, int width,
                                           int act) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t n = rows * (size_t)width, stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const size_t r = i / width;
    const int c = (int)(i - r * width);
    const size_t base = r * 2 * width + (size_t)(c / 8) * 16 + (c % 8);
    const float g = to_float(gate_up[base]);
    const float u = to_float(gate_up[base + 8]);
    out[i] = from_float<T>(round_to<T>(activate(g, act)) * u);
  }
}

// The same for bfloat16 with 16-byte accesses: one thread takes one group of eight gate values and the eight
// up values behind them.
__global__ void act_mul_interleaved_vec_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, size_t rows,
                                               int width, int act) {
  const int groups = width / 8;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t n = rows * (size_t)groups, stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const size_t r = i / groups;
    const int b = (int)(i - r * groups);
    const bf16* src = gate_up + r * 2 * width + (size_t)b * 16;
    const Vec16<bf16> g = load16(src);
    const Vec16<bf16> u = load16(src + 8);
    Vec16<bf16> o;
#pragma unroll
    for (int k = 0; k < 8; ++k) o.set(k, round_to<bf16>(activate(g.get(k), act)) * u.get(k));
    store16(out + r * width + (size_t)b * 8, o);
  }
}

static int grid_for(size_t n, int block) {
  size_t g = (n + block - 1) / block;
  const size_t cap = 148 * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

template <typename T>
int launch_embedding(const int* ids, const void* table, void* out, int tokens, int width, int vocab,
                     int* error_flag, cudaStream_t s) {
  if (tokens == 0) return 0;
  return (int)launch_pdl(tokens, embedding_kernel<T>, dim3(tokens), dim3(128), 0, s, ids, (const T*)table, (T*)out, width,
                         vocab, error_flag);
}

template <typename T>
int launch_rmsnorm(void* x, const void* delta, const void* weight, void* out, const int* rows, int out_rows,
                   int width, float eps, int write_residual, cudaStream_t s) {
  if (out_rows == 0) return 0;
  constexpr int N = Vec16<T>::N;
  const bool vector_ok = width % N == 0 && aligned16(x) && aligned16(weight) && aligned16(out) &&
                         (!delta || aligned16(delta)) && ((size_t)width * sizeof(T)) % 16 == 0;
  const int need = vector_ok ? (width / N + 255) / 256 : 99;
  T* xp = (T*)x;
  const T *dp = (const T*)delta, *wp = (const T*)weight;
  T* op = (T*)out;
  if (need <= 1) return (int)launch_pdl(out_rows, rmsnorm_reg_kernel<T, 1>, dim3(out_rows), dim3(256), 0, s, xp, dp, wp, op, rows, width, eps, write_residual);
  if (need <= 2) return (int)launch_pdl(out_rows, rmsnorm_reg_kernel<T, 2>, dim3(out_rows), dim3(256), 0, s, xp, dp, wp, op, rows, width, eps, write_residual);
  if (need <= 4) return (int)launch_pdl(out_rows, rmsnorm_reg_kernel<T, 4>, dim3(out_rows), dim3(256), 0, s, xp, dp, wp, op, rows, width, eps, write_residual);
  const int block = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  return (int)launch_pdl(out_rows, rmsnorm_kernel<T>, dim3(out_rows), dim3(block), 0, s, xp, dp, wp, op, rows, width, eps,
                         write_residual);
}

template <typename T>
int launch_act_mul(const void* gate_up, void* out, size_t rows, int width, int act, cudaStream_t s) {
  if (rows == 0) return 0;
  constexpr int N = Vec16<T>::N;
  if (width % N == 0 && aligned16(gate_up) && aligned16(out)) {
    const size_t n = rows * (size_t)(width / N);
    act_mul_vec_kernel<T><<<grid_for(n, 256), 256, 0, s>>>((const T*)gate_up, (T*)out, rows, width, act);
  } else {
    act_mul_kernel<T><<<grid_for(rows * (size_t)width, 256), 256, 0, s>>>((const T*)gate_up, (T*)out, rows, width, act);
  }
  LI_LAUNCH_CHECK();
}

// tokens[dst[i]] = source[src[i]] for every i with dst[i] >= 0: token ids that were sampled on the device a step ago
// take their places in this step's batch without a trip through the host.
__global__ void scatter_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ dst, const int* __restrict__ src,
                                      const int* __restrict__ source, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int d = dst[i];
  if (d >= 0) tokens[d] = source[src[i]];
}

// A step's batch from pinned host memory (read by the kernel itself, over the bus) into its place on the device, and
// then the late tokens into theirs: one launch of one block instead of a copy and a launch.
__global__ void __launch_bounds__(1024) stage_batch_kernel(int* __restrict__ device, const int* __restrict__ host, int words,
                                                           int* __restrict__ tokens, const int* __restrict__ dst,
                                                           const int* __restrict__ src, const int* __restrict__ source,
                                                           int n_late) {
  for (int i = threadIdx.x; i < words; i += blockDim.x) device[i] = host[i];
  if (n_late <= 0 || source == nullptr) return;
  __syncthreads();
  for (int i = threadIdx.x; i < n_late; i += blockDim.x) {
    const int d = dst[i];
    if (d >= 0) tokens[d] = source[src[i]];
  }
}

}  // namespace li

using namespace li;

// device[0 .. words) = host[0 .. words), then tokens[dst[i]] = source[src[i]] wherever dst[i] >= 0 (tokens, dst and
// src lie inside `device`; source may be null: nothing is placed then).  `host` must be page-locked memory that the
// device can read in place; where it cannot, LI_ERR_UNSUPPORTED is returned and nothing is launched.
LI_EXPORT int li_stage_batch(int* device, const int* host, int words, int* tokens, const int* dst, const int* src,
                             const int* source, int n_late, cudaStream_t stream) {
  if (words <= 0) return 0;
  void* mapped = nullptr;
  if (cudaHostGetDevicePointer(&mapped, const_cast<int*>(host), 0) != cudaSuccess || mapped == nullptr) {
    cudaGetLastError();
    return LI_ERR_UNSUPPORTED;
  }
  stage_batch_kernel<<<1, 1024, 0, stream>>>(device, static_cast<const int*>(mapped), words, tokens, dst, src, source, n_late);
  LI_LAUNCH_CHECK();
}

LI_EXPORT int li_scatter_tokens(int* tokens, const int* dst, const int* src, const int* source, int n,
                                cudaStream_t stream) {
  if (n <= 0) return 0;
  scatter_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(tokens, dst, src, source, n);
  LI_LAUNCH_CHECK();
}

// out[t, :] = table[ids[t], :].  An id outside [0, vocab) sets *error_flag (if given) and yields zeros.
LI_EXPORT int li_embedding(int dtype, const int* ids, const void* table, void* out, int tokens, int width, int vocab,
                           int* error_flag, cudaStream_t stream) {
  return dtype == kFloat32 ? launch_embedding<float>(ids, table, out, tokens, width, vocab, error_flag, stream)
                           : launch_embedding<bf16>(ids, table, out, tokens, width, vocab, error_flag, stream);
}

// out[r] = weight * norm(x[rows ? rows[r] : r] (+ delta[same row])); with write_residual the sum is stored to x.
LI_EXPORT int li_rmsnorm(int dtype, void* x, const void* delta, const void* weight, void* out, const int* rows,
                         int out_rows, int width, float eps, int write_residual, cudaStream_t stream) {
  return dtype == kFloat32
             ? launch_rmsnorm<float>(x, delta, weight, out, rows, out_rows, width, eps, write_residual, stream)
             : launch_rmsnorm<bf16>(x, delta, weight, out, rows, out_rows, width, eps, write_residual, stream);
}

LI_EXPORT int li_add(int dtype, void* x, const void* delta, size_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  if (dtype == kFloat32)
    add_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>((float*)x, (const float*)delta, n);
  else
    add_kernel<bf16><<<grid_for(n, 256), 256, 0, stream>>>((bf16*)x, (const bf16*)delta, n);
  LI_LAUNCH_CHECK();
}

LI_EXPORT int li_add_bias(int dtype, void* out, const void* bias, size_t rows, int width, cudaStream_t stream) {
  if (rows == 0) return 0;
  const size_t n = rows * (size_t)width;
  if (dtype == kFloat32)
    add_bias_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>((float*)out, (const float*)bias, rows, width);
  else
    add_bias_kernel<bf16><<<grid_for(n, 256), 256, 0, stream>>>((bf16*)out, (const bf16*)bias, rows, width);
  LI_LAUNCH_CHECK();
}

// out[r, c] = act(gate_up[r, c]) * gate_up[r, width + c];  act: 0 silu, 1 gelu (erf), 2 gelu (tanh), 3 relu.
LI_EXPORT int li_act_mul(int dtype, const void* gate_up, void* out, size_t rows, int width, int act,
                         cudaStream_t stream) {
  if (act < 0 || act > 3) return LI_ERR_UNSUPPORTED;
  return dtype == kFloat32 ? launch_act_mul<float>(gate_up, out, rows, width, act, stream)
                           : launch_act_mul<bf16>(gate_up, out, rows, width, act, stream);
}

// As li_act_mul for a gate_up interleaved in eights; width must be a multiple of 8.
LI_EXPORT int li_act_mul_interleaved(int dtype, const void* gate_up, void* out, size_t rows, int width, int act,
                                     cudaStream_t stream) {
  if (act < 0 || act > 3 || (width % 8)) return LI_ERR_UNSUPPORTED;
  if (rows == 0) return 0;
  const size_t n = rows * (size_t)width;
  if (dtype == kFloat32)
    act_mul_interleaved_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>((const float*)gate_up, (float*)out, rows,
                                                                            width, act);
  else if (aligned16(gate_up) && aligned16(out))
    act_mul_interleaved_vec_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>((const bf16*)gate_up, (bf16*)out, rows,
                                                                             width, act);
  else
    act_mul_interleaved_kernel<bf16><<<grid_for(n, 256), 256, 0, stream>>>((const bf16*)gate_up, (bf16*)out, rows,
                                                                          width, act);
  LI_LAUNCH_CHECK();
}
