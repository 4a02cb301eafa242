// Shared helpers of the liteinfer_b200 kernels (sm_100a).
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and a
// stream, launches, and returns the launch's cudaError_t as an int (0 = ok); the
// Python side turns a non-zero value into an exception.  Nothing here allocates.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define LI_EXPORT extern "C" __attribute__((visibility("default")))

// Error codes above cudaError_t's range: a size the kernel refuses.
#define LI_ERR_UNSUPPORTED 100001
#define LI_ERR_ALIGNMENT 100002

#define LI_LAUNCH_CHECK() return (int)cudaGetLastError()

namespace li {

// dtype codes shared with Python (liteinfer_b200/ops/kernels.py).
constexpr int kFloat32 = 0;
constexpr int kBFloat16 = 1;

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float x) { return __float2bfloat16_rn(x); }

// Rounds through T and back: the value a tensor of dtype T would hold.
template <typename T> __device__ __forceinline__ float round_to(float x) { return to_float(from_float<T>(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of the additions depends only on blockDim, never on the data or the grid.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

template <typename T> struct Vec16;  // 16 bytes of T
template <> struct Vec16<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ float get(int i) const { return (&raw.x)[i]; }
  __device__ __forceinline__ void set(int i, float v) { (&raw.x)[i] = v; }
};
template <> struct Vec16<bf16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ float get(int i) const {
    return __bfloat162float(reinterpret_cast<const bf16*>(&raw)[i]);
  }
  __device__ __forceinline__ void set(int i, float v) {
    reinterpret_cast<bf16*>(&raw)[i] = __float2bfloat16_rn(v);
  }
};

template <typename T> __device__ __forceinline__ Vec16<T> load16(const T* p) {
  Vec16<T> v;
  v.raw = *reinterpret_cast<const decltype(v.raw)*>(p);
  return v;
}
template <typename T> __device__ __forceinline__ void store16(T* p, const Vec16<T>& v) {
  *reinterpret_cast<decltype(v.raw)*>(p) = v.raw;
}

// ---- rotary pairs ---------------------------------------------------------------------------------
// (a, b) = dimensions (j, j + half) of a head, rotated by the angle whose cosine and sine are c and s.  Every
// product and sum is rounded on its own, whichever kernel the rotation is part of, so that all of them agree
// to the bit (and with a plain a*c - b*s written in any tensor library).
__device__ __forceinline__ float rotate_lo(float a, float b, float c, float s) {
  return __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
}
__device__ __forceinline__ float rotate_hi(float a, float b, float c, float s) {
  return __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
}
// Eight pairs at once: a and b hold dimensions j..j+7 and j+half..j+half+7; cosv and sinv point at entry j.
__device__ __forceinline__ void rotate_eight(const Vec16<bf16>& a, const Vec16<bf16>& b, const float* cosv,
                                             const float* sinv, Vec16<bf16>& lo, Vec16<bf16>& hi) {
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float x = a.get(e), y = b.get(e), c = cosv[e], s = sinv[e];
    lo.set(e, rotate_lo(x, y, c, s));
    hi.set(e, rotate_hi(x, y, c, s));
  }
}

// ---- programmatic dependent launch -------------------------------------------------------------
// Every kernel of this library is launched so that it may start while the kernel before it in the
// stream is still running.  What a kernel does before `grid_dependency_wait()` must not read what
// earlier kernels write, nor write anything at all: only prefetches of weights belong there.  After the
// wait, everything earlier kernels wrote is visible.  `grid_launch_dependents()` lets the next kernel
// start its own prologue.  Both are no-ops when the kernel was launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" :::); }

// LITEINFER_PDL: 0 = every kernel launched the ordinary way; 1 (default) = every kernel of this library that
// calls grid_dependency_wait() may start early; 2 = of those only the weight-streaming products.  Measured with
// mode 1 against mode 0 on B200 (Llama 1B shape): 1.43 against 1.54 ms per decode step at batch 8 when it was
// introduced; later, across all widths, 2.38 against 2.43 ms at batch 64 and 4.64 against 4.80 ms for a prompt of
// 2,048 tokens (library kernels in between neither trigger nor start early: the order around them is the usual one).
inline int pdl_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("LITEINFER_PDL");
    mode = e ? atoi(e) : 1;
  }
  return mode;
}
inline bool pdl_enabled(long /*rows of the step*/) { return pdl_mode() == 1; }

// Launches `kernel`, with programmatic stream serialization when `early` (it may then start before the kernel
// ahead of it has finished, and must call grid_dependency_wait() before it reads that kernel's results).
template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_maybe_early(bool early, void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = early ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, KernelArgs(args)...);
}

// Launches `kernel` of a step that is `rows` rows wide, early when the mode and the width allow it.
template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_pdl(long rows, void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl_enabled(rows) ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, KernelArgs(args)...);
}

__host__ __device__ inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace li
