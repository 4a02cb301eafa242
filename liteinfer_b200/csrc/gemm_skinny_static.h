// A variant of the decode matrix product for callers that cannot allocate device memory.
//
// This entry point has no counterpart in ValeGian/liteinfer: that engine reaches every kernel
// through PyTorch, whose allocator hands out whatever scratch a kernel needs.  Some hosts of this
// library are not in that position: a plug-in running inside another process's CUDA context under
// a memory budget it does not own, a real-time loop that must not touch the driver's allocator
// once it is warm, a sandbox whose policy forbids cudaMalloc outright.  For them the scratch of
// the k-sliced product lives in a fixed array inside the library.
//
//   out[M, N] = x[M, K] @ w[N, K]^T (+ bias[N])        bfloat16, row-major, 1 <= M <= 64
//
// The kernel template is li_gemm_skinny's (gemm_skinny.cu), run with the plan of narrow blocks and
// k slices (the form that needs scratch); li_gemm_skinny itself may choose wide blocks instead, so
// the two add their products in different orders and may differ in the last bit of a result.
//
// Limits and rules
//   * The scratch is LI_STATIC_SCRATCH_FLOATS floats (1 MiB) plus LI_STATIC_COUNTERS counters
//     (4 KiB) of device memory per GPU, held from the moment the library is loaded on that GPU
//     until the process exits.  A product whose slices need more is refused with
//     LI_ERR_STATIC_SCRATCH_TOO_SMALL and nothing is launched; li_gemm_skinny_static_needs() tells
//     beforehand how many floats a shape needs (0: the shape is not sliced and needs none).  Every
//     shape with M <= 16 fits; with more rows of x the long-k shapes (few rows of w) do not.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress).
//     Make that first call outside any stream capture, with the device current; later calls on
//     that device do no set-up.
//   * Nothing is allocated or freed, by this function or by anything it calls.
//   * All calls share the one array, and it keeps what the last call left there.  The arrival
//     counters are cleared on the stream before every launch; the partial sums need no clearing
//     (every slot that is read was written by the same launch).  Two calls whose kernels may
//     overlap on the GPU (different streams, or graphs replayed side by side) race on the array:
//     order them.
//   * K must be a multiple of 8 and x, w 16-byte aligned, as for li_gemm_skinny.
//   * The first call on a device must come from one thread at a time (the look-up of the array's
//     address is not locked), and the device's primary context is assumed: the address is kept per
//     device ordinal, so a host that runs two CUDA contexts on one device must make its calls in
//     the context that made the first.
//
// Returns 0, a cudaError_t, or one of the LI_ERR_* codes; li_static_error_string() names them.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#define LI_STATIC_SCRATCH_FLOATS (1u << 18)
#define LI_STATIC_COUNTERS 1024
#define LI_ERR_UNSUPPORTED 100001              /* sizes the kernel refuses: M outside 1..64, K not a multiple of 8 */
#define LI_ERR_ALIGNMENT 100002                /* x or w not 16-byte aligned */
#define LI_ERR_STATIC_SCRATCH_TOO_SMALL 100003

#ifdef __cplusplus
extern "C" {
#endif

int li_gemm_skinny_static(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                          cudaStream_t stream);

// Floats of scratch that out[M, N] = x[M, K] w^T needs (0 when k is not sliced), for checking a
// shape against LI_STATIC_SCRATCH_FLOATS without launching anything.
size_t li_gemm_skinny_static_needs(int M, int N, int K);

const char* li_static_error_string(int code);

#ifdef __cplusplus
}
#endif
