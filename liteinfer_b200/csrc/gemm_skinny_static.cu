// li_gemm_skinny_static: the k-sliced decode product with its scratch in a file-scope device array,
// for callers that cannot allocate.  The contract is in gemm_skinny_static.h.
#include "gemm_skinny_static.h"

#include "gemm_skinny.cuh"

namespace li {

// The scratch itself.  In host code these names are stand-ins, not device addresses: the address a
// kernel may use comes from cudaGetSymbolAddress, once per device (below).
static __device__ __align__(256) float static_scratch[LI_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) unsigned static_counters[LI_STATIC_COUNTERS];

constexpr int kMaxDevices = 64;
struct DeviceScratch {
  float* scratch;
  unsigned* counters;
  bool ready;
};
static DeviceScratch device_scratch[kMaxDevices];

// Looks up the arrays' addresses on the current device the first time it is asked for them.
static cudaError_t scratch_of_current_device(DeviceScratch** found) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  DeviceScratch& slot = device_scratch[device];
  if (!slot.ready) {
    float* scratch = nullptr;
    unsigned* counters = nullptr;
    e = cudaGetSymbolAddress((void**)&scratch, static_scratch);
    if (e != cudaSuccess) return e;
    e = cudaGetSymbolAddress((void**)&counters, static_counters);
    if (e != cudaSuccess) return e;
    slot.scratch = scratch;
    slot.counters = counters;
    slot.ready = true;
  }
  *found = &slot;
  return cudaSuccess;
}

static int tiles_of(int M) { return M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8)); }

template <int NT>
static int launch_static(const SkinnyParams& p, cudaStream_t s) {
  const dim3 grid((p.N + 15) / 16, p.num_slices);
  gemm_skinny_kernel<NT><<<grid, kSkinnyWarps * 32, 0, s>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace li

using namespace li;

extern "C" __attribute__((visibility("default")))
size_t li_gemm_skinny_static_needs(int M, int N, int K) {
  if (M < 1 || N < 1 || K < 1) return 0;
  const int slices = skinny_slices(N, K, nullptr);
  if (slices <= 1) return 0;
  return (size_t)((N + 15) / 16) * slices * 16 * 8 * tiles_of(M);
}

extern "C" __attribute__((visibility("default")))
const char* li_static_error_string(int code) {
  switch (code) {
    case 0: return "ok";
    case LI_ERR_UNSUPPORTED: return "unsupported sizes: need 1 <= M <= 64 and K a positive multiple of 8";
    case LI_ERR_ALIGNMENT: return "x and w must be 16-byte aligned";
    case LI_ERR_STATIC_SCRATCH_TOO_SMALL:
      return "the product's k slices need more scratch than the library's fixed array holds "
             "(LI_STATIC_SCRATCH_FLOATS floats, LI_STATIC_COUNTERS counters)";
    default: return cudaGetErrorString((cudaError_t)code);
  }
}

extern "C" __attribute__((visibility("default")))
int li_gemm_skinny_static(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                          cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || N < 0 || M > 64 || K < 8 || (K % 8)) return LI_ERR_UNSUPPORTED;
  if (!aligned16(x) || !aligned16(w)) return LI_ERR_ALIGNMENT;
  SkinnyParams p{(const bf16*)x, (const bf16*)w, (const bf16*)bias, (bf16*)out, M, N, K, 0, 1, -1, nullptr, nullptr};
  p.num_slices = skinny_slices(N, K, &p.slice_k);
  const int tiles = (N + 15) / 16;
  if (p.num_slices > 1) {
    if (li_gemm_skinny_static_needs(M, N, K) > LI_STATIC_SCRATCH_FLOATS || tiles > LI_STATIC_COUNTERS)
      return LI_ERR_STATIC_SCRATCH_TOO_SMALL;
    DeviceScratch* mine = nullptr;
    cudaError_t e = scratch_of_current_device(&mine);
    if (e != cudaSuccess) return (int)e;
    p.scratch = mine->scratch;
    p.counters = mine->counters;
    // The counters must start at zero; the array keeps whatever an earlier (perhaps aborted) call left.
    e = cudaMemsetAsync(mine->counters, 0, (size_t)tiles * sizeof(unsigned), stream);
    if (e != cudaSuccess) return (int)e;
  }
  switch (tiles_of(M)) {
    case 1: return launch_static<1>(p, stream);
    case 2: return launch_static<2>(p, stream);
    case 4: return launch_static<4>(p, stream);
    default: return launch_static<8>(p, stream);
  }
}
