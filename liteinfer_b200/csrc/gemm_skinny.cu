// out[M, N] = x[M, K] @ w[N, K]^T (+ bias) for bfloat16 and a handful of rows
// (M <= 64): the matrix product of a decode step, where every weight is read
// once and the time is the time to stream w from HBM.
//
// The weights are the 16-row operand of mma.sync m16n8k16 and the few rows of x
// are its 8-wide operand, so no tensor-core work is wasted on padding M.  Each
// thread reads its weights straight from global memory as 16-byte vectors in
// fragment order (the k index inside a 32-wide block is permuted the same way
// for both operands, which a sum over k does not notice), all loads of a block
// in flight at once, no shared-memory staging; x comes through L1/L2.
//
// Work unit: one block = 16 rows of w x one slice of k.  The warps of a block
// (4; 8 or 16 where the weight has few rows: the output and down projections; 2 where it has very many)
// take interleaved 32-wide k blocks and add their partial sums through shared
// memory in a fixed order.  When k is also cut into several slices every block
// writes its 16 x M partial tile to scratch memory and bumps the tile's counter;
// the block that arrives last adds the slices in slice order, writes the result
// and resets the counter.  Nothing waits on anything, and the order of every sum
// is fixed, so a row's result depends neither on the batch nor on which block
// came last.
//
// Optional epilogue for a gated feed-forward: with `gated_act >= 0` the rows of w
// are interleaved in groups of eight (eight gate rows, then their eight up rows),
// and the block writes act(gate) * up, N/2 columns wide.
#include "gemm_skinny.cuh"

namespace li {

template <int NT, int kWarps = kSkinnyWarps>
int launch_skinny(const SkinnyParams& p, cudaStream_t s) {
  const dim3 grid((p.N + 15) / 16, p.num_slices);
  if (p.norm_weight)
    return (int)launch_maybe_early(pdl_mode() >= 1, gemm_skinny_kernel<NT, kWarps, true>, grid, dim3(kWarps * 32), 0, s, p);
  return (int)launch_maybe_early(pdl_mode() >= 1, gemm_skinny_kernel<NT, kWarps>, grid, dim3(kWarps * 32), 0, s, p);
}

}  // namespace li

using namespace li;

// How the kernel would run these sizes: returns the slices of k; *warps (optional) the warps per block,
// *slice_k (optional) the k per slice.
// The plan depends on the weight's shape only, so that a row of x meets the same order of sums in any batch.
LI_EXPORT int li_gemm_skinny_plan(int N, int K, int* warps, int* slice_k) { return skinny_plan(N, K, warps, slice_k); }

// bfloat16 only; 1 <= M <= 64; K a multiple of 8 and 16-byte aligned rows.  scratch (float) and counters
// (unsigned, all zero) are needed when li_gemm_skinny_plan(N, K) > 1: scratch_floats must be at least
// tiles * slices * 16 * 8 * ceil(M/8) and num_counters at least tiles, with tiles = ceil(N/16).
// gated_act: -1 plain; 0 silu, 1 gelu, 2 gelu-tanh, 3 relu on rows interleaved in eights (N a multiple of 16);
// out is then [M, N/2].
static int run_skinny(SkinnyParams p, float* scratch, size_t scratch_floats, unsigned* counters, int num_counters,
                      cudaStream_t stream) {
  const int M = p.M, N = p.N, K = p.K;
  int warps = kSkinnyWarps;
  p.num_slices = li_gemm_skinny_plan(N, K, &warps, &p.slice_k);
  const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
  const int tiles = (N + 15) / 16;
  if (p.num_slices > 1) {
    const size_t need = (size_t)tiles * p.num_slices * 16 * 8 * nt;
    if (!scratch || !counters || scratch_floats < need || num_counters < tiles) {
      // Not enough scratch: run unsplit, which needs none.
      p.num_slices = 1;
      p.slice_k = (K + 31) / 32 * 32;
    }
  }
  switch (nt * 100 + warps) {
    case 102: return launch_skinny<1, 2>(p, stream);
    case 104: return launch_skinny<1, 4>(p, stream);
    case 108: return launch_skinny<1, 8>(p, stream);
    case 116: return launch_skinny<1, 16>(p, stream);
    case 202: return launch_skinny<2, 2>(p, stream);
    case 204: return launch_skinny<2, 4>(p, stream);
    case 208: return launch_skinny<2, 8>(p, stream);
    case 216: return launch_skinny<2, 16>(p, stream);
    case 402: return launch_skinny<4, 2>(p, stream);
    case 404: return launch_skinny<4, 4>(p, stream);
    case 408: return launch_skinny<4, 8>(p, stream);
    case 416: return launch_skinny<4, 16>(p, stream);
    case 802: return launch_skinny<8, 2>(p, stream);
    case 804: return launch_skinny<8, 4>(p, stream);
    case 808: return launch_skinny<8, 8>(p, stream);
    default: return launch_skinny<8, 16>(p, stream);
  }
}

LI_EXPORT int li_gemm_skinny(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                             int gated_act, float* scratch, size_t scratch_floats, unsigned* counters,
                             int num_counters, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M > 64 || K < 8 || (K % 8)) return LI_ERR_UNSUPPORTED;
  if (gated_act > 3 || (gated_act >= 0 && (N % 16))) return LI_ERR_UNSUPPORTED;
  if (!aligned16(x) || !aligned16(w)) return LI_ERR_ALIGNMENT;
  SkinnyParams p{(const bf16*)x, (const bf16*)w, (const bf16*)bias, (bf16*)out, M, N, K, 0, 1, gated_act,
                 scratch, counters};
  return run_skinny(p, scratch, scratch_floats, counters, num_counters, stream);
}

// The same product with the steps around it fused in (either, both or neither):
//   norm_weight != null: x holds unnormalised rows (row m is x[x_rows[m]] when x_rows is given); the product is
//     that of weight * x / rms(x), where rms uses in_sumsq [in_parts][in_stride], the sums of squares of every
//     row of x in parts.  The weight multiply is rounded to bfloat16; 1 / rms multiplies the 32-bit sums.
//   out_sumsq != null (plain product only): out [M, N] is added to, out = round(out + round(product + bias)), and
//     out_sumsq [ceil(N/16)][out_stride] receives the sums of squares of the new rows, one part per 16 columns.
LI_EXPORT int li_gemm_skinny_fused(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                                   int gated_act, float* scratch, size_t scratch_floats, unsigned* counters,
                                   int num_counters, const void* norm_weight, const float* in_sumsq, int in_parts,
                                   int in_stride, float eps, const int* x_rows, float* out_sumsq, int out_stride,
                                   cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M > 64 || K < 8 || (K % 8)) return LI_ERR_UNSUPPORTED;
  if (gated_act > 3 || (gated_act >= 0 && (N % 16))) return LI_ERR_UNSUPPORTED;
  if (out_sumsq && (gated_act >= 0 || out_stride < M)) return LI_ERR_UNSUPPORTED;
  if (norm_weight && (!in_sumsq || in_parts < 1)) return LI_ERR_UNSUPPORTED;
  if (!aligned16(x) || !aligned16(w) || (norm_weight && !aligned16(norm_weight))) return LI_ERR_ALIGNMENT;
  SkinnyParams p{(const bf16*)x, (const bf16*)w, (const bf16*)bias, (bf16*)out, M, N, K, 0, 1, gated_act,
                 scratch, counters};
  p.norm_weight = (const bf16*)norm_weight;
  p.in_sumsq = in_sumsq;
  p.in_parts = in_parts;
  p.in_stride = in_stride;
  p.eps = eps;
  p.x_rows = norm_weight ? x_rows : nullptr;
  p.out_sumsq = out_sumsq;
  p.out_stride = out_stride;
  return run_skinny(p, scratch, scratch_floats, counters, num_counters, stream);
}
