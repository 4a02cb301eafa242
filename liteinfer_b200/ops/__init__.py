"""The engine's kernels: thin Python faces over the CUDA libraries in `csrc/`."""

from liteinfer_b200.ops.kernels import (  # noqa: F401
    ACTIVATIONS,
    act_mul,
    act_mul_interleaved,
    add_,
    add_bias_,
    argmax,
    embedding,
    decode_splits_for,
    gemm_error_flag,
    gemm_simt,
    gemm_tcgen05,
    gated_linear,
    gated_linear_supported,
    gemm_skinny,
    gemm_skinny_slices,
    mma_attention_supports,
    linear,
    paged_attention,
    paged_attention_generic,
    paged_attention_mma,
    rmsnorm,
    rope_kv_write,
    sample,
)
from liteinfer_b200.ops.library import KernelLibraryError, build_all  # noqa: F401
