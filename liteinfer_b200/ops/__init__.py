"""The engine's kernels: thin Python faces over the CUDA libraries in `csrc/`."""

from liteinfer_b200.ops.kernels import (  # noqa: F401
    ACTIVATIONS,
    act_mul,
    add_,
    add_bias_,
    argmax,
    embedding,
    decode_splits_for,
    gemm_simt,
    gemm_skinny,
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
