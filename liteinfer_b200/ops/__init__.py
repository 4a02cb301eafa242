"""The engine's kernels: thin Python faces over the CUDA libraries in `csrc/`."""

from liteinfer_b200.ops.kernels import (  # noqa: F401
    ACTIVATIONS,
    act_mul,
    add_,
    add_bias_,
    argmax,
    embedding,
    gemm_simt,
    linear,
    paged_attention,
    rmsnorm,
    rope_kv_write,
    sample,
)
from liteinfer_b200.ops.library import KernelLibraryError, build_all  # noqa: F401
