"""Python faces of the CUDA kernels in `liteinfer_b200/csrc`.

Every function checks its tensors (device, dtype, contiguity, shapes), launches
on torch's current stream and raises when the launch is refused.  None of them
has a CPU or library path: a tensor that is not on a CUDA device raises
`KernelLibraryError`.  The parts of a model call these functions through the
module (`from liteinfer_b200 import ops` then `ops.rmsnorm(...)`), never by a
bound name, so tests can stand in for a single kernel.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_size_t, c_void_p

from dataclasses import dataclass

import torch

from liteinfer_b200.ops.library import KernelLibraryError, load

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
ACTIVATIONS = {"silu": 0, "gelu": 1, "gelu_pytorch_tanh": 2, "gelu_tanh": 2, "relu": 3}

_ERRORS = {
    100001: "the kernel refuses these sizes (unsupported shape or option)",
    100002: "the kernel needs 16-byte aligned rows",
}

_functions: dict[str, ctypes._CFuncPtr] = {}

_SIGNATURES = {
    "li_embedding": ("elementwise", [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "li_scatter_tokens": ("elementwise", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "li_stage_batch": ("elementwise", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "li_rmsnorm": ("elementwise", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                                   c_int, c_void_p]),
    "li_add": ("elementwise", [c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
    "li_add_bias": ("elementwise", [c_int, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "li_act_mul": ("elementwise", [c_int, c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p]),
    "li_act_mul_interleaved": ("elementwise", [c_int, c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p]),
    "li_rope_kv_write": ("rope_cache", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                        c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "li_paged_attention_generic": ("attention_generic", [
        c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "li_paged_attention_mma": ("attention_mma", [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "li_paged_attention_stream": ("attention_stream", [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "li_paged_attention_stream_supports": ("attention_stream", [c_int, c_int, c_int, c_int]),
    "li_paged_attention_stream_capacity": ("attention_stream", [c_int]),
    "li_paged_attention_stream_cluster_capacity": ("attention_stream", [c_int, c_int]),
    "li_paged_attention_mma_counters": ("attention_mma", [c_int, c_int, c_int, c_int]),
    "li_paged_attention_mma_decode_capacity": ("attention_mma", [c_int]),
    "li_paged_attention_tcgen05": ("attention_tcgen05", [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p]),
    "li_paged_attention_tcgen05_supports": ("attention_tcgen05", [c_int, c_int, c_int, c_int]),
    "li_gemm_skinny": ("gemm_skinny", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                       c_void_p, c_size_t, c_void_p, c_int, c_void_p]),
    "li_gemm_skinny_fused": ("gemm_skinny", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                             c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                             c_float, c_void_p, c_void_p, c_int, c_void_p]),
    "li_gemm_skinny_plan": ("gemm_skinny", [c_int, c_int, c_void_p, c_void_p]),
    "li_gemm_stream": ("gemm_stream", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                       c_int, c_void_p, c_void_p]),
    "li_gemm_stream_supports": ("gemm_stream", [c_int, c_int, c_int]),
    "li_gemm_tcgen05": ("gemm_tcgen05", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                         c_void_p]),
    "li_gemm_simt": ("gemm_simt", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "li_argmax": ("sampling", [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                               c_void_p]),
    "li_sample": ("sampling", [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p]),
}


def _fn(name: str):
    fn = _functions.get(name)
    if fn is None:
        library, argtypes = _SIGNATURES[name]
        fn = getattr(load(library), name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _functions[name] = fn
    return fn


# Launches of this package's own kernels since import (library products are not counted).
launch_count = 0


def _check(code: int, name: str) -> None:
    global launch_count
    if code == 0:
        launch_count += 1
        return
    if code in _ERRORS:
        raise KernelLibraryError(f"{name}: {_ERRORS[code]}")
    raise KernelLibraryError(f"{name}: CUDA error {code} at launch")


_pinned_stream: int | None = None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream if _pinned_stream is None else _pinned_stream


class on_current_stream:
    """Within this context every kernel of this module goes to the stream that was current when it was entered,
    without asking for it again at every launch (a step of a model launches a few hundred kernels; the lookup
    was a noticeable part of a step's host time).  Contexts nest; leave the stream alone inside."""

    def __enter__(self):
        global _pinned_stream
        self.before = _pinned_stream
        _pinned_stream = torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else None
        return self

    def __exit__(self, *exc):
        global _pinned_stream
        _pinned_stream = self.before
        return False


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelLibraryError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _on_gpu(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelLibraryError(
                "liteinfer_b200 kernels run on a CUDA device only; there is no CPU path "
                f"(got a tensor on {t.device})")
        if not t.is_contiguous():
            raise KernelLibraryError("kernels take contiguous tensors")


class _Scratch:
    """Per-device scratch that split kernels leave partial results in, and their arrival counters.

    The counters are zero between launches (the kernels reset them); the buffers live as long as the
    process, so CUDA graphs may hold their addresses."""

    GEMM_FLOATS = 1 << 21
    GEMM_COUNTERS = 1 << 12
    ATTENTION_COUNTERS = 1 << 16
    ARGMAX_ROWS = 4096

    def __init__(self, device: torch.device) -> None:
        self.gemm = torch.empty(self.GEMM_FLOATS, dtype=torch.float32, device=device)
        self.gemm_counters = torch.zeros(self.GEMM_COUNTERS, dtype=torch.int32, device=device)
        self.attention_counters = torch.zeros(self.ATTENTION_COUNTERS, dtype=torch.int32, device=device)
        self.argmax_value = torch.empty(self.ARGMAX_ROWS * 32, dtype=torch.float32, device=device)
        self.argmax_index = torch.empty(self.ARGMAX_ROWS * 32, dtype=torch.int32, device=device)
        self.argmax_counters = torch.zeros(self.ARGMAX_ROWS, dtype=torch.int32, device=device)
        # Error flags that kernels raise and the engine reads where it synchronises anyway: [0] the number of a
        # bounded wait that gave up (tcgen05 and TMA kernels), [1] a token id outside the embedding table.
        self.errors = torch.zeros(2, dtype=torch.int32, device=device)
        self.gemm_error = self.errors[0:1]
        self.token_error = self.errors[1:2]


_scratch: dict[torch.device, _Scratch] = {}


def normalise_device(device: torch.device | str) -> torch.device:
    """`cuda` and `cuda:0` are one device (torch compares and hashes them apart): the index is filled in with the
    current device's."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device() if torch.cuda.is_available() else 0)
    return device


def scratch_for(device: torch.device | str) -> _Scratch:
    device = normalise_device(device)
    found = _scratch.get(device)
    if found is None:
        found = _scratch[device] = _Scratch(device)
    return found


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _int32(t: torch.Tensor | None, what: str) -> None:
    if t is not None and t.dtype != torch.int32:
        raise KernelLibraryError(f"{what} must be int32, got {t.dtype}")


# ------------------------------------------------------------------ row-wise
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
              error_flag: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[ids[t]].  An id outside the table sets `error_flag[0]` and gives a zero row."""
    _on_gpu(ids, table, out, error_flag)
    _int32(ids, "ids")
    _int32(error_flag, "error_flag")
    tokens, width = out.shape
    assert ids.numel() == tokens and table.shape[1] == width and table.dtype == out.dtype
    _check(_fn("li_embedding")(_code(out), ids.data_ptr(), table.data_ptr(), out.data_ptr(), tokens, width,
                               table.shape[0], _ptr(error_flag), _stream()), "embedding")
    return out


def scatter_tokens(tokens: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, source: torch.Tensor) -> torch.Tensor:
    """tokens[dst[i]] = source[src[i]] wherever dst[i] >= 0 (all int32): sampled token ids that never left the
    device take their places in the next step's batch."""
    _on_gpu(tokens, dst, src, source)
    for t, what in ((tokens, "tokens"), (dst, "dst"), (src, "src"), (source, "source")):
        _int32(t, what)
    assert dst.numel() == src.numel()
    _check(_fn("li_scatter_tokens")(tokens.data_ptr(), dst.data_ptr(), src.data_ptr(), source.data_ptr(), dst.numel(),
                                    _stream()), "scatter_tokens")
    return tokens


# Batches up to this many 32-bit words are brought to the device by a kernel that reads the pinned buffer in place
# (one block; a copy engine's latency is longer than that for a few kilobytes, shorter for many).
STAGE_KERNEL_MAX_WORDS = 16384


def stage_batch(device: torch.Tensor, host: torch.Tensor, tokens: torch.Tensor, dst: torch.Tensor, src: torch.Tensor,
                source: torch.Tensor | None) -> bool:
    """device[:] = host[:] (int32; `host` pinned), then tokens[dst[i]] = source[src[i]] wherever dst[i] >= 0, in one
    launch.  False (and nothing done) where the buffer is too large for that or the device cannot read `host` in
    place: the caller then copies and scatters."""
    _on_gpu(device, tokens, dst, src, source)
    for t, what in ((device, "device"), (host, "host"), (tokens, "tokens"), (dst, "dst"), (src, "src")):
        _int32(t, what)
    words = device.numel()
    if words > STAGE_KERNEL_MAX_WORDS or host.numel() != words or not host.is_pinned():
        return False
    code = _fn("li_stage_batch")(device.data_ptr(), host.data_ptr(), words, tokens.data_ptr(), dst.data_ptr(),
                                 src.data_ptr(), _ptr(source), dst.numel() if source is not None else 0, _stream())
    if code == 100001:        # LI_ERR_UNSUPPORTED: the device cannot read this host memory in place
        return False
    _check(code, "stage_batch")
    return True


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            delta: torch.Tensor | None = None, rows: torch.Tensor | None = None,
            write_residual: bool = False) -> torch.Tensor:
    """out[r] = weight * rmsnorm(x[row] (+ delta[row])), row = rows[r] if rows is given else r.

    With `write_residual` the sum x + delta is stored back into x (the residual
    stream moves on in place); statistics and the sum are 32-bit.
    """
    _on_gpu(x, weight, out, delta, rows)
    _int32(rows, "rows")
    width = x.shape[-1]
    out_rows = out.shape[0]
    assert weight.numel() == width and out.shape[-1] == width and x.dtype == out.dtype == weight.dtype
    assert delta is None or (delta.shape == x.shape and delta.dtype == x.dtype)
    assert rows is not None or out_rows == x.shape[0]
    assert rows is None or rows.numel() == out_rows
    assert not (write_residual and delta is None)
    _check(_fn("li_rmsnorm")(_code(x), x.data_ptr(), _ptr(delta), weight.data_ptr(), out.data_ptr(), _ptr(rows),
                             out_rows, width, float(eps), int(write_residual), _stream()), "rmsnorm")
    return out


def add_(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += delta, summed in 32-bit."""
    _on_gpu(x, delta)
    assert x.shape == delta.shape and x.dtype == delta.dtype
    _check(_fn("li_add")(_code(x), x.data_ptr(), delta.data_ptr(), x.numel(), _stream()), "add")
    return x


def add_bias_(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    _on_gpu(out, bias)
    assert out.shape[-1] == bias.numel() and out.dtype == bias.dtype
    _check(_fn("li_add_bias")(_code(out), out.data_ptr(), bias.data_ptr(), out.numel() // bias.numel(),
                              bias.numel(), _stream()), "add_bias")
    return out


def act_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str) -> torch.Tensor:
    """out = act(gate_up[:, :w]) * gate_up[:, w:], w = out.shape[1]."""
    _on_gpu(gate_up, out)
    rows, width = out.shape
    assert gate_up.shape == (rows, 2 * width) and gate_up.dtype == out.dtype
    if activation not in ACTIVATIONS:
        raise KernelLibraryError(f"activation {activation!r} has no kernel; known: {sorted(ACTIVATIONS)}")
    _check(_fn("li_act_mul")(_code(out), gate_up.data_ptr(), out.data_ptr(), rows, width, ACTIVATIONS[activation],
                             _stream()), "act_mul")
    return out


# ------------------------------------------------------------- matrix product
@dataclass
class RowStats:
    """What a product leaves behind when it has added its result into the residual stream itself: the sums of
    squares of the stream's new rows, in parts (one per 16 columns the product wrote), [parts, rows] float32.
    The norm that follows needs nothing else of the rows' statistics."""

    sumsq: torch.Tensor


@dataclass
class PendingNorm:
    """A root-mean-square norm that has not run yet: `x` (the residual stream, sums done), the norm's weight and
    eps, the rows' statistics, and optionally the rows that are wanted (int32 indices).  `linear` and
    `gated_linear` take one in place of x and fold the norm into the product where their kernel can; anything
    else calls `materialise()`."""

    x: torch.Tensor
    weight: torch.Tensor
    eps: float
    stats: RowStats
    rows: torch.Tensor | None = None

    @property
    def shape(self) -> tuple[int, int]:
        return ((self.x.shape[0] if self.rows is None else self.rows.numel()), self.x.shape[1])

    @property
    def dtype(self) -> torch.dtype:
        return self.x.dtype

    @property
    def device(self) -> torch.device:
        return self.x.device

    def materialise(self) -> torch.Tensor:
        from liteinfer_b200 import ops      # through the module, so that a stand-in kernel is found
        out = torch.empty(self.shape, dtype=self.x.dtype, device=self.x.device)
        return ops.rmsnorm(self.x, self.weight, self.eps, out, rows=self.rows)


# LITEINFER_FUSED_NORM=1: the weight-streaming products add into the residual stream themselves and fold the norm
# after it into the next product, which takes 32 launches out of a decode step of 16 layers.  Off by default: measured
# on B200 at the 1B shape, a norm launched early costs 1.3 us between two products (its launch hides behind the
# product's weights, which are asked for before the wait), while multiplying x by the norm's weight inside the
# product's loop costs more (gate_up at 8 rows 20.9 against 15.2 us, the head 130 against 91): 1.17 against 1.06 ms
# per decode step at batch 8.
FUSED_NORM = os.environ.get("LITEINFER_FUSED_NORM", "0") == "1"


# LITEINFER_GEMM_STREAM=0: products of at most 16 rows run on the kernel that loads its weights through registers
# (gemm_skinny) instead of the persistent kernel with per-warp TMA rings (gemm_stream).
GEMM_STREAM = os.environ.get("LITEINFER_GEMM_STREAM", "1") != "0"


def _streams(M: int, N: int, K: int) -> bool:
    """Whether the weight-streaming kernel runs a bfloat16 product of these sizes."""
    if K % 8 or K < 8 or M <= 0:
        return False
    return M <= SKINNY_MAX_ROWS or (M <= SKINNY_MAX_ROWS_SMALL and N <= SKINNY_SMALL_WEIGHT_ROWS)


def linear(x: "torch.Tensor | PendingNorm", weight: torch.Tensor, out: torch.Tensor | None,
           bias: torch.Tensor | None = None, residual: torch.Tensor | None = None) -> "torch.Tensor | RowStats":
    """out[M, N] = x[M, K] @ weight[N, K]^T (+ bias).

    float32 runs the FFMA kernel (a true 32-bit product: tensor cores have no such
    mode).  bfloat16 hands the product to the library GEMM, as the reference's
    `nn.Linear` does (liteinfer/models/llama.py:108-110,137-140), with 32-bit
    accumulation, except for a handful of rows, which the weight-streaming kernel takes.

    `x` may be a `PendingNorm`: the weight-streaming kernel then normalises on its way in; any other path runs
    the norm first.  With `residual` [M, N] the weight-streaming kernel adds its result into it
    (residual = round(residual + round(product))) and returns the new rows' `RowStats`, `out` being unused; any
    other path returns the product in `out`, for the caller to add.
    """
    pending = x if isinstance(x, PendingNorm) else None
    M, K = x.shape
    N = weight.shape[0]
    fused = x.dtype == torch.bfloat16 and _streams(M, N, K)
    if pending is not None and not fused:
        x, pending = pending.materialise(), None
    if residual is not None and not (fused and FUSED_NORM):
        residual = None
    if out is None and residual is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    _on_gpu(x if pending is None else pending.x, weight, out, bias, residual)
    assert weight.shape[1] == K and x.dtype == weight.dtype
    assert residual is None or (residual.shape == (M, N) and residual.dtype == x.dtype)
    assert out is None or (out.shape == (M, N) and out.dtype == x.dtype)
    if x.dtype == torch.float32:
        _check(_fn("li_gemm_simt")(0, x.data_ptr(), weight.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K,
                                   _stream()), "gemm_simt")
        return out
    if fused:
        return _skinny(x, weight, out, bias, -1, residual)
    if M > 0:
        torch.mm(x, weight.t(), out=out)
        if bias is not None:
            add_bias_(out, bias)
    return out


# Rows of x up to which the weight-streaming kernel runs the bfloat16 product (measured on B200: beyond
# eight rows the library product streams the weights faster).
SKINNY_MAX_ROWS = 8
# ...except for weights of few rows (the projections around the attention, the down projection), where the kernel
# still wins at 9 to 16 rows of x: 5.4 against 5.8 us (3072 x 2048), 4.7 against 5.6 (2048 x 2048), 11.3 against
# 13.2 (2048 x 8192); inside a step of 12 sequences 1.219 against 1.245 ms, of 16 sequences 1.315 against 1.330.
SKINNY_MAX_ROWS_SMALL = 16
SKINNY_SMALL_WEIGHT_ROWS = 4096
NUM_SMS = 148


def _skinny(x, weight, out, bias, gated_act: int, residual: torch.Tensor | None = None, rings: bool = True):
    """A weight-streaming kernel, with what `x` (a tensor or a PendingNorm) and `residual` ask to be fused in:
    the persistent kernel with TMA rings where it takes the sizes (and `rings`), else the one that loads through
    registers."""
    M, K = x.shape
    N = weight.shape[0]
    pending = x if isinstance(x, PendingNorm) else None
    ws = scratch_for(weight.device)
    if pending is None and rings and GEMM_STREAM and M <= 16:
        # The persistent kernel that streams the weights through per-warp TMA rings.
        stats = None
        if residual is not None:
            stats = RowStats(torch.empty((-(-N // 16), M), dtype=torch.float32, device=weight.device))
        code = _fn("li_gemm_stream")(x.data_ptr(), weight.data_ptr(), _ptr(bias),
                                     (residual if residual is not None else out).data_ptr(), M, N, K, gated_act,
                                     _ptr(stats.sumsq if stats is not None else None), M if stats is not None else 0,
                                     ws.gemm_error.data_ptr(), _stream())
        if code != 100001:          # sizes it refuses go to the kernel below
            _check(code, "gemm_stream")
            return stats if stats is not None else out
    if pending is None and residual is None:
        _check(_fn("li_gemm_skinny")(x.data_ptr(), weight.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, gated_act,
                                     ws.gemm.data_ptr(), ws.gemm.numel(), ws.gemm_counters.data_ptr(),
                                     ws.gemm_counters.numel(), _stream()), "gemm_skinny")
        return out
    stats = None
    if residual is not None:
        stats = RowStats(torch.empty((-(-N // 16), M), dtype=torch.float32, device=weight.device))
    source = pending.x if pending is not None else x
    _int32(pending.rows if pending is not None else None, "rows")
    _check(_fn("li_gemm_skinny_fused")(
        source.data_ptr(), weight.data_ptr(), _ptr(bias), (residual if residual is not None else out).data_ptr(),
        M, N, K, gated_act, ws.gemm.data_ptr(), ws.gemm.numel(), ws.gemm_counters.data_ptr(),
        ws.gemm_counters.numel(),
        _ptr(pending.weight if pending is not None else None),
        _ptr(pending.stats.sumsq if pending is not None else None),
        pending.stats.sumsq.shape[0] if pending is not None else 0,
        pending.stats.sumsq.shape[1] if pending is not None else 0,
        float(pending.eps) if pending is not None else 0.0,
        _ptr(pending.rows if pending is not None else None),
        _ptr(stats.sumsq if stats is not None else None), M if stats is not None else 0, _stream()), "gemm_skinny_fused")
    return stats if stats is not None else out


def gemm_skinny(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """The weight-streaming bfloat16 product for at most 64 rows of x."""
    _on_gpu(x, weight, out, bias)
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and out.shape == (M, N) and x.dtype == weight.dtype == out.dtype == torch.bfloat16
    return _skinny(x, weight, out, bias, -1, rings=False)


def gemm_stream(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
                gated_activation: str | None = None, residual: torch.Tensor | None = None):
    """The persistent weight-streaming product (per-warp TMA rings) for at most 16 rows of x: out = x @ weight^T
    (+ bias); with `gated_activation`, act(gate) * up on a weight interleaved in eights (out is [M, N/2]); with
    `residual` [M, N] the result is added into it and the new rows' `RowStats` are returned (`out` unused)."""
    _on_gpu(x, weight, out, bias, residual)
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and x.dtype == weight.dtype == torch.bfloat16
    act = -1 if gated_activation is None else ACTIVATIONS[gated_activation]
    stats = None
    if residual is not None:
        stats = RowStats(torch.empty((-(-N // 16), M), dtype=torch.float32, device=weight.device))
    _check(_fn("li_gemm_stream")(x.data_ptr(), weight.data_ptr(), _ptr(bias),
                                 (residual if residual is not None else out).data_ptr(), M, N, K, act,
                                 _ptr(stats.sumsq if stats is not None else None), M if stats is not None else 0,
                                 scratch_for(x.device).gemm_error.data_ptr(), _stream()), "gemm_stream")
    return stats if stats is not None else out


def gemm_tcgen05(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
                 gated_activation: str | None = None) -> torch.Tensor:
    """The tcgen05 / TMA / tensor-memory product for bfloat16: out = x @ weight^T (+ bias), or with
    `gated_activation` act(gate) * up on a weight whose rows are interleaved in eights (out is [M, N/2]).

    `gemm_error_flag(device)` tells afterwards whether a wait inside the kernel ever gave up."""
    _on_gpu(x, weight, out, bias)
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and x.dtype == weight.dtype == out.dtype == torch.bfloat16
    assert out.shape == ((M, N) if gated_activation is None else (M, N // 2))
    act = -1 if gated_activation is None else ACTIVATIONS[gated_activation]
    _check(_fn("li_gemm_tcgen05")(x.data_ptr(), weight.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, act,
                                  scratch_for(x.device).gemm_error.data_ptr(), _stream()), "gemm_tcgen05")
    return out


def gemm_error_flag(device: torch.device | str) -> int:
    """0, or the number of the wait that gave up in a tcgen05 or TMA kernel since the flag was last cleared
    (synchronises the device)."""
    return error_flags(device)[0]


def token_error_flag(device: torch.device | str) -> torch.Tensor:
    """The device's flag that the embedding kernel raises for a token id outside its table."""
    return scratch_for(device).token_error


def error_flags(device: torch.device | str) -> tuple[int, int]:
    """(the number of a bounded wait that gave up, whether a token id lay outside an embedding table) since the
    flags were last read; reading clears them (one small copy that synchronises the device)."""
    flags = scratch_for(device).errors
    wait, token = flags.tolist()
    if wait or token:
        flags.zero_()
    return int(wait), int(token)


def gemm_simt(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """The FFMA product for either dtype (32-bit accumulation, fixed summation order)."""
    _on_gpu(x, weight, out, bias)
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and out.shape == (M, N) and x.dtype == weight.dtype == out.dtype
    _check(_fn("li_gemm_simt")(_code(x), x.data_ptr(), weight.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K,
                               _stream()), "gemm_simt")
    return out


def gemm_skinny_plan(N: int, K: int) -> tuple[int, int]:
    """(warps per block, slices of k) with which the weight-streaming kernel runs a weight [N, K]."""
    warps = ctypes.c_int(0)
    slices = int(_fn("li_gemm_skinny_plan")(N, K, ctypes.byref(warps), None))
    return warps.value, slices


def gemm_skinny_slices(N: int, K: int) -> int:
    """Into how many slices the weight-streaming kernel cuts k for a weight of [N, K]."""
    return gemm_skinny_plan(N, K)[1]


# Rows of x from which the gated product runs on the tcgen05 kernel (pairs of CTAs on 256 x 256 tiles) with the
# activation in its epilogue.  Measured on B200 at 2,048 rows x 16,384 x 2,048: 100 us, against 95 us for the
# library product plus 25 us for the activation kernel inside a step.  LITEINFER_TCGEN05_GATED=0 turns it off.
TCGEN05_MIN_ROWS = 256 if os.environ.get("LITEINFER_TCGEN05_GATED", "1") != "0" else 1 << 30


def gated_linear_supported(x: "torch.Tensor | PendingNorm", weight: torch.Tensor) -> bool:
    """Whether product, activation and multiply can be one kernel for this x: at most 8 rows (the
    weight-streaming kernel) or at least `TCGEN05_MIN_ROWS` (the tcgen05 kernel)."""
    M, K = x.shape
    return (x.dtype == torch.bfloat16 and K % 8 == 0 and K >= 8 and weight.shape[0] % 16 == 0
            and (0 < M <= SKINNY_MAX_ROWS or M >= TCGEN05_MIN_ROWS))


def gated_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, activation: str,
                 bias: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N/2] = act(gate) * up, where `weight` [N, K] holds gate and up rows interleaved in eights
    (rows 16b..16b+7 are gate rows 8b..8b+7, rows 16b+8..16b+15 their up rows): product, activation and
    multiply in one kernel (bfloat16)."""
    M, K = x.shape
    N = weight.shape[0]
    if isinstance(x, PendingNorm) and M > SKINNY_MAX_ROWS:
        x = x.materialise()
    _on_gpu(x.x if isinstance(x, PendingNorm) else x, weight, out, bias)
    assert weight.shape[1] == K and out.shape == (M, N // 2) and gated_linear_supported(x, weight)
    if M <= SKINNY_MAX_ROWS:
        return _skinny(x, weight, out, bias, ACTIVATIONS[activation])
    return gemm_tcgen05(x, weight, out, bias, activation)


def act_mul_interleaved(gate_up: torch.Tensor, out: torch.Tensor, activation: str) -> torch.Tensor:
    """`act_mul` for a gate_up whose columns are interleaved in eights like `gated_linear`'s weight rows."""
    _on_gpu(gate_up, out)
    rows, width = out.shape
    assert gate_up.shape == (rows, 2 * width) and gate_up.dtype == out.dtype and width % 8 == 0
    _check(_fn("li_act_mul_interleaved")(_code(out), gate_up.data_ptr(), out.data_ptr(), rows, width,
                                         ACTIVATIONS[activation], _stream()), "act_mul_interleaved")
    return out


# ------------------------------------------------------------ cache and mixer
def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                  block_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                  inv_freq: torch.Tensor | None, heads: int, kv_heads: int, head_dim: int,
                  rotary_dim: int, store: bool = True) -> None:
    """Rotates q (in place) and k, and stores k and v of every token into its page
    (with `store` False only q is rotated; the pages are left alone).

    qkv: [tokens, (heads + 2*kv_heads) * head_dim].  k_pool, v_pool:
    [pages, kv_heads, page_size, head_dim].  block_table: [seqs, max_pages] int32.
    """
    _on_gpu(qkv, positions, seq_of_token, block_table, k_pool, v_pool, inv_freq)
    _int32(positions, "positions"); _int32(seq_of_token, "seq_of_token"); _int32(block_table, "block_table")
    tokens = qkv.shape[0]
    pages, kvh, page_size, hd = k_pool.shape
    assert (kvh, hd) == (kv_heads, head_dim) and v_pool.shape == k_pool.shape
    assert qkv.shape[1] == (heads + 2 * kv_heads) * head_dim
    assert k_pool.dtype == qkv.dtype == v_pool.dtype
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rotary_dim)
    _check(_fn("li_rope_kv_write")(_code(qkv), qkv.data_ptr(), positions.data_ptr(), seq_of_token.data_ptr(),
                                   block_table.data_ptr(), block_table.stride(0), k_pool.data_ptr(),
                                   v_pool.data_ptr(), _ptr(inv_freq), tokens, heads, kv_heads, head_dim,
                                   rotary_dim if inv_freq is not None else 0, page_size, pages if store else 0, _stream()),
           "rope_kv_write")


_decode_capacity: dict[tuple[int, bool], int] = {}


def decode_capacity(head_dim: int, streaming: bool = False) -> int:
    """Blocks of the decode attention launch that the device holds at once (asked of the occupancy calculator
    once per head size and kernel); without a device, what a B200 holds."""
    key = (head_dim, streaming)
    if key not in _decode_capacity:
        blocks = 0
        if torch.cuda.is_available():
            name = "li_paged_attention_stream_capacity" if streaming else "li_paged_attention_mma_decode_capacity"
            blocks = int(_fn(name)(head_dim))
        _decode_capacity[key] = blocks or ((3 if streaming else 5) if head_dim <= 64 else 2) * NUM_SMS
    return _decode_capacity[key]


def decode_splits_for(num_decode: int, kv_heads: int, max_context_len: int, head_dim: int = 64,
                      streaming: bool = False) -> int:
    """Blocks that share one sequence's keys in a decode launch: as many as still run as one wave when the
    batch is narrow (a launch a little over one wave takes as long as two), never fewer than two key tiles
    each, at most 32 (liteinfer/engine/model_runner.py:250-272 and paged_kernels.py:645-693 choose likewise)."""
    tiles = -(-max_context_len // 64)
    if tiles < 4:
        return 1
    pairs = max(1, num_decode * kv_heads)
    splits = max(1, min(decode_capacity(head_dim, streaming) // pairs, tiles // 2, 32))
    if streaming and cluster_merge_wanted() and splits > 1:
        # The streaming kernel can merge the splits of a sequence through distributed shared memory when they are
        # one thread-block cluster (16 blocks at most) and every cluster of the launch is resident at once: then a
        # count that allows it is worth more than the last few splits (see attention_stream.cu for the figures).
        for fewer in range(min(splits, 16), max(1, splits // 2) - 1, -1):
            if fewer > 1 and cluster_capacity(head_dim, fewer) >= pairs:
                return fewer
    return splits


def cluster_merge_wanted() -> bool:
    """The switch LITEINFER_ATTN_CLUSTER_MERGE=1 (off by default; the kernel's entry point reads the same variable)."""
    return os.environ.get("LITEINFER_ATTN_CLUSTER_MERGE", "0") == "1"


_cluster_capacity: dict[tuple[int, int], int] = {}


def cluster_capacity(head_dim: int, splits: int) -> int:
    """Clusters of `splits` blocks of the streaming decode kernel that the device holds at once (0: none)."""
    key = (head_dim, splits)
    if key not in _cluster_capacity:
        clusters = 0
        if torch.cuda.is_available():
            clusters = int(_fn("li_paged_attention_stream_cluster_capacity")(head_dim, splits))
        _cluster_capacity[key] = clusters
    return _cluster_capacity[key]


def paged_attention_generic(q, q_row_stride, out, k_pool, v_pool, block_table, query_start_loc, context_lens,
                            num_seqs, max_q_len, heads, kv_heads, head_dim, scale, window=0) -> torch.Tensor:
    """The plain SIMT kernel: any dtype, head size up to 256, any grouping."""
    _on_gpu(q, out, k_pool, v_pool, block_table, query_start_loc, context_lens)
    pages, kvh, page_size, hd = k_pool.shape
    _check(_fn("li_paged_attention_generic")(
        _code(q), q.data_ptr(), q_row_stride, out.data_ptr(), out.stride(0), k_pool.data_ptr(), v_pool.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), query_start_loc.data_ptr(), context_lens.data_ptr(),
        num_seqs, max_q_len, heads, kv_heads, head_dim, page_size, pages, float(scale), int(window), _stream()),
        "paged_attention_generic")
    return out


def paged_attention_mma(q, q_row_stride, out, k_pool, v_pool, block_table, query_start_loc, context_lens,
                        seq_index, num_seqs, max_q_len, heads, kv_heads, head_dim, scale, window=0,
                        num_splits=1, newest=None, streaming=False) -> torch.Tensor:
    """The tensor-core kernel (bfloat16, head size 64 or 128); `num_splits` > 1 splits every sequence's keys
    over that many blocks, the last of which merges the partial results.  `newest` (NewestToken, single-token
    sequences only): q is unrotated and the newest key and value are not in their pages yet; the kernel
    rotates q and the key and stores key and value itself.  `streaming` (single-token sequences, sizes that
    `stream_attention_supports` allows): the kernel that passes K and V through registers only."""
    _on_gpu(q, out, k_pool, v_pool, block_table, query_start_loc, context_lens, seq_index)
    pages, kvh, page_size, hd = k_pool.shape
    partial_out = partial_lse = counters = None
    if num_splits > 1:
        total = q.shape[0] * heads * num_splits
        partial_out = torch.empty((total, head_dim), dtype=torch.float32, device=q.device)
        partial_lse = torch.empty((total,), dtype=torch.float32, device=q.device)
        need = int(_fn("li_paged_attention_mma_counters")(num_seqs, max_q_len, heads, kv_heads))
        counters = scratch_for(q.device).attention_counters
        if need > counters.numel():
            counters = torch.zeros(need, dtype=torch.int32, device=q.device)
    tail = (_ptr(newest.inv_freq if newest else None), _ptr(newest.k if newest else None),
            _ptr(newest.v if newest else None), int(newest.store) if newest else 0)
    if streaming:
        assert max_q_len == 1
        _check(_fn("li_paged_attention_stream")(
            q.data_ptr(), q_row_stride, out.data_ptr(), out.stride(0), k_pool.data_ptr(), v_pool.data_ptr(),
            block_table.data_ptr(), block_table.stride(0), query_start_loc.data_ptr(), context_lens.data_ptr(),
            _ptr(seq_index), num_seqs, heads, kv_heads, head_dim, page_size, pages, float(scale), int(window),
            int(num_splits), _ptr(partial_out), _ptr(partial_lse), _ptr(counters), *tail,
            scratch_for(q.device).gemm_error.data_ptr(), _stream()), "paged_attention_stream")
        return out
    _check(_fn("li_paged_attention_mma")(
        q.data_ptr(), q_row_stride, out.data_ptr(), out.stride(0), k_pool.data_ptr(), v_pool.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), query_start_loc.data_ptr(), context_lens.data_ptr(),
        _ptr(seq_index), num_seqs, max_q_len, heads, kv_heads, head_dim, page_size, pages, float(scale),
        int(window), int(num_splits), _ptr(partial_out), _ptr(partial_lse), _ptr(counters), *tail, _stream()),
        "paged_attention_mma")
    return out


@dataclass
class NewestToken:
    """The unrotated key and value projections of each sequence's newest token (views with the row stride of
    q) and the rotary frequencies, for the decode kernel that rotates and stores them itself."""
    inv_freq: torch.Tensor     # [head_dim / 2] float32
    k: torch.Tensor
    v: torch.Tensor
    store: bool = True         # False: the pages are another layer's and already hold the token


def fused_decode_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, rotary_dim: int, plan) -> bool:
    """Whether a step's attention can run as one launch that also rotates q and k and writes the cache: every
    sequence brings one token, all of the head is rotated, and the tensor-core decode kernel takes the sizes."""
    return (plan is not None and plan.num_prefill == 0 and plan.num_decode > 0 and rotary_dim == head_dim
            and mma_attention_supports(dtype, heads, kv_heads, head_dim) and heads // kv_heads <= 16)


def paged_attention_tcgen05(q, q_row_stride, out, k_pool, v_pool, block_table, query_start_loc, context_lens,
                            seq_index, num_seqs, max_q_len, heads, kv_heads, head_dim, scale, window=0) -> torch.Tensor:
    """The tcgen05 / TMA / tensor-memory attention kernel for prompts and portions (bfloat16, head size 64,
    pages of 16, 32 or 64 tokens, groups of at most 128 heads).  `gemm_error_flag(device)` tells afterwards whether a
    wait inside the kernel ever gave up."""
    _on_gpu(q, out, k_pool, v_pool, block_table, query_start_loc, context_lens, seq_index)
    pages, kvh, page_size, hd = k_pool.shape
    _check(_fn("li_paged_attention_tcgen05")(
        q.data_ptr(), q_row_stride, out.data_ptr(), out.stride(0), k_pool.data_ptr(), v_pool.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), query_start_loc.data_ptr(), context_lens.data_ptr(),
        _ptr(seq_index), num_seqs, max_q_len, heads, kv_heads, head_dim, page_size, pages, float(scale),
        int(window), scratch_for(q.device).gemm_error.data_ptr(), _stream()), "paged_attention_tcgen05")
    return out


def tcgen05_attention_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(
        _fn("li_paged_attention_tcgen05_supports")(heads, kv_heads, head_dim, page_size))


def stream_attention_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether single-token sequences can go through the kernel that streams K and V through registers.
    LITEINFER_DECODE_STREAM=0 keeps them on the shared-memory kernel."""
    return (dtype == torch.bfloat16 and os.environ.get("LITEINFER_DECODE_STREAM", "1") != "0"
            and bool(_fn("li_paged_attention_stream_supports")(heads, kv_heads, head_dim, page_size)))


def mma_attention_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and heads // kv_heads <= 64


def paged_attention(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_pool: torch.Tensor,
                    v_pool: torch.Tensor, block_table: torch.Tensor, query_start_loc: torch.Tensor,
                    context_lens: torch.Tensor, num_seqs: int, max_q_len: int, heads: int, kv_heads: int,
                    head_dim: int, scale: float, window: int = 0, plan=None,
                    decode_splits: int | None = None, newest: "NewestToken | None" = None) -> torch.Tensor:
    """Attention of each sequence's newest queries over its pages (any mix of portions and single tokens).

    q: the tensor holding the queries, head h of token t at q[t, h*head_dim:...]
    with `q_row_stride` elements between tokens (the fused qkv buffer is passed as
    it is).  out: [tokens, heads*head_dim].  bfloat16 with head size 64 or 128 runs
    on tensor cores; with a `plan` (AttentionPlan) the sequences that bring one
    token go through a launch that splits their keys over several blocks, the
    others through an unsplit one.  Everything else runs the plain SIMT kernel.
    `newest`: only where `fused_decode_supports` said yes; see `paged_attention_mma`.
    """
    _on_gpu(q, out, k_pool, v_pool, block_table, query_start_loc, context_lens)
    _int32(block_table, "block_table"); _int32(query_start_loc, "query_start_loc"); _int32(context_lens, "context_lens")
    pages, kvh, page_size, hd = k_pool.shape
    assert (kvh, hd) == (kv_heads, head_dim) and q.dtype == out.dtype == k_pool.dtype == v_pool.dtype
    if newest is not None and not fused_decode_supports(q.dtype, heads, kv_heads, head_dim, head_dim, plan):
        raise ValueError("the decode kernel with the rotary encoding fused in does not take this step")
    if not mma_attention_supports(q.dtype, heads, kv_heads, head_dim):
        return paged_attention_generic(q, q_row_stride, out, k_pool, v_pool, block_table, query_start_loc,
                                       context_lens, num_seqs, max_q_len, heads, kv_heads, head_dim, scale, window)
    common = (q, q_row_stride, out, k_pool, v_pool, block_table, query_start_loc, context_lens)
    if plan is None:
        return paged_attention_mma(*common, None, num_seqs, max_q_len, heads, kv_heads, head_dim, scale, window)
    if plan.num_prefill:
        many = (paged_attention_tcgen05 if tcgen05_attention_supports(q.dtype, heads, kv_heads, head_dim, page_size)
                else paged_attention_mma)
        many(*common, plan.prefill_seqs, plan.num_prefill, plan.max_prefill_query_len, heads, kv_heads, head_dim,
             scale, window)
    if plan.num_decode:
        bound = plan.max_decode_context_len if window <= 0 else min(plan.max_decode_context_len, window)
        streaming = stream_attention_supports(q.dtype, heads, kv_heads, head_dim, page_size)
        splits = decode_splits or decode_splits_for(plan.num_decode, kv_heads, bound, head_dim, streaming)
        paged_attention_mma(*common, plan.decode_seqs, plan.num_decode, 1, heads, kv_heads, head_dim, scale,
                            window, splits, newest, streaming)
    return out


# ------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _on_gpu(logits, out)
    _int32(out, "out")
    rows, vocab = logits.shape
    ws = scratch_for(logits.device)
    _check(_fn("li_argmax")(_code(logits), logits.data_ptr(), rows, vocab, out.data_ptr(), ws.argmax_value.data_ptr(),
                            ws.argmax_index.data_ptr(), ws.argmax_counters.data_ptr(), ws.ARGMAX_ROWS, _stream()),
           "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """One token per row: temperature, top-k, top-p, then the draw `uniform[r]` in [0, 1)."""
    _on_gpu(logits, temperature, top_k, top_p, uniform, out)
    _int32(out, "out"); _int32(top_k, "top_k")
    rows, vocab = logits.shape
    for t in (temperature, top_p, uniform):
        assert t.dtype == torch.float32 and t.numel() == rows
    _check(_fn("li_sample")(_code(logits), logits.data_ptr(), rows, vocab, temperature.data_ptr(), top_k.data_ptr(),
                            top_p.data_ptr(), uniform.data_ptr(), out.data_ptr(), _stream()), "sample")
    return out
