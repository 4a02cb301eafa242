"""Norm parts.  Interface of a norm:

    tensor_specs() -> {local name: TensorSpec}
    bind(tensors)                      # {local name: device tensor}
    forward(x, delta=None, rows=None, out=None) -> Tensor

`forward` normalises `x` [tokens, size].  With `delta` the sum x + delta is
what is normalised, and it is stored back into `x` (the residual stream moves on
in place) unless `rows` is given.  With `rows` (int32 indices) only those rows are
produced: the final norm computes just the rows whose logits are wanted.

Two optional abilities, which a block asks for only of a norm that declares them
(`apply_norm` in parts/block.py): `reads_row_stats`: `delta` may be an
`ops.RowStats` (the part before has already added its result into `x` and hands
on the new rows' sums of squares); `defers`: with `lazy=True` and such statistics
the norm does not run but returns an `ops.PendingNorm`, which the next part's
first product folds in.
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.registry import register_norm
from liteinfer_b200.parts.spec import TensorSpec


class RMSNorm:
    """y = weight * round(x * rsqrt(mean(x^2) + eps)), statistics in 32-bit.

    liteinfer/models/llama.py:35-48.
    """

    def __init__(self, size: int, eps: float, dtype: torch.dtype, device: torch.device) -> None:
        self.size, self.eps, self.dtype, self.device = size, float(eps), dtype, device
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), init="ones_normal")}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    reads_row_stats = True
    defers = True

    def forward(self, x: torch.Tensor, delta: "torch.Tensor | ops.RowStats | None" = None,
                rows: torch.Tensor | None = None, out: torch.Tensor | None = None, lazy: bool = False):
        if isinstance(delta, ops.RowStats):
            if lazy and out is None:
                return ops.PendingNorm(x, self.weight, self.eps, delta, rows)
            delta = None            # x holds the sum already
        n = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty((n, self.size), dtype=x.dtype, device=x.device)
        return ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows,
                           write_residual=delta is not None and rows is None)


register_norm("rmsnorm", RMSNorm)
