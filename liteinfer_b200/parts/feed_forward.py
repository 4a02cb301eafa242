"""Feed-forward parts.  Interface of a feed-forward:

    tensor_specs() / bind(tensors)
    forward(x, ctx) -> Tensor [tokens, hidden]
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.context import StepContext
from liteinfer_b200.parts.registry import register_feed_forward
from liteinfer_b200.parts.spec import TensorSpec


class GatedMLP:
    """down(act(gate(x)) * up(x)) — liteinfer/models/llama.py:105-114.

    gate and up are one product against the concatenated weights; the activation
    and the multiply are one kernel.
    """

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str, dtype: torch.dtype,
                 device: torch.device, bias: bool = False) -> None:
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} has no kernel; known: {sorted(ops.ACTIVATIONS)}")
        self.hidden_size, self.intermediate_size, self.activation, self.bias = (
            hidden_size, intermediate_size, activation, bias)
        self.gate_up_weight = self.gate_up_bias = self.down_weight = self.down_bias = None
        self.interleaved = False

    def tensor_specs(self) -> dict[str, TensorSpec]:
        i, h = self.intermediate_size, self.hidden_size
        specs = {"gate_proj.weight": TensorSpec((i, h)), "up_proj.weight": TensorSpec((i, h)),
                 "down_proj.weight": TensorSpec((h, i))}
        if self.bias:
            specs.update({"gate_proj.bias": TensorSpec((i,), init="zeros"), "up_proj.bias": TensorSpec((i,), init="zeros"),
                          "down_proj.bias": TensorSpec((h,), init="zeros")})
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        # bfloat16: gate and up rows interleaved in eights, the layout whose product, activation and
        # multiply one decode kernel can do together; otherwise gate rows first, then up rows.
        self.interleaved = gate.dtype == torch.bfloat16 and self.intermediate_size % 8 == 0
        self.gate_up_weight = self._pair(gate, up)
        self.down_weight = tensors["down_proj.weight"]
        if self.bias:
            self.gate_up_bias = self._pair(tensors["gate_proj.bias"], tensors["up_proj.bias"])
            self.down_bias = tensors["down_proj.bias"]

    def _pair(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        if not self.interleaved:
            return torch.cat([gate, up])
        rest = gate.shape[1:]
        stacked = torch.stack([gate.reshape(-1, 8, *rest), up.reshape(-1, 8, *rest)], dim=1)
        return stacked.reshape(2 * gate.shape[0], *rest).contiguous()

    takes_pending_norm = True       # x may be an ops.PendingNorm: the gate_up product folds the norm in
    adds_to_residual = True         # the down projection adds into the residual stream where its kernel can

    def forward(self, x, ctx: StepContext, residual: torch.Tensor | None = None):
        tokens = x.shape[0]
        hidden = torch.empty((tokens, self.intermediate_size), dtype=x.dtype, device=x.device)
        if self.interleaved and ops.gated_linear_supported(x, self.gate_up_weight):
            ops.gated_linear(x, self.gate_up_weight, hidden, self.activation, self.gate_up_bias)
        else:
            gate_up = torch.empty((tokens, 2 * self.intermediate_size), dtype=x.dtype, device=x.device)
            ops.linear(x, self.gate_up_weight, gate_up, self.gate_up_bias)
            if self.interleaved:
                ops.act_mul_interleaved(gate_up, hidden, self.activation)
            else:
                ops.act_mul(gate_up, hidden, self.activation)
        return ops.linear(hidden, self.down_weight, None, self.down_bias, residual=residual)


register_feed_forward("gated_mlp", GatedMLP)
