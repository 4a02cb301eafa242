"""Position-encoding parts.  Interface of a position encoding:

    tensor_specs() / bind(tensors)     # most have no tensors
    rotary() -> RotaryTable | None     # the fused path: the mixer's kernel rotates q and k itself
    apply(q, k, ctx) -> None           # otherwise: change q and k in place before k is stored

A mixer asks `rotary()` first.  An encoding that is not a rotation of pairs
returns None there and does its work in `apply`.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from liteinfer_b200.parts.registry import register_position_encoding
from liteinfer_b200.parts.spec import TensorSpec


@dataclass
class RotaryTable:
    inv_freq: torch.Tensor   # [rotary_dim / 2] float32 on the device
    rotary_dim: int
    attention_scaling: float = 1.0


def rotary_inverse_frequencies(head_dim: int, theta: float, rope_type: str = "default", factor: float = 1.0,
                               low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                               original_max_position_embeddings: int = 0) -> torch.Tensor:
    """inv_freq [head_dim / 2] in float32 (CPU).

    default: theta^(-2i/d) (liteinfer/models/llama.py:66-71).  linear: divided by
    `factor`.  llama3 (llama.py:73-74 takes it from the rope registry): a
    wavelength 2*pi/f longer than original/low is divided by factor, shorter than
    original/high is kept, between them the two are blended with weight
    (original/wavelength - low) / (high - low).
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    if rope_type == "default":
        return inv_freq
    if rope_type == "linear":
        return inv_freq / factor
    if rope_type != "llama3":
        raise ValueError(f"rope_type {rope_type!r} is not supported")
    original = float(original_max_position_embeddings)
    wavelen = 2 * math.pi / inv_freq
    long_wave = wavelen > original / low_freq_factor
    short_wave = wavelen < original / high_freq_factor
    scaled = torch.where(long_wave, inv_freq / factor, inv_freq)
    smooth = (original / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    blended = (1 - smooth) * scaled / factor + smooth * scaled
    return torch.where(~long_wave & ~short_wave, blended, scaled)


class RotaryEmbedding:
    """Half-split rotary embedding: dimension j pairs with j + rotary_dim/2 (llama.py:89-102)."""

    def __init__(self, head_dim: int, theta: float, dtype: torch.dtype, device: torch.device,
                 rotary_dim: int | None = None, rope_type: str = "default", factor: float = 1.0,
                 low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                 original_max_position_embeddings: int = 0) -> None:
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        inv_freq = rotary_inverse_frequencies(self.rotary_dim, theta, rope_type, factor, low_freq_factor,
                                              high_freq_factor, original_max_position_embeddings)
        self.table = RotaryTable(inv_freq.to(device), self.rotary_dim, 1.0)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        pass

    def rotary(self) -> RotaryTable | None:
        return self.table

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx) -> None:  # the fused path covers it
        raise NotImplementedError


class NoPositionEncoding:
    """Leaves q and k as they are."""

    def __init__(self, dtype: torch.dtype, device: torch.device) -> None:
        pass

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        pass

    def rotary(self) -> RotaryTable | None:
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx) -> None:
        pass


register_position_encoding("rotary", RotaryEmbedding)
register_position_encoding("none", NoPositionEncoding)
