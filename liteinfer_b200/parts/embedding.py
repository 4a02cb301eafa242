"""Token embedding and output head.

Interface of an embedding: tensor_specs() / bind(tensors) / forward(token_ids) -> [tokens, hidden].
Interface of a head: tensor_specs() / bind(tensors) / forward(x [rows, hidden]) -> logits [rows, vocab].
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.registry import register_embedding, register_head
from liteinfer_b200.parts.spec import TensorSpec


class TokenEmbedding:
    """h[t] = table[token[t]] — liteinfer/models/llama.py:204,217."""

    def __init__(self, vocab_size: int, hidden_size: int, dtype: torch.dtype, device: torch.device) -> None:
        self.vocab_size, self.hidden_size, self.dtype, self.device = vocab_size, hidden_size, dtype, device
        self.weight: torch.Tensor | None = None
        # Set by the kernel when a token id lies outside the table; the step function reads it.
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=device)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = torch.empty((token_ids.numel(), self.hidden_size), dtype=self.weight.dtype, device=token_ids.device)
        return ops.embedding(token_ids, self.weight, out, self.error_flag)


class LinearHead:
    """logits = x @ weight^T, no bias — liteinfer/models/llama.py:245,277.  A tied head
    is bound to the embedding's tensor by the loader (llama.py:246-247)."""

    def __init__(self, vocab_size: int, hidden_size: int, dtype: torch.dtype, device: torch.device) -> None:
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty((x.shape[0], self.vocab_size), dtype=x.dtype, device=x.device)
        return ops.linear(x, self.weight, out)


register_embedding("token_embedding", TokenEmbedding)
register_head("linear", LinearHead)
