"""Block arrangements: how a layer's mixer, feed-forward and norms are wired.

Interface of a block:

    roles = {role: registry}                # its parts by role, and the registry each is built from
                                            # ("mixer", "feed_forward", "norm", "position")
    __init__(parts: {role: built part})
    forward(hidden, delta, ctx, cache) -> (hidden, delta)

A block may have any roles (two mixers side by side, a third norm); it hands
each part what it needs of `cache`, where every part finds its own pages or
state under the name its need declared.

The residual stream travels as a pair: `hidden` [tokens, hidden_size] and a
`delta` not yet added to it (None at the first layer).  A block's first norm
adds the pending delta while it normalises, so the sum costs no pass of its own;
what the block returns is again (hidden, pending delta).
"""

from __future__ import annotations

import torch

from liteinfer_b200.parts.context import LayerCache, StepContext
from liteinfer_b200.parts.registry import register_block


class PreNormResidualBlock:
    """h = h + mixer(norm(h)); h = h + feed_forward(norm(h)) — liteinfer/models/llama.py:174-192."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, parts: dict) -> None:
        self.mixer_norm = parts["mixer_norm"]
        self.mixer = parts["mixer"]
        self.feed_forward_norm = parts["feed_forward_norm"]
        self.feed_forward = parts["feed_forward"]

    def forward(self, hidden: torch.Tensor, delta: torch.Tensor | None, ctx: StepContext,
                cache: LayerCache) -> tuple[torch.Tensor, torch.Tensor]:
        normed = self.mixer_norm.forward(hidden, delta)
        mixed = self.mixer.forward(normed, ctx, cache)
        normed = self.feed_forward_norm.forward(hidden, mixed)
        return hidden, self.feed_forward.forward(normed, ctx)


register_block("prenorm_residual", PreNormResidualBlock)
