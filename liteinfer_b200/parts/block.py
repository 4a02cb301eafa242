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
what the block returns is again (hidden, pending delta).  Where a part's last
product can add into the stream itself (`adds_to_residual`), the pending delta
is instead an `ops.RowStats`: the sum is made, and the next norm gets the rows'
statistics for nothing (`apply_norm`, `run_part`).
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.context import LayerCache, StepContext
from liteinfer_b200.parts.registry import register_block


def apply_norm(norm, hidden: torch.Tensor, delta, consumer=None, rows: torch.Tensor | None = None):
    """Runs `norm` on the residual stream, whatever form the pending `delta` has (None, a tensor still to be
    added, or `ops.RowStats` of a sum already made), using what the norm and the part that reads its result say
    they can do: a norm that `defers` hands a consumer that `takes_pending_norm` the unfinished norm."""
    if isinstance(delta, ops.RowStats) and not getattr(norm, "reads_row_stats", False):
        delta = None                # the sum is in `hidden` already; a plain norm needs no more
    lazy = (isinstance(delta, ops.RowStats) and getattr(norm, "defers", False)
            and getattr(consumer, "takes_pending_norm", False))
    if lazy:
        return norm.forward(hidden, delta, rows=rows, lazy=True)
    return norm.forward(hidden, delta) if rows is None else norm.forward(hidden, delta, rows=rows)


def run_part(part, normed, hidden: torch.Tensor, *args):
    """A mixer's or feed-forward's contribution to the residual stream: a part that `adds_to_residual` is given
    the stream and may add to it itself (it then returns `ops.RowStats`); what any part returns is the pending
    delta of the next norm."""
    if getattr(part, "adds_to_residual", False):
        return part.forward(normed, *args, residual=hidden)
    return part.forward(normed, *args)


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
        normed = apply_norm(self.mixer_norm, hidden, delta, self.mixer)
        mixed = run_part(self.mixer, normed, hidden, ctx, cache)
        normed = apply_norm(self.feed_forward_norm, hidden, mixed, self.feed_forward)
        return hidden, run_part(self.feed_forward, normed, hidden, ctx)


register_block("prenorm_residual", PreNormResidualBlock)
