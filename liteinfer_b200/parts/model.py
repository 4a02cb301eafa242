"""A model put together from a `ModelSpec`: embedding, layers in schedule order, final norm, head.

This class knows no architecture.  It builds every part the spec names from the
registries, tells the loader which checkpoint tensors the parts want (local
names behind the spec's prefixes), tells the cache manager what every stop of
the schedule must keep, and runs a step: embed the tokens, walk the schedule,
normalise only the rows whose logits are wanted, project them.
"""

from __future__ import annotations

import torch

import liteinfer_b200.parts.attention  # noqa: F401  (registers the built-in parts)
import liteinfer_b200.parts.block  # noqa: F401
import liteinfer_b200.parts.embedding  # noqa: F401
import liteinfer_b200.parts.feed_forward  # noqa: F401
import liteinfer_b200.parts.norm  # noqa: F401
import liteinfer_b200.parts.position  # noqa: F401
from liteinfer_b200.parts.block import apply_norm
from liteinfer_b200.parts.context import LayerCache, StepContext
from liteinfer_b200.parts.registry import BLOCKS, build_part
from liteinfer_b200.parts.spec import ModelSpec, TensorSpec

class Layer:
    """One layer: its block class says which roles it has and from which registry each is built
    (`roles = {"mixer": "mixer", "mixer_norm": "norm", ...}`); the layer's spec names a part for every role."""

    def __init__(self, spec, dtype: torch.dtype, device: torch.device) -> None:
        if spec.block not in BLOCKS:
            raise ValueError(f"no block of kind {spec.block!r} is registered; known: {sorted(BLOCKS)}")
        self.spec = spec
        roles = dict(BLOCKS[spec.block].roles)
        if set(roles) != set(spec.parts):
            raise ValueError(f"block {spec.block!r} has the roles {sorted(roles)}, the layer names parts for "
                             f"{sorted(spec.parts)}")
        self.parts = {role: build_part(roles[role], spec.parts[role], dtype=dtype, device=device) for role in roles}
        self.block = BLOCKS[spec.block](self.parts)

    def cache_needs(self) -> tuple:
        needs: list = []
        for part in self.parts.values():
            if hasattr(part, "cache_needs"):
                needs.extend(part.cache_needs())
        return tuple(needs)


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.spec, self.dtype, self.device = spec, dtype, device
        self.embedding = build_part("embedding", spec.embedding, dtype=dtype, device=device)
        self.layers = [Layer(layer, dtype, device) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, dtype=dtype, device=device)
        self.head = build_part("head", spec.head, dtype=dtype, device=device)
        self.schedule = spec.schedule

    # ------------------------------------------------------------- tensors
    def _named_parts(self):
        yield self.spec.embedding_prefix, self.embedding
        for layer in self.layers:
            for role, part in layer.parts.items():
                yield layer.spec.prefixes[role], part
        yield self.spec.final_norm_prefix, self.final_norm
        yield self.spec.head_prefix, self.head

    def tensor_specs(self) -> dict[str, TensorSpec]:
        """Checkpoint name -> spec of every tensor the parts read, in a fixed order."""
        specs: dict[str, TensorSpec] = {}
        for prefix, part in self._named_parts():
            for local, spec in part.tensor_specs().items():
                name = prefix + local
                if name in specs and specs[name] != spec:
                    raise ValueError(f"two parts want tensor {name!r} with different specs")
                specs[name] = spec
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Hand every part its tensors (by checkpoint name, already on the device)."""
        for prefix, part in self._named_parts():
            part.bind({local: tensors[prefix + local] for local in part.tensor_specs()})

    @property
    def graph_safe(self) -> bool:
        """Whether a step of this model may be captured into a CUDA graph: every part launches kernels only.
        A part that reads device values on the host in `forward` sets `graph_safe = False`."""
        return all(getattr(part, "graph_safe", True) for _, part in self._named_parts())

    def weight_bytes(self) -> int:
        seen: dict[int, int] = {}
        for _, part in self._named_parts():
            for value in vars(part).values():
                if isinstance(value, torch.Tensor):
                    seen[value.data_ptr()] = value.numel() * value.element_size()
        return sum(seen.values())

    # --------------------------------------------------------------- cache
    def cache_needs(self) -> list[tuple]:
        """What each layer (by index) must keep between steps."""
        return [layer.cache_needs() for layer in self.layers]

    # ------------------------------------------------------------- forward
    def hidden(self, ctx: StepContext, caches: list[LayerCache]) -> tuple[torch.Tensor, torch.Tensor | None]:
        """Runs the schedule; returns the residual stream and the delta still to be added."""
        hidden = self.embedding.forward(ctx.token_ids)
        delta = None
        for stop, entry in enumerate(self.schedule):
            hidden, delta = self.layers[entry.layer].block.forward(hidden, delta, ctx, caches[stop])
        return hidden, delta

    def forward(self, ctx: StepContext, caches: list[LayerCache]) -> torch.Tensor:
        """Logits [ctx.num_logit_rows, vocab] at `ctx.logit_rows`."""
        hidden, delta = self.hidden(ctx, caches)
        if ctx.num_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=hidden.dtype, device=hidden.device)
        normed = apply_norm(self.final_norm, hidden, delta, self.head, rows=ctx.logit_rows)
        return self.head.forward(normed)
