"""Data that describes a model: which parts, with which sizes, run in which order.

A model here is not a class per architecture but a `ModelSpec`: an embedding, a
tuple of `LayerSpec` (each naming its block arrangement, mixer, feed-forward,
norms and the prefix of its tensor names), a `schedule` that says in which order
layers run (a layer may be named twice, or read another layer's cache), a final
norm and a head.  An architecture is a function from its typed configuration to
such a spec (`liteinfer_b200/config/registry.py`); the parts themselves never
learn which model they are in.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part reads.

    kind: "weight" is kept in the engine's dtype (bfloat16 or float32); "int" is
    an integer table kept as int32; "f32" stays 32-bit whatever the engine dtype.
    init: how the random-weights mode draws it: "normal" (N(0, 0.02)),
    "ones_normal" (1 + N(0, 0.01)), "zeros", or a function `(shape, generator) ->
    float32 tensor` for a part whose parameters need a distribution of their own
    (a decay kept in log space, a gate that must be positive).
    """

    shape: tuple[int, ...]
    kind: str = "weight"
    init: str | Callable[[tuple[int, ...], Any], Any] = "normal"


@dataclass(frozen=True)
class PartSpec:
    """A part by registry kind plus its constructor parameters."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __hash__(self) -> int:  # params is a dict; specs are compared by identity of content
        return hash((self.kind, tuple(sorted((k, repr(v)) for k, v in self.params.items()))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (`block`) of a mixer, a feed-forward and norms.

    `prefixes` maps the role of each part in the block ("mixer", "feed_forward",
    "mixer_norm", "feed_forward_norm", ...) to the prefix of its tensor names in
    the checkpoint, e.g. {"mixer": "model.layers.3.self_attn."}.
    """

    block: str
    parts: Mapping[str, PartSpec]
    prefixes: Mapping[str, str]


@dataclass(frozen=True)
class ScheduleEntry:
    """One stop of the forward pass: run `layer`.  `cache_of` is the index of an
    earlier stop of the schedule whose cache this stop reads instead of keeping
    one of its own (None: its own); such a stop stores nothing."""

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    embedding_prefix: str
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    final_norm_prefix: str
    head: PartSpec
    head_prefix: str
    # Tensor names that may be absent from a checkpoint because they alias another
    # tensor (a tied head): {absent name: name it reads instead}.
    tied: Mapping[str, str] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if not self.schedule:
            raise ValueError("a model's schedule names no layer")
        for stop, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule names layer {entry.layer}, but there are {len(self.layers)}")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < stop:
                    raise ValueError(f"stop {stop} reads the cache of stop {entry.cache_of}, which is not an earlier stop")
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ValueError(f"stop {stop} reads the cache of stop {entry.cache_of}, which keeps none of its own")
