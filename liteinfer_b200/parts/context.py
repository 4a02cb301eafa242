"""What a part sees of one step, and of its layer's cache.

`StepContext` is the batch as tensors on the device: a flat run of tokens, each
sequence's queries laid end to end, plus where each sequence's context ends and
which pages or state slot hold it.  Parts read it; only the step function
builds it.  `LayerCache` is the slice of the cache manager's storage that
belongs to one stop of the schedule.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass(frozen=True)
class KVNeed:
    """A part that keeps keys and values per token: `window` None keeps every
    token, a number keeps the newest `window` of them.  `name` is the key under
    which the part finds its pages in its layer's `LayerCache.kvs`; a layer whose
    parts declare several needs gives each its own name.  Needs that are equal
    apart from the name share a group of pages."""

    kv_heads: int
    head_dim: int
    window: int | None = None
    name: str = field(default="kv", compare=False)


@dataclass(frozen=True)
class StateNeed:
    """A part that keeps a fixed-size state per request, of `shape` per request.
    `kind`: "weight" (engine dtype) or "f32".  `name`: its key in `LayerCache.states`."""

    shape: tuple[int, ...]
    kind: str = "f32"
    name: str = "state"


@dataclass
class KVCacheView:
    k_pool: torch.Tensor       # [pages, kv_heads, page_size, head_dim] of this layer
    v_pool: torch.Tensor
    group: int                 # index into StepContext.block_tables
    page_size: int


@dataclass
class LayerCache:
    """What one stop of the schedule keeps: pages and states, each under its need's name."""

    kvs: dict[str, KVCacheView] = field(default_factory=dict)
    states: dict[str, torch.Tensor] = field(default_factory=dict)   # each [slots, *StateNeed.shape]
    read_only: bool = False             # this stop reads another stop's cache and stores nothing

    @property
    def kv(self) -> KVCacheView | None:
        """The pages of a layer that keeps one set of them (the one named "kv", else the only one)."""
        return self.kvs.get("kv") or (next(iter(self.kvs.values())) if len(self.kvs) == 1 else None)

    @property
    def state(self) -> torch.Tensor | None:
        """The state of a layer that keeps one (the one named "state", else the only one)."""
        found = self.states.get("state")
        if found is None and len(self.states) == 1:
            found = next(iter(self.states.values()))
        return found


@dataclass
class AttentionPlan:
    """How a step's sequences are dealt to the attention kernels: those that bring one
    token (their keys may be split over several blocks) and those that bring more."""

    num_decode: int = 0
    decode_seqs: torch.Tensor | None = None     # [num_decode] int32 batch rows with one query
    decode_tokens: torch.Tensor | None = None   # [num_decode] int32 their token rows
    num_prefill: int = 0
    prefill_seqs: torch.Tensor | None = None    # [num_prefill] int32 batch rows with several queries
    max_prefill_query_len: int = 0
    max_decode_context_len: int = 0             # host bound on the decode rows' context (sizes the splits)


@dataclass
class StepContext:
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor          # [T] int32
    positions: torch.Tensor          # [T] int32, position of each token in its sequence
    seq_of_token: torch.Tensor       # [T] int32, row of the batch each token belongs to
    query_start_loc: torch.Tensor    # [B+1] int32, prefix sums of the sequences' query counts
    context_lens: torch.Tensor       # [B] int32, tokens each sequence holds after this step
    block_tables: list[torch.Tensor]  # per KV group: [B, max_pages] int32, page of each logical block (-1: none)
    state_slots: torch.Tensor        # [B] int32, fixed-size state slot of each sequence
    logit_rows: torch.Tensor         # [R] int32, token rows whose logits are wanted
    num_logit_rows: int
    max_query_len: int
    max_context_len: int
    query_lens: tuple[int, ...] = ()       # host copy
    host_context_lens: tuple[int, ...] = ()  # host copy
    decode_splits: int | None = None       # EngineConfig.paged_decode_splits
    plan: AttentionPlan | None = None
    extras: dict = field(default_factory=dict)

    @property
    def is_decode_only(self) -> bool:
        return self.max_query_len == 1
