"""The step function: one batch of (request, its next tokens) through the model, from the cache.

`ModelRunner.step` takes any mix of entries — a whole prompt, a portion of
one cut anywhere, a single decoded token — runs exactly the tokens it is given
as one batch, and returns logits only at the places asked for.  What the
requests computed earlier is read from the cache; what this step computes is
written there.  The cache changes only if the step succeeds.

The reference's `ModelRunner.execute` (liteinfer/engine/model_runner.py:137-172)
has the same contract on `Sequence` objects and returns one row per sequence;
here the batch is plain token ids so that the scheduler's engine and the
trace-replay program drive the very same function, and rows are computed only
where `want` asks.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from liteinfer_b200.cache.manager import CacheManager
from liteinfer_b200.parts.context import StepContext
from liteinfer_b200.parts.model import Model


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them whose logits are wanted."""

    request_id: str
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


class ModelRunner:
    def __init__(self, model: Model, cache: CacheManager, decode_splits: int | None = None) -> None:
        self.model, self.cache = model, cache
        self.device = model.device
        self.decode_splits = decode_splits
        self.layer_caches = cache.layer_caches()
        self._pinned = self.device.type == "cuda"
        self.num_steps = 0

    # ---------------------------------------------------------------- batch
    def _validate(self, entries: list[StepEntry]) -> None:
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen: set[str] = set()
        vocab = self.model.spec.vocab_size
        for entry in entries:
            if entry.request_id in seen:
                raise ValueError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            n = len(entry.tokens)
            if n < 1:
                raise ValueError(f"request {entry.request_id!r} brings no tokens")
            if min(entry.tokens) < 0 or max(entry.tokens) >= vocab:
                raise ValueError(f"request {entry.request_id!r} has a token id outside [0, {vocab})")
            for place in entry.want:
                if not 0 <= place < n:
                    raise ValueError(f"request {entry.request_id!r} wants logits at {place}, but brings {n} tokens")

    def build_context(self, entries: list[StepEntry]) -> StepContext:
        """The batch as device tensors (one staging buffer, one host-to-device copy)."""
        cache = self.cache
        starts = [cache.length(e.request_id) for e in entries]
        counts = [len(e.tokens) for e in entries]
        totals = [s + c for s, c in zip(starts, counts)]
        B, T = len(entries), sum(counts)
        R = sum(len(e.want) for e in entries)
        widths = [max(len(cache.block_table(g, e.request_id)) for e in entries) for g in range(len(cache.groups))]

        sizes = [T, T, T, B + 1, B, B, R] + [B * w for w in widths]
        offsets = np.concatenate(([0], np.cumsum(sizes)))
        host = torch.empty(int(offsets[-1]), dtype=torch.int32, pin_memory=self._pinned)
        flat = host.numpy()
        tok, pos, seq, qsl, ctxl, slots, rows = (flat[offsets[i]:offsets[i + 1]] for i in range(7))
        cursor = 0
        row_cursor = 0
        qsl[0] = 0
        for i, entry in enumerate(entries):
            n = counts[i]
            tok[cursor:cursor + n] = entry.tokens
            pos[cursor:cursor + n] = np.arange(starts[i], totals[i], dtype=np.int32)
            seq[cursor:cursor + n] = i
            for place in entry.want:
                rows[row_cursor] = cursor + place
                row_cursor += 1
            cursor += n
            qsl[i + 1] = cursor
            ctxl[i] = totals[i]
            slots[i] = cache.state_slot(entry.request_id)
        for g, width in enumerate(widths):
            table = flat[offsets[7 + g]:offsets[8 + g]].reshape(B, width) if width else None
            if table is None:
                continue
            table.fill(-1)
            for i, entry in enumerate(entries):
                blocks = cache.block_table(g, entry.request_id)
                table[i, :len(blocks)] = blocks

        dev = host.to(self.device, non_blocking=True)
        part = [dev[int(offsets[i]):int(offsets[i + 1])] for i in range(len(sizes))]
        tables = [part[7 + g].view(B, widths[g]) if widths[g] else
                  torch.full((B, 1), -1, dtype=torch.int32, device=self.device) for g in range(len(widths))]
        return StepContext(
            num_tokens=T, num_seqs=B, token_ids=part[0], positions=part[1], seq_of_token=part[2],
            query_start_loc=part[3], context_lens=part[4], block_tables=tables, state_slots=part[5],
            logit_rows=part[6], num_logit_rows=R, max_query_len=max(counts), max_context_len=max(totals),
            query_lens=tuple(counts), host_context_lens=tuple(totals), decode_splits=self.decode_splits,
        )

    # ----------------------------------------------------------------- step
    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        """Logits [number of wanted places, vocab], in the order of `entries` and of each entry's `want`."""
        self._validate(entries)
        ids = [e.request_id for e in entries]
        totals = [self.cache.length(e.request_id) + len(e.tokens) for e in entries]
        self.cache.reserve(ids, totals)   # raises before anything changes
        try:
            ctx = self.build_context(entries)
            logits = self.model.forward(ctx, self.layer_caches)
        except BaseException:
            self.cache.rollback(ids)
            raise
        for request_id, total in zip(ids, totals):
            self.cache.commit(request_id, total)
        self.num_steps += 1
        return logits

    def enable_decode_graphs(self, max_num_seqs: int, max_model_len: int) -> None:
        """Replay steps that hold single decoded tokens only from CUDA graphs."""
        self._graphs_wanted = (max_num_seqs, max_model_len)

    def release(self, request_id: str) -> None:
        """The request is finished: what it holds is given back."""
        self.cache.release(request_id)
