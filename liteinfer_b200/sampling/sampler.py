"""Sampler: logits -> token ids, one kernel launch for the whole batch.

liteinfer/sampling/sampler.py:19-63 takes greedy rows together in one arg-max
and loops over the stochastic rows (temperature, top-k, softmax, top-p,
multinomial with a per-request generator).  Here both kinds are one launch: a
batch of only greedy rows runs the arg-max kernel, any other batch the
sampling kernel, which treats a row with temperature 0 or top_k 1 as arg-max.

Random numbers come from the host: every request owns a `random.Random` stream
(seeded by `SamplingParams.seed` alone, or for unseeded requests by the engine's
seed and a key the caller gives), and each sampled token consumes one uniform number from it.  What a
request draws therefore does not depend on which other requests share its
batch.
"""

from __future__ import annotations

import random

import torch

from liteinfer_b200 import ops
from liteinfer_b200.sampling.params import SamplingParams


class Sampler:
    def __init__(self, seed: int = 42) -> None:
        self.seed = seed
        self._streams: dict[str, random.Random] = {}

    def _stream(self, params: SamplingParams, key: str | None) -> random.Random:
        stream_key = params.id if key is None else f"{params.id}/{key}"
        stream = self._streams.get(stream_key)
        if stream is None:
            if params.seed is not None:
                # Every request with this seed draws the same numbers: the same prompt gives the same tokens.
                stream = random.Random(params.seed)
            else:
                stream = random.Random(f"{self.seed}/{stream_key}")
            self._streams[stream_key] = stream
        return stream

    def forget(self, params: SamplingParams, key: str | None = None) -> None:
        """Drop the random stream of a finished request."""
        self._streams.pop(params.id if key is None else f"{params.id}/{key}", None)

    def __call__(self, logits: torch.Tensor, params: list[SamplingParams],
                 keys: list[str | None] | None = None) -> torch.Tensor:
        """One token id per row of `logits` [batch, vocab]; int32 on the logits' device.

        `keys` tells apart requests that share one SamplingParams object (a list of
        prompts generated with the same parameters): each key gets its own stream.
        """
        if logits.ndim != 2:
            raise ValueError(f"expected 2D logits, got shape {tuple(logits.shape)}")
        if len(params) != logits.shape[0]:
            raise ValueError(f"params length {len(params)} != batch size {logits.shape[0]}")
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        if rows == 0:
            return out
        if all(p.greedy for p in params):
            return ops.argmax(logits, out)
        keys = keys or [None] * rows
        host = torch.empty((4, rows), dtype=torch.float32, pin_memory=logits.is_cuda)
        for i, p in enumerate(params):
            host[0, i] = 0.0 if p.greedy else p.temperature
            host[1, i] = p.top_p
            host[2, i] = 0.0 if p.greedy else self._stream(p, keys[i]).random()
            host[3, i] = 0.0
        top_k = torch.tensor([p.top_k if p.top_k > 0 else 0 for p in params], dtype=torch.int32,
                             pin_memory=logits.is_cuda)
        dev = host.to(logits.device, non_blocking=True)
        return ops.sample(logits, dev[0], top_k.to(logits.device, non_blocking=True), dev[1], dev[2], out)
