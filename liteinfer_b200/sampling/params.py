"""Sampling parameters: the names, defaults and checks of liteinfer/sampling/params.py:9-49."""

from __future__ import annotations

import uuid
from dataclasses import dataclass, field


@dataclass
class SamplingParams:
    temperature: float = 1.0   # 0 is greedy
    top_p: float = 1.0         # in (0, 1]
    top_k: int = -1            # -1 disables; 1 is greedy

    max_tokens: int = 64
    min_tokens: int = 0        # early stops (EOS, stop ids, stop strings) wait for this many tokens
    ignore_eos: bool = False
    stop: list[str] | None = None
    stop_token_ids: list[int] | None = None

    seed: int | None = None    # None: the engine's seed and the request's number decide the stream

    # Stable identity of this object, so that per-request random streams can be keyed
    # by it (liteinfer/sampling/params.py:23-27).
    _id: str = field(default_factory=lambda: uuid.uuid4().hex, init=False, repr=False, compare=False)

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k != -1 and self.top_k < 1:
            raise ValueError("top_k must be -1 (disabled) or >= 1")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.min_tokens < 0:
            raise ValueError("min_tokens must be >= 0")
        if self.min_tokens > self.max_tokens:
            raise ValueError("min_tokens must be <= max_tokens")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1

    @property
    def id(self) -> str:
        return self._id
