"""What a request asks of the sampler and of the rules that end it.

The fields, their defaults and their meanings are those of liteinfer/sampling/params.py:9-49, since a user of that
engine passes the same object here: temperature 0 (or top_k 1) is greedy; top_k -1 switches the cut off; top_p is
applied to the probabilities that top_k left; `min_tokens` holds back EOS, stop ids and stop strings, never the
length limits.
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass, field

_serial = itertools.count()

# (what must hold, what to say when it does not); each takes the parameters object.
_RULES = (
    (lambda p: p.temperature >= 0, "temperature is {temperature}: it cannot be negative (0 means greedy)"),
    (lambda p: 0.0 < p.top_p <= 1.0, "top_p is {top_p}: it is a probability mass in (0, 1]"),
    (lambda p: p.top_k == -1 or p.top_k >= 1, "top_k is {top_k}: use -1 for no cut or a count of at least 1"),
    (lambda p: p.max_tokens >= 1, "max_tokens is {max_tokens}: a request produces at least one token"),
    (lambda p: 0 <= p.min_tokens <= p.max_tokens, "min_tokens is {min_tokens}: it lies between 0 and max_tokens ({max_tokens})"),
)


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1

    max_tokens: int = 64
    min_tokens: int = 0
    ignore_eos: bool = False
    stop: list[str] | None = None
    stop_token_ids: list[int] | None = None

    seed: int | None = None    # None: the engine's seed and the request's number decide the stream

    # A number of its own for every object: requests that share one parameters object are told apart by the key
    # the sampler is given with them, objects by this.
    _serial: int = field(default_factory=lambda: next(_serial), init=False, repr=False, compare=False)

    def __post_init__(self) -> None:
        for holds, message in _RULES:
            if not holds(self):
                raise ValueError(message.format(**vars(self)))

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1

    @property
    def id(self) -> str:
        return f"params-{self._serial}"
