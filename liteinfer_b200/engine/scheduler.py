"""The scheduler: which requests compute how many tokens in the next step.

The policy is the reference's (liteinfer/engine/scheduler.py:1-104): every step
spends a token budget; running requests come first, in admission order, each
granted what it owes (the rest of its prompt, or its one sampled token) clamped
by what is left of the budget; then waiting requests are admitted while budget
and free seats (`max_num_seqs`) remain.  A prompt larger than what is left is
cut: it takes all that is left and continues next step, so at most one request
is part-way through its prompt and nothing is admitted behind it.

One decision is added where the reference leaves it to failure
(liteinfer/engine/async_llm_engine.py:73-85,244-248 sheds requests after the pool
refused a step): when a `page_gate` is given, a waiting request is admitted only
if the cache can hold it to its end beside everything already running, so
newcomers wait instead of being aborted.  Without a gate, or for a request that
can never fit, running out of pages is still possible; the engine then sheds by
the reference's tiers.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable

from liteinfer_b200.config.engine_config import EngineConfig
from liteinfer_b200.engine.sequence import Sequence, SequenceStatus


@dataclass
class SchedulerOutput:
    seqs: list[Sequence] = field(default_factory=list)
    num_scheduled_tokens: dict[str, int] = field(default_factory=dict)

    @property
    def is_empty(self) -> bool:
        return not self.seqs


class Scheduler:
    def __init__(self, config: EngineConfig,
                 page_gate: Callable[[Sequence, list[Sequence]], bool] | None = None) -> None:
        """`page_gate(seq, admitted)` says whether the cache can take `seq` now, beside the requests
        `admitted` earlier in this same step (which hold no pages yet)."""
        self.config = config
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.page_gate = page_gate

    def add(self, sequence: Sequence) -> None:
        sequence.status = SequenceStatus.WAITING
        self.waiting.append(sequence)

    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput()
        budget = self.config.token_budget

        for seq in self.running:
            if budget == 0:
                break
            if not seq.is_finished:
                budget -= self._grant(out, seq, budget)

        admitted: list[Sequence] = []
        while budget > 0 and self.waiting and len(self.running) < self.config.max_num_seqs:
            seq = self.waiting[0]
            if self.page_gate is not None and not self.page_gate(seq, admitted):
                # Wait for pages rather than fail — unless nothing runs at all, in which case
                # waiting would never end and the request is let through to fail on its own.
                if self.running:
                    break
            self.waiting.popleft()
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            admitted.append(seq)
            budget -= self._grant(out, seq, budget)
        return out

    @staticmethod
    def _grant(out: SchedulerOutput, seq: Sequence, budget: int) -> int:
        num_tokens = min(seq.num_uncomputed_tokens, budget)
        assert num_tokens > 0, f"{seq.request_id} was scheduled with nothing to compute"
        out.seqs.append(seq)
        out.num_scheduled_tokens[seq.request_id] = num_tokens
        return num_tokens

    def remove_finished(self) -> list[Sequence]:
        finished = [s for s in self.running if s.is_finished]
        self.running = [s for s in self.running if not s.is_finished]
        return finished

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)


def rows_to_shed(seqs: list[Sequence]) -> list[Sequence]:
    """What a step the cache could not hold gives up, least invested first
    (liteinfer/engine/async_llm_engine.py:73-85): requests that have computed nothing
    yet; failing that, prompts part-way; failing that, everything."""
    newcomers = [seq for seq in seqs if seq.num_computed_tokens == 0]
    prompts = [seq for seq in seqs if not seq.is_prompt_computed]
    return newcomers or prompts or seqs
