"""The scheduler: which requests compute how many tokens in the next step.

The policy is the reference's (liteinfer/engine/scheduler.py:49-104): a step has a budget of tokens; requests that
hold a seat are served first, oldest first, each with what it owes (the rest of its prompt, or its one sampled
token) as far as the budget reaches; then requests from the queue take the seats and the budget that are left.  A
prompt that does not fit what is left takes all of it and goes on in the next step, which is why at most one
request is ever part-way through its prompt and nothing is seated behind it.

Here the scheduler plans against the cache it schedules for.  It is given the cache manager's ledger (anything
with `can_hold(final_lengths, largest_step)`), and seats a request only if the cache can hold it to its end beside
every seated request grown to its own end: each group of the cache is asked what a request of that length costs it
(a window bounds that), and a model without pages is held by its state slots alone.  A seated request therefore
never runs out of pages, and a newcomer waits instead of being shed, where the reference admits by seats only and
sheds after the pool refused a step (liteinfer/engine/async_llm_engine.py:73-85,244-248).  Without a ledger the
scheduler admits by seats as the reference does; the engine still sheds by tiers if a step is refused
(`shed_order`).  A request that could never fit is seated when nothing else is, so that it fails alone instead of
waiting for ever.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Protocol

from liteinfer_b200.config.engine_config import EngineConfig
from liteinfer_b200.engine.sequence import Sequence, SequenceStatus


class CacheLedger(Protocol):
    def can_hold(self, final_lengths: list[int], largest_step: int) -> bool: ...


@dataclass
class StepPlan:
    """What one step computes: (request, number of its next tokens), in the order of the batch."""

    grants: list[tuple[Sequence, int]] = field(default_factory=list)

    @property
    def is_empty(self) -> bool:
        return not self.grants

    @property
    def seqs(self) -> list[Sequence]:
        return [seq for seq, _ in self.grants]

    @property
    def num_scheduled_tokens(self) -> dict[str, int]:
        return {seq.request_id: count for seq, count in self.grants}

    @property
    def num_tokens(self) -> int:
        return sum(count for _, count in self.grants)


class Scheduler:
    def __init__(self, config: EngineConfig, ledger: CacheLedger | None = None) -> None:
        self.seats = config.max_num_seqs
        self.budget = config.token_budget
        self.ledger = ledger
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []      # the seated requests, oldest first (finished ones until they are retired)

    def add(self, sequence: Sequence) -> None:
        sequence.status = SequenceStatus.WAITING
        self.waiting.append(sequence)

    # ------------------------------------------------------------------ planning
    def _fits(self, newcomer: Sequence) -> bool:
        if self.ledger is None:
            return True
        ends = [s.final_length for s in self.running if not s.is_finished]
        return self.ledger.can_hold([*ends, newcomer.final_length], self.budget)

    def schedule(self) -> StepPlan:
        plan = StepPlan()
        left = self.budget

        def serve(seq: Sequence) -> None:
            nonlocal left
            owed = seq.num_uncomputed_tokens
            if owed < 1:
                raise AssertionError(f"{seq.request_id} holds a seat but owes no token")
            take = min(owed, left)
            plan.grants.append((seq, take))
            left -= take

        for seq in self.running:
            if left == 0:
                break
            if seq.wants_step:
                serve(seq)
        while left > 0 and self.waiting and len(self.running) < self.seats:
            newcomer = self.waiting[0]
            someone_runs = any(not s.is_finished for s in self.running)
            if someone_runs and not self._fits(newcomer):
                break                   # it waits for pages; what runs will give some back
            self.waiting.popleft()
            newcomer.status = SequenceStatus.RUNNING
            self.running.append(newcomer)
            serve(newcomer)
        return plan

    # ------------------------------------------------------------------ retiring
    def remove_finished(self, ready=None) -> list[Sequence]:
        """The seated requests that have finished (and are `ready`, where the caller has a say: a request whose
        last token has not been read yet keeps its seat) give up their seats; they are returned so that the caller
        can give back what they hold."""
        gone = [s for s in self.running if s.is_finished and (ready is None or ready(s))]
        if gone:
            self.running = [s for s in self.running if s not in gone]
        return gone

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)


def shed_order(seqs: list[Sequence]) -> list[Sequence]:
    """Which requests of a step that the cache refused are given up: those that have the least to lose.  Requests
    that have computed nothing yet; if there are none, requests still in their prompt; if there are none either, all
    of them (the tiers of liteinfer/engine/async_llm_engine.py:73-85)."""
    for tier in (lambda s: s.num_computed_tokens == 0, lambda s: not s.is_prompt_computed):
        chosen = [seq for seq in seqs if tier(seq)]
        if chosen:
            return chosen
    return list(seqs)


rows_to_shed = shed_order
