"""A request in flight, and the rules that end it.

The reference keeps the request's state in `Sequence` (liteinfer/engine/sequence.py:12-74: status, token lists,
`num_computed_tokens`) and ends it by `resolve_stop_status` (liteinfer/engine/stopping.py:9-37: `min_tokens` gates
EOS, stop ids and stop strings, never the length limits; the stop rules come before the length).  The same
behaviour is arranged here for an engine that launches a step before it has read the tokens of the step before:

  * the rules of a request are worked out once, at admission (`StopRules`): the set of token ids that end it, the
    strings that end it, and the number of produced tokens at which its length ends it;
  * what ends a request by *count* is known when a token is launched, what ends it by *value* only when the
    token has been read, so the two are asked separately;
  * a sampled token whose value is still on the device stands in the output list as `PENDING`.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from liteinfer_b200.sampling.params import SamplingParams

PENDING = -1        # a sampled token that the host has not read yet


class SequenceStatus(str, Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED_STOPPED = "finished_stopped"   # EOS, a stop token or a stop string
    FINISHED_LENGTH = "finished_length"     # max_tokens or max_model_len
    FINISHED_ABORTED = "finished_aborted"   # failed or shed


_FINISHED = frozenset({SequenceStatus.FINISHED_STOPPED, SequenceStatus.FINISHED_LENGTH,
                       SequenceStatus.FINISHED_ABORTED})

FINISH_REASONS = {
    SequenceStatus.FINISHED_STOPPED: "stop",
    SequenceStatus.FINISHED_LENGTH: "length",
    SequenceStatus.FINISHED_ABORTED: "abort",
}


class StopRules:
    """When a request ends, from its sampling parameters, the tokenizer's end-of-sequence ids and the room its
    prompt leaves in `max_model_len`."""

    def __init__(self, params: SamplingParams, eos_token_ids=(), room: int | None = None) -> None:
        enders = set(params.stop_token_ids or ())
        if not params.ignore_eos:
            enders.update(eos_token_ids)
        self.enders = frozenset(enders)
        self.strings = tuple(params.stop or ())
        self.not_before = params.min_tokens
        # Produced tokens at which the length ends the request: max_tokens, or the context being full.
        self.length_limit = params.max_tokens if room is None else min(params.max_tokens, max(room, 0))

    @property
    def reads_text(self) -> bool:
        return bool(self.strings)

    def ended_by_length(self, produced: int) -> bool:
        return produced >= self.length_limit

    def ended_by_value(self, produced: int, token: int, text: str) -> bool:
        """Whether the `produced`-th token, `token`, ends the request by what it is (the text is what the request
        has produced up to and including it)."""
        if produced < self.not_before:
            return False
        return token in self.enders or any(s in text for s in self.strings)

    def status_after(self, produced: int, token: int, text: str) -> SequenceStatus | None:
        if self.ended_by_value(produced, token, text):
            return SequenceStatus.FINISHED_STOPPED
        if self.ended_by_length(produced):
            return SequenceStatus.FINISHED_LENGTH
        return None


@dataclass
class Sequence:
    request_id: str
    prompt: str
    prompt_token_ids: list[int]
    sampling_params: SamplingParams
    output_token_ids: list[int] = field(default_factory=list)
    status: SequenceStatus = SequenceStatus.WAITING
    output_text: str = ""
    # Tokens whose keys and values are in the cache (or on their way there in a launched step); the rest of
    # len(self) is what the next step has to compute.
    num_computed_tokens: int = 0
    detokenizer: object | None = None
    rules: StopRules | None = None
    # Tokens the request may hold at most (prompt and output): what the cache must have room for.
    final_length: int = 0
    # The token that ends the request by its length has been launched (its value is still to be read): the request
    # runs no further step, though it is not finished before that token has arrived.
    last_token_launched: bool = False

    def __post_init__(self) -> None:
        if self.rules is None:
            self.rules = StopRules(self.sampling_params)
        if not self.final_length:
            self.final_length = len(self.prompt_token_ids) + self.rules.length_limit

    @property
    def is_finished(self) -> bool:
        return self.status in _FINISHED

    @property
    def wants_step(self) -> bool:
        """Whether the scheduler has anything to give this request."""
        return self.status not in _FINISHED and not self.last_token_launched

    def __len__(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def num_uncomputed_tokens(self) -> int:
        return len(self) - self.num_computed_tokens

    @property
    def is_prompt_computed(self) -> bool:
        return self.num_computed_tokens >= len(self.prompt_token_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self.output_token_ids)

    @property
    def num_unread_tokens(self) -> int:
        """Sampled tokens at the end of the output whose values are still on the device."""
        n = 0
        for token in reversed(self.output_token_ids):
            if token != PENDING:
                break
            n += 1
        return n

    @property
    def read_token_ids(self) -> list[int]:
        """The output tokens whose values the host has (all of them once the request is finished)."""
        unread = self.num_unread_tokens
        return self.output_token_ids[:len(self.output_token_ids) - unread] if unread else list(self.output_token_ids)

    def next_tokens(self, count: int) -> list[int]:
        """The `count` tokens after the computed ones: from the prompt or from the output, never both
        (liteinfer/engine/model_runner.py:62-79)."""
        start, end = self.num_computed_tokens, self.num_computed_tokens + count
        if count < 1 or end > len(self):
            raise ValueError(f"{self.request_id}: cannot compute {count} tokens from {start} of {len(self)}")
        n_prompt = len(self.prompt_token_ids)
        if end <= n_prompt:
            return self.prompt_token_ids[start:end]
        if start >= n_prompt:
            return self.output_token_ids[start - n_prompt:end - n_prompt]
        raise ValueError(f"{self.request_id}: a portion may not span the prompt's end")


def resolve_stop_status(seq: Sequence, last_token_id: int, eos_token_ids, max_model_len: int) -> SequenceStatus | None:
    """The status that ends `seq` now that `last_token_id` is the last of its output, or None to go on: the rules
    worked out from the request's parameters, these end-of-sequence ids and this context limit."""
    rules = StopRules(seq.sampling_params, eos_token_ids, max_model_len - len(seq.prompt_token_ids))
    return rules.status_after(seq.num_output_tokens, last_token_id, seq.output_text)
