"""A request in flight, and the rules that end it.

liteinfer/engine/sequence.py:12-74 (status, token lists, `num_computed_tokens`)
and liteinfer/engine/stopping.py:9-37 (`min_tokens` gates EOS, stop ids and stop
strings, never the length limits).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from liteinfer_b200.sampling.params import SamplingParams


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


@dataclass
class Sequence:
    request_id: str
    prompt: str
    prompt_token_ids: list[int]
    sampling_params: SamplingParams
    output_token_ids: list[int] = field(default_factory=list)
    status: SequenceStatus = SequenceStatus.WAITING
    output_text: str = ""
    # Tokens whose keys and values are in the cache; the rest of len(self) is what the
    # next step has to compute (sequence.py:44-49).
    num_computed_tokens: int = 0
    detokenizer: object | None = None

    @property
    def is_finished(self) -> bool:
        return self.status in _FINISHED

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
    """The status that ends `seq` after `last_token_id`, or None to go on (stopping.py:9-37)."""
    params = seq.sampling_params
    num_output = seq.num_output_tokens
    if num_output >= params.min_tokens:
        hit_eos = last_token_id in eos_token_ids and not params.ignore_eos
        hit_stop_token = bool(params.stop_token_ids) and last_token_id in params.stop_token_ids
        if hit_eos or hit_stop_token:
            return SequenceStatus.FINISHED_STOPPED
        if params.stop and any(s in seq.output_text for s in params.stop):
            return SequenceStatus.FINISHED_STOPPED
    if num_output >= params.max_tokens or len(seq) >= max_model_len:
        return SequenceStatus.FINISHED_LENGTH
    return None
