"""Per-step records of what the engine did (liteinfer/engine/metrics.py:14-116)."""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class StepMetrics:
    step_idx: int
    num_seqs: int
    input_tokens: int      # tokens the forward computed
    prompt_tokens: int     # of those, prompt tokens
    new_tokens: int        # tokens sampled
    wall_time_s: float

    @property
    def phase(self) -> str:
        if self.prompt_tokens == 0:
            return "decode"
        return "prefill" if self.prompt_tokens == self.input_tokens else "mixed"


@dataclass
class EngineStats:
    steps: list[StepMetrics] = field(default_factory=list)
    num_requests_finished: int = 0
    num_requests_aborted: int = 0

    def record(self, step: StepMetrics) -> None:
        self.steps.append(step)

    @property
    def total_new_tokens(self) -> int:
        return sum(s.new_tokens for s in self.steps)

    @property
    def total_time_s(self) -> float:
        return sum(s.wall_time_s for s in self.steps)
