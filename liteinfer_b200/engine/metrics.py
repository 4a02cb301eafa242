"""What the engine records about its steps: counts, wall time, and where a step's time went.

liteinfer/engine/metrics.py:14-157 keeps a `StepMetrics` per step, totals per
stage of the loop (`TimeBreakdown`: forward, sample, deliver, schedule, loop)
and a `StepTimer` that synchronises the device at both ends of a stage.  Here
the stages are told apart without stopping the device: the host's share of a
stage is read off the host clock at the stage's ends, the device's share of
the forward and of the sampler off CUDA events recorded on the stream between
them and read after the step's one device-to-host copy has waited for the
stream anyway.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Callable


@dataclass
class StageTimes:
    """Seconds, of one step or summed over steps.

    Host clock: `schedule` (finished requests dropped, the batch chosen), `launch` (the step function: pages
    reserved, the batch staged and copied, kernels or a graph launched), `wait` (the sampler's launch and the
    blocking read of the sampled tokens: the host idles here while the device works), `finish` (tokens
    appended, stop rules, text), `loop` (everything, end of the last step to end of this one, so what the
    caller does between steps is in it).  Device clock: `forward_device`, `sample_device`.
    """

    schedule: float = 0.0
    launch: float = 0.0
    wait: float = 0.0
    finish: float = 0.0
    loop: float = 0.0
    forward_device: float = 0.0
    sample_device: float = 0.0

    def add(self, other: "StageTimes") -> None:
        for f in fields(self):
            setattr(self, f.name, getattr(self, f.name) + getattr(other, f.name))

    @property
    def unattributed(self) -> float:
        return max(0.0, self.loop - (self.schedule + self.launch + self.wait + self.finish))

    def shares(self) -> dict[str, float]:
        """Each host stage as a fraction of the loop's time (empty before the first step)."""
        if self.loop <= 0:
            return {}
        parts = {"schedule": self.schedule, "launch": self.launch, "wait": self.wait, "finish": self.finish,
                 "unattributed": self.unattributed}
        return {name: seconds / self.loop for name, seconds in parts.items()}


@dataclass
class StepMetrics:
    step_idx: int
    num_seqs: int
    input_tokens: int      # tokens the forward computed
    prompt_tokens: int     # of those, prompt tokens
    new_tokens: int        # tokens sampled
    wall_time_s: float     # from the start of the step function to the end of the stop rules
    stages: StageTimes | None = None
    ended_at: float = 0.0  # host clock at the end of the step

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
    time: StageTimes = field(default_factory=StageTimes)
    listeners: list[Callable[[StepMetrics], None]] = field(default_factory=list)

    def record(self, step: StepMetrics) -> None:
        self.steps.append(step)
        if step.stages is not None:
            self.time.add(step.stages)
        for listener in self.listeners:
            listener(step)

    def on_step(self, listener: Callable[[StepMetrics], None]) -> None:
        self.listeners.append(listener)

    @property
    def total_new_tokens(self) -> int:
        return sum(s.new_tokens for s in self.steps)

    @property
    def total_time_s(self) -> float:
        return sum(s.wall_time_s for s in self.steps)
