"""The engine: requests in, tokens out, one `step()` at a time.

One step is what liteinfer/engine/async_llm_engine.py:228-264 does: the requests that finished give back what they
hold, the scheduler spends the token budget, every scheduled request's tokens run through the step function as one
batch, the requests whose prompt is now complete are sampled, the stop rules are applied.  A step that the cache
cannot hold sheds one tier of requests (:73-85) and the rest go on; any other failure aborts the step's requests
only (:249-251).

Here the host does not wait for a step's tokens before it launches the next step.  The sampled token ids stay on
the device and are copied from there into the next batch (`StepEntry.late`); what a request's next step needs of
the host is only that it goes on, and the rules that end a request by count (max_tokens, the context limit) are
known at launch.  So `step()` plans and launches step n + 1 first and then reads the tokens of step n, which has
finished long since or is just finishing: the device always has its next step queued, and planning, staging and
the stop rules run beside it.  A request that step n's token ends by its value (EOS, a stop id, a stop string) has
then been launched once too often; that token is dropped when it arrives, and what the launch wrote lies in pages
that are given back with the request.  `EngineConfig.async_scheduling=False` reads every step's tokens before
the next launch, as the reference does.

`EngineCore` is synchronous and owns everything on the device.  `LLM` drives it directly; `AsyncLLM` drives it
from an asyncio task.  What `step()` returns is one step late under pipelining: the requests whose tokens were
read in this call.
"""

from __future__ import annotations

import logging
import time
from dataclasses import dataclass, field

import torch

from liteinfer_b200.cache.manager import CacheManager
from liteinfer_b200.cache.pages import CacheExhaustedError
from liteinfer_b200.config.engine_config import EngineConfig
from liteinfer_b200.engine.loading import make_runner, resolve_model_path
from liteinfer_b200.engine.metrics import EngineStats, StageTimes, StepMetrics
from liteinfer_b200.engine.runner import ModelRunner, StepEntry
from liteinfer_b200.engine.scheduler import Scheduler, shed_order
from liteinfer_b200.engine.sequence import PENDING, Sequence, SequenceStatus, StopRules
from liteinfer_b200.sampling.params import SamplingParams
from liteinfer_b200.sampling.sampler import Sampler
from liteinfer_b200.tokenizer import IncrementalDetokenizer, load_tokenizer
from liteinfer_b200.weights.loader import load_model

_LOGGER = logging.getLogger(__name__)


class EngineOverloaded(RuntimeError):
    """The waiting queue is full; the request was not accepted (async_llm_engine.py:58-64)."""


@dataclass
class StepResult:
    sampled: list[Sequence] = field(default_factory=list)            # requests whose new token was read in this call
    released: list[Sequence] = field(default_factory=list)           # finished earlier, evicted now
    aborted: list[tuple[Sequence, Exception]] = field(default_factory=list)


@dataclass
class _Launched:
    """A step that is on the device: whom it samples, where their tokens will be, and when it was launched."""

    seqs: list[Sequence]                 # the sampled requests, in the order of the rows
    places: list[int]                    # index of each one's pending token in its output
    sampled: torch.Tensor | None         # int32 [len(seqs)] on the device
    host_copy: torch.Tensor | None       # the same in pinned host memory, on its way since the step was launched
    copied: object | None                # the CUDA event behind that copy
    num_seqs: int
    input_tokens: int
    prompt_tokens: int
    t_begin: float
    t_start: float
    t_launched: float
    events: list | None


def _cdiv(a: int, b: int) -> int:
    return -(-a // b)


class EngineCore:
    def __init__(self, config: EngineConfig, text_every_step: bool = True) -> None:
        """`text_every_step` False: a request's text is decoded when it finishes (and step by step only if it
        has stop strings, which must be looked for in the text); nobody reads it earlier in a batch call."""
        self.config = config
        self.text_every_step = text_every_step
        self.device = config.resolved_device()
        self.stats = EngineStats()
        self.sampler = Sampler(config.seed)
        self.scheduler = Scheduler(config)
        self.pipelined = config.async_scheduling if config.async_scheduling is not None else True
        self.runner: ModelRunner | None = None
        self.tokenizer = None
        self.model_config = None
        self._step_idx = 0
        self._last_step_end = 0.0
        self._in_flight: _Launched | None = None
        self._event_sets: list[list] = []   # CUDA events that mark the forward and the sampler of a step on the stream
        self._host_buffers: list[tuple[torch.Tensor, object]] = []   # pinned buffers for the sampled tokens, with their events
        self._copy_stream = None            # the stream those copies run on (made at the first one)
        self._sampled_ready = None

    # ----------------------------------------------------------------- load
    def load(self) -> None:
        model_dir = resolve_model_path(self.config.model)
        model, self.model_config = load_model(model_dir, self.config.dtype, self.device)
        eos = tuple(getattr(self.model_config, "eos_token_id", ()) or ())
        self.tokenizer = load_tokenizer(model_dir, model.spec.vocab_size, eos)
        num_pages = self._num_pages(model)
        self.runner = make_runner(model, self.config.dtype, self.device, self.config.block_size, num_pages,
                                  self.config.max_num_seqs, self.config.paged_decode_splits)
        cache = self.runner.cache
        self.scheduler.ledger = cache        # admission asks the cache what a request will cost it
        use_graphs = self.config.enable_cuda_graphs
        if use_graphs is None:
            use_graphs = self.device.type == "cuda"
        if use_graphs:
            if self.device.type != "cuda":
                raise ValueError("enable_cuda_graphs=True needs a CUDA device")
            self.runner.enable_decode_graphs(self.config.max_num_seqs, self.config.max_model_len)
        _LOGGER.info("cache: %d pages of %d tokens (%.2f GiB)", num_pages, self.config.block_size,
                     num_pages * cache.bytes_per_page() / 2 ** 30)

    def _num_pages(self, model) -> int:
        """liteinfer/engine/model_runner.py:324-387: as many pages as the configuration can ever
        address, unless memory affords fewer; `num_gpu_blocks` overrides both."""
        cfg = self.config
        if cfg.num_gpu_blocks is not None:
            return cfg.num_gpu_blocks
        reachable = cfg.max_num_seqs * _cdiv(cfg.max_model_len, cfg.block_size)
        per_page = CacheManager.bytes_per_page_for(model.cache_needs(), model.schedule, cfg.block_size, cfg.dtype)
        if self.device.type != "cuda" or per_page == 0:
            return max(1, reachable)
        free, total = torch.cuda.mem_get_info(self.device)
        element = torch.empty((), dtype=cfg.dtype).element_size()
        widest = min(cfg.token_budget, cfg.max_num_seqs * cfg.max_model_len)
        activations = widest * model.spec.hidden_size * element * 32 + cfg.max_num_seqs * model.spec.vocab_size * 8
        budget = free - int(total * (1.0 - cfg.gpu_memory_utilization)) - activations
        affordable = max(0, budget // per_page)
        if affordable < reachable:
            servable = affordable * cfg.block_size // max(1, cfg.max_model_len)
            _LOGGER.warning(
                "the cache holds %d pages but max_num_seqs=%d x max_model_len=%d can address %d; "
                "about %d full-length requests fit at once", affordable, cfg.max_num_seqs, cfg.max_model_len,
                reachable, servable)
        if affordable < 1:
            raise RuntimeError("no memory is left for the cache; lower gpu_memory_utilization's complement, "
                               "max_num_batched_tokens or the model size")
        return int(min(affordable, reachable))

    # ------------------------------------------------------------- requests
    @property
    def num_waiting(self) -> int:
        return len(self.scheduler.waiting)

    def add_request(self, request_id: str, prompt: str | list[int], params: SamplingParams) -> Sequence:
        """Tokenize and queue one request.  A bad request raises and touches nothing else
        (async_llm_engine.py:207-222: empty and over-long prompts are refused)."""
        if isinstance(prompt, str):
            token_ids = self.tokenizer.encode(prompt)
            text = prompt
        else:
            token_ids = [int(t) for t in prompt]
            vocab = self.runner.model.spec.vocab_size
            if any(not 0 <= t < vocab for t in token_ids):
                raise ValueError(f"a prompt token id lies outside the vocabulary [0, {vocab})")
            text = self.tokenizer.decode(token_ids)
        if not token_ids:
            raise ValueError(f"prompt {prompt!r} encodes to no tokens")
        if len(token_ids) >= self.config.max_model_len:
            raise ValueError(f"prompt has {len(token_ids)} tokens, >= max_model_len={self.config.max_model_len}")
        rules = StopRules(params, self.tokenizer.eos_token_ids, self.config.max_model_len - len(token_ids))
        seq = Sequence(request_id=request_id, prompt=text, prompt_token_ids=list(token_ids), sampling_params=params,
                       detokenizer=IncrementalDetokenizer(), rules=rules)
        if not self.has_unfinished():
            self._last_step_end = 0.0
        self.scheduler.add(seq)
        return seq

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._in_flight is not None

    # ----------------------------------------------------------------- step
    def step(self) -> StepResult:
        result = StepResult()
        t_begin = time.perf_counter()
        # Requests that have finished and whose last token has been read give back what they hold.
        for seq in self.scheduler.remove_finished(ready=lambda s: s.num_unread_tokens == 0):
            self.runner.release(seq.request_id)
            self.sampler.forget(seq.sampling_params, seq.request_id)
            result.released.append(seq)
        before = self._in_flight
        self._in_flight = self._launch(result, t_begin, before)
        if before is not None:
            self._collect(before, result)
        if not self.pipelined and self._in_flight is not None:
            self._collect(self._in_flight, result)
            self._in_flight = None
        if self._in_flight is None and before is None:
            self._last_step_end = 0.0      # idle: the next step's loop time starts with that step
        return result

    def _launch(self, result: StepResult, t_begin: float, before: _Launched | None) -> _Launched | None:
        """Plans the next step and puts it on the device; None if there is nothing to run (or it was refused)."""
        plan = self.scheduler.schedule()
        if plan.is_empty:
            return None
        row_of = {id(seq): row for row, seq in enumerate(before.seqs)} if before is not None else {}
        entries: list[StepEntry] = []
        prompt_tokens = 0
        for seq, count in plan.grants:
            if not seq.is_prompt_computed:
                prompt_tokens += count
            completes = seq.num_computed_tokens + count >= len(seq.prompt_token_ids)
            tokens = seq.next_tokens(count)
            late = None
            if tokens[-1] == PENDING:       # sampled by the step before this one, still on the device
                late = row_of[id(seq)]
            entries.append(StepEntry(seq.request_id, tokens, (count - 1,) if completes else (), late))

        timed = self.config.collect_stats
        events = self._events() if timed else None
        start = time.perf_counter()
        try:
            if events:
                events[0].record()
            # The logits are sampled from on this stream before the next step is launched: no copy of them.
            logits = self.runner.step(entries, before.sampled if before is not None else None, borrow=True)
            if events:
                events[1].record()
        except CacheExhaustedError as error:
            self._abort(shed_order(plan.seqs), error, result)
            return None
        except Exception as error:  # the pass failed, so its requests cannot continue
            self._abort(plan.seqs, error, result)
            return None

        sampling, places = [], []
        for (seq, count), entry in zip(plan.grants, entries):
            seq.num_computed_tokens += count
            if entry.want:
                sampling.append(seq)
        sampled = host_copy = copied = None
        if sampling:
            sampled = self.sampler(logits, [s.sampling_params for s in sampling], [s.request_id for s in sampling])
            if events:
                events[2].record()
            if self.device.type == "cuda":
                # The tokens start for the host now, behind this step's sampling: a copy asked for later would queue
                # behind the step launched meanwhile.  They travel on a stream of their own, so that the next step
                # (which reads them on the device) does not wait for the copy either.
                host_copy, copied = self._host_buffers.pop() if self._host_buffers else (
                    torch.empty(self.config.max_num_seqs, dtype=torch.int32, pin_memory=True), torch.cuda.Event())
                if self._copy_stream is None:
                    self._copy_stream = torch.cuda.Stream(self.device)
                    self._sampled_ready = torch.cuda.Event()
                self._sampled_ready.record()
                self._copy_stream.wait_event(self._sampled_ready)
                with torch.cuda.stream(self._copy_stream):
                    host_copy[:len(sampling)].copy_(sampled, non_blocking=True)
                    copied.record()
                sampled.record_stream(self._copy_stream)
            for seq in sampling:
                places.append(len(seq.output_token_ids))
                seq.output_token_ids.append(PENDING)
                if seq.rules.ended_by_length(len(seq.output_token_ids)):
                    seq.last_token_launched = True      # known without the token's value: no further step
        return _Launched(sampling, places, sampled, host_copy, copied, len(entries), sum(len(e.tokens) for e in entries),
                         prompt_tokens, t_begin, start, time.perf_counter(), events)

    def _collect(self, step: _Launched, result: StepResult) -> None:
        """Reads a launched step's tokens (the one device-to-host copy of a step), puts them in their places and
        applies the rules that need their values."""
        t_wait = time.perf_counter()
        if step.host_copy is not None:
            step.copied.synchronize()
            token_ids = step.host_copy[:len(step.seqs)].tolist()
            self._host_buffers.append((step.host_copy, step.copied))
        else:
            token_ids = step.sampled.tolist() if step.sampled is not None else []
        t_read = time.perf_counter()
        for seq, place, token_id in zip(step.seqs, step.places, token_ids):
            if seq.status == SequenceStatus.FINISHED_ABORTED or place >= len(seq.output_token_ids):
                continue                    # aborted meanwhile, or ended by an earlier token: this one is dropped
            seq.output_token_ids[place] = int(token_id)
            produced = place + 1
            needs_text = self.text_every_step or seq.rules.reads_text
            if needs_text:
                seq.output_text = seq.detokenizer.update(self.tokenizer, seq.output_token_ids[:produced])
            status = seq.rules.status_after(produced, int(token_id), seq.output_text)
            if status is not None:
                del seq.output_token_ids[produced:]         # a token launched after this one is not the request's
                seq.status = status
            if seq.is_finished:
                if not needs_text:          # the detokenizer catches up on everything it has not seen
                    seq.output_text = seq.detokenizer.catch_up(self.tokenizer, seq.output_token_ids)
                self.stats.num_requests_finished += 1
            result.sampled.append(seq)
        if self.config.collect_stats:
            now = time.perf_counter()
            stages = StageTimes(schedule=step.t_start - step.t_begin, launch=step.t_launched - step.t_start,
                                wait=t_read - t_wait, finish=now - t_read,
                                loop=now - (self._last_step_end or step.t_begin))
            if step.events:
                if step.sampled is None:
                    step.events[1].synchronize()        # a step that samples nothing: nothing was read, wait for it here
                # (otherwise the read above waited for the copy behind the step, so the events have happened)
                stages.forward_device = step.events[0].elapsed_time(step.events[1]) * 1e-3
                if step.sampled is not None:
                    stages.sample_device = step.events[1].elapsed_time(step.events[2]) * 1e-3
                self._event_sets.append(step.events)
            self._last_step_end = now
            self.stats.record(StepMetrics(self._step_idx, step.num_seqs, step.input_tokens, step.prompt_tokens,
                                          len(step.seqs), now - step.t_start, stages, now))
        self._step_idx += 1
        if self._step_idx % 256 == 1:
            self.runner.check_kernels()

    def _events(self):
        if self.device.type != "cuda":
            return None
        if self._event_sets:
            return self._event_sets.pop()
        return [torch.cuda.Event(enable_timing=True) for _ in range(3)]

    def _abort(self, seqs: list[Sequence], error: Exception, result: StepResult) -> None:
        for seq in seqs:
            seq.status = SequenceStatus.FINISHED_ABORTED
            del seq.output_token_ids[len(seq.output_token_ids) - seq.num_unread_tokens:]    # tokens never read
            self.stats.num_requests_aborted += 1
            result.aborted.append((seq, error))

    def close(self) -> None:
        if self.runner is not None:
            self.runner.check_kernels()
        self.runner = None
        self._in_flight = None
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
