"""The engine: requests in, tokens out, one `step()` at a time.

One step is what liteinfer/engine/async_llm_engine.py:228-264 does: drop the
requests that finished (their pages go back), let the scheduler spend the token
budget, run every scheduled request's tokens through the step function as one
batch, sample the requests whose prompt is now complete, apply the stop rules.
A step that the cache cannot hold sheds one tier of requests (:73-85) and the
rest go on; any other failure aborts the step's requests only (:249-251).

`EngineCore` is synchronous and owns everything on the device.  `LLM` drives it
directly; `AsyncLLM` drives it from an asyncio task.
"""

from __future__ import annotations

import logging
import time
from dataclasses import dataclass, field

import torch

from liteinfer_b200.cache.manager import CacheManager
from liteinfer_b200.cache.pages import CacheExhaustedError
from liteinfer_b200.config.engine_config import EngineConfig
from liteinfer_b200.engine.loading import resolve_model_path
from liteinfer_b200.engine.metrics import EngineStats, StageTimes, StepMetrics
from liteinfer_b200.engine.runner import ModelRunner, StepEntry
from liteinfer_b200.engine.scheduler import Scheduler, rows_to_shed
from liteinfer_b200.engine.sequence import Sequence, SequenceStatus, resolve_stop_status
from liteinfer_b200.sampling.params import SamplingParams
from liteinfer_b200.sampling.sampler import Sampler
from liteinfer_b200.tokenizer import IncrementalDetokenizer, load_tokenizer
from liteinfer_b200.weights.loader import load_model

_LOGGER = logging.getLogger(__name__)


class EngineOverloaded(RuntimeError):
    """The waiting queue is full; the request was not accepted (async_llm_engine.py:58-64)."""


@dataclass
class StepResult:
    sampled: list[Sequence] = field(default_factory=list)            # requests that got a token this step
    released: list[Sequence] = field(default_factory=list)           # finished earlier, evicted now
    aborted: list[tuple[Sequence, Exception]] = field(default_factory=list)


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
        self.scheduler = Scheduler(config, page_gate=self._pages_free_for)
        self.runner: ModelRunner | None = None
        self.tokenizer = None
        self.model_config = None
        self._step_idx = 0
        self._last_step_end = 0.0
        self._events = None     # three CUDA events that mark the forward and the sampler on the stream

    # ----------------------------------------------------------------- load
    def load(self) -> None:
        model_dir = resolve_model_path(self.config.model)
        model, self.model_config = load_model(model_dir, self.config.dtype, self.device)
        eos = tuple(getattr(self.model_config, "eos_token_id", ()) or ())
        self.tokenizer = load_tokenizer(model_dir, model.spec.vocab_size, eos)
        num_pages = self._num_pages(model)
        cache = CacheManager(model.cache_needs(), model.schedule, self.config.block_size, num_pages,
                             self.config.max_num_seqs, self.config.dtype, self.device)
        self.runner = ModelRunner(model, cache, self.config.paged_decode_splits)
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
    def _pages_free_for(self, seq: Sequence, admitted: list[Sequence]) -> bool:
        """Admission gate: can the cache hold this request to its very end, beside every request that is
        running (those admitted earlier in this step are among them), each grown to its own end?  Each group of
        the cache says what a request of that length costs it (a window bounds what it holds there), and a model
        that keeps no pages is held by its state slots alone.  With this rule a step of admitted requests never
        runs out of pages; requests wait for room instead."""
        def end_of(s: Sequence) -> int:
            return min(len(s.prompt_token_ids) + s.sampling_params.max_tokens, self.config.max_model_len)

        live = [s for s in self.scheduler.running if not s.is_finished and s is not seq]
        return self.runner.cache.can_hold([end_of(s) for s in [seq, *live]], self.config.token_budget)

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
        seq = Sequence(request_id=request_id, prompt=text, prompt_token_ids=list(token_ids), sampling_params=params,
                       detokenizer=IncrementalDetokenizer())
        if not self.scheduler.has_unfinished():
            self._last_step_end = 0.0
        self.scheduler.add(seq)
        return seq

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    # ----------------------------------------------------------------- step
    def step(self) -> StepResult:
        result = StepResult()
        timed = self.config.collect_stats
        t_begin = time.perf_counter()
        for seq in self.scheduler.remove_finished():
            self.runner.release(seq.request_id)
            self.sampler.forget(seq.sampling_params, seq.request_id)
            result.released.append(seq)
        sched = self.scheduler.schedule()
        if sched.is_empty:
            self._last_step_end = 0.0      # idle: the next step's loop time starts with that step
            return result

        entries: list[StepEntry] = []
        prompt_tokens = 0
        for seq in sched.seqs:
            count = sched.num_scheduled_tokens[seq.request_id]
            if not seq.is_prompt_computed:
                prompt_tokens += count
            completes = seq.num_computed_tokens + count >= len(seq.prompt_token_ids)
            entries.append(StepEntry(seq.request_id, seq.next_tokens(count), (count - 1,) if completes else ()))

        events = self._stream_events() if timed else None
        start = time.perf_counter()
        try:
            if events:
                events[0].record()
            logits = self.runner.step(entries)
            if events:
                events[1].record()
        except CacheExhaustedError as error:
            self._abort(rows_to_shed(sched.seqs), error, result)
            return result
        except Exception as error:  # the pass failed, so its requests cannot continue
            self._abort(sched.seqs, error, result)
            return result

        for seq, entry in zip(sched.seqs, entries):
            seq.num_computed_tokens += len(entry.tokens)
        sampling = [seq for seq, entry in zip(sched.seqs, entries) if entry.want]
        t_launched = t_read = time.perf_counter()
        if sampling:
            sampled = self.sampler(logits, [s.sampling_params for s in sampling], [s.request_id for s in sampling])
            if events:
                events[2].record()
            token_ids = sampled.tolist()       # one device-to-host read per step
            t_read = time.perf_counter()
            for seq, token_id in zip(sampling, token_ids):
                seq.output_token_ids.append(int(token_id))
                needs_text = self.text_every_step or bool(seq.sampling_params.stop)
                if needs_text:
                    seq.output_text = seq.detokenizer.update(self.tokenizer, seq.output_token_ids)
                status = resolve_stop_status(seq, int(token_id), self.tokenizer.eos_token_ids,
                                             self.config.max_model_len)
                if status is not None:
                    if not needs_text:      # the detokenizer catches up on everything it has not seen
                        seq.output_text = seq.detokenizer.catch_up(self.tokenizer, seq.output_token_ids)
                    seq.status = status
                    self.stats.num_requests_finished += 1
            result.sampled = sampling
        if timed:
            if self.device.type == "cuda" and not sampling:
                torch.cuda.synchronize(self.device)
                t_read = time.perf_counter()
            now = time.perf_counter()
            stages = StageTimes(schedule=start - t_begin, launch=t_launched - start, wait=t_read - t_launched,
                                finish=now - t_read, loop=now - (self._last_step_end or t_begin))
            if events:      # the read above waited for the stream, so the events have happened
                stages.forward_device = events[0].elapsed_time(events[1]) * 1e-3
                if sampling:
                    stages.sample_device = events[1].elapsed_time(events[2]) * 1e-3
            self._last_step_end = now
            self.stats.record(StepMetrics(self._step_idx, len(entries), sum(len(e.tokens) for e in entries),
                                          prompt_tokens, len(sampling), now - start, stages, now))
        self._step_idx += 1
        if self._step_idx % 256 == 1:
            self.runner.check_kernels()
        return result

    def _stream_events(self):
        if self.device.type != "cuda":
            return None
        if self._events is None:
            self._events = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        return self._events

    def _abort(self, seqs: list[Sequence], error: Exception, result: StepResult) -> None:
        for seq in seqs:
            seq.status = SequenceStatus.FINISHED_ABORTED
            self.stats.num_requests_aborted += 1
            result.aborted.append((seq, error))

    def close(self) -> None:
        if self.runner is not None:
            self.runner.check_kernels()
        self.runner = None
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
