"""`AsyncLLM`: continuous batching behind an asyncio interface (liteinfer/async_llm.py:15-112).

    async with AsyncLLM("path/to/model") as llm:
        results = await llm.generate(prompts, SamplingParams(max_tokens=64))
        async for event in llm.stream(prompt, SamplingParams(max_tokens=64)):
            ...

One background task runs engine steps and yields to the event loop between
them; each request has a queue of `StreamEvent`s ended by None, or by the error
that ended it (liteinfer/engine/async_llm_engine.py:1-28,127-193).
"""

from __future__ import annotations

import asyncio
from collections.abc import AsyncGenerator
from itertools import count

from liteinfer_b200.config.engine_config import EngineConfig
from liteinfer_b200.engine.core import EngineCore, EngineOverloaded
from liteinfer_b200.engine.outputs import RequestOutput, StreamEvent
from liteinfer_b200.engine.sequence import FINISH_REASONS, Sequence
from liteinfer_b200.sampling.params import SamplingParams

_IDLE_POLL_S = 0.05


class AsyncLLM:
    def __init__(self, model: str, **engine_kwargs) -> None:
        self.config = EngineConfig(model=str(model), **engine_kwargs)
        self.engine = EngineCore(self.config)
        self._ids = count(0)
        self._queues: dict[str, asyncio.Queue] = {}
        self._final_only: set[str] = set()
        self._pending: asyncio.Queue = asyncio.Queue()
        self._task: asyncio.Task | None = None
        self._shutdown = asyncio.Event()

    # ------------------------------------------------------------ lifecycle
    async def start(self) -> None:
        self.engine.load()
        self._task = asyncio.create_task(self._run_loop())

    async def stop(self) -> None:
        self._shutdown.set()
        if self._task is not None:
            await self._task
            self._task = None
        self.engine.close()

    async def __aenter__(self) -> AsyncLLM:
        await self.start()
        return self

    async def __aexit__(self, *_) -> None:
        await self.stop()

    # ----------------------------------------------------------------- loop
    @property
    def num_waiting(self) -> int:
        return self._pending.qsize() + self.engine.num_waiting

    async def _run_loop(self) -> None:
        try:
            while not self._shutdown.is_set():
                while not self._pending.empty():
                    self._admit(self._pending.get_nowait())
                if self.engine.has_unfinished():
                    self._deliver(self.engine.step())
                else:
                    try:
                        self._admit(await asyncio.wait_for(self._pending.get(), timeout=_IDLE_POLL_S))
                    except asyncio.TimeoutError:
                        pass
                await asyncio.sleep(0)
        except BaseException as error:
            # Only this loop ever completes a request: if it dies, every waiter must hear of it.
            failure = error if isinstance(error, Exception) else RuntimeError(repr(error))
            for request_id in list(self._queues):
                self._fail(request_id, failure)
            raise

    def _admit(self, item) -> None:
        request_id, prompt, params = item
        try:
            self.engine.add_request(request_id, prompt, params)
        except Exception as error:   # a bad request fails only itself
            self._fail(request_id, error)

    def _forget(self, request_id: str):
        self._final_only.discard(request_id)
        return self._queues.pop(request_id, None)

    def _fail(self, request_id: str, error: Exception) -> None:
        queue = self._forget(request_id)
        if queue is not None:
            queue.put_nowait(error)

    def _event(self, seq: Sequence) -> StreamEvent:
        return StreamEvent(seq.request_id, seq.prompt, list(seq.output_token_ids), seq.output_text,
                           seq.is_finished, FINISH_REASONS.get(seq.status) if seq.is_finished else None)

    def _deliver(self, result) -> None:
        for seq in result.released:
            queue = self._forget(seq.request_id)
            if queue is not None:
                queue.put_nowait(None)
        for seq, error in result.aborted:
            self._fail(seq.request_id, error)
        for seq in result.sampled:
            queue = self._queues.get(seq.request_id)
            if queue is not None and (seq.is_finished or seq.request_id not in self._final_only):
                queue.put_nowait(self._event(seq))

    # ------------------------------------------------------------------ API
    async def _generate_stream(self, request_id: str, prompt, params: SamplingParams,
                               stream_tokens: bool = True) -> AsyncGenerator[StreamEvent, None]:
        if self._task is None or self._task.done():
            raise RuntimeError("engine loop is not running; call start() first")
        if self.num_waiting >= self.config.max_waiting_seqs:
            raise EngineOverloaded(f"{self.num_waiting} requests already waiting "
                                   f"(max_waiting_seqs={self.config.max_waiting_seqs}); retry later")
        queue: asyncio.Queue = asyncio.Queue()
        self._queues[request_id] = queue
        if not stream_tokens:
            self._final_only.add(request_id)
        self._pending.put_nowait((request_id, prompt, params))
        while True:
            item = await queue.get()
            if item is None:
                return
            if isinstance(item, Exception):
                raise item
            yield item

    async def generate(self, prompts, sampling_params: SamplingParams | None = None) -> list[RequestOutput]:
        """Submit all prompts and await their completions, in the order given."""
        if isinstance(prompts, str) or (isinstance(prompts, list) and prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        params = sampling_params or SamplingParams()
        slots = asyncio.Semaphore(self.config.max_waiting_seqs)

        async def collect(prompt, request_id: str) -> RequestOutput:
            final: StreamEvent | None = None
            async with slots:
                async for event in self._generate_stream(request_id, prompt, params, stream_tokens=False):
                    final = event
            assert final is not None
            return RequestOutput(request_id, final.prompt, final.text, final.output_token_ids,
                                 final.finish_reason or "stop")

        ids = [f"req-{next(self._ids)}" for _ in prompts]
        return list(await asyncio.gather(*(collect(p, r) for p, r in zip(prompts, ids))))

    async def stream(self, prompt, sampling_params: SamplingParams | None = None) -> AsyncGenerator[StreamEvent, None]:
        """Submit one prompt and stream its events token by token."""
        request_id = f"req-{next(self._ids)}"
        async for event in self._generate_stream(request_id, prompt, sampling_params or SamplingParams()):
            yield event
