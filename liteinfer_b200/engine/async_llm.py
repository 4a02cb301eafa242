"""`AsyncLLM`: continuous batching behind an asyncio interface (liteinfer/async_llm.py:15-112).

    async with AsyncLLM("path/to/model") as llm:
        results = await llm.generate(prompts, SamplingParams(max_tokens=64))
        async for event in llm.stream(prompt, SamplingParams(max_tokens=64)):
            ...

One background task runs engine steps and yields to the event loop between
them (liteinfer/engine/async_llm_engine.py:1-28,127-193).  A streamed request has a
queue of `StreamEvent`s ended by None, or by the error that ended it; a request of a
batch call has a future that its last event resolves, and no events before that.
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
        self._queues: dict[str, asyncio.Queue] = {}        # streamed requests: their events, then None or an error
        self._futures: dict[str, asyncio.Future] = {}       # batch requests: resolved with the final event
        self._pending: asyncio.Queue = asyncio.Queue()
        self._room = asyncio.Event()                        # set whenever the queue of accepted requests shrinks
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
            for request_id in [*self._queues, *self._futures]:
                self._fail(request_id, failure)
            raise

    def _admit(self, item) -> None:
        request_id, prompt, params = item
        try:
            self.engine.add_request(request_id, prompt, params)
        except Exception as error:   # a bad request fails only itself
            self._fail(request_id, error)

    def _fail(self, request_id: str, error: Exception) -> None:
        """The request ends with `error`, whichever way its caller is listening."""
        queue = self._queues.pop(request_id, None)
        if queue is not None:
            queue.put_nowait(error)
        future = self._futures.pop(request_id, None)
        if future is not None and not future.done():
            future.set_exception(error)

    def _event(self, seq: Sequence) -> StreamEvent:
        return StreamEvent(seq.request_id, seq.prompt, seq.read_token_ids, seq.output_text,
                           seq.is_finished, FINISH_REASONS.get(seq.status) if seq.is_finished else None)

    def _deliver(self, result) -> None:
        """Hands a step's outcome to whoever waits for it: every new token to a stream, only the last to a batch
        call (which would throw the others away), the end of a stream when the request's seat is given up."""
        for seq, error in result.aborted:
            self._fail(seq.request_id, error)
        for seq in result.sampled:
            queue = self._queues.get(seq.request_id)
            if queue is not None:
                queue.put_nowait(self._event(seq))
            elif seq.is_finished:
                future = self._futures.pop(seq.request_id, None)
                if future is not None and not future.done():
                    future.set_result(self._event(seq))
        for seq in result.released:
            queue = self._queues.pop(seq.request_id, None)
            if queue is not None:
                queue.put_nowait(None)
        self._room.set()

    # ------------------------------------------------------------------ API
    def _accept(self, request_id: str, prompt, params: SamplingParams) -> None:
        """Queues a request for the loop, or refuses it when the loop is down or the queue is full."""
        if self._task is None or self._task.done():
            raise RuntimeError("engine loop is not running; call start() first")
        if self.num_waiting >= self.config.max_waiting_seqs:
            raise EngineOverloaded(f"{self.num_waiting} requests already waiting "
                                   f"(max_waiting_seqs={self.config.max_waiting_seqs}); retry later")
        self._pending.put_nowait((request_id, prompt, params))

    async def generate(self, prompts, sampling_params: SamplingParams | None = None) -> list[RequestOutput]:
        """Submit all prompts and await their completions, in the order given.  A long list is fed in as the queue
        of accepted requests has room (`max_waiting_seqs`), so a batch call never trips the overload check."""
        if isinstance(prompts, str) or (isinstance(prompts, list) and prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        params = sampling_params or SamplingParams()
        loop = asyncio.get_running_loop()
        waiting: list[tuple[str, asyncio.Future]] = []
        for prompt in prompts:
            while self.num_waiting >= self.config.max_waiting_seqs:
                self._room.clear()
                await self._room.wait()
            request_id = f"req-{next(self._ids)}"
            future = loop.create_future()
            self._futures[request_id] = future
            try:
                self._accept(request_id, prompt, params)
            except BaseException:
                self._futures.pop(request_id, None)
                raise
            waiting.append((request_id, future))
        finals = await asyncio.gather(*(future for _, future in waiting), return_exceptions=True)
        for final in finals:
            if isinstance(final, BaseException):
                raise final
        return [RequestOutput(request_id, final.prompt, final.text, final.output_token_ids, final.finish_reason or "stop")
                for (request_id, _), final in zip(waiting, finals)]

    async def stream(self, prompt, sampling_params: SamplingParams | None = None) -> AsyncGenerator[StreamEvent, None]:
        """Submit one prompt and stream its events token by token; an error that ends the request is raised here."""
        request_id = f"req-{next(self._ids)}"
        queue: asyncio.Queue = asyncio.Queue()
        self._queues[request_id] = queue
        try:
            self._accept(request_id, prompt, sampling_params or SamplingParams())
        except BaseException:
            self._queues.pop(request_id, None)
            raise
        while True:
            item = await queue.get()
            if item is None:
                return
            if isinstance(item, Exception):
                raise item
            yield item
