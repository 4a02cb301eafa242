"""`LLM`: synchronous offline generation (liteinfer/llm.py:14-68).

    llm = LLM("path/to/model", dtype="bfloat16", max_num_seqs=8)
    outputs = llm.generate(["5 17 3", "9 9"], SamplingParams(max_tokens=16, temperature=0))
    llm.close()

Keyword arguments are `EngineConfig` fields.  Prompts are strings (tokenized by
the model's tokenizer) or lists of token ids.  Outputs come back in the order
the prompts were given.
"""

from __future__ import annotations

from itertools import count

from liteinfer_b200.config.engine_config import EngineConfig
from liteinfer_b200.engine.core import EngineCore
from liteinfer_b200.engine.outputs import RequestOutput
from liteinfer_b200.engine.sequence import FINISH_REASONS
from liteinfer_b200.sampling.params import SamplingParams


class LLM:
    def __init__(self, model: str, **engine_kwargs) -> None:
        self.config = EngineConfig(model=str(model), **engine_kwargs)
        self.engine = EngineCore(self.config, text_every_step=False)   # a batch call hands text out at the end only
        self.engine.load()
        self._ids = count(0)

    @property
    def stats(self):
        return self.engine.stats

    @property
    def tokenizer(self):
        return self.engine.tokenizer

    def generate(self, prompts: str | list[int] | list[str] | list[list[int]],
                 sampling_params: SamplingParams | list[SamplingParams] | None = None) -> list[RequestOutput]:
        """Generate completions, returned in the order the prompts were given.

        A request that fails (empty or over-long prompt, shed when the cache ran out)
        raises its error after the others have finished.
        """
        if isinstance(prompts, str) or (isinstance(prompts, list) and prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        if isinstance(sampling_params, list):
            if len(sampling_params) != len(prompts):
                raise ValueError("one SamplingParams per prompt, or one for all")
            params = sampling_params
        else:
            params = [sampling_params or SamplingParams()] * len(prompts)

        engine = self.engine
        pending = list(zip([f"req-{next(self._ids)}" for _ in prompts], prompts, params))
        order = [request_id for request_id, _, _ in pending]
        done: dict[str, RequestOutput] = {}
        failed: dict[str, Exception] = {}
        live: dict[str, object] = {}
        while pending or engine.has_unfinished():
            # The batch call paces itself against the queue cap (liteinfer/async_llm.py:76-79).
            while pending and engine.num_waiting < self.config.max_waiting_seqs:
                request_id, prompt, p = pending.pop(0)
                try:
                    live[request_id] = engine.add_request(request_id, prompt, p)
                except Exception as error:
                    failed[request_id] = error
            result = engine.step()
            for seq, error in result.aborted:
                failed[seq.request_id] = error
                live.pop(seq.request_id, None)
            for seq in result.sampled:
                if seq.is_finished:
                    done[seq.request_id] = RequestOutput(seq.request_id, seq.prompt, seq.output_text,
                                                         list(seq.output_token_ids), FINISH_REASONS[seq.status])
                    live.pop(seq.request_id, None)
        if failed:
            raise next(iter(failed.values()))
        return [done[request_id] for request_id in order]

    def close(self) -> None:
        self.engine.close()

    def __enter__(self) -> LLM:
        return self

    def __exit__(self, *_) -> None:
        self.close()
