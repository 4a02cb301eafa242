"""`python -m liteinfer_b200 bench`: throughput and latency of the engine on synthetic requests.

The reference's benchmark script (benchmarks/cli.py:209-265) makes a dataset of prompts of a stated length
(`dataset --isl --osl -n`), runs it in two modes (`run --mode throughput|latency|both`) and reports

  throughput  every request offered at once: output tokens/s, requests/s, wall time (benchmarks/stats.py:53-62);
  latency     one request at a time: time to the first token, time per further token derived as
              (e2e - ttft) / (osl - 1), and end-to-end time, as percentiles (stats.py:65-82).

Here `bench run` does both steps with the same option names and the same summaries.  There is no corpus and
no tokenizer on the machines this runs on, so the prompts are seeded uniform-random token ids of the stated
lengths; `--isl mixed` draws lengths from a log-normal spread with the median (17) and 99th percentile
(1,286) the reference reports for its corpus (benchmarks/dataset.py:14-19), capped at `--max-isl`.  Output
length is forced as the reference forces it (`min_tokens = max_tokens = osl`, `ignore_eos`;
benchmarks/adapters.py:70-72); two warm-up rounds at the width of the run come before the clock
(benchmarks/harness.py:110-122); the clock is the host's, with the device synchronised on both sides.
"""

from __future__ import annotations

import json
import math
import random
import time
from pathlib import Path

WARMUP_TOKENS = 32
WARMUP_ROUNDS = 2
DEFAULT_MAX_MIXED_ISL = 2048


def percentile(values: list[float], p: float) -> float:
    """The p-th percentile with linear interpolation between neighbours (what the reference's summaries use,
    benchmarks/stats.py:17-30)."""
    import numpy as np

    return float(np.percentile(np.asarray(values, dtype=np.float64), p))


def make_prompts(vocab_size: int, isl: int | None, num_samples: int, max_isl: int, seed: int) -> list[list[int]]:
    """Seeded token-id prompts: all `isl` long, or (isl None) of log-normally spread lengths up to `max_isl`."""
    rng = random.Random(seed)
    sigma = math.log(1286 / 17) / 2.326          # 99th percentile 1,286 at a median of 17
    prompts = []
    for _ in range(num_samples):
        n = isl if isl is not None else max(1, min(max_isl, round(17 * math.exp(rng.gauss(0.0, sigma)))))
        prompts.append([rng.randrange(vocab_size) for _ in range(n)])
    return prompts


def throughput_summary(output_tokens: int, num_requests: int, wall_time_s: float) -> dict:
    """Every request offered at once: what came out per second of wall time (benchmarks/stats.py:53-62)."""
    per_second = 1.0 / wall_time_s
    return {"output_tokens_per_s": output_tokens * per_second, "requests_per_s": num_requests * per_second,
            "wall_time_s": wall_time_s}


def latency_summary(ttft_s: list[float], e2e_s: list[float], osl: int) -> dict:
    """One request at a time: percentiles of the time to the first token, of the time per further token (derived:
    what is left of the end-to-end time spread over the osl - 1 further tokens) and of the end-to-end time
    (benchmarks/stats.py:65-82)."""
    if osl < 2:
        raise ValueError("latency mode needs --osl >= 2 to derive the time per further token")
    series = {"ttft": ttft_s, "itl": [(whole - first) / (osl - 1) for first, whole in zip(ttft_s, e2e_s, strict=True)]}
    summary = {f"{name}_p{p}_ms": percentile(values, p) * 1e3 for name, values in series.items() for p in (50, 95, 99)}
    summary["e2e_p50_ms"] = percentile(e2e_s, 50) * 1e3
    return summary


def _sync(llm) -> None:
    import torch

    if llm.engine.device.type == "cuda":
        torch.cuda.synchronize(llm.engine.device)


def _timed_generate(llm, prompts, tokens: int) -> tuple[float, list[int]]:
    from liteinfer_b200.sampling.params import SamplingParams

    params = SamplingParams(temperature=0.0, max_tokens=tokens, min_tokens=tokens, ignore_eos=True)
    _sync(llm)
    start = time.perf_counter()
    outs = llm.generate(prompts, params)
    _sync(llm)
    return time.perf_counter() - start, [len(o.token_ids) for o in outs]


def _check_lengths(counts: list[int], expected: int) -> None:
    wrong = [c for c in counts if c != expected]
    if wrong:
        raise RuntimeError(f"{len(wrong)}/{len(counts)} requests returned {wrong[0]} tokens instead of {expected}: "
                           "the forced output length did not hold, so the run is not comparable")


def run(llm, prompts: list[list[int]], osl: int, mode: str) -> dict:
    """The summaries of `mode` ("throughput", "latency" or "both") for these prompts on a loaded engine."""
    out: dict = {}
    width = llm.config.max_num_seqs
    if mode in ("throughput", "both"):
        warm = [prompts[i % len(prompts)] for i in range(width)]
        for _ in range(WARMUP_ROUNDS):
            _timed_generate(llm, warm, min(WARMUP_TOKENS, osl))
        llm.stats.steps.clear()
        wall, counts = _timed_generate(llm, prompts, osl)
        _check_lengths(counts, osl)
        phases: dict[str, int] = {}
        for step in llm.stats.steps:
            phases[step.phase] = phases.get(step.phase, 0) + 1
        out["throughput"] = {**throughput_summary(sum(counts), len(counts), wall), "step_phases": phases}
    if mode in ("latency", "both"):
        for _ in range(WARMUP_ROUNDS):
            _timed_generate(llm, prompts[:1], 1)
            _timed_generate(llm, prompts[:1], min(WARMUP_TOKENS, osl))
        ttft, e2e = [], []
        for prompt in prompts:
            first, _ = _timed_generate(llm, [prompt], 1)          # a pass that ends at the first token
            whole, counts = _timed_generate(llm, [prompt], osl)
            _check_lengths(counts, osl)
            ttft.append(first)
            e2e.append(whole)
        out["latency"] = latency_summary(ttft, e2e, osl)
    return out


def main(args) -> int:
    from liteinfer_b200.engine.llm import LLM

    isl = None if args.isl == "mixed" else int(args.isl)
    longest = args.max_isl if isl is None else isl
    engine = {k: getattr(args, k) for k in ("dtype", "device", "max_num_seqs", "max_num_batched_tokens", "block_size",
                                            "num_gpu_blocks", "gpu_memory_utilization", "paged_decode_splits",
                                            "enable_cuda_graphs", "seed")}
    engine["max_model_len"] = max(args.max_model_len, longest + args.osl + 1)
    with LLM(args.model, **engine) as llm:
        vocab = llm.engine.runner.model.spec.vocab_size
        prompts = make_prompts(vocab, isl, args.num_samples, args.max_isl, args.dataset_seed)
        summary = run(llm, prompts, args.osl, args.mode)
    result = {"model": args.model, "mode": args.mode, "max_num_seqs": args.max_num_seqs,
              "dataset": {"target_isl": isl, "target_osl": args.osl, "max_isl": args.max_isl if isl is None else None,
                          "num_samples": len(prompts), "input_tokens": sum(len(p) for p in prompts),
                          "data": "seeded uniform-random token ids"},
              "summary": summary}
    print(json.dumps(result))
    if args.results_dir:
        shape = f"isl{'mixed' if isl is None else isl}_osl{args.osl}"
        path = Path(args.results_dir) / f"liteinfer_b200__{args.mode}__{shape}.json"
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(json.dumps(result, indent=1))
    return 0
