"""Headline benchmark: decode tokens/s of the Llama 3.2 1B shape on one B200, with prefill and roofline figures.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 with every
sequence near the benchmark context (4,096), timed on the device over K decode
steps of the engine's own step function and sampler.  `e2e` is the same measured
through the Python entry point (`LLM.generate`: host token ids in, host token
ids out; every step its inputs travel from pinned host memory to the device, read
in place by the kernel that stages the batch, and the sampled tokens travel back
to the host).  `prefill` times one 2,048-token prompt,
`roofline` relates the decode step to the bytes it must read, `points` holds
decode at batch 1 and 64.  Weights are random (seeded) and token ids synthetic.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 128256, "hidden_size": 2048, "intermediate_size": 8192,
    "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "max_position_embeddings": 131072, "hidden_act": "silu",
}
# The other shapes of the reference's configurations, for `--shape` (the default run and the contract are the 1B shape).
LLAMA_3B = dict(LLAMA_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, head_dim=128)
LLAMA_8B = dict(LLAMA_1B, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, head_dim=128,
                tie_word_embeddings=False,
                rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                              "original_max_position_embeddings": 8192})
SHAPES = {"1b": ("Llama 3.2 1B", LLAMA_1B, 4096), "3b": ("Llama 3.2 3B", LLAMA_3B, 4096),
          "8b": ("Llama 3.1 8B", LLAMA_8B, 8192)}
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = 16
# A40 decode step of the reference at batch 8 (docs/benchmarks.md:749-753: 6.41 ms -> 1,248 tok/s).
BASELINE_DECODE_B8_TOKS = 1248.0


def _find_number(tree, key: str):
    """The first number stored under `key` anywhere in a JSON tree (the file's layout is the driver's)."""
    if isinstance(tree, dict):
        value = tree.get(key)
        if isinstance(value, (int, float)) and not isinstance(value, bool):
            return float(value)
        if isinstance(value, dict):
            for inner in ("value", "median", "mean"):
                if isinstance(value.get(inner), (int, float)):
                    return float(value[inner])
        for child in tree.values():
            found = _find_number(child, key)
            if found is not None:
                return found
    elif isinstance(tree, list):
        for child in tree:
            found = _find_number(child, key)
            if found is not None:
                return found
    return None


def measured_peaks() -> dict:
    """Copy bandwidth (GB/s) and bfloat16 product throughput (TFLOP/s) to measure against: the driver's
    measurements if it left them, else the stated fallback.  `bf16_tflops_burst` is the library product timed
    alone, `bf16_tflops` the same held for seconds under the power cap; a prefill step of a few milliseconds
    timed alone is measured against the burst figure."""
    fallback = {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "bf16_tflops_burst": 1590.0, "source": "fallback"}
    path = ROOT / "MEASURED_PEAKS.json"
    if not path.is_file():
        return fallback
    try:
        raw = json.loads(path.read_text())
    except (OSError, ValueError):
        return fallback
    hbm = _find_number(raw, "hbm_gbs")
    burst = _find_number(raw, "bf16_tflops")
    flops = _find_number(raw, "bf16_tflops_sustained") or burst
    if hbm is not None and hbm < 100:          # given in TB/s
        hbm *= 1000.0
    if flops is not None and flops > 100000:   # given in GFLOP/s
        flops, burst = flops / 1000.0, (burst or flops) / 1000.0
    if not hbm or not flops:
        return fallback
    return {"hbm_gbs": hbm, "bf16_tflops": flops, "bf16_tflops_burst": burst or flops, "source": "measured"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self._proc = None

    def start(self) -> None:
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self._proc = None

    def _read(self) -> None:
        for line in self._proc.stdout:
            self.samples.append([f.strip() for f in line.split(",")])

    def stop(self) -> dict:
        if self._proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self._proc.terminate()
        rows = [s for s in self.samples if len(s) >= 6 and s[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in rows), "sm_max_mhz": int(rows[0][1]),
                "reasons": reasons, "samples": len(rows)}


def _fill_cache(runner, ids: list[str], lengths: list[int]) -> None:
    """Gives every request `length` tokens of cache without computing them: pages are taken through the
    cache manager and hold small random values (a decode step's time does not depend on what they are)."""
    runner.cache.reserve(ids, lengths)
    for request_id, n in zip(ids, lengths):
        runner.cache.commit(request_id, n)


def _decode_rate(runner, sampler, params, batch: int, start_len: int, steps: int, warmup: int, vocab: int):
    """(tokens/s, ms per step, launches of own kernels per step) of `steps` decode steps at `batch`."""
    import torch

    from liteinfer_b200.engine.runner import StepEntry
    from liteinfer_b200.ops import kernels

    ids = [f"b{batch}-{i}" for i in range(batch)]
    _fill_cache(runner, ids, [start_len] * batch)
    g = torch.Generator().manual_seed(batch)
    tokens = torch.randint(0, vocab, (batch,), generator=g).tolist()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = 0
    for i in range(warmup + steps):
        if i == warmup:
            torch.cuda.synchronize()
            launches = kernels.launch_count + getattr(runner, "graph_launches", 0)
            start.record()
        logits = runner.step([StepEntry(r, [t], (0,)) for r, t in zip(ids, tokens)])
        sampled = sampler(logits, [params] * batch, ids)
        tokens = sampled.tolist()
    stop.record()
    torch.cuda.synchronize()
    launches = kernels.launch_count + getattr(runner, "graph_launches", 0) - launches
    ms = start.elapsed_time(stop) / steps
    for r in ids:
        runner.release(r)
    return batch / ms * 1e3, ms, launches // steps


def run_ours(args) -> dict:
    import torch

    from liteinfer_b200 import LLM, SamplingParams
    from liteinfer_b200.engine.runner import StepEntry
    from liteinfer_b200.ops import kernels
    from liteinfer_b200.sampling.sampler import Sampler
    from liteinfer_b200.weights.random_init import write_random_model

    model_name, shape, CONTEXT = SHAPES[args.shape]     # the context length of the chosen shape
    cfg = dict(shape)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    peaks = measured_peaks()
    steps, warmup, batch = args.steps, max(3, args.warmup), 8
    greedy = SamplingParams(temperature=0.0, max_tokens=warmup + steps + 1, ignore_eos=True)

    with tempfile.TemporaryDirectory() as tmp:
        model_dir = write_random_model(cfg, Path(tmp) / "llama-1b", seed=0)
        decode_start = CONTEXT - (warmup + steps) - 1
        llm = LLM(str(model_dir), dtype="bfloat16", device="cuda:0", max_num_seqs=64, max_model_len=CONTEXT + 1,
                  block_size=PAGE, max_num_batched_tokens=8192, gpu_memory_utilization=0.5)
        runner = llm.engine.runner
        model = runner.model
        for group in runner.cache.groups:                      # random cache contents
            group.pool.normal_(0.0, 0.5)
        vocab, hidden = cfg["vocab_size"], cfg["hidden_size"]
        sampler = Sampler(0)

        g = torch.Generator().manual_seed(7)
        if args.section == "decode":
            value, ms, launches = _decode_rate(runner, sampler, greedy, args.batch, decode_start, steps, warmup, vocab)
            llm.close()
            return {"section": "decode", "batch": args.batch, "value": value, "ms_per_step": ms,
                    "gpu_launches": launches * steps}

        # ---- prefill: one prompt of 2,048 tokens, logits at its last token
        prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=g).tolist()
        times = []
        for i in range(3 + 3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            runner.step([StepEntry("prefill", prompt, (PREFILL_TOKENS - 1,))])
            b.record()
            torch.cuda.synchronize()
            runner.release("prefill")
            if i >= 3:
                times.append(a.elapsed_time(b))
        prefill_ms = statistics.median(times)
        layers = cfg["num_hidden_layers"]
        q, kv, inter = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"], cfg["intermediate_size"]
        linear_params = layers * (hidden * (q + 2 * kv) + q * hidden + 3 * hidden * inter)
        attn_flops = layers * 4 * cfg["num_attention_heads"] * cfg["head_dim"] * PREFILL_TOKENS * (PREFILL_TOKENS + 1) / 2
        prefill_flops = 2 * linear_params * PREFILL_TOKENS + attn_flops + 2 * hidden * vocab
        prefill = {"value": PREFILL_TOKENS / prefill_ms * 1e3, "tokens": PREFILL_TOKENS, "ms": prefill_ms,
                   "frac": prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops_burst"] * 1e12),
                   "frac_of_sustained": prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)}
        if args.section == "prefill":
            llm.close()
            return {"section": "prefill", **prefill}

        # ---- decode, device-timed
        clocks = ClockSampler()
        clocks.start()
        value, ms, launches = _decode_rate(runner, sampler, greedy, batch, decode_start, steps, warmup, vocab)
        clock_record = clocks.stop()
        b1, _, _ = _decode_rate(runner, sampler, greedy, 1, decode_start, steps, warmup, vocab)
        b64, _, _ = _decode_rate(runner, sampler, greedy, 64, decode_start, steps, warmup, vocab)

        # ---- roofline of the batch-8 decode step: every weight once, plus the live requests' cache
        element = 2
        weight_bytes = (linear_params + hidden * vocab + (2 * layers + 1) * hidden) * element
        mean_ctx = decode_start + warmup + steps / 2
        kv_bytes = batch * mean_ctx * layers * 2 * kv * element
        achieved = (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "of": peaks["source"]}

        # ---- end to end through LLM.generate: host ids in, host ids out
        prompts = [torch.randint(0, vocab, (decode_start,), generator=g).tolist() for _ in range(batch)]
        llm.generate(prompts, greedy)          # once untimed: every graph the timed run replays is captured here
        llm.stats.steps.clear()
        outs = llm.generate(prompts, greedy)
        assert all(len(o.token_ids) == warmup + steps + 1 for o in outs)
        # A step's time end to end: from the end of the step before it to its own end (scheduling, the step
        # function, sampling, the read of the tokens, the stop rules and the loop around them).
        decode_steps = [s for s in llm.stats.steps if s.phase == "decode" and s.num_seqs == batch][-steps:]
        e2e_ms = sum(s.stages.loop for s in decode_steps) / len(decode_steps) * 1e3
        stage_us = {name: round(sum(getattr(s.stages, name) for s in decode_steps) / len(decode_steps) * 1e6, 1)
                    for name in ("schedule", "launch", "wait", "finish", "forward_device", "sample_device")}
        pages = -(-CONTEXT // PAGE)
        e2e = {"value": batch / e2e_ms * 1e3, "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 4 * (3 * batch + (batch + 1) + 3 * batch + batch * pages),
               "d2h_bytes_per_step": 4 * batch, "stage_us": stage_us}
        llm.close()

    # ---- the reference's two larger configurations (full depth), each reported as a few flat numbers
    points = {"decode_b1": b1, "decode_b64": b64}
    workloads = {}
    if args.shape == "1b" and not args.layers and not args.no_workloads:
        args.workload = "all"
        workloads = run_workloads(args)
        for name, result in workloads.items():
            for key, number in result.items():
                if key in ("output_tok_s", "decode_hbm_frac", "decode_b1_tok_s", "decode_b8_tok_s", "decode_b64_tok_s",
                           "decode_b1_hbm_frac", "decode_b8_hbm_frac", "decode_b64_hbm_frac", "failed"):
                    points[f"w{name}_{key}"] = number

    return {
        "metric": f"decode tok/s at batch 8 ({model_name} shape)", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / BASELINE_DECODE_B8_TOKS if args.shape == "1b" and not args.layers else None, "dtype": "bf16", "data": "synthetic ids, random weights",
        "impl": "ours",
        "config": {"model": model_name.lower().replace(" ", "-") + "-shape", "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "hidden": hidden, "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": inter, "vocab": vocab, "global_batch": batch,
                   "seq_len": CONTEXT, "page_size": PAGE, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (weights and cache are read every step)",
                   "baseline": "reference A40 batch-8 decode, 1248 tok/s"},
        "clocks": clock_record, "e2e": e2e, "gpu_launches": launches * steps,
        "prefill": prefill, "roofline": roofline, "points": points, "workloads": workloads,
    }


def _shape_numbers(cfg: dict) -> dict:
    layers, hidden, vocab = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    linear = layers * (hidden * (q + 2 * kv) + q * hidden + 3 * hidden * cfg["intermediate_size"])
    return {"weight_bytes": (linear + hidden * vocab + (2 * layers + 1) * hidden) * 2,     # every weight a step reads, once
            "kv_bytes_per_token": layers * 2 * kv * 2}


def workload_3b(args, peaks: dict) -> dict:
    """The reference's serving workload at the Llama 3.2 3B layer sizes: 64 requests with prompts of 128 to 2,048
    tokens (uniform, seeded) and 256 forced output tokens each, all offered at once to `LLM.generate` (continuous
    batching under a token budget of 8,192).  One untimed run of the same requests comes first, as the reference's
    harness warms up (benchmarks/harness.py:110-122).  Reported: output tokens per second over the whole run, and
    for its decode steps the bytes they had to read (weights once, the live requests' cache) over their time."""
    import random

    import torch

    from liteinfer_b200 import LLM, SamplingParams
    from liteinfer_b200.weights.random_init import write_random_model

    cfg = dict(LLAMA_3B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    numbers = _shape_numbers(cfg)
    rng = random.Random(3)
    lengths = [rng.randint(128, 2048) for _ in range(64)]
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in lengths]
    params = SamplingParams(temperature=0.0, max_tokens=256, min_tokens=256, ignore_eos=True)
    with tempfile.TemporaryDirectory() as tmp:
        model_dir = write_random_model(cfg, Path(tmp) / "llama-3b", seed=0)
        with LLM(str(model_dir), dtype="bfloat16", device="cuda:0", max_num_seqs=64, max_model_len=2048 + 256 + 1,
                 block_size=PAGE, max_num_batched_tokens=8192) as llm:
            llm.generate(prompts, params)                       # warm-up: every graph this run needs is captured
            steps: list[tuple[str, float, int]] = []
            scheduler = llm.engine.scheduler
            llm.stats.on_step(lambda m: steps.append(
                (m.phase, m.stages.loop, sum(len(s) for s in scheduler.running if not s.is_finished))))
            torch.cuda.synchronize()
            start = time.perf_counter()
            outs = llm.generate(prompts, params)
            torch.cuda.synchronize()
            wall = time.perf_counter() - start
    assert all(len(o.token_ids) == 256 for o in outs)
    decode = [(t, held) for phase, t, held in steps if phase == "decode"]
    decode_bytes = sum(numbers["weight_bytes"] + held * numbers["kv_bytes_per_token"] for _, held in decode)
    decode_s = sum(t for t, _ in decode)
    return {"model": "llama-3.2-3b-shape", "layers": cfg["num_hidden_layers"], "layers_full": LLAMA_3B["num_hidden_layers"],
            "requests": 64, "prompt_tokens": sum(lengths), "output_tokens": 64 * 256, "wall_s": wall,
            "output_tok_s": 64 * 256 / wall, "total_tok_s": (sum(lengths) + 64 * 256) / wall, "steps": len(steps),
            "decode_steps": len(decode), "decode_ms_per_step": decode_s / max(1, len(decode)) * 1e3,
            "decode_hbm_frac": decode_bytes / decode_s / 1e9 / peaks["hbm_gbs"] if decode_s else None}


def workload_8b(args, peaks: dict) -> dict:
    """Decode at the Llama 3.1 8B layer sizes with every sequence at a context of 8,192: batch 1, 8 and 64, the cache
    sized for 64 such sequences (68.7 GB beside 16 GB of weights).  Tokens per second of the step function and the
    sampler, device-timed, and the fraction of the copy bandwidth that the bytes of a step come to."""
    from liteinfer_b200 import LLM, SamplingParams
    from liteinfer_b200.sampling.sampler import Sampler
    from liteinfer_b200.weights.random_init import write_random_model

    cfg = dict(LLAMA_8B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    numbers = _shape_numbers(cfg)
    context, steps, warmup = 8192, args.steps, max(3, args.warmup)
    start_len = context - (warmup + steps) - 1
    greedy = SamplingParams(temperature=0.0, max_tokens=warmup + steps + 1, ignore_eos=True)
    out = {"model": "llama-3.1-8b-shape", "layers": cfg["num_hidden_layers"], "layers_full": LLAMA_8B["num_hidden_layers"],
           "context": context}
    with tempfile.TemporaryDirectory() as tmp:
        model_dir = write_random_model(cfg, Path(tmp) / "llama-8b", seed=0)
        pages = 64 * (-(-(context + 1) // PAGE)) + 16
        with LLM(str(model_dir), dtype="bfloat16", device="cuda:0", max_num_seqs=64, max_model_len=context + 1,
                 block_size=PAGE, max_num_batched_tokens=8192, num_gpu_blocks=pages) as llm:
            runner = llm.engine.runner
            for group in runner.cache.groups:
                group.pool.normal_(0.0, 0.5)
            out["cache_gb"] = pages * runner.cache.bytes_per_page() / 1e9
            for batch in (1, 8, 64):
                value, ms, _ = _decode_rate(runner, Sampler(0), greedy, batch, start_len, steps, warmup, cfg["vocab_size"])
                nbytes = numbers["weight_bytes"] + batch * (start_len + warmup + steps / 2) * numbers["kv_bytes_per_token"]
                out[f"decode_b{batch}_tok_s"] = value
                out[f"decode_b{batch}_ms"] = ms
                out[f"decode_b{batch}_hbm_frac"] = nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]
    return out


def run_workloads(args) -> dict:
    """The two larger configurations of the reference's benchmark set; a failure is reported, not raised."""
    peaks = measured_peaks()
    results = {}
    for name, fn in (("3b", workload_3b), ("8b", workload_8b)):
        if args.workload not in ("all", name):
            continue
        try:
            started = time.perf_counter()
            results[name] = {**fn(args, peaks), "took_s": round(time.perf_counter() - started, 1)}
        except Exception as error:  # noqa: BLE001
            results[name] = {"failed": f"{type(error).__name__}: {str(error)[:200]}"}
    return results


def run_reference(args) -> dict:
    """The unmodified reference through its own public API: `baseline/_ref` holds its package (put there by
    `baseline/install_reference.py`), `baseline/reference_arm.py` drives it.  Whatever keeps it from running
    here (the package missing, a dependency missing on this box, its Triton kernels failing to compile for
    this GPU) is printed as the reason for `unavailable`."""
    if not (ROOT / "baseline" / "_ref" / "liteinfer").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref holds no copy of the reference package "
                "(run python baseline/install_reference.py <reference checkout> where one exists)"}
    try:
        sys.path.insert(0, str(ROOT / "baseline"))
        from reference_arm import run  # noqa: PLC0415
        helpers = {"ClockSampler": ClockSampler, "peaks": measured_peaks(), "baseline_toks": BASELINE_DECODE_B8_TOKS}
        return run(args, LLAMA_1B, CONTEXT, PAGE, helpers)
    except Exception as error:  # noqa: BLE001
        import traceback
        traceback.print_exc()
        return {"impl": "reference", "unavailable": f"{type(error).__name__}: {str(error)[:300]}"}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    parser.add_argument("--section", default="all", choices=["all", "decode", "prefill"],
                        help="run one part only (for profiling); the JSON line then lacks the other parts")
    parser.add_argument("--batch", type=int, default=8, help="decode batch of --section decode")
    parser.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="layer sizes: Llama 3.2 1B (the contract's), 3B or 3.1 8B")
    parser.add_argument("--workload", default="none", choices=["none", "3b", "8b", "all"],
                        help="run the reference's larger configurations instead (64 requests under continuous batching "
                             "at the 3B sizes; decode at a context of 8,192 at the 8B sizes) and print their line")
    parser.add_argument("--no-workloads", action="store_true",
                        help="leave the 3B and 8B configurations out of the default run (they add about 80 s)")
    args = parser.parse_args()
    if args.gpus != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print("liteinfer_b200 is a single-GPU engine: bench.py runs at --gpus 1 only")
        return 2
    if args.workload != "none" and args.impl == "ours":
        print(json.dumps({"impl": "ours", "workloads": run_workloads(args)}))
        return 0
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
