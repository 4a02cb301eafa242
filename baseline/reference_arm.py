"""The reference arm of bench.py: the unmodified reference package, driven through its own public API.

Nothing of liteinfer_b200 runs inside the timed regions: the model folder is
the one the random-weights mode writes (plus a word-level tokenizer, which the
reference's `LLM` wants in the folder: one word per token id, as the
reference's own test fixture builds it, tests/integration/tiny_llama.py:41-49),
and from there on everything is `baseline/_ref/liteinfer`: its loader, cache,
Triton paged attention, decode graphs, sampler and engine loop with their
defaults.

Two measurements, the same two as for this repository's arm:

  device-timed   K decode steps of `ModelRunner.execute` (liteinfer/engine/model_runner.py:137-172) at
                 batch 8 with contexts just below the benchmark context, each followed by the reference's
                 `Sampler` and one `.tolist()`, between CUDA events, after W warm-up steps (the first of
                 which capture the decode graph, liteinfer/engine/cuda_graphs.py:151-181)
  end to end     the same batch through `LLM.generate` (liteinfer/llm.py:14-68): the time between the ends
                 of consecutive decode steps of its engine loop, host strings in, host tokens out
"""

from __future__ import annotations

import json
import statistics
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent


def write_tokenizer(model_dir: Path, vocab_size: int) -> None:
    """A word-level tokenizer with one word per token id ("t17" is id 17; ids 0 and 1 are "<unk>" and "<eos>")."""
    from tokenizers import Tokenizer as HFTokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import WhitespaceSplit
    from transformers import PreTrainedTokenizerFast

    vocab = {"<unk>": 0, "<eos>": 1, **{f"t{i}": i for i in range(2, vocab_size)}}
    tok = HFTokenizer(WordLevel(vocab=vocab, unk_token="<unk>"))
    tok.pre_tokenizer = WhitespaceSplit()
    PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<eos>", unk_token="<unk>").save_pretrained(str(model_dir))


def as_text(token_ids: list[int]) -> str:
    return " ".join(f"t{i}" for i in token_ids)


def _decode_rate(runner, sampler_cls, seq_cls, params, batch: int, start_len: int, steps: int, warmup: int,
                 vocab: int, budget: int):
    """(tokens/s, ms per step) of `steps` decode steps of the reference's step function at `batch`."""
    import torch

    g = torch.Generator().manual_seed(batch)
    seqs = [seq_cls(request_id=f"b{batch}-{i}", prompt="",
                    prompt_token_ids=torch.randint(2, vocab, (start_len,), generator=g).tolist(),
                    sampling_params=params) for i in range(batch)]
    sampler = sampler_cls()
    # The prompts, a token budget's worth per step (as its scheduler would cut them).
    for seq in seqs:
        while not seq.is_prompt_computed:
            runner.execute([seq], [min(budget, seq.num_uncomputed_tokens)])
        seq.output_token_ids.append(int(torch.randint(2, vocab, (1,), generator=g)))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(warmup + steps):
        if i == warmup:
            torch.cuda.synchronize()
            start.record()
        logits = runner.execute(seqs, [1] * batch)
        sampled = sampler(logits, [params] * batch)
        for seq, token in zip(seqs, sampled.tolist()):
            seq.output_token_ids.append(token)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    for seq in seqs:
        runner.release_sequence(seq)
    return batch / ms * 1e3, ms


def run(args, shape: dict, context: int, page: int, helpers: dict) -> dict:
    """`helpers`: bench.py's ClockSampler class, its peaks and the published baseline figure."""
    import tempfile

    import torch

    from liteinfer_b200.weights.random_init import write_random_model

    sys.path.insert(0, str(HERE / "_ref"))
    import liteinfer  # the reference package
    from liteinfer import LLM, SamplingParams
    from liteinfer.config import EngineConfig
    from liteinfer.engine.model_runner import ModelRunner
    from liteinfer.engine.sequence import Sequence
    from liteinfer.sampling.sampler import Sampler

    if not str(Path(liteinfer.__file__).resolve()).startswith(str(HERE / "_ref")):
        raise RuntimeError(f"the reference was imported from {liteinfer.__file__}, not from baseline/_ref")

    cfg = dict(shape)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    device = getattr(args, "device", None) or "cuda"
    steps, warmup, batch = args.steps, max(3, args.warmup), 8
    vocab, hidden = cfg["vocab_size"], cfg["hidden_size"]
    budget = 8192
    engine_kwargs = dict(dtype=torch.bfloat16, device=device, max_num_seqs=64, max_model_len=context + 1,
                         block_size=page, max_num_batched_tokens=budget, gpu_memory_utilization=0.5)
    params = SamplingParams(temperature=0.0, max_tokens=warmup + steps + 1, ignore_eos=True)
    decode_start = context - (warmup + steps) - 1
    on_cuda = torch.device(device).type == "cuda"

    with tempfile.TemporaryDirectory() as tmp:
        model_dir = write_random_model(cfg, Path(tmp) / "llama", seed=0)
        write_tokenizer(model_dir, vocab)

        # ---- the step function alone, device-timed
        runner = ModelRunner(EngineConfig(model=str(model_dir), **engine_kwargs))
        runner.load_model()
        points = {}
        prefill = None
        if on_cuda:
            g = torch.Generator().manual_seed(7)
            tokens = 2048
            prompt = torch.randint(2, vocab, (tokens,), generator=g).tolist()
            times = []
            for i in range(6):
                seq = Sequence(request_id=f"prefill-{i}", prompt="", prompt_token_ids=prompt, sampling_params=params)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                a.record()
                runner.execute([seq])
                b.record()
                torch.cuda.synchronize()
                runner.release_sequence(seq)
                if i >= 3:
                    times.append(a.elapsed_time(b))
            prefill_ms = statistics.median(times)
            layers = cfg["num_hidden_layers"]
            q = cfg["num_attention_heads"] * cfg["head_dim"]
            kv = cfg["num_key_value_heads"] * cfg["head_dim"]
            inter = cfg["intermediate_size"]
            linear_params = layers * (hidden * (q + 2 * kv) + q * hidden + 3 * hidden * inter)
            flops = (2 * linear_params * tokens + layers * 4 * q * tokens * (tokens + 1) / 2 + 2 * hidden * vocab)
            prefill = {"value": tokens / prefill_ms * 1e3, "tokens": tokens, "ms": prefill_ms,
                       "frac": flops / (prefill_ms * 1e-3) / (helpers["peaks"]["bf16_tflops_burst"] * 1e12)}
            clocks = helpers["ClockSampler"]()
            clocks.start()
            value, ms = _decode_rate(runner, Sampler, Sequence, params, batch, decode_start, steps, warmup, vocab, budget)
            clock_record = clocks.stop()
            for width in (1, 64):
                points[f"decode_b{width}"], _ = _decode_rate(runner, Sampler, Sequence, params, width, decode_start,
                                                             steps, warmup, vocab, budget)
            weight_bytes = (linear_params + hidden * vocab + (2 * layers + 1) * hidden) * 2
            kv_bytes = batch * (decode_start + warmup + steps / 2) * layers * 2 * kv * 2
            achieved = (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9
            peak = helpers["peaks"]["hbm_gbs"]
            roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                        "of": helpers["peaks"]["source"]}
        else:       # a CPU run only checks that the arm drives the reference; it times nothing
            value = ms = 0.0
            clock_record, roofline = {}, {}
        attention = runner.attn_implementation
        graphs = runner.captured_decode_widths
        del runner
        if on_cuda:
            torch.cuda.empty_cache()

        # ---- end to end through LLM.generate: host strings in, host tokens out
        g = torch.Generator().manual_seed(11)
        prompts = [as_text(torch.randint(2, vocab, (decode_start,), generator=g).tolist()) for _ in range(batch)]
        llm = LLM(str(model_dir), **engine_kwargs)
        ends: list[tuple[float, str, int]] = []
        llm.stats.on_step(lambda step: ends.append((time.perf_counter(), step.phase.value, step.num_seqs)))
        llm.generate(prompts, params)          # once untimed: its decode graphs are captured here
        ends.clear()
        outs = llm.generate(prompts, params)
        assert all(len(o.token_ids) == warmup + steps + 1 for o in outs), [len(o.token_ids) for o in outs]
        gaps = [b[0] - a[0] for a, b in zip(ends, ends[1:]) if b[1] == "decode" and b[2] == batch][-steps:]
        e2e_ms = sum(gaps) / len(gaps) * 1e3
        llm.close()

    e2e = {"value": batch / e2e_ms * 1e3, "unit": "tokens/s", "ms_per_step": e2e_ms,
           # per decode step the reference copies tokens and positions (int64), write slots, the slot table of
           # every context position (int64) and the context lengths (liteinfer/engine/model_runner.py:215-244)
           "h2d_bytes_per_step": 8 * 2 * batch + 8 * batch + 8 * batch * context + 4 * batch,
           "d2h_bytes_per_step": 8 * batch}
    return {
        "metric": "decode tok/s at batch 8 (llama 3.2 1b shape)", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / helpers["baseline_toks"] if value and not args.layers else None, "dtype": "bf16",
        "data": "synthetic ids, random weights", "impl": "reference",
        "config": {"model": "llama-3.2-1b-shape", "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "hidden": hidden, "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": vocab,
                   "global_batch": batch, "seq_len": context, "page_size": page, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (weights and cache are read every step)",
                   "reference_version": getattr(liteinfer, "__version__", "?"), "attention": attention,
                   "graph_widths": len(graphs)},
        "clocks": clock_record, "e2e": e2e, "gpu_launches": None,
        "prefill": prefill, "roofline": roofline, "points": points,
    }


if __name__ == "__main__":
    print(json.dumps({"note": "run through bench.py --impl reference"}))
