"""Generation through the entry points on the GPU: greedy against the plain implementation, long decoding,
the first tokens of a sequence, sampling through the kernel, the command line."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_llama
import replay_harness as rh
import tiny_configs

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_d", "tiny_e"])
def test_greedy_generation_float32_equals_plain(model_dirs, name):
    from liteinfer_b200 import LLM, SamplingParams

    config, _, page = tiny_configs.ALL[name]
    prompts = [tiny_configs.prompt(config["vocab_size"], n, i) for i, n in enumerate((1, 9, 40, 17))]
    raw, weights = plain_llama.read_model(model_dirs[name])
    expected = [plain_llama.greedy(raw, weights, p, 8, device="cuda") for p in prompts]
    with LLM(str(model_dirs[name]), dtype="float32", block_size=page, max_num_seqs=3, max_model_len=128,
             max_num_batched_tokens=24) as llm:
        outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
        assert llm.engine.runner.graph_replays > 0            # decode steps went through CUDA graphs
    assert [o.token_ids for o in outs] == expected


@pytest.mark.parametrize("name", ["tiny_b", "tiny_d", "tiny_e"])
def test_greedy_generation_bfloat16_picks_a_top_token_of_the_plain_run(model_dirs, name):
    """In bfloat16 one rounding can flip an arg-max between near-equal logits (random weights give flat
    logits), so the check is on logits, along the engine's own tokens: what the engine picked is, in the
    plain 32-bit run, the maximum or within bfloat16's drift of it, at every step."""
    from liteinfer_b200 import LLM, SamplingParams

    config, _, page = tiny_configs.ALL[name]
    prompt = tiny_configs.prompt(config["vocab_size"], 30, 5)
    raw, weights = plain_llama.read_model(model_dirs[name])
    exact = plain_llama.forward(raw, weights, prompt, device="cuda")
    drift = float((plain_llama.forward(raw, weights, prompt, torch.bfloat16, "cuda") - exact).abs().max())
    with LLM(str(model_dirs[name]), dtype="bfloat16", block_size=page, max_num_seqs=2, max_model_len=128) as llm:
        got = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))[0].token_ids
    assert len(got) == 12
    tokens = list(prompt)
    for step, token in enumerate(got):
        logits = plain_llama.forward(raw, weights, tokens, device="cuda")[-1]
        assert float(logits.max() - logits[token]) <= 4 * drift, f"step {step}: token {token} is not near the top"
        tokens.append(token)


def test_long_decoding_and_first_tokens(model_dirs, tmp_path):
    """A request of two tokens decoded for 400 steps: the first tokens of a sequence, then many pages, one token at
    a time, in float32 against the plain implementation's logits at every position."""
    config, _, page = tiny_configs.ALL["tiny_d"]
    tokens = tiny_configs.prompt(config["vocab_size"], 402, 9)
    expected = rh.expected_logits(model_dirs["tiny_d"], {"x": tokens}, device="cuda")
    trace = rh.Trace()
    trace.add([("d-x", tokens[:2], [0, 1])])
    for i in range(2, len(tokens)):
        trace.add([("d-x", tokens[i:i + 1], [0])], end=["d-x"] if i == len(tokens) - 1 else [])
    for dtype, bound in (("float32", 3e-5), ("bfloat16", None)):
        results = rh.run_program(trace, model_dirs["tiny_d"], dtype, tmp_path / dtype, config["vocab_size"], page)
        worst, where = rh.worst_error(results, rh.gather_expected(trace, expected))
        if bound is None:
            plain_bf16 = rh.expected_logits(model_dirs["tiny_d"], {"x": tokens}, dtype=torch.bfloat16, device="cuda")
            bound = 2 * float((plain_bf16["x"] - expected["x"]).abs().max())
        assert worst <= bound, f"{dtype}: worst difference {worst} at step {where}"


def test_sampling_through_the_engine_is_seeded_and_spread(model_dirs):
    from liteinfer_b200 import LLM, SamplingParams

    config, _, page = tiny_configs.ALL["tiny_a"]
    prompt = tiny_configs.prompt(config["vocab_size"], 6, 0)
    with LLM(str(model_dirs["tiny_a"]), dtype="bfloat16", block_size=page, max_num_seqs=8, max_model_len=64) as llm:
        params = SamplingParams(temperature=1.0, top_k=50, top_p=0.95, max_tokens=10, seed=11, ignore_eos=True)
        a = llm.generate([prompt], params)[0].token_ids
        b = llm.generate([prompt], SamplingParams(temperature=1.0, top_k=50, top_p=0.95, max_tokens=10, seed=11,
                                                  ignore_eos=True))[0].token_ids
        c = llm.generate([prompt], SamplingParams(temperature=1.0, top_k=50, top_p=0.95, max_tokens=10, seed=12,
                                                  ignore_eos=True))[0].token_ids
        many = llm.generate([prompt] * 6, SamplingParams(temperature=1.5, max_tokens=10, ignore_eos=True))
    assert a == b and a != c
    assert len({tuple(o.token_ids) for o in many}) > 1     # requests sharing one params object draw apart


def test_command_line_generates(model_dirs):
    config, _, page = tiny_configs.ALL["tiny_a"]
    prompt = tiny_configs.prompt(config["vocab_size"], 5, 0)
    raw, weights = plain_llama.read_model(model_dirs["tiny_a"])
    cmd = [sys.executable, "-m", "liteinfer_b200", "generate", "--model", str(model_dirs["tiny_a"]),
           "--prompt-ids", " ".join(map(str, prompt)), "--temperature", "0", "--max-tokens", "5", "--dtype", "float32",
           "--block-size", str(page), "--max-model-len", "64", "--max-num-seqs", "2"]
    done = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    record = json.loads(done.stdout.strip().splitlines()[-1])
    assert record["token_ids"] == plain_llama.greedy(raw, weights, prompt, 5) and record["finish_reason"] == "length"
