"""The engine at the widths of Llama 3.2 1B (hidden 2048, 32 heads / 8 KV heads of 64, intermediate 8192,
vocabulary 128,256, llama3 rotary scaling), with two layers so that it stays quick: the kernels that only real
sizes reach (the tcgen05 attention, the library and weight-streaming products, the split arg-max) inside the
whole model, in float32 and bfloat16, against the plain implementation."""

from __future__ import annotations

import pytest
import torch

import plain_llama
import replay_harness as rh
import tiny_configs

pytestmark = pytest.mark.gpu

WIDE = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 128256, "hidden_size": 2048, "intermediate_size": 8192,
    "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "max_position_embeddings": 131072, "hidden_act": "silu",
}


@pytest.fixture(scope="module")
def wide_model(tmp_path_factory):
    from liteinfer_b200.weights.random_init import write_random_model

    return write_random_model(WIDE, tmp_path_factory.mktemp("wide") / "wide", seed=4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_model_replay(wide_model, dtype):
    from liteinfer_b200 import ops
    from liteinfer_b200.config.engine_config import parse_dtype
    from liteinfer_b200.engine.loading import build_runner

    requests = {f"r{i}": tiny_configs.prompt(WIDE["vocab_size"], n, i) for i, n in enumerate((300, 70, 9))}
    exact = rh.expected_logits(wide_model, requests, device="cuda")
    trace = rh.Trace()
    rh.whole(trace, {"r0": requests["r0"]})
    rh.mixed(trace, requests, chunk=128, decode_tail=6)
    runner = build_runner(wide_model, parse_dtype(dtype), "cuda:0", 16, -(-trace.max_tokens // 16), 4)
    if dtype == "bfloat16":
        runner.enable_decode_graphs(4, 512)
    results = rh.run_in_process(runner, trace)
    worst, where = rh.worst_error(results, rh.gather_expected(trace, exact))
    assert ops.gemm_error_flag("cuda:0") == 0
    if dtype == "float32":
        assert worst < 1e-4, f"worst difference {worst} at step {where}"
    else:
        plain_bf16 = rh.expected_logits(wide_model, requests, dtype=torch.bfloat16, device="cuda")
        drift = max(float((plain_bf16[k] - exact[k]).abs().max()) for k in exact)
        assert worst <= 2 * drift, f"worst difference {worst} at step {where}; plain bfloat16 drifts {drift}"


def test_wide_model_greedy_tokens(wide_model):
    from liteinfer_b200 import LLM, SamplingParams

    prompt = tiny_configs.prompt(WIDE["vocab_size"], 40, 7)
    raw, weights = plain_llama.read_model(wide_model)
    with LLM(str(wide_model), dtype="float32", max_num_seqs=2, max_model_len=128) as llm:
        got = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))[0].token_ids
    assert got == plain_llama.greedy(raw, weights, prompt, 4, device="cuda")
