"""Configuration: config.json keys, defaults, refusals, the architecture registry, engine knobs."""

from __future__ import annotations

import json

import pytest
import torch

import tiny_configs
from liteinfer_b200.config.engine_config import EngineConfig, parse_dtype
from liteinfer_b200.config.model_config import ConfigError, LlamaConfig
from liteinfer_b200.config.registry import ARCHITECTURES, resolve, resolve_model_dir


def test_llama_config_reads_its_keys():
    cfg = LlamaConfig.from_dict(tiny_configs.TINY_B)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers) == (1000, 96, 320, 3)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.num_kv_groups) == (6, 3, 16, 2)
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 500000.0 and not cfg.tie_word_embeddings
    assert cfg.rope_scaling.rope_type == "llama3" and cfg.rope_scaling.factor == 32.0
    assert cfg.rope_scaling.original_max_position_embeddings == 64


def test_defaults_follow_the_architecture():
    raw = {k: v for k, v in tiny_configs.TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "hidden_act")}
    cfg = LlamaConfig.from_dict(raw)
    assert cfg.num_key_value_heads == cfg.num_attention_heads      # no grouping unless said
    assert cfg.head_dim == cfg.hidden_size // cfg.num_attention_heads
    assert cfg.hidden_act == "silu" and cfg.rope_scaling.rope_type == "default"
    assert not cfg.attention_bias and not cfg.mlp_bias


def test_rope_parameters_spelling_is_read_too():
    raw = dict(tiny_configs.TINY_B)
    scaling = raw.pop("rope_scaling")
    theta = raw.pop("rope_theta")
    raw["rope_parameters"] = {**scaling, "rope_theta": theta}
    assert LlamaConfig.from_dict(raw) == LlamaConfig.from_dict(tiny_configs.TINY_B)


def test_round_trip_through_config_json():
    for cfg, _, _ in tiny_configs.ALL.values():
        typed = LlamaConfig.from_dict(cfg)
        assert LlamaConfig.from_dict(json.loads(json.dumps(typed.to_dict()))) == typed


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads"])
def test_a_missing_size_is_refused(key):
    raw = {k: v for k, v in tiny_configs.TINY_A.items() if k != key}
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(raw)


def test_options_a_config_leaves_out_take_the_architectures_defaults():
    """No size has a default; the options do, as through the reference's configuration class: KV heads = heads,
    head size = hidden / heads, rotary base 10,000 unscaled, eps 1e-6, untied head, silu, no biases."""
    raw = {k: tiny_configs.TINY_A[k] for k in ("architectures", "vocab_size", "hidden_size", "intermediate_size",
                                               "num_hidden_layers", "num_attention_heads")}
    cfg = LlamaConfig.from_dict(raw)
    assert cfg.num_key_value_heads == cfg.num_attention_heads and cfg.head_dim == cfg.hidden_size // cfg.num_attention_heads
    assert cfg.rope_theta == 10000.0 and cfg.rope_scaling.rope_type == "default" and cfg.rms_norm_eps == 1e-6
    assert not cfg.tie_word_embeddings and cfg.hidden_act == "silu" and not cfg.attention_bias and not cfg.mlp_bias


@pytest.mark.parametrize("change,match", [
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"), ({"hidden_act": "swish9"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_type"), ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "original_max_position_embeddings"),
])
def test_values_the_engine_cannot_run_are_refused(change, match):
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_dict({**tiny_configs.TINY_A, **change})


def test_registry_maps_the_name_to_the_model():
    arch, cfg = resolve(tiny_configs.TINY_A)
    assert arch.name == "LlamaForCausalLM" and arch is ARCHITECTURES["LlamaForCausalLM"]
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 2 and [e.layer for e in spec.schedule] == [0, 1]
    assert spec.tied == {"lm_head.weight": "model.embed_tokens.weight"}
    assert spec.layers[1].prefixes["mixer"] == "model.layers.1.self_attn."
    assert spec.layers[0].parts["mixer"].params["kv_heads"] == 2
    untied = arch.build_spec(LlamaConfig.from_dict(tiny_configs.TINY_B))
    assert untied.tied == {}


def test_registry_refusals(tmp_path):
    with pytest.raises(ConfigError, match="unsupported architecture 'GPT9'.*LlamaForCausalLM"):
        resolve({**tiny_configs.TINY_A, "architectures": ["GPT9"]})
    with pytest.raises(ConfigError, match="architectures"):
        resolve({k: v for k, v in tiny_configs.TINY_A.items() if k != "architectures"})
    with pytest.raises(FileNotFoundError, match="config.json"):
        resolve_model_dir(tmp_path)


def test_engine_config_checks_and_budget():
    cfg = EngineConfig(model="m")
    assert cfg.dtype == torch.bfloat16 and cfg.block_size == 16 and cfg.max_num_seqs == 32
    assert cfg.token_budget == 32 * 4096
    assert EngineConfig(model="m", max_num_batched_tokens=64).token_budget == 64
    assert EngineConfig(model="m", dtype="float32").dtype == torch.float32
    for bad in ({"max_num_seqs": 0}, {"max_model_len": 0}, {"block_size": 0}, {"max_num_batched_tokens": 8},
                {"max_waiting_seqs": 0}, {"paged_decode_splits": 0}, {"gpu_memory_utilization": 0.0},
                {"gpu_memory_utilization": 1.5}, {"attn_implementation": "sdpa"}, {"dtype": "float16"},
                {"num_gpu_blocks": 0}):
        with pytest.raises(ValueError):
            EngineConfig(model="m", **bad)
    assert parse_dtype("bf16") == torch.bfloat16


def test_cuda_and_cuda_0_are_one_device():
    """Scratch buffers and error flags are kept per device; `cuda` must find what `cuda:0` left."""
    import torch

    from liteinfer_b200.ops import normalise_device

    assert normalise_device("cuda") == normalise_device("cuda:0") == torch.device("cuda", 0)
    assert normalise_device("cuda:1") == torch.device("cuda", 1) and normalise_device("cpu") == torch.device("cpu")
