"""Weights: bound by name, converted to the engine dtype, one error for every mismatch; the random-weights mode."""

from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import tiny_configs
from liteinfer_b200.weights.loader import WeightsError, load_model
from liteinfer_b200.weights.random_init import random_tensors, write_random_model


def test_random_weights_mode_writes_a_model_folder(tmp_path):
    config, seed, _ = tiny_configs.ALL["tiny_a"]
    folder = write_random_model(config, tmp_path / "m", seed)
    assert (folder / "config.json").is_file() and (folder / "model.safetensors").is_file()
    tensors = load_file(str(folder / "model.safetensors"))
    assert "lm_head.weight" not in tensors                   # tied: the head is not stored
    assert tensors["model.embed_tokens.weight"].shape == (512, 64)
    assert tensors["model.layers.1.mlp.gate_proj.weight"].shape == (176, 64)
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    w = tensors["model.layers.0.self_attn.q_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = tensors["model.norm.weight"].float()
    assert abs(float(n.mean()) - 1.0) < 0.01 and 0.003 < float(n.std()) < 0.02
    again = random_tensors(config, seed)
    assert all(torch.equal(again[k], tensors[k]) for k in tensors)
    other = random_tensors(config, seed + 1)
    assert not torch.equal(other["model.norm.weight"], tensors["model.norm.weight"])
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["LlamaForCausalLM"]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_loader_binds_by_name_in_the_engine_dtype(model_dirs, dtype):
    model, config = load_model(model_dirs["tiny_b"], dtype, "cpu")
    stored = load_file(str(model_dirs["tiny_b"] / "model.safetensors"))
    layer = model.layers[2].parts
    q, k, v = (stored[f"model.layers.2.self_attn.{n}_proj.weight"] for n in "qkv")
    assert torch.equal(layer["mixer"].qkv_weight, torch.cat([q, k, v]).to(dtype))
    assert layer["mixer"].qkv_weight.dtype == dtype
    assert torch.equal(model.head.weight, stored["lm_head.weight"].to(dtype))
    assert model.head.weight.data_ptr() != model.embedding.weight.data_ptr()
    assert config.num_hidden_layers == 3


def test_a_tied_head_reads_the_embedding(model_dirs, tmp_path):
    model, _ = load_model(model_dirs["tiny_a"], torch.bfloat16, "cpu")
    assert model.head.weight.data_ptr() == model.embedding.weight.data_ptr()
    # A tied checkpoint that stores the head as well is still read (the stored head is not used).
    tensors = load_file(str(model_dirs["tiny_a"] / "model.safetensors"))
    tensors["lm_head.weight"] = torch.zeros_like(tensors["model.embed_tokens.weight"])
    (tmp_path / "config.json").write_text((model_dirs["tiny_a"] / "config.json").read_text())
    save_file(tensors, str(tmp_path / "model.safetensors"))
    model, _ = load_model(tmp_path, torch.bfloat16, "cpu")
    assert torch.equal(model.head.weight, tensors["model.embed_tokens.weight"])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(model_dirs, tmp_path):
    tensors = load_file(str(model_dirs["tiny_b"] / "model.safetensors"))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.extra.weight"] = torch.zeros(3)
    tensors["model.norm.weight"] = torch.zeros(95, dtype=torch.bfloat16)
    tensors["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(48, 95, dtype=torch.bfloat16)
    (tmp_path / "config.json").write_text((model_dirs["tiny_b"] / "config.json").read_text())
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightsError) as info:
        load_model(tmp_path, torch.bfloat16, "cpu")
    error = info.value
    assert set(error.missing) == {"model.layers.1.mlp.up_proj.weight", "lm_head.weight"}
    assert error.unexpected == ["model.layers.0.extra.weight"]
    assert {w[0] for w in error.wrong_shape} == {"model.norm.weight", "model.layers.2.self_attn.k_proj.weight"}
    text = str(error)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (2)", "model.norm.weight is [95], expected [96]"):
        assert needle in text


def test_no_safetensors_is_file_not_found(tmp_path, model_dirs):
    (tmp_path / "config.json").write_text((model_dirs["tiny_a"] / "config.json").read_text())
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_model(tmp_path, torch.bfloat16, "cpu")


def test_float32_checkpoints_are_converted(tmp_path):
    config, seed, _ = tiny_configs.ALL["tiny_c"]
    folder = write_random_model(config, tmp_path / "m", seed, dtype=torch.float32)
    model, _ = load_model(folder, torch.bfloat16, "cpu")
    assert model.embedding.weight.dtype == torch.bfloat16
    assert model.layers[0].parts["mixer"].qkv_bias is not None and model.layers[0].parts["feed_forward"].down_bias is not None
