"""The plain implementation against the reference's own logits (tests/golden) and against itself."""

from __future__ import annotations

from pathlib import Path

import pytest
import torch

import plain_llama
import tiny_configs

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", list(tiny_configs.ALL))
def test_plain_matches_reference_golden(tmp_path, name):
    """tests/golden/<name>.pt holds logits of liteinfer's LlamaForCausalLM (float32, CPU, eager) on the
    model that the random-weights mode writes for this configuration and seed in float32."""
    from liteinfer_b200.weights.random_init import write_random_model

    config, seed, _ = tiny_configs.ALL[name]
    golden = torch.load(GOLDEN / f"{name}.pt")
    assert golden["seed"] == seed
    model_dir = write_random_model(config, tmp_path / name, seed, dtype=torch.float32)
    raw, weights = plain_llama.read_model(model_dir)
    assert torch.equal(plain_llama.rope_inverse_frequencies(raw), golden["inv_freq"])
    logits = plain_llama.forward(raw, weights, golden["tokens"])
    torch.testing.assert_close(logits, golden["logits"], rtol=1e-5, atol=1e-5)


def test_a_prefix_does_not_see_what_follows(model_dirs):
    raw, weights = plain_llama.read_model(model_dirs["tiny_b"])
    tokens = tiny_configs.prompt(raw["vocab_size"], 30, 0)
    full = plain_llama.forward(raw, weights, tokens)
    part = plain_llama.forward(raw, weights, tokens[:11])
    torch.testing.assert_close(full[:11], part, rtol=1e-5, atol=1e-6)


def test_window_attention_of_the_plain_implementation():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(12, 2, 8, generator=g) for _ in range(3))
    full = plain_llama.causal_attention(q, k, v, 0.3)
    wide = plain_llama.causal_attention(q, k, v, 0.3, window=12)
    torch.testing.assert_close(full, wide)
    narrow = plain_llama.causal_attention(q, k, v, 0.3, window=1)
    torch.testing.assert_close(narrow, v)      # each query sees only itself


def test_rope_pairs_are_half_split():
    cos, sin = plain_llama.rope_tables(torch.tensor([0.5, 0.25]), torch.tensor([3]), torch.float32)
    x = torch.arange(4.0).view(1, 1, 4)
    y = plain_llama.apply_rope(x, cos, sin)[0, 0]
    a0, a1 = 3 * 0.5, 3 * 0.25
    want = torch.tensor([0 * torch.cos(torch.tensor(a0)) - 2 * torch.sin(torch.tensor(a0)),
                         1 * torch.cos(torch.tensor(a1)) - 3 * torch.sin(torch.tensor(a1)),
                         2 * torch.cos(torch.tensor(a0)) + 0 * torch.sin(torch.tensor(a0)),
                         3 * torch.cos(torch.tensor(a1)) + 1 * torch.sin(torch.tensor(a1))])
    torch.testing.assert_close(y, want)
