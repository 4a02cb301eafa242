"""Trace replay on the GPU through bin/trace_run, in 32-bit and in bfloat16, against the plain implementation.

One child process per (configuration, dtype) replays, as one long trace: every
request alone and whole; most of it in one step and the last 32 tokens one by
one; portions of changing size down to two tokens; and up to four live requests
mixed, with a pool so small that pages are used again.
"""

from __future__ import annotations

import pytest
import torch

import replay_harness as rh
import tiny_configs

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": (5, 17, 33, 70, 129), "tiny_b": (1, 9, 40, 64, 100), "tiny_c": (3, 50, 66),
           "tiny_d": (2, 70, 130, 300), "tiny_e": (3, 66, 140, 260)}


def _requests(vocab: int, lengths) -> dict[str, list[int]]:
    return {f"r{i}": tiny_configs.prompt(vocab, n, i) for i, n in enumerate(lengths)}


def _trace(requests) -> rh.Trace:
    trace = rh.Trace()
    rh.whole(trace, requests)
    rh.tail_decoded(trace, requests)
    rh.portions(trace, requests)
    rh.mixed(trace, requests)
    return trace


@pytest.mark.parametrize("name", list(LENGTHS))
def test_float32_replay_matches_plain(model_dirs, tmp_path, name):
    config, _, page = tiny_configs.ALL[name]
    requests = _requests(config["vocab_size"], LENGTHS[name])
    trace = _trace(requests)
    expected = rh.gather_expected(trace, rh.expected_logits(model_dirs[name], requests))
    results = rh.run_program(trace, model_dirs[name], "float32", tmp_path / "out", config["vocab_size"], page)
    worst, where = rh.worst_error(results, expected)
    # Logits are O(1); float32 sums over at most a few hundred terms.
    assert worst < 2e-5, f"worst difference {worst} at step {where}: {trace.steps[where]}"


@pytest.mark.parametrize("name", list(LENGTHS))
def test_float32_cuts_agree_bit_for_bit(model_dirs, tmp_path, name):
    """The 32-bit kernels add in an order that depends on a token's position only, so every
    way of cutting gives the same bits."""
    config, _, page = tiny_configs.ALL[name]
    requests = _requests(config["vocab_size"], LENGTHS[name])
    trace = _trace(requests)
    results = rh.run_program(trace, model_dirs[name], "float32", tmp_path / "out", config["vocab_size"], page)
    seen: dict[tuple[str, int], torch.Tensor] = {}
    for wanted, got in zip(trace.wanted, results):
        for row, (rid, pos) in enumerate(wanted):
            key = (rid.split("-", 1)[1], pos)
            if key in seen:
                assert torch.equal(seen[key], got[row]), f"{rid} position {pos} differs between cuts"
            else:
                seen[key] = got[row]


@pytest.mark.parametrize("name", list(LENGTHS))
def test_bfloat16_replay_stays_within_bfloat16_drift(model_dirs, tmp_path, name):
    """bfloat16 against the 32-bit plain run: no further off than twice what the plain
    implementation itself drifts when run in bfloat16 (the reference's own criterion,
    tests/integration/test_token_budget_gpu.py:70-77)."""
    config, _, page = tiny_configs.ALL[name]
    requests = _requests(config["vocab_size"], LENGTHS[name])
    trace = _trace(requests)
    exact = rh.expected_logits(model_dirs[name], requests)
    plain_bf16 = rh.expected_logits(model_dirs[name], requests, dtype=torch.bfloat16)
    drift = max(float((plain_bf16[k] - exact[k]).abs().max()) for k in exact)
    results = rh.run_program(trace, model_dirs[name], "bfloat16", tmp_path / "out", config["vocab_size"], page)
    worst, where = rh.worst_error(results, rh.gather_expected(trace, exact))
    assert worst <= 2 * drift, f"worst difference {worst} at step {where}; plain bfloat16 drifts {drift}"
