"""The step function, the cache and the batch builder, driven on a CPU with the stand-in kernels.

What is under test here is the host side: positions, block tables, page reuse,
the order of the returned rows.  The same traces run on the GPU through
bin/trace_run in test_replay_gpu.py.
"""

from __future__ import annotations

import pytest
import torch

import replay_harness as rh
import tiny_configs


def _requests(vocab: int, lengths, seed0: int = 0) -> dict[str, list[int]]:
    return {f"r{i}": tiny_configs.prompt(vocab, n, seed0 + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("name,lengths", [("tiny_a", (5, 17, 33, 70)), ("tiny_b", (1, 9, 40, 64, 100)),
                                           ("tiny_c", (3, 50)), ("tiny_d", (2, 70, 130))])
def test_all_cuts_match_plain_on_cpu(cpu_kernels, model_dirs, name, lengths):
    from liteinfer_b200.engine.loading import build_runner

    config, _, page = tiny_configs.ALL[name]
    requests = _requests(config["vocab_size"], lengths)
    expected = rh.expected_logits(model_dirs[name], requests)
    trace = rh.Trace()
    rh.whole(trace, requests)
    rh.tail_decoded(trace, requests)
    rh.portions(trace, requests)
    rh.mixed(trace, requests)
    assert trace.max_live <= 4
    runner = build_runner(model_dirs[name], torch.float32, "cpu", page, -(-trace.max_tokens // page), 4)
    results = rh.run_in_process(runner, trace)
    worst, where = rh.worst_error(results, rh.gather_expected(trace, expected))
    assert worst < 2e-5, f"worst difference {worst} at step {where}"
    assert not runner.cache.live_requests
    for group in runner.cache.groups:
        assert group.allocator.num_held == 0


def test_failed_step_changes_nothing(cpu_kernels, model_dirs):
    from liteinfer_b200.cache.pages import OutOfPagesError
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    config, _, page = tiny_configs.ALL["tiny_a"]
    runner = build_runner(model_dirs["tiny_a"], torch.float32, "cpu", page, 2, 4)
    tokens = tiny_configs.prompt(config["vocab_size"], 40, 0)
    runner.step([StepEntry("a", tokens[:20], [19])])
    with pytest.raises(OutOfPagesError):
        runner.step([StepEntry("a", tokens[20:22], [1]), StepEntry("b", tokens[:17], [16])])
    assert runner.cache.length("a") == 20 and not runner.cache.has("b")
    runner.cache.check_invariants()
    with pytest.raises(ValueError):
        runner.step([StepEntry("a", [config["vocab_size"]], [0])])
    with pytest.raises(ValueError):
        runner.step([StepEntry("a", [1], [1])])
    out = runner.step([StepEntry("a", tokens[20:22], [0, 1])])
    assert out.shape == (2, config["vocab_size"])
