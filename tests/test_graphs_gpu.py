"""Decode steps replayed from CUDA graphs give the logits of the same steps launched kernel by kernel."""

from __future__ import annotations

import pytest
import torch

import tiny_configs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype", [("tiny_b", torch.float32), ("tiny_d", torch.bfloat16), ("tiny_a", torch.bfloat16)])
def test_graph_replay_equals_eager(model_dirs, name, dtype):
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    config, _, page = tiny_configs.ALL[name]
    vocab = config["vocab_size"]
    prompts = {f"r{i}": tiny_configs.prompt(vocab, n, i) for i, n in enumerate((5, 40, 290))}
    forced = {r: tiny_configs.prompt(vocab, 20, 50 + i) for i, r in enumerate(prompts)}
    runs = []
    for graphs in (False, True):
        runner = build_runner(model_dirs[name], dtype, "cuda:0", page, 80, 4)
        if graphs:
            runner.enable_decode_graphs(4, 400)
        rows = [runner.step([StepEntry(r, t, (len(t) - 1,)) for r, t in prompts.items()])]
        live = list(prompts)
        for step in range(20):
            if step == 8:
                runner.release(live.pop(0))            # the batch narrows: another graph
            tokens = [forced[r][step] for r in live]      # forced tokens keep both runs on one path
            rows.append(runner.step([StepEntry(r, [t], (0,)) for r, t in zip(live, tokens)]))
        runs.append(rows)
        if graphs:
            assert runner.graph_replays == 21 and len(runner._graphs) == 2 and len(runner._padded_graphs) == 1   # the prompts too
    for eager, replayed in zip(*runs):
        assert eager.shape == replayed.shape
        if name == "tiny_d":
            # A graph splits the keys by the longest context it may ever see, the eager step by the one
            # it has: the same sums in another order.
            torch.testing.assert_close(eager.float(), replayed.float(), rtol=2 ** -6, atol=2 ** -6)
        else:
            assert torch.equal(eager, replayed)


@pytest.mark.parametrize("name,dtype", [("tiny_b", torch.float32), ("tiny_d", torch.bfloat16)])
def test_graph_rows_follow_the_requests(model_dirs, name, dtype):
    """A graph's staged batch keeps a request's rows from step to step; they must follow when the same width is
    filled by other requests, when requests change places, and when a request named again is a new one."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    config, _, page = tiny_configs.ALL[name]
    vocab = config["vocab_size"]
    prompts = {f"r{i}": tiny_configs.prompt(vocab, n, 7 + i) for i, n in enumerate((5, 40, 130, 23, 64))}
    forced = {r: tiny_configs.prompt(vocab, 40, 90 + i) for i, r in enumerate(prompts)}
    plan = [(["r0", "r1", "r2"], 6), (["r0", "r3", "r2"], 5), (["r2", "r0", "r3"], 9), (["r3", "r4", "r0"], 4),
            (["r1", "r4", "r0"], 7)]            # r1 comes back after it was released: the same name, a new request
    runs = []
    for graphs in (False, True):
        runner = build_runner(model_dirs[name], dtype, "cuda:0", page, 120, 4)
        if graphs:
            runner.enable_decode_graphs(4, 400)
        rows, live, taken = [], [], {r: 0 for r in prompts}
        for members, steps in plan:
            for r in [r for r in live if r not in members]:
                runner.release(r)
                taken[r] = 0
            for r in [r for r in members if r not in live]:
                rows.append(runner.step([StepEntry(r, prompts[r], (len(prompts[r]) - 1,))]))
            live = members
            for _ in range(steps):
                tokens = [forced[r][taken[r]] for r in live]
                for r in live:
                    taken[r] += 1
                rows.append(runner.step([StepEntry(r, [t], (0,)) for r, t in zip(live, tokens)]))
        runs.append(rows)
        if graphs:
            assert runner.graph_replays == sum(steps for _, steps in plan) + 6     # and the six prompts, padded
    for eager, replayed in zip(*runs):
        assert eager.shape == replayed.shape
        if dtype == torch.float32:
            assert torch.equal(eager, replayed)
        else:
            torch.testing.assert_close(eager.float(), replayed.float(), rtol=2 ** -6, atol=2 ** -6)
