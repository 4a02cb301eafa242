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
            assert runner.graph_replays == 20 and len(runner._graphs) == 2
    for eager, replayed in zip(*runs):
        assert eager.shape == replayed.shape
        if name == "tiny_d":
            # A graph splits the keys by the longest context it may ever see, the eager step by the one
            # it has: the same sums in another order.
            torch.testing.assert_close(eager.float(), replayed.float(), rtol=2 ** -6, atol=2 ** -6)
        else:
            assert torch.equal(eager, replayed)
