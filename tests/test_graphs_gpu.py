"""Decode steps replayed from CUDA graphs give the logits of the same steps launched kernel by kernel."""

from __future__ import annotations

import pytest
import torch

import tiny_configs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype", [("tiny_b", torch.float32), ("tiny_d", torch.bfloat16), ("tiny_a", torch.bfloat16), ("tiny_e", torch.bfloat16)])
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
        if name in ("tiny_d", "tiny_e"):
            # A graph splits the keys by the longest context it may ever see, the eager step by the one
            # it has: the same sums in another order.
            torch.testing.assert_close(eager.float(), replayed.float(), rtol=2 ** -6, atol=2 ** -6)
        else:
            assert torch.equal(eager, replayed)


@pytest.mark.parametrize("name,dtype", [("tiny_b", torch.float32), ("tiny_d", torch.bfloat16), ("tiny_e", torch.bfloat16)])
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


@pytest.mark.parametrize("name,dtype", [("tiny_b", torch.float32), ("tiny_a", torch.float32), ("tiny_d", torch.bfloat16), ("tiny_e", torch.bfloat16)])
def test_padded_graphs_equal_eager_over_random_steps(model_dirs, name, dtype):
    """Steps of every kind (portions of prompts down to two tokens, alone or beside single tokens, logits wanted
    anywhere, nowhere, or at more places than there are sequences) replayed from graphs of padded shapes against
    the same steps launched kernel by kernel.  Shapes repeat with other real sizes inside them, so a graph's buffers
    hold what a larger step left there; requests end and their pages are used again."""
    import random

    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    config, _, page = tiny_configs.ALL[name]
    vocab = config["vocab_size"]
    rng = random.Random(11)
    eager = build_runner(model_dirs[name], dtype, "cuda:0", page, 64, 4)
    replayed = build_runner(model_dirs[name], dtype, "cuda:0", page, 64, 4)
    replayed.enable_decode_graphs(4, 64 * page)
    live: dict[str, int] = {}              # request -> tokens it still owes before it ends
    born = 0
    worst = 0.0
    for step in range(120):
        while len(live) < 4 and (not live or rng.random() < 0.4):
            live[f"q{born}"] = rng.randint(3, 90)
            born += 1
        entries = []
        for request, owed in list(live.items()):
            if rng.random() < 0.15:
                continue                                    # sits this step out
            n = 1 if rng.random() < 0.5 else rng.randint(2, min(owed, 40)) if owed >= 2 else 1
            n = min(n, owed)
            tokens = [rng.randrange(vocab) for _ in range(n)]
            kind = rng.random()
            want = () if kind < 0.2 else (n - 1,) if kind < 0.7 else tuple(sorted(rng.sample(range(n), rng.randint(1, n))))
            entries.append(StepEntry(request, tokens, want))
            live[request] = owed - n
        if not entries:
            continue
        a, b = eager.step(entries), replayed.step(entries)
        assert a.shape == b.shape
        if dtype == torch.float32:
            assert torch.equal(a, b), f"step {step}: {[(e.request_id, len(e.tokens), e.want) for e in entries]}"
        elif a.numel():
            worst = max(worst, float((a.float() - b.float()).abs().max()))
        for request in [r for r, owed in live.items() if owed == 0]:
            eager.release(request)
            replayed.release(request)
            del live[request]
        replayed.cache.check_invariants()
    assert worst <= 2 ** -6, worst
    assert replayed.graph_replays >= 100 and 5 <= len(replayed._padded_graphs) <= 60
    replayed.check_kernels()


def test_a_wait_that_gave_up_is_reported(model_dirs):
    """Kernels that wait on mbarriers poll a bounded number of times and then raise a flag on the device instead of
    hanging; the engine reads it where it synchronises anyway.  The flag is set here by the host (no kernel is
    made to give up): `check_kernels` must raise, name the wait, and clear the flag, whichever way the device was
    named."""
    from liteinfer_b200 import ops
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.ops.kernels import scratch_for

    config, _, page = tiny_configs.ALL["tiny_a"]
    runner = build_runner(model_dirs["tiny_a"], torch.bfloat16, "cuda", page, 8, 2)      # "cuda", not "cuda:0"
    runner.check_kernels()
    scratch_for("cuda:0").gemm_error.fill_(7)
    with pytest.raises(RuntimeError, match="wait number 7"):
        runner.check_kernels()
    runner.check_kernels()                                  # reading cleared it
    ops.token_error_flag("cuda").fill_(1)
    with pytest.raises(RuntimeError, match="outside the vocabulary"):
        runner.check_kernels()
    assert ops.error_flags("cuda:0") == (0, 0)
