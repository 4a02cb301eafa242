"""The engine loop, the entry points and the sampler's host side, on a CPU with the stand-in kernels."""

from __future__ import annotations

import asyncio

import pytest
import torch

import plain_llama
import tiny_configs


def _prompts(vocab, lengths):
    return [tiny_configs.prompt(vocab, n, i) for i, n in enumerate(lengths)]


def test_greedy_generation_through_llm_matches_plain(cpu_kernels, model_dirs):
    from liteinfer_b200 import LLM, SamplingParams

    config, _, page = tiny_configs.ALL["tiny_b"]
    prompts = _prompts(config["vocab_size"], (3, 30, 11, 1))
    raw, weights = plain_llama.read_model(model_dirs["tiny_b"])
    expected = [plain_llama.greedy(raw, weights, p, 5) for p in prompts]
    # a budget of 16 tokens cuts the 30-token prompt into portions that run beside the others' decodes
    with LLM(str(model_dirs["tiny_b"]), dtype="float32", device="cpu", block_size=page, max_num_seqs=3,
             max_model_len=64, max_num_batched_tokens=16) as llm:
        outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
        assert [o.token_ids for o in outs] == expected
        assert [o.finish_reason for o in outs] == ["length"] * 4
        assert [o.request_id for o in outs] == ["req-0", "req-1", "req-2", "req-3"]
        assert outs[0].text == " ".join(map(str, expected[0]))        # no tokenizer.json: text is ids
        phases = {s.phase for s in llm.stats.steps}
        assert "mixed" in phases and "decode" in phases
        assert max(s.input_tokens for s in llm.stats.steps) <= 16
        assert llm.engine.runner.cache.live_requests == [] or True
        # strings work too: the tokenizer of a folder without tokenizer.json reads ids
        again = llm.generate(" ".join(map(str, prompts[0])), SamplingParams(temperature=0.0, max_tokens=5))
        assert again[0].token_ids == expected[0]


def test_stop_rules_through_the_engine(cpu_kernels, model_dirs):
    from liteinfer_b200 import LLM, SamplingParams

    config, _, page = tiny_configs.ALL["tiny_a"]
    prompt = tiny_configs.prompt(config["vocab_size"], 7, 0)
    with LLM(str(model_dirs["tiny_a"]), dtype="float32", device="cpu", block_size=page, max_model_len=32) as llm:
        free = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8))[0].token_ids
        stop_at = free[2]
        cut = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8, stop_token_ids=[stop_at]))[0]
        assert cut.finish_reason == "stop" and cut.token_ids == free[:free.index(stop_at) + 1]
        gated = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8, min_tokens=6,
                                                      stop_token_ids=[stop_at]))[0]
        assert len(gated.token_ids) >= 6
        # A stop string is looked for in the text, which is then decoded at every step (otherwise at the end only).
        text_stop = " " + str(free[3])
        by_text = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8, stop=[text_stop]))[0]
        first = next(n for n in range(1, 9) if text_stop in " ".join(map(str, free[:n])))
        assert by_text.finish_reason == "stop" and by_text.token_ids == free[:first]
        assert by_text.text == " ".join(map(str, free[:first]))
        long = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=100))[0]
        assert long.finish_reason == "length" and len(prompt) + len(long.token_ids) == 32   # max_model_len
        with pytest.raises(ValueError, match="max_model_len"):
            llm.generate([list(range(40))], SamplingParams(max_tokens=1))
        with pytest.raises(ValueError, match="no tokens"):
            llm.generate([""], SamplingParams(max_tokens=1))


def test_newcomers_wait_for_pages_and_nothing_is_lost(cpu_kernels, model_dirs):
    """Six requests through a cache that holds two of them: all finish, none is aborted, every page comes back."""
    from liteinfer_b200 import LLM, SamplingParams

    config, _, page = tiny_configs.ALL["tiny_a"]
    prompts = _prompts(config["vocab_size"], (20, 25, 18, 30, 9, 22))
    raw, weights = plain_llama.read_model(model_dirs["tiny_a"])
    with LLM(str(model_dirs["tiny_a"]), dtype="float32", device="cpu", block_size=page, max_num_seqs=4,
             max_model_len=64, num_gpu_blocks=5) as llm:
        outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
        assert [o.token_ids for o in outs] == [plain_llama.greedy(raw, weights, p, 4) for p in prompts]
        assert llm.stats.num_requests_aborted == 0
        cache = llm.engine.runner.cache
        llm.engine.step()                                   # evicts what finished last
        assert all(g.allocator.num_held == 0 for g in cache.groups) and cache.slots.num_held == 0


def test_running_out_of_pages_while_decoding_sheds_the_least_invested(cpu_kernels, model_dirs):
    """Two requests fill the cache while decoding; the step that does not fit aborts one tier and the other goes on."""
    from liteinfer_b200.cache.pages import CacheExhaustedError
    from liteinfer_b200.config.engine_config import EngineConfig
    from liteinfer_b200.engine.core import EngineCore
    from liteinfer_b200.sampling.params import SamplingParams

    config, _, page = tiny_configs.ALL["tiny_a"]          # pages of 16 tokens
    engine = EngineCore(EngineConfig(model=str(model_dirs["tiny_a"]), dtype="float32", device="cpu",
                                     block_size=page, max_num_seqs=4, max_model_len=128, num_gpu_blocks=3))
    engine.load()
    engine.scheduler.ledger = None                          # admit regardless, as the reference does
    params = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    a = engine.add_request("a", tiny_configs.prompt(config["vocab_size"], 30, 0), params)
    b = engine.add_request("b", tiny_configs.prompt(config["vocab_size"], 14, 1), params)
    aborted = []
    for _ in range(60):
        if not engine.has_unfinished():
            break
        result = engine.step()
        aborted += result.aborted
    # a needs its third page at 33 tokens, b its second at 17: the pool of three cannot hold both.
    assert len(aborted) == 2 or len(aborted) == 1
    assert all(isinstance(error, CacheExhaustedError) for _, error in aborted)
    assert engine.stats.num_requests_aborted == len(aborted)
    finished = [s for s in (a, b) if s.status.value == "finished_length"]
    assert len(finished) + len(aborted) == 2
    engine.step()
    assert all(g.allocator.num_held == 0 for g in engine.runner.cache.groups)


def test_a_failing_step_aborts_only_its_requests(cpu_kernels, model_dirs, monkeypatch):
    from liteinfer_b200 import LLM, SamplingParams

    config, _, page = tiny_configs.ALL["tiny_a"]
    with LLM(str(model_dirs["tiny_a"]), dtype="float32", device="cpu", block_size=page, max_model_len=64) as llm:
        runner = llm.engine.runner
        real = runner.model.forward
        calls = {"n": 0}

        def flaky(ctx, caches):
            calls["n"] += 1
            if calls["n"] == 2:
                raise RuntimeError("boom")
            return real(ctx, caches)

        monkeypatch.setattr(runner.model, "forward", flaky)
        with pytest.raises(RuntimeError, match="boom"):
            llm.generate([tiny_configs.prompt(config["vocab_size"], 5, 0)], SamplingParams(temperature=0.0, max_tokens=4))
        monkeypatch.setattr(runner.model, "forward", real)
        out = llm.generate([tiny_configs.prompt(config["vocab_size"], 5, 0)], SamplingParams(temperature=0.0, max_tokens=4))
        assert len(out[0].token_ids) == 4                   # the engine is still usable, the cache was rolled back
        runner.cache.check_invariants()


def test_async_llm_generates_and_streams(cpu_kernels, model_dirs):
    from liteinfer_b200 import AsyncLLM, SamplingParams

    config, _, page = tiny_configs.ALL["tiny_b"]
    prompts = _prompts(config["vocab_size"], (4, 12, 7))
    raw, weights = plain_llama.read_model(model_dirs["tiny_b"])
    expected = [plain_llama.greedy(raw, weights, p, 4) for p in prompts]

    async def run():
        async with AsyncLLM(str(model_dirs["tiny_b"]), dtype="float32", device="cpu", block_size=page,
                            max_num_seqs=2, max_model_len=64) as llm:
            outs = await llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
            events = [e async for e in llm.stream(prompts[1], SamplingParams(temperature=0.0, max_tokens=4,
                                                                              ignore_eos=True))]
            with pytest.raises(ValueError):
                await llm.generate([[]], SamplingParams(max_tokens=1))
            return outs, events

    outs, events = asyncio.run(run())
    assert [o.token_ids for o in outs] == expected
    assert [len(e.output_token_ids) for e in events] == [1, 2, 3, 4]
    assert events[-1].is_finished and events[-1].finish_reason == "length" and not events[0].is_finished
    assert events[-1].output_token_ids == expected[1]


def test_sampling_params_checks():
    from liteinfer_b200 import SamplingParams

    for bad in ({"temperature": -1}, {"top_p": 0.0}, {"top_p": 1.5}, {"top_k": 0}, {"max_tokens": 0},
                {"min_tokens": -1}, {"min_tokens": 9, "max_tokens": 3}):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    assert SamplingParams(temperature=0).greedy and SamplingParams(top_k=1).greedy and not SamplingParams().greedy
    assert SamplingParams().id != SamplingParams().id


def test_sampler_streams_do_not_depend_on_the_batch(cpu_kernels):
    """A seeded request draws the same tokens alone and beside others; greedy rows are the arg-max."""
    from liteinfer_b200 import SamplingParams
    from liteinfer_b200.sampling.sampler import Sampler

    g = torch.Generator().manual_seed(0)
    logits = torch.randn(3, 50, generator=g)
    seeded = SamplingParams(temperature=1.0, top_k=20, top_p=0.9, seed=7)
    alone = [int(Sampler(1)(logits[1:2], [seeded], ["r"])[0]) for _ in range(1)]
    sampler = Sampler(99)
    mixed = sampler(logits, [SamplingParams(temperature=0.0), seeded, SamplingParams(temperature=0.8)], ["a", "r", "c"])
    assert int(mixed[1]) == alone[0] and int(mixed[0]) == int(torch.argmax(logits[0]))
    draws_a = [int(Sampler(5)(logits[2:3], [SamplingParams(temperature=1.5, seed=3)], ["x"])[0]) for _ in range(2)]
    assert draws_a[0] == draws_a[1]                                    # same seed, same first draw
    s = Sampler(5)
    p = SamplingParams(temperature=1.5, seed=3)
    many = {int(s(logits[2:3], [p], ["x"])[0]) for _ in range(40)}
    assert len(many) > 3                                               # the stream advances between steps
    with pytest.raises(ValueError):
        s(logits, [p])


def test_sample_rule_properties():
    """The row-by-row rule the kernel is tested against: top-k keeps exactly k, the entry crossing p is kept."""
    from torch_kernels import sample_row

    logits = torch.tensor([1.0, 3.0, 3.0, 2.0, -1.0])
    draws = {sample_row(logits, 1.0, 2, 1.0, u / 100) for u in range(100)}
    assert draws == {1, 2}                                             # ties at the top: exactly two survive
    draws = {sample_row(logits, 1.0, 3, 1.0, u / 100) for u in range(100)}
    assert draws == {1, 2, 3}
    probs = torch.softmax(logits, -1)
    p_just_below_top_two = float(probs[1] + probs[2]) - 1e-3
    draws = {sample_row(logits, 1.0, 0, p_just_below_top_two, u / 200) for u in range(200)}
    assert draws == {1, 2}                                             # the second entry crosses p and is kept
    draws = {sample_row(logits, 1.0, 0, float(probs[1]) - 1e-3, u / 50) for u in range(50)}
    assert draws == {1}
    assert sample_row(logits, 0.0, 0, 1.0, 0.5) == 1                   # temperature 0: the first arg-max


def test_bench_run_reports_the_references_summaries(cpu_kernels, model_dirs, capsys):
    """`bench run` on a CPU with the stand-in kernels: forced output lengths, the two modes' fields."""
    import json

    from liteinfer_b200.benchmark import make_prompts, percentile
    from liteinfer_b200.cli import main

    assert percentile([1.0, 2.0, 3.0, 4.0], 50) == 2.5 and percentile([5.0], 99) == 5.0
    mixed = make_prompts(100, None, 200, 64, 0)
    assert all(1 <= len(p) <= 64 for p in mixed) and len({len(p) for p in mixed}) > 10
    assert make_prompts(100, 7, 3, 64, 0) == make_prompts(100, 7, 3, 64, 0)
    code = main(["bench", "run", "--model", str(model_dirs["tiny_a"]), "--isl", "9", "--osl", "4", "-n", "5",
                 "--dtype", "float32", "--device", "cpu", "--max-num-seqs", "2", "--max-model-len", "32"])
    assert code == 0
    result = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert result["dataset"]["num_samples"] == 5 and result["dataset"]["input_tokens"] == 45
    assert set(result["summary"]["throughput"]) == {"output_tokens_per_s", "requests_per_s", "wall_time_s", "step_phases"}
    assert set(result["summary"]["latency"]) == {"ttft_p50_ms", "ttft_p95_ms", "ttft_p99_ms", "itl_p50_ms",
                                                 "itl_p95_ms", "itl_p99_ms", "e2e_p50_ms"}
    assert result["summary"]["throughput"]["output_tokens_per_s"] > 0


def test_padded_shapes_of_the_step_graphs():
    """The ladder that steps are rounded up to before they are replayed from a graph: never below the step, less
    than 16 tokens or an eighth of the next power of two above it, few distinct shapes, and stable (a padded size
    pads to itself)."""
    from liteinfer_b200.engine.runner import _pow2, _token_bucket

    shapes = set()
    for n in range(1, 8193):
        padded = _token_bucket(n)
        shapes.add(padded)
        assert padded >= n and _token_bucket(padded) == padded
        assert padded - n < max(16, _pow2(n) // 8)
    assert len(shapes) <= 48
    assert [_pow2(n) for n in (0, 1, 2, 3, 4, 5, 33, 64)] == [1, 1, 2, 4, 4, 8, 64, 64]


def test_steps_launched_ahead_give_the_same_outputs(cpu_kernels, model_dirs):
    """The engine launches a step before it has read the tokens of the step before.  With every kind of ending
    (a stop id early or late, min_tokens, max_tokens, the context limit), prompts cut by the budget and a cache
    that makes newcomers wait, the outputs are those of the engine that reads every step before the next."""
    from liteinfer_b200 import LLM, SamplingParams

    config, _, page = tiny_configs.ALL["tiny_a"]
    vocab = config["vocab_size"]
    prompts = _prompts(vocab, (5, 21, 9, 30, 2, 14, 17, 40))
    common = dict(dtype="float32", device="cpu", block_size=page, max_num_seqs=3, max_model_len=48,
                  max_num_batched_tokens=12, num_gpu_blocks=7)
    with LLM(str(model_dirs["tiny_a"]), async_scheduling=False, **common) as llm:
        free = [o.token_ids for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))]
    params = [
        SamplingParams(temperature=0.0, max_tokens=12, stop_token_ids=[free[0][0]]),            # the very first token ends it
        SamplingParams(temperature=0.0, max_tokens=12, stop_token_ids=[free[1][4]]),
        SamplingParams(temperature=0.0, max_tokens=12, stop_token_ids=[free[2][1]], min_tokens=5),
        SamplingParams(temperature=0.0, max_tokens=100),                                          # the context limit
        SamplingParams(temperature=0.0, max_tokens=1),
        SamplingParams(temperature=0.0, max_tokens=12, stop=[" " + str(free[5][3])]),            # a stop string
        SamplingParams(temperature=0.7, top_k=5, seed=3, max_tokens=9),                           # a seeded stream
        SamplingParams(temperature=0.0, max_tokens=7, stop_token_ids=[free[7][6]]),              # stop id and length at once
    ]
    runs = []
    for ahead in (False, True):
        with LLM(str(model_dirs["tiny_a"]), async_scheduling=ahead, **common) as llm:
            outs = llm.generate(prompts, params)
            runs.append([(o.token_ids, o.finish_reason, o.text) for o in outs])
            assert llm.stats.num_requests_aborted == 0
            llm.engine.step()
            cache = llm.engine.runner.cache
            cache.check_invariants()
            assert all(g.allocator.num_held == 0 for g in cache.groups) and cache.slots.num_held == 0
            assert not llm.engine.has_unfinished()
    assert runs[0] == runs[1]
    assert runs[1][0][0] == free[0][:1] and runs[1][0][1] == "stop"
    assert runs[1][3][1] == "length" and len(prompts[3]) + len(runs[1][3][0]) == 48
    assert all(-1 not in tokens for tokens, _, _ in runs[1])
