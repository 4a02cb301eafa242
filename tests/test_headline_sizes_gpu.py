"""What the benchmark times, checked against plain implementations at the benchmark's own sizes.

Kernel level, against tests/torch_kernels.py in 32-bit arithmetic: the tcgen05 attention on one prompt of 2,048
tokens (33 key tiles a block, every block of queries) and on four portions of 2,048 queries that end contexts of
4,096 keys, at head sizes 64 and 128, with and without a window; the decode attention on 8 and 64 single-token
sequences over 4,000 to 4,096 keys with the splits the engine would choose, rotary encoding and cache write fused
in, every slot that no request owns holding NaN.

Model level, at the widths of Llama 3.2 1B with two layers, in bfloat16 and float32, against tests/plain_llama.py
on the GPU: one whole prompt of 2,048 tokens; one step of 2,500 tokens (above the largest padded graph: launched
kernel by kernel); a portion of 512 tokens beside three single tokens whose contexts exceed 3,000.
"""

from __future__ import annotations

import pytest
import torch

import plain_llama
import tiny_configs
import torch_kernels as ref
from test_wide_model_gpu import WIDE

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _randn(*shape, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(BF16)


def _case(heads, kv_heads, d, page, q_lens, ctx_lens, seed=0):
    """Shuffled pages holding random keys and values for every earlier token of every context, NaN elsewhere;
    the new tokens' q, k, v in one fused buffer."""
    g = torch.Generator().manual_seed(seed)
    B = len(q_lens)
    per = [-(-c // page) for c in ctx_lens]
    num_pages = sum(per) + 5
    perm = torch.randperm(num_pages, generator=g)
    table = torch.full((B, max(per) + 1), -1, dtype=torch.int32)
    at = 0
    for s, n in enumerate(per):
        table[s, :n] = perm[at:at + n].to(torch.int32)
        at += n
    table = table.cuda()
    k_pool = torch.full((num_pages, kv_heads, page, d), float("nan"), dtype=BF16, device="cuda")
    v_pool = torch.full_like(k_pool, float("nan"))
    for s in range(B):
        old = ctx_lens[s] - q_lens[s]
        if not old:
            continue
        pos = torch.arange(old, device="cuda")
        pages = table[s].long()[pos // page]
        k_pool[pages, :, pos % page] = _randn(old, kv_heads, d, seed=seed + 10 + s)
        v_pool[pages, :, pos % page] = _randn(old, kv_heads, d, seed=seed + 500 + s)
    T = sum(q_lens)
    qkv = _randn(T, (heads + 2 * kv_heads) * d, seed=seed + 1)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    starts = [0]
    for q in q_lens:
        starts.append(starts[-1] + q)
    positions = torch.cat([torch.arange(c - q, c) for q, c in zip(q_lens, ctx_lens)]).to(torch.int32).cuda()
    seq_of = torch.cat([torch.full((q,), s) for s, q in enumerate(q_lens)]).to(torch.int32).cuda()
    return dict(qkv=qkv, k_pool=k_pool, v_pool=v_pool, table=table, qsl=i32(starts), ctx=i32(ctx_lens),
                positions=positions, seq_of=seq_of, B=B, T=T)


def _inv_freq(d):
    return (1.0 / (500000.0 ** (torch.arange(0, d, 2).float() / d))).cuda()


@pytest.mark.parametrize("d,heads,kv_heads", [(64, 8, 2), (128, 6, 2)])
@pytest.mark.parametrize("q_lens,ctx_lens,window", [([2048], [2048], 0), ([2048] * 4, [4096] * 4, 0),
                                                    ([2048, 1000], [2048, 4096], 1000)])
def test_tcgen05_attention_at_the_benchmark_sizes(d, heads, kv_heads, q_lens, ctx_lens, window):
    from liteinfer_b200 import ops

    case = _case(heads, kv_heads, d, 16, q_lens, ctx_lens, seed=d)
    qkv, k_pool, v_pool = case["qkv"], case["k_pool"], case["v_pool"]
    inv_freq = _inv_freq(d)
    ref.rope_kv_write(qkv, case["positions"], case["seq_of"], case["table"], k_pool, v_pool, inv_freq, heads,
                      kv_heads, d, d)
    rest = (k_pool, v_pool, case["table"], case["qsl"], case["ctx"])
    tail = (case["B"], max(q_lens), heads, kv_heads, d, d ** -0.5, window)
    want = ref.paged_attention(qkv, qkv.shape[1], torch.empty(case["T"], heads * d, dtype=BF16, device="cuda"),
                               *rest, *tail)
    out = torch.full((case["T"], heads * d), float("nan"), dtype=BF16, device="cuda")
    assert ops.tcgen05_attention_supports(BF16, heads, kv_heads, d, 16)
    ops.paged_attention_tcgen05(qkv, qkv.shape[1], out, *rest, None, *tail)
    assert ops.gemm_error_flag("cuda:0") == 0
    assert torch.isfinite(out.float()).all()
    torch.testing.assert_close(out.float(), want.float(), rtol=2 ** -6, atol=2 ** -6)


def test_tcgen05_attention_finds_one_key_among_2048():
    """One key made to dominate for the queries behind it: each of them returns that key's value, whichever tile
    and page it lies in, and the queries before it do not see it."""
    from liteinfer_b200 import ops

    heads, kv_heads, d, n = 4, 1, 64, 2048
    for far in (0, 63, 64, 1023, 2000):
        case = _case(heads, kv_heads, d, 16, [n], [n], seed=far)
        qkv, k_pool, v_pool = case["qkv"], case["k_pool"], case["v_pool"]
        direction = torch.nn.functional.normalize(_randn(d, seed=9).float(), dim=0)
        qkv[:, :heads * d] = (direction * 6).to(BF16).repeat(heads)        # every query points the same way
        qkv[:, heads * d:(heads + 1) * d] = _randn(n, d, seed=3, scale=0.05)
        qkv[far, heads * d:(heads + 1) * d] = (direction * 6).to(BF16)
        ref.rope_kv_write(qkv, case["positions"], case["seq_of"], case["table"], k_pool, v_pool, None, heads,
                          kv_heads, d, 0)
        out = torch.empty(n, heads * d, dtype=BF16, device="cuda")
        ops.paged_attention_tcgen05(qkv, qkv.shape[1], out, k_pool, v_pool, case["table"], case["qsl"], case["ctx"],
                                    None, 1, n, heads, kv_heads, d, 1.0, 0)
        value = qkv[far, (heads + 1) * d:].float()
        got = out.view(n, heads, d).float()
        torch.testing.assert_close(got[far:], value.expand(n - far, heads, d), rtol=3e-2, atol=3e-2)
        if far:
            assert float((got[:far] - value).abs().mean()) > 0.3
    assert ops.gemm_error_flag("cuda:0") == 0


@pytest.mark.parametrize("batch", [8, 64])
@pytest.mark.parametrize("d,heads,kv_heads", [(64, 32, 8), (128, 24, 8)])
def test_decode_attention_at_the_benchmark_context(batch, d, heads, kv_heads):
    """Single tokens of `batch` sequences over 4,000 to 4,096 keys, through the launch the engine uses (keys split
    over as many blocks as one wave holds, the last block merging; rotary encoding of q and the newest key and
    their cache write inside the kernel), against rotate-and-store and attention in plain torch."""
    from liteinfer_b200 import ops
    from liteinfer_b200.parts.context import AttentionPlan

    g = torch.Generator().manual_seed(batch + d)
    ctx_lens = [4096, 4000, 4033] + torch.randint(4000, 4097, (batch - 3,), generator=g).tolist()
    q_lens = [1] * batch
    case = _case(heads, kv_heads, d, 16, q_lens, ctx_lens, seed=batch)
    inv_freq = _inv_freq(d)
    rows = torch.arange(batch, dtype=torch.int32, device="cuda")
    plan = AttentionPlan(num_decode=batch, decode_seqs=rows, decode_tokens=rows, num_prefill=0,
                         prefill_seqs=rows[:0], max_prefill_query_len=0, max_decode_context_len=4097)
    q_width, kv_width = heads * d, kv_heads * d
    rest = (case["table"], case["qsl"], case["ctx"], batch, 1, heads, kv_heads, d, d ** -0.5, 0)

    qkv, k_ref, v_ref = case["qkv"].clone(), case["k_pool"].clone(), case["v_pool"].clone()
    ref.rope_kv_write(qkv, case["positions"], case["seq_of"], case["table"], k_ref, v_ref, inv_freq, heads, kv_heads, d, d)
    want = ref.paged_attention(qkv, qkv.shape[1], torch.empty(batch, q_width, dtype=BF16, device="cuda"),
                               k_ref, v_ref, *rest)

    qkv, k_pool, v_pool = case["qkv"].clone(), case["k_pool"].clone(), case["v_pool"].clone()
    assert ops.fused_decode_supports(BF16, heads, kv_heads, d, d, plan)
    assert ops.stream_attention_supports(BF16, heads, kv_heads, d, 16)
    splits = ops.decode_splits_for(batch, kv_heads, 4097, d, True)
    assert (splits > 1) == (batch == 8)
    newest = ops.NewestToken(inv_freq, qkv[:, q_width:], qkv[:, q_width + kv_width:])
    got = ops.paged_attention(qkv, qkv.shape[1], torch.full((batch, q_width), float("nan"), dtype=BF16, device="cuda"),
                              k_pool, v_pool, *rest, plan=plan, newest=newest)
    assert ops.gemm_error_flag("cuda:0") == 0
    torch.testing.assert_close(got.float(), want.float(), rtol=2 ** -6, atol=2 ** -6)
    # The pages: exactly the newest token's slots were written, with the rotated key and the value.
    for mine, theirs in ((k_pool, k_ref), (v_pool, v_ref)):
        assert torch.equal(torch.isnan(mine.float()), torch.isnan(theirs.float()))
        torch.testing.assert_close(torch.nan_to_num(mine.float()), torch.nan_to_num(theirs.float()),
                                   rtol=2 ** -7, atol=2 ** -7)


# ------------------------------------------------------------------------------------------------ model level
@pytest.fixture(scope="module")
def wide_model(tmp_path_factory):
    from liteinfer_b200.weights.random_init import write_random_model

    return write_random_model(WIDE, tmp_path_factory.mktemp("headline") / "wide", seed=6)


def _plain_rows(model_dir, tokens, rows, dtype):
    """Logits of the plain implementation at `rows` of one whole sequence (the head only where asked)."""
    raw, weights = plain_llama.read_model(model_dir)
    hidden = plain_llama.hidden_states(raw, weights, tokens, dtype, "cuda")
    head = weights["model.embed_tokens.weight"].to(device="cuda", dtype=dtype)
    return plain_llama.linear(hidden[rows], head).float()


def _runner(model_dir, dtype, tokens_held, graphs=True):
    from liteinfer_b200.engine.loading import build_runner

    runner = build_runner(model_dir, dtype, "cuda:0", 16, -(-tokens_held // 16) + 8, 4)
    if graphs:
        runner.enable_decode_graphs(4, 4096)
    return runner


def _check(runner, got, want, exact, dtype):
    from liteinfer_b200 import ops

    assert ops.gemm_error_flag("cuda:0") == 0
    assert torch.isfinite(got.float()).all()
    worst = float((got.float() - exact).abs().max())
    if dtype == torch.float32:
        assert worst < 2e-4, worst
    else:
        drift = float((want - exact).abs().max())       # what the plain implementation drifts in bfloat16
        assert worst <= 2 * drift, f"worst difference {worst}; plain bfloat16 drifts {drift}"


@pytest.mark.parametrize("dtype", [torch.float32, BF16])
@pytest.mark.parametrize("length", [2048, 2500])
def test_a_whole_prompt_of_benchmark_length(wide_model, dtype, length):
    """2,048 tokens: the benchmark's prefill, replayed from the largest padded graph.  2,500: above it."""
    from liteinfer_b200.engine.runner import StepEntry

    tokens = tiny_configs.prompt(WIDE["vocab_size"], length, 21)
    rows = [0, 15, 16, 63, 64, 127, 128, 1000, 2047, length - 1]
    runner = _runner(wide_model, dtype, length)
    got = runner.step([StepEntry("a", tokens, rows)])
    assert runner.graph_replays == (1 if length <= 2048 else 0)
    exact = _plain_rows(wide_model, tokens, rows, torch.float32)
    want = _plain_rows(wide_model, tokens, rows, dtype)
    _check(runner, got, want, exact, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, BF16])
def test_a_portion_beside_long_decoding_rows(wide_model, dtype):
    """Three requests hold more than 3,000 tokens each and bring one token; a fourth brings 512 tokens of its
    prompt, of which it holds 700 already: one step, the decode rows' keys split beside the unsplit portion."""
    from liteinfer_b200.engine.runner import StepEntry

    vocab = WIDE["vocab_size"]
    lengths = {"d0": 3001, "d1": 3500, "d2": 4000, "p": 700 + 512}
    requests = {r: tiny_configs.prompt(vocab, n, 30 + i) for i, (r, n) in enumerate(lengths.items())}
    runner = _runner(wide_model, dtype, sum(-(-n // 64) * 64 for n in lengths.values()))
    for r in ("d0", "d1", "d2"):
        held = requests[r][:-1]
        for at in range(0, len(held), 2048):
            runner.step([StepEntry(r, held[at:at + 2048], ())])
    runner.step([StepEntry("p", requests["p"][:700], ())])
    entries = [StepEntry("d0", requests["d0"][-1:], (0,)), StepEntry("p", requests["p"][700:], (0, 255, 511)),
               StepEntry("d1", requests["d1"][-1:], (0,)), StepEntry("d2", requests["d2"][-1:], (0,))]
    got = runner.step(entries)
    where = [("d0", [3000]), ("p", [700, 955, 1211]), ("d1", [3499]), ("d2", [3999])]
    exact = torch.cat([_plain_rows(wide_model, requests[r], rows, torch.float32) for r, rows in where])
    want = torch.cat([_plain_rows(wide_model, requests[r], rows, dtype) for r, rows in where])
    _check(runner, got, want, exact, dtype)
    runner.cache.check_invariants()
