"""Each CUDA kernel alone against its plain torch reference (tests/torch_kernels.py), at other sizes
than the engine's tiny models: widths that are no power of two, head sizes in steps of 16,
odd group sizes, pages of odd length."""

from __future__ import annotations

import pytest
import torch

import torch_kernels as ref

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2 ** -7, atol=2 ** -7)


def _randn(*shape, dtype, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [64, 100, 2048, 3000])
def test_embedding(dtype, width):
    from liteinfer_b200 import ops

    table = _randn(777, width, dtype=dtype)
    ids = torch.tensor([0, 776, 5, 5, 123, 1000, -1], dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.embedding(ids, table, torch.empty(7, width, dtype=dtype, device="cuda"), flag)
    assert torch.equal(out[:5], table[ids[:5].long()])
    assert torch.equal(out[5:], torch.zeros_like(out[5:])) and int(flag) == 1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [64, 100, 2048, 5000])
def test_rmsnorm_variants(dtype, width):
    from liteinfer_b200 import ops

    x = _randn(37, width, dtype=dtype, seed=1, scale=3.0)
    delta = _randn(37, width, dtype=dtype, seed=2)
    w = (1 + 0.1 * _randn(width, dtype=torch.float32, seed=3)).to(dtype)
    rows = torch.tensor([36, 0, 5, 5], dtype=torch.int32, device="cuda")
    for kwargs in ({}, {"delta": delta, "write_residual": True}, {"delta": delta, "rows": rows}, {"rows": rows}):
        xa, xb = x.clone(), x.clone()
        n = 4 if "rows" in kwargs else 37
        got = ops.rmsnorm(xa, w, 1e-5, torch.empty(n, width, dtype=dtype, device="cuda"), **kwargs)
        want = ref.rmsnorm(xb, w, 1e-5, torch.empty(n, width, dtype=dtype, device="cuda"), **kwargs)
        torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))
        torch.testing.assert_close(xa.float(), xb.float(), **_tol(dtype))   # the residual stream moved on (or not)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_pytorch_tanh", "relu"])
@pytest.mark.parametrize("width", [176, 100, 8192])
def test_act_mul(dtype, act, width):
    from liteinfer_b200 import ops

    gu = _randn(19, 2 * width, dtype=dtype, scale=2.0)
    got = ops.act_mul(gu, torch.empty(19, width, dtype=dtype, device="cuda"), act)
    want = ref.act_mul(gu, torch.empty(19, width, dtype=dtype, device="cuda"), act)
    torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_add_and_bias(dtype):
    from liteinfer_b200 import ops

    x, d, b = _randn(9, 100, dtype=dtype), _randn(9, 100, dtype=dtype, seed=5), _randn(100, dtype=dtype, seed=6)
    torch.testing.assert_close(ops.add_(x.clone(), d).float(), (x.float() + d.float()).to(dtype).float())
    torch.testing.assert_close(ops.add_bias_(x.clone(), b).float(), (x.float() + b.float()).to(dtype).float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (7, 1000, 96), (130, 100, 50), (64, 128256 // 64, 2048), (3, 5, 7)])
def test_gemm_simt(dtype, M, N, K):
    from liteinfer_b200 import ops

    x, w, b = _randn(M, K, dtype=dtype), _randn(N, K, dtype=dtype, seed=1, scale=0.05), _randn(N, dtype=dtype, seed=2)
    got = ops.gemm_simt(x, w, torch.empty(M, N, dtype=dtype, device="cuda"), b)
    want = (x.double() @ w.double().t() + b.double())
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2 ** -7, atol=2 ** -7)
    torch.testing.assert_close(got.double(), want, **tol)


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    from liteinfer_b200 import ops

    x, w = _randn(70, 320, dtype=torch.float32), _randn(1000, 320, dtype=torch.float32, seed=1)
    full = ops.gemm_simt(x, w, torch.empty(70, 1000, device="cuda"))
    one = ops.gemm_simt(x[33:34].contiguous(), w, torch.empty(1, 1000, device="cuda"))
    assert torch.equal(full[33:34], one)


@pytest.mark.parametrize("M,N,K", [(1, 3072, 2048), (8, 2048, 8192), (64, 1000, 96), (300, 512, 64), (2048, 256, 2048)])
def test_linear_bfloat16(M, N, K):
    from liteinfer_b200 import ops

    x, w = _randn(M, K, dtype=torch.bfloat16), _randn(N, K, dtype=torch.bfloat16, seed=1, scale=0.05)
    got = ops.linear(x, w, torch.empty(M, N, dtype=torch.bfloat16, device="cuda"))
    want = x.double() @ w.double().t()
    torch.testing.assert_close(got.double(), want, rtol=2 ** -7, atol=2 ** -7)


def _paged_case(dtype, heads, kv_heads, head_dim, page_size, q_lens, ctx_lens, seed=0, poison=True):
    """Random pool, shuffled pages, sequences with given new-query and context lengths."""
    g = torch.Generator().manual_seed(seed)
    B = len(q_lens)
    pages_per = [-(-c // page_size) for c in ctx_lens]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    width = max(pages_per) + 2
    table = torch.full((B, width), -1, dtype=torch.int32)
    at = 0
    for s, n in enumerate(pages_per):
        table[s, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    T = sum(q_lens)
    row = (heads + 2 * kv_heads) * head_dim
    qkv = _randn(T, row, dtype=dtype, seed=seed + 1)
    fill = float("nan") if poison else 0.0
    k_pool = torch.full((num_pages, kv_heads, page_size, head_dim), fill, dtype=dtype, device="cuda")
    v_pool = torch.full_like(k_pool, fill)
    # Earlier tokens of every context: random keys and values written straight into the pages.
    for s in range(B):
        old = ctx_lens[s] - q_lens[s]
        kk = _randn(old, kv_heads, head_dim, dtype=dtype, seed=seed + 10 + s)
        vv = _randn(old, kv_heads, head_dim, dtype=dtype, seed=seed + 50 + s)
        for p in range(old):
            page = int(table[s, p // page_size])
            k_pool[page, :, p % page_size] = kk[p]
            v_pool[page, :, p % page_size] = vv[p]
    qsl = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    ctx = torch.tensor(ctx_lens, dtype=torch.int32, device="cuda")
    positions = torch.cat([torch.arange(c - q, c) for q, c in zip(q_lens, ctx_lens)]).to(torch.int32).cuda()
    seq_of = torch.cat([torch.full((q,), s) for s, q in enumerate(q_lens)]).to(torch.int32).cuda()
    return dict(qkv=qkv, k_pool=k_pool, v_pool=v_pool, table=table.cuda(), qsl=qsl, ctx=ctx, positions=positions,
                seq_of=seq_of, B=B, T=T)


ATTENTION_SHAPES = [  # heads, kv_heads, head_dim, page_size
    (4, 2, 16, 16), (6, 3, 48, 8), (10, 2, 80, 5), (8, 8, 64, 16), (32, 8, 128, 16), (3, 1, 32, 64), (2, 1, 256, 16),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", ATTENTION_SHAPES)
@pytest.mark.parametrize("window", [0, 7])
def test_rope_write_then_attention(dtype, heads, kv_heads, head_dim, page_size, window):
    """Portions, whole prompts and single tokens in one launch, over shuffled pages with NaN in every unwritten slot."""
    from liteinfer_b200 import ops

    q_lens, ctx_lens = [1, 40, 1, 7, 33, 2], [90, 60, 3, 7, 33, 65]
    case = _paged_case(dtype, heads, kv_heads, head_dim, page_size, q_lens, ctx_lens)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, head_dim, 2).float() / head_dim))).cuda()
    outs = []
    for impl in (ops, ref):
        qkv, k_pool, v_pool = case["qkv"].clone(), case["k_pool"].clone(), case["v_pool"].clone()
        impl.rope_kv_write(qkv, case["positions"], case["seq_of"], case["table"], k_pool, v_pool, inv_freq, heads,
                           kv_heads, head_dim, head_dim)
        out = torch.empty(case["T"], heads * head_dim, dtype=dtype, device="cuda")
        impl.paged_attention(qkv, qkv.shape[1], out, k_pool, v_pool, case["table"], case["qsl"], case["ctx"],
                             case["B"], max(q_lens), heads, kv_heads, head_dim, head_dim ** -0.5, window)
        outs.append((qkv, k_pool, v_pool, out))
    for got, want in zip(outs[0], outs[1]):
        written = ~torch.isnan(want.float())
        assert torch.equal(torch.isnan(got.float()), ~written)      # nothing written outside the requests' slots
        torch.testing.assert_close(got.float()[written], want.float()[written], **_tol(dtype))
    assert torch.isfinite(outs[0][3].float()).all()


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(dtype):
    """One key among hundreds is made to dominate: the output must be that key's value, wherever its page lies."""
    from liteinfer_b200 import ops

    heads, kv_heads, d, page = 4, 2, 64, 16
    ctx = 700
    for far in (0, 15, 16, 333, 698):
        case = _paged_case(dtype, heads, kv_heads, d, page, [1], [ctx], seed=far, poison=True)
        qkv, k_pool, v_pool = case["qkv"], case["k_pool"], case["v_pool"]
        # the new token's own key/value must be in the pool too (position ctx-1)
        ops.rope_kv_write(qkv, case["positions"], case["seq_of"], case["table"], k_pool, v_pool, None, heads,
                          kv_heads, d, 0)
        q = qkv[:, :heads * d].view(1, heads, d)
        pg, off = int(case["table"][0, far // page]), far % page
        for h in range(kv_heads):
            k_pool[pg, h, off] = (q[0, h * 2].float() * 8).to(dtype)    # aligned with the first head of the group
        out = torch.empty(1, heads * d, dtype=dtype, device="cuda")
        ops.paged_attention(qkv, qkv.shape[1], out, k_pool, v_pool, case["table"], case["qsl"], case["ctx"], 1, 1,
                            heads, kv_heads, d, 1.0)
        for h in range(kv_heads):
            torch.testing.assert_close(out.view(heads, d)[h * 2].float(), v_pool[pg, h, off].float(),
                                       rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edge(dtype):
    """With a window of w the key at distance w-1 is seen and the key at distance w is not."""
    from liteinfer_b200 import ops

    heads, kv_heads, d, page, w, ctx = 2, 1, 32, 8, 11, 50
    for distance, seen in ((w - 1, True), (w, False)):
        case = _paged_case(dtype, heads, kv_heads, d, page, [1], [ctx], seed=3, poison=False)
        qkv, k_pool, v_pool = case["qkv"], case["k_pool"], case["v_pool"]
        ops.rope_kv_write(qkv, case["positions"], case["seq_of"], case["table"], k_pool, v_pool, None, heads,
                          kv_heads, d, 0)
        far = ctx - 1 - distance
        pg, off = int(case["table"][0, far // page]), far % page
        k_pool[pg, 0, off] = (qkv[0, :d].float() * 10).to(dtype)
        v_pool[pg, 0, off] = 100.0
        out = torch.empty(1, heads * d, dtype=dtype, device="cuda")
        ops.paged_attention(qkv, qkv.shape[1], out, k_pool, v_pool, case["table"], case["qsl"], case["ctx"], 1, 1,
                            heads, kv_heads, d, 1.0, w)
        assert (out[0, :d].float().mean() > 50) == seen


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab", [512, 1000, 128256])
def test_argmax(dtype, vocab):
    from liteinfer_b200 import ops

    logits = _randn(5, vocab, dtype=dtype)
    logits[2, vocab - 1] = 50.0
    logits[3, 7] = logits[3, 300] = 60.0     # equal values: the lower index wins
    got = ops.argmax(logits, torch.empty(5, dtype=torch.int32, device="cuda"))
    want = ref.argmax(logits.cpu(), torch.empty(5, dtype=torch.int32))
    assert got.cpu().tolist() == want.tolist() and got[2] == vocab - 1 and got[3] == 7


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab", [50, 1000])
def test_sample_matches_the_rule(dtype, vocab):
    """Temperature, top-k and top-p, with ties at the boundaries, against the row-by-row rule."""
    from liteinfer_b200 import ops

    g = torch.Generator().manual_seed(0)
    rows = 24
    logits = (torch.randn(rows, vocab, generator=g) * 2).to(dtype)
    logits[1, 3] = logits[1, 17] = logits[1, 30] = logits[1].float().max() + 1     # ties at the top
    logits[2] = logits[2].float().round().to(dtype)                               # many ties everywhere
    temps = torch.tensor([0.0, 1.0, 0.7, 2.5] * 6)
    top_k = torch.tensor([0, 1, 2, 5, 0, 40, 3, 0, vocab, vocab + 5, 7, 0] * 2, dtype=torch.int32)
    top_p = torch.tensor([1.0, 0.9, 0.5, 1.0, 0.1, 0.95] * 4)
    for trial in range(4):
        u = torch.rand(rows, generator=g)
        got = ops.sample(logits.cuda(), temps.cuda(), top_k.cuda(), top_p.cuda(), u.cuda(),
                         torch.empty(rows, dtype=torch.int32, device="cuda")).cpu()
        for r in range(rows):
            want = ref.sample_row(logits[r], float(temps[r]), int(top_k[r]), float(top_p[r]), float(u[r]))
            if int(got[r]) != want:
                # A draw that lands within rounding of a boundary of the running sum may fall either side of it.
                lo = ref.sample_row(logits[r], float(temps[r]), int(top_k[r]), float(top_p[r]), max(0.0, float(u[r]) - 1e-5))
                hi = ref.sample_row(logits[r], float(temps[r]), int(top_k[r]), float(top_p[r]), min(0.999999, float(u[r]) + 1e-5))
                assert int(got[r]) in (lo, hi), f"row {r}: got {int(got[r])}, rule gives {want}"


def test_sample_distribution():
    """Many draws of one row follow softmax(logits / T) restricted to the top-k."""
    from liteinfer_b200 import ops

    vocab, n = 40, 20000
    g = torch.Generator().manual_seed(1)
    row = torch.randn(vocab, generator=g)
    logits = row.repeat(n, 1).cuda()
    u = torch.rand(n, generator=g).cuda()
    got = ops.sample(logits, torch.full((n,), 0.8).cuda(), torch.full((n,), 10, dtype=torch.int32).cuda(),
                     torch.ones(n).cuda(), u, torch.empty(n, dtype=torch.int32, device="cuda")).cpu()
    keep = torch.topk(row, 10).indices
    p = torch.zeros(vocab)
    p[keep] = torch.softmax(row[keep] / 0.8, -1)
    freq = torch.bincount(got.long(), minlength=vocab).float() / n
    assert float((freq - p).abs().max()) < 0.015
    assert set(got.tolist()) <= set(keep.tolist())


@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16, 17, 33, 64])
@pytest.mark.parametrize("N,K", [(3072, 2048), (2048, 8192), (1000, 96), (17, 40), (128256 // 8, 2048), (48, 16384)])
def test_gemm_skinny(M, N, K):
    from liteinfer_b200 import ops

    x, w = _randn(M, K, dtype=torch.bfloat16), _randn(N, K, dtype=torch.bfloat16, seed=1, scale=0.05)
    b = _randn(N, dtype=torch.bfloat16, seed=2)
    got = ops.gemm_skinny(x, w, torch.empty(M, N, dtype=torch.bfloat16, device="cuda"), b)
    want = x.double() @ w.double().t() + b.double()
    torch.testing.assert_close(got.double(), want, rtol=2 ** -7, atol=2 ** -7)


def test_gemm_skinny_rows_do_not_depend_on_the_batch():
    from liteinfer_b200 import ops

    x, w = _randn(64, 2048, dtype=torch.bfloat16), _randn(555, 2048, dtype=torch.bfloat16, seed=1, scale=0.05)
    full = ops.gemm_skinny(x, w, torch.empty(64, 555, dtype=torch.bfloat16, device="cuda"))
    for rows in (1, 8, 20):
        part = ops.gemm_skinny(x[:rows].contiguous(), w, torch.empty(rows, 555, dtype=torch.bfloat16, device="cuda"))
        assert torch.equal(part, full[:rows])


def test_linear_hands_narrow_batches_to_the_streaming_kernel():
    """Up to 8 rows of x always, up to 16 for weights of few rows: `linear` then gives what the kernel gives."""
    from liteinfer_b200 import ops

    for M, N, streams in ((8, 8192, True), (12, 2048, True), (16, 4096, True), (17, 2048, False), (12, 8192, False)):
        x, w = _randn(M, 512, dtype=torch.bfloat16), _randn(N, 512, dtype=torch.bfloat16, seed=1, scale=0.05)
        before = ops.kernels.launch_count
        out = ops.linear(x, w, torch.empty(M, N, dtype=torch.bfloat16, device="cuda"))
        assert (ops.kernels.launch_count > before) == streams     # library products are not counted
        torch.testing.assert_close(out.double(), x.double() @ w.double().t(), rtol=2 ** -7, atol=2 ** -7)
        if streams:
            assert torch.equal(out, ops.gemm_stream(x, w, torch.empty(M, N, dtype=torch.bfloat16, device="cuda")))


def test_gemm_skinny_refuses_what_it_cannot_do():
    from liteinfer_b200 import ops
    from liteinfer_b200.ops import KernelLibraryError

    x, w = _randn(65, 64, dtype=torch.bfloat16), _randn(16, 64, dtype=torch.bfloat16)
    with pytest.raises(KernelLibraryError, match="refuses"):
        ops.gemm_skinny(x, w, torch.empty(65, 16, dtype=torch.bfloat16, device="cuda"))
    x, w = _randn(2, 100, dtype=torch.bfloat16), _randn(16, 100, dtype=torch.bfloat16)
    with pytest.raises(KernelLibraryError, match="refuses"):
        ops.gemm_skinny(x, w, torch.empty(2, 16, dtype=torch.bfloat16, device="cuda"))
    # ...while `linear` takes any shape, by handing what the kernel refuses to the library product.
    out = ops.linear(x, w, torch.empty(2, 16, dtype=torch.bfloat16, device="cuda"))
    torch.testing.assert_close(out.double(), x.double() @ w.double().t(), rtol=2 ** -7, atol=2 ** -7)


def _plan_for(q_lens, ctx_lens):
    from liteinfer_b200.parts.context import AttentionPlan

    dec = [i for i, q in enumerate(q_lens) if q == 1]
    pre = [i for i, q in enumerate(q_lens) if q > 1]
    starts = [0]
    for q in q_lens:
        starts.append(starts[-1] + q)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    return AttentionPlan(num_decode=len(dec), decode_seqs=i32(dec), decode_tokens=i32([starts[i] for i in dec]),
                         num_prefill=len(pre), prefill_seqs=i32(pre),
                         max_prefill_query_len=max([q_lens[i] for i in pre], default=0),
                         max_decode_context_len=max([ctx_lens[i] for i in dec], default=0))


def _splits(splits, monkeypatch):
    """`"11 as a cluster"`: 11 splits with the streaming kernel's merge through a cluster switched on."""
    if isinstance(splits, str):
        monkeypatch.setenv("LITEINFER_ATTN_CLUSTER_MERGE", "1")
        return int(splits.split()[0])
    return splits


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", [(4, 2, 64, 16), (8, 8, 64, 8), (32, 8, 128, 16),
                                                               (6, 2, 128, 5), (64, 1, 64, 32), (5, 1, 64, 16)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("splits", [None, 1, 3, 32, "2 as a cluster", "11 as a cluster", "16 as a cluster"])
def test_tensor_core_attention_against_the_plain_kernel(heads, kv_heads, head_dim, page_size, window, splits,
                                                        monkeypatch):
    """Portions and single tokens, planned (split decode rows beside unsplit portions) or not, over
    contexts that straddle the 64-key tiles, with NaN in every slot no request owns."""
    from liteinfer_b200 import ops

    splits = _splits(splits, monkeypatch)
    q_lens = [1, 130, 1, 7, 64, 1, 1, 2]
    ctx_lens = [700, 190, 1, 7, 64, 63, 65, 129]
    case = _paged_case(torch.bfloat16, heads, kv_heads, head_dim, page_size, q_lens, ctx_lens)
    qkv, k_pool, v_pool = case["qkv"], case["k_pool"], case["v_pool"]
    ops.rope_kv_write(qkv, case["positions"], case["seq_of"], case["table"], k_pool, v_pool, None, heads, kv_heads,
                      head_dim, 0)
    args = (qkv, qkv.shape[1])
    rest = (k_pool, v_pool, case["table"], case["qsl"], case["ctx"], case["B"], max(q_lens), heads, kv_heads,
            head_dim, head_dim ** -0.5, window)
    want = ref.paged_attention(*args, torch.empty(case["T"], heads * head_dim, dtype=torch.bfloat16, device="cuda"), *rest)
    out = torch.full((case["T"], heads * head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
    plan = None if splits is None else _plan_for(q_lens, ctx_lens)
    got = ops.paged_attention(*args, out, *rest, plan=plan, decode_splits=splits if splits and splits > 1 else None)
    assert torch.isfinite(got.float()).all()
    torch.testing.assert_close(got.float(), want.float(), rtol=2 ** -6, atol=2 ** -6)


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", [(32, 8, 64, 16), (8, 8, 64, 8), (16, 1, 128, 16),
                                                               (6, 2, 128, 5), (5, 1, 64, 32)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("splits", [1, 3, 32, "11 as a cluster", "16 as a cluster"])
def test_decode_attention_with_rotary_and_cache_write_fused(heads, kv_heads, head_dim, page_size, window, splits,
                                                            monkeypatch):
    """One launch that rotates q and the newest key, stores key and value and attends, against the two
    launches it replaces: the same output and the same pages, to the bit; contexts end at, just before and
    just after the edges of pages and of 64-key tiles."""
    from liteinfer_b200 import ops

    splits = _splits(splits, monkeypatch)
    ctx_lens = [700, 1, 64, 65, 63, 129, 320, 16, 17]
    q_lens = [1] * len(ctx_lens)
    case = _paged_case(torch.bfloat16, heads, kv_heads, head_dim, page_size, q_lens, ctx_lens, seed=3)
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, head_dim, 2).float() / head_dim))).cuda()
    plan = _plan_for(q_lens, ctx_lens)
    rest = (case["table"], case["qsl"], case["ctx"], case["B"], 1, heads, kv_heads, head_dim, head_dim ** -0.5, window)
    q_width, kv_width = heads * head_dim, kv_heads * head_dim

    qkv, k_two, v_two = case["qkv"].clone(), case["k_pool"].clone(), case["v_pool"].clone()
    ops.rope_kv_write(qkv, case["positions"], case["seq_of"], case["table"], k_two, v_two, inv_freq, heads, kv_heads,
                      head_dim, head_dim)
    want = ops.paged_attention(qkv, qkv.shape[1], torch.empty(case["T"], q_width, dtype=torch.bfloat16, device="cuda"),
                               k_two, v_two, *rest, plan=plan, decode_splits=splits)

    qkv, k_one, v_one = case["qkv"].clone(), case["k_pool"].clone(), case["v_pool"].clone()
    assert ops.fused_decode_supports(torch.bfloat16, heads, kv_heads, head_dim, head_dim, plan)
    newest = ops.NewestToken(inv_freq, qkv[:, q_width:], qkv[:, q_width + kv_width:])
    got = ops.paged_attention(qkv, qkv.shape[1], torch.empty(case["T"], q_width, dtype=torch.bfloat16, device="cuda"),
                              k_one, v_one, *rest, plan=plan, decode_splits=splits, newest=newest)
    assert torch.equal(got, want)
    for one, two in ((k_one, k_two), (v_one, v_two)):
        assert torch.equal(torch.isnan(one.float()), torch.isnan(two.float()))
        assert torch.equal(torch.nan_to_num(one.float()), torch.nan_to_num(two.float()))

    # A layer that reads another layer's pages: the newest token is there already and nothing is written.
    frozen_k, frozen_v = k_two.clone(), v_two.clone()
    newest = ops.NewestToken(inv_freq, qkv[:, q_width:], qkv[:, q_width + kv_width:], store=False)
    again = ops.paged_attention(qkv, qkv.shape[1], torch.empty_like(got), frozen_k, frozen_v, *rest, plan=plan,
                                decode_splits=splits, newest=newest)
    assert torch.equal(again, want)
    assert torch.equal(torch.nan_to_num(frozen_k.float()), torch.nan_to_num(k_two.float()))


def test_tensor_core_attention_finds_one_far_key_under_splits():
    from liteinfer_b200 import ops

    heads, kv_heads, d, page, ctx = 8, 2, 128, 16, 3000
    for far in (0, 63, 64, 1500, 2998):
        case = _paged_case(torch.bfloat16, heads, kv_heads, d, page, [1], [ctx], seed=far)
        qkv, k_pool, v_pool = case["qkv"], case["k_pool"], case["v_pool"]
        ops.rope_kv_write(qkv, case["positions"], case["seq_of"], case["table"], k_pool, v_pool, None, heads,
                          kv_heads, d, 0)
        q = qkv[:, :heads * d].view(1, heads, d)
        pg, off = int(case["table"][0, far // page]), far % page
        for h in range(kv_heads):
            k_pool[pg, h, off] = (q[0, h * 4].float() * 4).to(torch.bfloat16)
        out = torch.empty(1, heads * d, dtype=torch.bfloat16, device="cuda")
        ops.paged_attention(qkv, qkv.shape[1], out, k_pool, v_pool, case["table"], case["qsl"], case["ctx"], 1, 1,
                            heads, kv_heads, d, 1.0, 0, plan=_plan_for([1], [ctx]))
        for h in range(kv_heads):
            torch.testing.assert_close(out.view(heads, d)[h * 4].float(), v_pool[pg, h, off].float(),
                                       rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("words,n_late", [(40, 0), (2105, 8), (16384, 64), (16385, 3)])
def test_stage_batch_equals_copy_and_scatter(words, n_late):
    """The kernel that reads a pinned batch in place and places the late tokens gives what the copy followed by the
    scatter gives; a batch beyond its limit is refused (the caller copies)."""
    from liteinfer_b200 import ops

    g = torch.Generator().manual_seed(words)
    tok_len, n = 16, max(n_late, 1)                      # layout: tokens [0, 16), dst [20, 20 + n), src after it
    host = torch.randint(0, 1000, (words,), generator=g, dtype=torch.int32)
    dst = torch.full((n,), -1, dtype=torch.int32)
    places = torch.randperm(tok_len, generator=g).to(torch.int32)
    for i in range(0, min(n_late, 2 * tok_len), 2):      # every second entry names a place, each place once
        dst[i] = places[i // 2]
    host[20:20 + n] = dst
    host[20 + n:20 + 2 * n] = torch.randint(0, 32, (n,), generator=g, dtype=torch.int32)
    host = host.pin_memory()
    source = torch.randint(0, 50000, (32,), generator=g, dtype=torch.int32).cuda()
    views = lambda t: (t[:tok_len], t[20:20 + n], t[20 + n:20 + 2 * n])
    want = host.cuda()
    if n_late:
        ops.scatter_tokens(*views(want), source)
    device = torch.full((words,), -7, dtype=torch.int32, device="cuda")
    done = ops.stage_batch(device, host, *views(device), source if n_late else None)
    assert done == (words <= ops.kernels.STAGE_KERNEL_MAX_WORDS)
    if done:
        torch.cuda.synchronize()
        assert torch.equal(device, want)


def test_split_policy():
    from liteinfer_b200.ops import decode_splits_for

    assert decode_splits_for(1, 8, 100) == 1            # fewer than four key tiles: nothing to split
    assert decode_splits_for(1, 8, 4096) == 32
    assert 2 <= decode_splits_for(8, 8, 4096) <= 16
    assert decode_splits_for(64, 8, 4096) == 1


def test_split_policy_with_the_cluster_merge(monkeypatch):
    """With the switch on, the streaming kernel gets a count whose splits can be one cluster each, all of them
    resident at once."""
    from liteinfer_b200.ops import decode_splits_for, kernels

    monkeypatch.setenv("LITEINFER_ATTN_CLUSTER_MERGE", "1")
    for batch in (1, 4, 8, 16):
        chosen = decode_splits_for(batch, 8, 4096, 64, True)
        assert 2 <= chosen <= 16 and kernels.cluster_capacity(64, chosen) >= batch * 8, (batch, chosen)


def _interleave(gate, up):
    rest = gate.shape[1:]
    return torch.stack([gate.reshape(-1, 8, *rest), up.reshape(-1, 8, *rest)], dim=1).reshape(2 * gate.shape[0], *rest).contiguous()


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("inter,K,act", [(8192, 2048, "silu"), (112, 120, "gelu_pytorch_tanh"), (176, 64, "relu")])
@pytest.mark.parametrize("with_bias", [False, True])
def test_gated_linear_is_product_activation_and_multiply_in_one(M, inter, K, act, with_bias):
    from liteinfer_b200 import ops

    dt = torch.bfloat16
    x = _randn(M, K, dtype=dt)
    gate, up = _randn(inter, K, dtype=dt, seed=1, scale=0.05), _randn(inter, K, dtype=dt, seed=2, scale=0.05)
    bg, bu = _randn(inter, dtype=dt, seed=3), _randn(inter, dtype=dt, seed=4)
    w = _interleave(gate, up)
    b = _interleave(bg, bu) if with_bias else None
    got = ops.gated_linear(x, w, torch.empty(M, inter, dtype=dt, device="cuda"), act, b)
    # the same thing in two kernels, through the same layout: bit for bit
    gu = ops.linear(x, w, torch.empty(M, 2 * inter, dtype=dt, device="cuda"), b)
    two = ops.act_mul_interleaved(gu, torch.empty(M, inter, dtype=dt, device="cuda"), act)
    assert torch.equal(got, two)
    # and the plain formula on the plain layout
    gu_plain = torch.cat([x.double() @ gate.double().t() + (bg.double() if with_bias else 0),
                          x.double() @ up.double().t() + (bu.double() if with_bias else 0)], dim=1).to(dt)
    want = ref.act_mul(gu_plain, torch.empty(M, inter, dtype=dt, device="cuda"), act)
    torch.testing.assert_close(got.float(), want.float(), rtol=2 ** -6, atol=2 ** -6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_act_mul_interleaved(dtype):
    from liteinfer_b200 import ops

    gu = _randn(5, 2 * 176, dtype=dtype, scale=2.0)
    got = ops.act_mul_interleaved(gu, torch.empty(5, 176, dtype=dtype, device="cuda"), "silu")
    want = ref.act_mul_interleaved(gu, torch.empty(5, 176, dtype=dtype, device="cuda"), "silu")
    torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))


def test_skinny_slices_leave_their_counters_at_zero():
    from liteinfer_b200 import ops
    from liteinfer_b200.ops.kernels import scratch_for

    # Few rows of w: wide blocks; very few and a long k: slices of k as well.
    assert ops.gemm_skinny_plan(16384, 2048) == (2, 1) and ops.gemm_skinny_plan(3072, 2048) == (8, 1)
    assert ops.gemm_skinny_plan(8192, 2048) == (8, 1) and ops.gemm_skinny_plan(9600, 64) == (4, 1)
    assert ops.gemm_skinny_plan(2048, 8192) == (16, 1) and ops.gemm_skinny_plan(64, 32768) == (16, 4)
    x, w = _randn(8, 32768, dtype=torch.bfloat16), _randn(64, 32768, dtype=torch.bfloat16, seed=1, scale=0.02)
    outs = [ops.gemm_skinny(x, w, torch.empty(8, 64, dtype=torch.bfloat16, device="cuda")) for _ in range(3)]
    torch.testing.assert_close(outs[0].double(), x.double() @ w.double().t(), rtol=2 ** -7, atol=2 ** -6)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    torch.cuda.synchronize()
    assert int(scratch_for(x.device).gemm_counters.abs().sum()) == 0
    assert int(scratch_for(x.device).attention_counters.abs().sum()) == 0


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (2048, 2048, 2048), (300, 1000, 96), (77, 136, 40), (129, 3072, 2048),
                                   (1024, 16384, 512), (256, 2048, 8192)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_gemm_tcgen05(M, N, K, with_bias):
    """The tcgen05 / TMA / tensor-memory product against a float64 product, at sizes that leave ragged tiles in
    every direction, for the kernel of single CTAs (fewer than 256 rows or columns) and the one of CTA pairs; no
    wait inside the kernel may have given up."""
    from liteinfer_b200 import ops

    x, w = _randn(M, K, dtype=torch.bfloat16), _randn(N, K, dtype=torch.bfloat16, seed=1, scale=0.05)
    b = _randn(N, dtype=torch.bfloat16, seed=2) if with_bias else None
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tcgen05(x, w, out, b)
    want = x.double() @ w.double().t() + (b.double() if with_bias else 0)
    assert ops.gemm_error_flag("cuda:0") == 0
    torch.testing.assert_close(out.double(), want, rtol=2 ** -7, atol=2 ** -6)


@pytest.mark.parametrize("M,inter,K,act", [(2048, 8192, 2048, "silu"), (130, 176, 64, "gelu_pytorch_tanh"),
                                           (500, 112, 120, "relu"), (300, 504, 96, "silu"), (257, 128, 4096, "gelu")])
def test_gemm_tcgen05_gated_epilogue(M, inter, K, act):
    """act(gate) * up in the product's epilogue equals the library product followed by the activation kernel,
    bit for bit without a bias (the same sums rounded at the same places)."""
    from liteinfer_b200 import ops

    dt = torch.bfloat16
    x = _randn(M, K, dtype=dt)
    w = _interleave(_randn(inter, K, dtype=dt, seed=1, scale=0.05), _randn(inter, K, dtype=dt, seed=2, scale=0.05))
    got = ops.gemm_tcgen05(x, w, torch.empty(M, inter, dtype=dt, device="cuda"), None, act)
    gu = ops.linear(x, w, torch.empty(M, 2 * inter, dtype=dt, device="cuda"))
    two = ops.act_mul_interleaved(gu, torch.empty(M, inter, dtype=dt, device="cuda"), act)
    assert ops.gemm_error_flag("cuda:0") == 0
    # the library may add its products in another order: a rounding of the bfloat16 product apart at most
    torch.testing.assert_close(got.float(), two.float(), rtol=2 ** -6, atol=2 ** -6)


@pytest.mark.parametrize("heads,kv_heads,page_size", [(4, 1, 16), (32, 8, 16), (8, 8, 32), (16, 2, 64), (128, 1, 16),
                                                      (24, 8, 16), (5, 1, 32), (7, 7, 16)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("d", [64, 128])
def test_tcgen05_attention_against_the_plain_kernel(heads, kv_heads, page_size, window, d, monkeypatch):
    """The tcgen05 / TMA / tensor-memory attention kernel: portions, whole prompts and single tokens over shuffled
    pages, NaN in every slot no request owns, contexts that straddle the 64-key tiles; no wait may give up."""
    from liteinfer_b200 import ops

    q_lens, ctx_lens = [1, 130, 1, 7, 64, 2, 257], [700, 190, 1, 7, 64, 129, 300]
    case = _paged_case(torch.bfloat16, heads, kv_heads, d, page_size, q_lens, ctx_lens)
    qkv, k_pool, v_pool = case["qkv"], case["k_pool"], case["v_pool"]
    ops.rope_kv_write(qkv, case["positions"], case["seq_of"], case["table"], k_pool, v_pool, None, heads, kv_heads, d, 0)
    rest = (k_pool, v_pool, case["table"], case["qsl"], case["ctx"])
    tail = (case["B"], max(q_lens), heads, kv_heads, d, d ** -0.5, window)
    want = ref.paged_attention(qkv, qkv.shape[1], torch.empty(case["T"], heads * d, dtype=torch.bfloat16, device="cuda"),
                               *rest, *tail)
    out = torch.full((case["T"], heads * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert ops.tcgen05_attention_supports(torch.bfloat16, heads, kv_heads, d, page_size)
    ops.paged_attention_tcgen05(qkv, qkv.shape[1], out, *rest, None, *tail)
    assert ops.gemm_error_flag("cuda:0") == 0
    assert torch.isfinite(out.float()).all()
    torch.testing.assert_close(out.float(), want.float(), rtol=2 ** -6, atol=2 ** -6)


def test_tcgen05_attention_refuses_what_it_cannot_do():
    from liteinfer_b200 import ops

    assert not ops.tcgen05_attention_supports(torch.bfloat16, 129, 1, 64, 16)    # a group larger than a block's rows
    assert not ops.tcgen05_attention_supports(torch.bfloat16, 4, 2, 96, 16)      # head size 96: the plain kernel
    assert not ops.tcgen05_attention_supports(torch.bfloat16, 4, 2, 64, 8)       # pages of 8
    assert not ops.tcgen05_attention_supports(torch.float32, 4, 2, 64, 16)


@pytest.mark.parametrize("M", [1, 5, 8, 13])
@pytest.mark.parametrize("N,K", [(3072, 2048), (2048, 8192), (1000, 96), (64, 32768)])
def test_streaming_product_adds_into_the_residual_stream(M, N, K, monkeypatch):
    """With `residual` the weight-streaming kernel adds its result into the stream itself (the same bits as the
    product followed by the 32-bit sum rounded once) and leaves the new rows' sums of squares in parts."""
    from liteinfer_b200 import ops

    monkeypatch.setattr(ops.kernels, "FUSED_NORM", True)       # the fusion is a switch (off by default)
    x, w = _randn(M, K, dtype=torch.bfloat16), _randn(N, K, dtype=torch.bfloat16, seed=1, scale=0.05)
    b = _randn(N, dtype=torch.bfloat16, seed=2)
    stream = _randn(M, N, dtype=torch.bfloat16, seed=3, scale=2.0)
    product = ops.linear(x, w, torch.empty(M, N, dtype=torch.bfloat16, device="cuda"), b)
    want = (stream.float() + product.float()).to(torch.bfloat16)
    got = stream.clone()
    stats = ops.linear(x, w, None, b, residual=got)
    assert isinstance(stats, ops.RowStats) and stats.sumsq.shape == (-(-N // 16), M)
    assert torch.equal(got, want)
    torch.testing.assert_close(stats.sumsq.sum(0), want.float().pow(2).sum(-1), rtol=1e-5, atol=1e-5)
    again = stream.clone()
    assert torch.equal(ops.linear(x, w, None, b, residual=again).sumsq, stats.sumsq) and torch.equal(again, got)


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("N,K,gated", [(3072, 2048, False), (16384, 2048, True), (1000, 96, False), (352, 64, True),
                                       (128256 // 4, 2048, False)])
def test_streaming_product_folds_the_norm_in(M, N, K, gated):
    """A pending norm as the product's input: weight * x / rms(x) with the statistics from the parts that the
    product before left, for all rows or for rows picked by index; against the norm kernel followed by the
    product, within bfloat16 rounding (the fused form rounds once less), and against float64."""
    from liteinfer_b200 import ops

    rows_total = M + 3
    hidden = _randn(rows_total, K, dtype=torch.bfloat16, seed=4, scale=3.0)
    wn = (1 + 0.1 * _randn(K, dtype=torch.float32, seed=5)).to(torch.bfloat16)
    w = _randn(N, K, dtype=torch.bfloat16, seed=1, scale=0.02)          # results of magnitude one
    # the statistics as a product of 7 column tiles would have left them
    parts = torch.stack([c.float().pow(2).sum(-1) for c in hidden.chunk(7, dim=1)])
    for rows in (None, torch.tensor(list(range(rows_total - 1, rows_total - 1 - M, -1)), dtype=torch.int32, device="cuda")):
        if rows is None:
            source, stats = hidden[:M].contiguous(), ops.RowStats(parts[:, :M].contiguous())
        else:
            source, stats = hidden, ops.RowStats(parts.contiguous())
        pending = ops.PendingNorm(source, wn, 1e-5, stats, rows)
        normed = pending.materialise()
        picked = source if rows is None else source[rows.long()]
        exact = (picked.double() / torch.sqrt(picked.double().pow(2).mean(-1, keepdim=True) + 1e-5)) * wn.double()
        if gated:
            got = ops.gated_linear(pending, w, torch.empty(M, N // 2, dtype=torch.bfloat16, device="cuda"), "silu")
            two = ops.gated_linear(normed, w, torch.empty(M, N // 2, dtype=torch.bfloat16, device="cuda"), "silu")
        else:
            got = ops.linear(pending, w, None)
            two = ops.linear(normed, w, None)
            torch.testing.assert_close(got.double(), exact @ w.double().t(), rtol=2 ** -6, atol=2 ** -6)
        # (the two-kernel form rounds the normalised row once more than the fused one: each is within a rounding of
        # the exact product, so they are within two of each other)
        torch.testing.assert_close(got.float(), two.float(), rtol=2 ** -5, atol=2 ** -5)


def test_fused_decode_layer_chain_matches_the_unfused_one(monkeypatch):
    """Norm -> product -> residual -> norm -> gated product -> product -> residual, as a decode step of five
    tokens runs it (two fused products per half layer), against the same chain kernel by kernel."""
    from liteinfer_b200.parts.block import apply_norm, run_part
    from liteinfer_b200.parts.feed_forward import GatedMLP
    from liteinfer_b200.parts.norm import RMSNorm
    from liteinfer_b200 import ops

    dev, dt, h, inter = torch.device("cuda:0"), torch.bfloat16, 256, 512
    norm = RMSNorm(h, 1e-5, dt, dev)
    hidden = _randn(5, h, dtype=dt, seed=2)
    norm.bind({"weight": (1 + 0.1 * _randn(h, dtype=torch.float32, seed=1)).to(dt)})
    mlp = GatedMLP(h, inter, "silu", dt, dev)
    mlp.bind({n: _randn(*s.shape, dtype=dt, seed=10 + i, scale=0.05) for i, (n, s) in enumerate(mlp.tensor_specs().items())})
    # unfused: materialised norms, deltas added by the next norm
    a = hidden.clone()
    d1 = mlp.forward(norm.forward(a, None), None)
    d2 = mlp.forward(norm.forward(a, d1), None)
    want = (a.float() + d2.float())
    # fused: the parts add into the stream and hand on statistics
    monkeypatch.setattr(ops.kernels, "FUSED_NORM", True)
    b = hidden.clone()
    s1 = run_part(mlp, apply_norm(norm, b, None, mlp), b, None)
    assert isinstance(s1, ops.RowStats)
    pending = apply_norm(norm, b, s1, mlp)
    assert isinstance(pending, ops.PendingNorm)
    s2 = run_part(mlp, pending, b, None)
    assert isinstance(s2, ops.RowStats)
    torch.testing.assert_close(b.float(), want, rtol=2 ** -6, atol=2 ** -6)
    torch.testing.assert_close(s2.sumsq.sum(0), b.float().pow(2).sum(-1), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(3072, 2048), (2048, 8192), (1000, 96), (17, 40), (128256 // 8, 2048), (48, 16384),
                                 (16384, 2048), (5000, 200)])
def test_gemm_stream(M, N, K):
    """The persistent product with per-warp TMA rings against a float64 product: tiles past N, chunks past K (a k
    that is no multiple of 128, of 64, or smaller than one chunk), more tiles than blocks and fewer."""
    from liteinfer_b200 import ops

    x, w = _randn(M, K, dtype=torch.bfloat16), _randn(N, K, dtype=torch.bfloat16, seed=1, scale=0.05)
    b = _randn(N, dtype=torch.bfloat16, seed=2)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    got = ops.gemm_stream(x, w, out, b)
    want = x.double() @ w.double().t() + b.double()
    assert ops.gemm_error_flag("cuda:0") == 0
    torch.testing.assert_close(got.double(), want, rtol=2 ** -7, atol=2 ** -6 if K > 4096 else 2 ** -7)
    again = ops.gemm_stream(x, w, torch.empty_like(out), b)
    assert torch.equal(got, again)


def test_gemm_stream_rows_do_not_depend_on_the_batch():
    from liteinfer_b200 import ops

    x, w = _randn(16, 2048, dtype=torch.bfloat16), _randn(555, 2048, dtype=torch.bfloat16, seed=1, scale=0.05)
    full = ops.gemm_stream(x, w, torch.empty(16, 555, dtype=torch.bfloat16, device="cuda"))
    for rows in (1, 5, 8, 12):
        part = ops.gemm_stream(x[:rows].contiguous(), w, torch.empty(rows, 555, dtype=torch.bfloat16, device="cuda"))
        assert torch.equal(part, full[:rows])


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("inter,K,act", [(8192, 2048, "silu"), (112, 120, "gelu_pytorch_tanh"), (176, 64, "relu")])
def test_gemm_stream_epilogues(M, inter, K, act):
    """act(gate) * up in the epilogue equals the product followed by the activation kernel; the residual sum equals
    the product followed by a 32-bit sum rounded once, and leaves the sums of squares of the new rows."""
    from liteinfer_b200 import ops

    dt = torch.bfloat16
    x = _randn(M, K, dtype=dt)
    w = _interleave(_randn(inter, K, dtype=dt, seed=1, scale=0.05), _randn(inter, K, dtype=dt, seed=2, scale=0.05))
    b = _interleave(_randn(inter, dtype=dt, seed=3), _randn(inter, dtype=dt, seed=4))
    gu = ops.gemm_stream(x, w, torch.empty(M, 2 * inter, dtype=dt, device="cuda"), b)
    two = ops.act_mul_interleaved(gu, torch.empty(M, inter, dtype=dt, device="cuda"), act)
    got = ops.gemm_stream(x, w, torch.empty(M, inter, dtype=dt, device="cuda"), b, act)
    assert torch.equal(got, two)
    stream = _randn(M, 2 * inter, dtype=dt, seed=9, scale=2.0)
    want = (stream.float() + gu.float()).to(dt)
    stats = ops.gemm_stream(x, w, None, b, residual=stream)
    assert torch.equal(stream, want)
    torch.testing.assert_close(stats.sumsq.sum(0), want.float().pow(2).sum(-1), rtol=1e-5, atol=1e-5)
    assert ops.gemm_error_flag("cuda:0") == 0


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("w,ctx", [(11, 50), (64, 129), (65, 129), (16, 81), (100, 700)])
def test_window_edge_on_the_tensor_core_paths(d, w, ctx, monkeypatch):
    """With a window of w the key at distance w - 1 is seen and the key at distance w is not, on every path that
    bfloat16 heads of 64 and 128 take: single tokens with their keys unsplit and split, through the kernel with
    TMA rings and the one with shared-memory tiles, with the rotary encoding and the cache write fused in, and a
    portion of three tokens through the tcgen05 kernel.  The edge falls inside a tile of 64 keys, on its first key,
    on its last, and on a page's edge."""
    from liteinfer_b200 import ops

    heads, kv_heads, page, dt = 8, 2, 16, torch.bfloat16
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, d, 2).float() / d))).cuda()

    def planted(q_len, distance, rotate):
        case = _paged_case(dt, heads, kv_heads, d, page, [q_len], [ctx], seed=w + distance, poison=False)
        qkv, k_pool, v_pool = case["qkv"], case["k_pool"], case["v_pool"]
        rotated = qkv.clone()          # what the queries look like once they are rotated (or not)
        ref.rope_kv_write(rotated, case["positions"], case["seq_of"], case["table"], k_pool.clone(), v_pool.clone(),
                          inv_freq if rotate else None, heads, kv_heads, d, d if rotate else 0, store=False)
        far = ctx - 1 - distance
        pg, off = int(case["table"][0, far // page]), far % page
        last = rotated[q_len - 1, :heads * d].view(heads, d)
        for h in range(kv_heads):
            k_pool[pg, h, off] = (last[h * (heads // kv_heads)].float() * 10).to(dt)
            v_pool[pg, h, off] = 100.0
        return case, qkv, k_pool, v_pool

    def sees(out, q_len):
        return float(out[q_len - 1].view(heads, d)[0].float().mean()) > 50

    for distance, seen in ((w - 1, True), (w, False)):
        # single tokens, keys and values already in their pages
        for stream in ("1", "0"):
            monkeypatch.setenv("LITEINFER_DECODE_STREAM", stream)
            for splits in (1, 3):
                case, qkv, k_pool, v_pool = planted(1, distance, False)
                ops.rope_kv_write(qkv, case["positions"], case["seq_of"], case["table"], k_pool, v_pool, None, heads,
                                  kv_heads, d, 0)
                out = torch.empty(1, heads * d, dtype=dt, device="cuda")
                ops.paged_attention(qkv, qkv.shape[1], out, k_pool, v_pool, case["table"], case["qsl"], case["ctx"], 1, 1,
                                    heads, kv_heads, d, 1.0, w, plan=_plan_for([1], [ctx]), decode_splits=splits)
                assert sees(out, 1) == seen, (stream, splits, distance)
        monkeypatch.setenv("LITEINFER_DECODE_STREAM", "1")
        # the rotary encoding and the cache write inside the attention launch
        for splits in (1, 3):
            case, qkv, k_pool, v_pool = planted(1, distance, True)
            q_width, kv_width = heads * d, kv_heads * d
            newest = ops.NewestToken(inv_freq, qkv[:, q_width:], qkv[:, q_width + kv_width:])
            out = torch.empty(1, heads * d, dtype=dt, device="cuda")
            ops.paged_attention(qkv, qkv.shape[1], out, k_pool, v_pool, case["table"], case["qsl"], case["ctx"], 1, 1,
                                heads, kv_heads, d, 1.0, w, plan=_plan_for([1], [ctx]), decode_splits=splits, newest=newest)
            assert sees(out, 1) == seen, ("fused", splits, distance)
        # a portion of three tokens: the tcgen05 kernel
        case, qkv, k_pool, v_pool = planted(3, distance, False)
        ops.rope_kv_write(qkv, case["positions"], case["seq_of"], case["table"], k_pool, v_pool, None, heads, kv_heads, d, 0)
        assert ctx - 1 - distance < ctx - 3      # the planted key lies before the portion's own keys
        out = torch.empty(3, heads * d, dtype=dt, device="cuda")
        assert ops.tcgen05_attention_supports(dt, heads, kv_heads, d, page)
        ops.paged_attention(qkv, qkv.shape[1], out, k_pool, v_pool, case["table"], case["qsl"], case["ctx"], 1, 3,
                            heads, kv_heads, d, 1.0, w, plan=_plan_for([3], [ctx]))
        assert sees(out, 3) == seen, ("portion", distance)
    assert ops.gemm_error_flag("cuda:0") == 0
