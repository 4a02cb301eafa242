"""Times single kernels at the sizes of a decode or prefill step: `python -m liteinfer_b200.kernel_bench`.

Each case runs its kernel alone on inputs larger than the L2 cache (several
copies of the operands are cycled through), times it with CUDA events after a
warm-up, and prints one JSON line with the time, the bytes or flops the kernel
must move or do, and what that is per second.  `--kernel` picks one case, which
is what a profiler capture of a single kernel needs.
"""

from __future__ import annotations

import argparse
import json

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.context import AttentionPlan


def _time(fn, copies: int, iters: int = 20, warmup: int = 3) -> float:
    """Median microseconds of one fn(i % copies), measured on the device: `copies` calls are captured into a
    CUDA graph (so that the host's launch cost stays out of it) and the graph is replayed."""
    for i in range(warmup):
        fn(i % copies)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(copies):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3 / copies)
    times.sort()
    return times[len(times) // 2]


def skinny(M: int, N: int, K: int) -> dict:
    copies = max(2, (300 << 20) // (N * K * 2) + 1)
    w = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    us = _time(lambda i: ops.gemm_skinny(x, w[i], out), copies)
    nbytes = N * K * 2 + M * K * 2 + M * N * 2
    return {"kernel": "gemm_skinny", "M": M, "N": N, "K": K, "us": us, "GBps": nbytes / us / 1e3,
            "warps": ops.gemm_skinny_plan(N, K)[0], "slices": ops.gemm_skinny_plan(N, K)[1]}


def stream_gemm(M: int, N: int, K: int, gated: bool = False) -> dict:
    copies = max(2, (300 << 20) // (N * K * 2) + 1)
    w = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N // 2 if gated else N, device="cuda", dtype=torch.bfloat16)
    us = _time(lambda i: ops.gemm_stream(x, w[i], out, None, "silu" if gated else None), copies)
    return {"kernel": "gemm_stream" + ("+silu*up" if gated else ""), "M": M, "N": N, "K": K, "us": us,
            "GBps": N * K * 2 / us / 1e3, "wait_that_gave_up": ops.gemm_error_flag("cuda:0")}


def skinny_fused(M: int, N: int, K: int, norm: bool, residual: bool, gated: bool = False) -> dict:
    """The weight-streaming product with the norm before it folded in and / or the residual sum after it."""
    copies = max(2, (300 << 20) // (N * K * 2) + 1)
    w = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    wn = torch.ones(K, device="cuda", dtype=torch.bfloat16)
    stats = ops.RowStats(torch.rand(K // 16, M, device="cuda") * 16)
    source = ops.PendingNorm(x, wn, 1e-5, stats) if norm else x
    stream = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N // 2 if gated else N, device="cuda", dtype=torch.bfloat16)

    def run(i):
        if gated:
            ops.gated_linear(source, w[i], out, "silu")
        else:
            ops.linear(source, w[i], None if residual else out, residual=stream if residual else None)

    us = _time(run, copies)
    return {"kernel": "gemm_skinny" + ("+norm" if norm else "") + ("+residual" if residual else "") + ("+silu*up" if gated else ""),
            "M": M, "N": N, "K": K, "us": us, "GBps": N * K * 2 / us / 1e3}


def mlp_chain(M: int, fused: bool, hidden: int = 2048, inter: int = 8192) -> dict:
    """norm -> gate_up + activation -> down -> residual sum, as one decode layer's second half runs it: kernel by
    kernel (three launches, the sum inside the next norm) or fused (two launches)."""
    copies = 4
    gu = [torch.randn(2 * inter, hidden, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    dn = [torch.randn(hidden, inter, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    wn = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
    stream = torch.randn(M, hidden, device="cuda", dtype=torch.bfloat16)
    mid = torch.empty(M, inter, device="cuda", dtype=torch.bfloat16)
    delta = torch.zeros(M, hidden, device="cuda", dtype=torch.bfloat16)
    normed = torch.empty(M, hidden, device="cuda", dtype=torch.bfloat16)
    state = {"stats": ops.RowStats(torch.rand(hidden // 16, M, device="cuda") * 16)}

    def run(i):
        if fused:
            ops.gated_linear(ops.PendingNorm(stream, wn, 1e-5, state["stats"]), gu[i], mid, "silu")
            state["stats"] = ops.linear(mid, dn[i], None, residual=stream)
        else:
            ops.rmsnorm(stream, wn, 1e-5, normed, delta=delta, write_residual=True)
            ops.gated_linear(normed, gu[i], mid, "silu")
            ops.linear(mid, dn[i], delta)

    us = _time(run, copies)
    return {"kernel": "mlp half layer " + ("fused" if fused else "kernel by kernel"), "M": M, "us": us,
            "GBps": (3 * inter * hidden * 2) / us / 1e3}


def tcgen05_gemm(M: int, N: int, K: int, gated: bool = False) -> dict:
    copies = max(2, (300 << 20) // (N * K * 2) + 1)
    w = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N // 2 if gated else N, device="cuda", dtype=torch.bfloat16)
    us = _time(lambda i: ops.gemm_tcgen05(x, w[i], out, None, "silu" if gated else None), copies)
    return {"kernel": "gemm_tcgen05" + ("+silu*up" if gated else ""), "M": M, "N": N, "K": K, "us": us,
            "TFLOPs": 2.0 * M * N * K / us / 1e6, "wait_that_gave_up": ops.gemm_error_flag("cuda:0")}


def library_gemm(M: int, N: int, K: int) -> dict:
    copies = max(2, (300 << 20) // (N * K * 2) + 1)
    w = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    us = _time(lambda i: torch.mm(x, w[i].t(), out=out), copies)
    return {"kernel": "library_mm", "M": M, "N": N, "K": K, "us": us, "GBps": (N * K * 2) / us / 1e3,
            "TFLOPs": 2.0 * M * N * K / us / 1e6}


def attention(batch: int, q_len: int, ctx: int, heads: int = 32, kv_heads: int = 8, head_dim: int = 64,
              page: int = 16, splits: int | None = None) -> dict:
    pages_per = -(-ctx // page)
    copies = max(2, (300 << 20) // (batch * ctx * kv_heads * head_dim * 4) + 1)
    num_pages = pages_per * batch
    pools = [(torch.randn(num_pages, kv_heads, page, head_dim, device="cuda", dtype=torch.bfloat16),
              torch.randn(num_pages, kv_heads, page, head_dim, device="cuda", dtype=torch.bfloat16))
             for _ in range(copies)]
    table = torch.randperm(num_pages, device="cuda").to(torch.int32).view(batch, pages_per)
    T = batch * q_len
    qkv = torch.randn(T, (heads + 2 * kv_heads) * head_dim, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, heads * head_dim, device="cuda", dtype=torch.bfloat16)
    qsl = (torch.arange(batch + 1, device="cuda") * q_len).to(torch.int32)
    ctxl = torch.full((batch,), ctx, device="cuda", dtype=torch.int32)
    seqs = torch.arange(batch, device="cuda", dtype=torch.int32)
    if q_len == 1:
        plan = AttentionPlan(num_decode=batch, decode_seqs=seqs, decode_tokens=seqs, max_decode_context_len=ctx)
    else:
        plan = AttentionPlan(num_prefill=batch, prefill_seqs=seqs, max_prefill_query_len=q_len)

    def run(i):
        ops.paged_attention(qkv, qkv.shape[1], out, pools[i][0], pools[i][1], table, qsl, ctxl, batch, q_len, heads,
                            kv_heads, head_dim, head_dim ** -0.5, 0, plan=plan, decode_splits=splits)

    us = _time(run, copies)
    kv_bytes = batch * ctx * kv_heads * head_dim * 2 * 2
    flops = 4.0 * heads * head_dim * batch * (q_len * (ctx - q_len) + q_len * (q_len + 1) / 2)
    return {"kernel": "paged_attention", "batch": batch, "q_len": q_len, "ctx": ctx, "heads": heads,
            "kv_heads": kv_heads, "head_dim": head_dim, "us": us, "GBps": kv_bytes / us / 1e3,
            "TFLOPs": flops / us / 1e6,
            "splits": splits or (ops.decode_splits_for(batch, kv_heads, ctx, head_dim, ops.stream_attention_supports(
                torch.bfloat16, heads, kv_heads, head_dim, 16)) if q_len == 1 else 1)}


def rmsnorm(rows: int, width: int) -> dict:
    x = torch.randn(rows, width, device="cuda", dtype=torch.bfloat16)
    d = torch.randn(rows, width, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(width, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(x)
    us = _time(lambda i: ops.rmsnorm(x, w, 1e-5, out, delta=d, write_residual=True), 8)
    return {"kernel": "add_rmsnorm", "rows": rows, "width": width, "us": us, "GBps": rows * width * 2 * 4 / us / 1e3}


CASES = {
    "decode_attention_b8": lambda: attention(8, 1, 4096),
    "decode_attention_b1": lambda: attention(1, 1, 4096),
    "decode_attention_b64": lambda: attention(64, 1, 4096),
    "prefill_attention_2048": lambda: attention(1, 2048, 2048),
    "prefill_attention_4x2048_ctx4096": lambda: attention(4, 2048, 4096),
    "prefill_attention_512": lambda: attention(1, 512, 512),
    "prefill_attention_8192": lambda: attention(1, 8192, 8192),
    "prefill_attention_8192_page64": lambda: attention(1, 8192, 8192, page=64),
    "prefill_attention_8192_head128": lambda: attention(1, 8192, 8192, head_dim=128),
    "prefill_attention_4x2048_ctx4096_head128": lambda: attention(4, 2048, 4096, head_dim=128),
    "prefill_attention_16384": lambda: attention(1, 16384, 16384),
    "prefill_attention_32x1024": lambda: attention(32, 1024, 1024),
    "decode_attention_b8_ctx1024": lambda: attention(8, 1, 1024),
    "decode_attention_b8_ctx16384": lambda: attention(8, 1, 16384),
    "decode_attention_b1_ctx32768": lambda: attention(1, 1, 32768),
    "decode_attention_b64_ctx1024": lambda: attention(64, 1, 1024),
    "decode_attention_b256_ctx1024": lambda: attention(256, 1, 1024),
    "prefill_attention_2048_head128": lambda: attention(1, 2048, 2048, heads=32, kv_heads=8, head_dim=128),
    "skinny_qkv_b8": lambda: skinny(8, 3072, 2048),
    "skinny_o_b8": lambda: skinny(8, 2048, 2048),
    "skinny_gate_up_b8": lambda: skinny(8, 16384, 2048),
    "skinny_down_b8": lambda: skinny(8, 2048, 8192),
    "skinny_head_b8": lambda: skinny(8, 128256, 2048),
    "skinny_gate_up_silu_b8": lambda: skinny_fused(8, 16384, 2048, False, False, True),
    "skinny_gate_up_silu_norm_b8": lambda: skinny_fused(8, 16384, 2048, True, False, True),
    "skinny_gate_up_silu_norm_b1": lambda: skinny_fused(1, 16384, 2048, True, False, True),
    "skinny_qkv_norm_b8": lambda: skinny_fused(8, 3072, 2048, True, False),
    "skinny_down_residual_b8": lambda: skinny_fused(8, 2048, 8192, False, True),
    "skinny_o_residual_b8": lambda: skinny_fused(8, 2048, 2048, False, True),
    "skinny_head_norm_b8": lambda: skinny_fused(8, 128256, 2048, True, False),
    "stream_qkv_b8": lambda: stream_gemm(8, 3072, 2048),
    "stream_o_b8": lambda: stream_gemm(8, 2048, 2048),
    "stream_gate_up_silu_b8": lambda: stream_gemm(8, 16384, 2048, True),
    "stream_down_b8": lambda: stream_gemm(8, 2048, 8192),
    "stream_head_b8": lambda: stream_gemm(8, 128256, 2048),
    "stream_gate_up_silu_b1": lambda: stream_gemm(1, 16384, 2048, True),
    "stream_gate_up_silu_b16": lambda: stream_gemm(16, 16384, 2048, True),
    "mlp_chain_b8": lambda: mlp_chain(8, False),
    "mlp_chain_fused_b8": lambda: mlp_chain(8, True),
    "mlp_chain_b1": lambda: mlp_chain(1, False),
    "mlp_chain_fused_b1": lambda: mlp_chain(1, True),
    "skinny_gate_up_b16": lambda: skinny(16, 16384, 2048),
    "library_gate_up_b16": lambda: library_gemm(16, 16384, 2048),
    "skinny_gate_up_b32": lambda: skinny(32, 16384, 2048),
    "library_gate_up_b32": lambda: library_gemm(32, 16384, 2048),
    "skinny_gate_up_b64": lambda: skinny(64, 16384, 2048),
    "library_down_b8": lambda: library_gemm(8, 2048, 8192),
    "library_qkv_b8": lambda: library_gemm(8, 3072, 2048),
    "library_gate_up_b64": lambda: library_gemm(64, 16384, 2048),
    "tcgen05_gate_up_2048": lambda: tcgen05_gemm(2048, 16384, 2048),
    "tcgen05_gate_up_silu_2048": lambda: tcgen05_gemm(2048, 16384, 2048, gated=True),
    "tcgen05_down_2048": lambda: tcgen05_gemm(2048, 2048, 8192),
    "tcgen05_qkv_2048": lambda: tcgen05_gemm(2048, 3072, 2048),
    "tcgen05_gate_up_b64": lambda: tcgen05_gemm(64, 16384, 2048),
    "tcgen05_down_b64": lambda: tcgen05_gemm(64, 2048, 8192),
    "library_down_b64": lambda: library_gemm(64, 2048, 8192),
    "library_qkv_b64": lambda: library_gemm(64, 3072, 2048),
    "library_o_b64": lambda: library_gemm(64, 2048, 2048),
    "library_head_b64": lambda: library_gemm(64, 128256, 2048),
    "library_gate_up_b24": lambda: library_gemm(24, 16384, 2048),
    "library_qkv_2048": lambda: library_gemm(2048, 3072, 2048),
    "library_gate_up_2048": lambda: library_gemm(2048, 16384, 2048),
    "library_down_2048": lambda: library_gemm(2048, 2048, 8192),
    "add_rmsnorm_b8": lambda: rmsnorm(8, 2048),
    "add_rmsnorm_2048": lambda: rmsnorm(2048, 2048),
}


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--kernel", default="all", help="all, or names of cases separated by commas: " + ", ".join(CASES))
    args = parser.parse_args()
    names = list(CASES) if args.kernel == "all" else args.kernel.split(",")
    for name in names:
        result = CASES[name]()
        print(json.dumps({"case": name, **{k: (round(v, 2) if isinstance(v, float) else v) for k, v in result.items()}}),
              flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
