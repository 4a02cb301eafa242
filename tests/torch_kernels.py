"""Plain torch stand-ins for the CUDA kernels, with the kernels' own signatures.

Two uses, both in tests only.  (1) `-m gpu` kernel tests compare each CUDA
kernel with the function of the same name here, on inputs of other sizes than
the engine's.  (2) `-m "not gpu"` tests patch these functions over
`liteinfer_b200.ops` (the `cpu_kernels` fixture) so that the step function, the
cache and the scheduler can be driven on a CPU; the product itself has no such
path.  Everything computes in float32 and rounds where the kernels round.
"""

from __future__ import annotations

import math

import torch

from liteinfer_b200.cache import addressing


def _r(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return x.to(dtype).float()


def embedding(ids, table, out, error_flag=None):
    bad = (ids < 0) | (ids >= table.shape[0])
    out.copy_(table[ids.long().clamp(0, table.shape[0] - 1)])
    out[bad] = 0
    if error_flag is not None and bool(bad.any()):
        error_flag.fill_(1)
    return out


def scatter_tokens(tokens, dst, src, source):
    live = dst >= 0
    tokens[dst[live].long()] = source[src[live].long()]
    return tokens


def rmsnorm(x, weight, eps, out, delta=None, rows=None, write_residual=False):
    dtype = x.dtype
    src = x if rows is None else x[rows.long()]
    v = src.float()
    if delta is not None:
        d = delta if rows is None else delta[rows.long()]
        v = _r(v + d.float(), dtype)
        if write_residual:
            x.copy_(v.to(dtype))
    inv = 1.0 / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    out.copy_((weight.float() * _r(v * inv, dtype)).to(dtype))
    return out


def add_(x, delta):
    x.copy_((x.float() + delta.float()).to(x.dtype))
    return x


def add_bias_(out, bias):
    out.copy_((out.float() + bias.float()).to(out.dtype))
    return out


def _activate(x, activation):
    if activation == "silu":
        return x / (1.0 + torch.exp(-x))
    if activation == "gelu":
        return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))
    if activation in ("gelu_pytorch_tanh", "gelu_tanh"):
        return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))
    if activation == "relu":
        return torch.relu(x)
    raise ValueError(activation)


def act_mul(gate_up, out, activation):
    w = out.shape[1]
    g, u = gate_up[:, :w].float(), gate_up[:, w:].float()
    out.copy_((_r(_activate(g, activation), out.dtype) * u).to(out.dtype))
    return out


def act_mul_interleaved(gate_up, out, activation):
    rows, w = out.shape
    pairs = gate_up.float().view(rows, w // 8, 2, 8)
    g, u = pairs[:, :, 0].reshape(rows, w), pairs[:, :, 1].reshape(rows, w)
    out.copy_((_r(_activate(g, activation), out.dtype) * u).to(out.dtype))
    return out


def gated_linear_supported(x, weight):
    return False


def gated_linear(x, weight, out, activation, bias=None):
    gate_up = torch.empty(x.shape[0], weight.shape[0], dtype=x.dtype, device=x.device)
    linear(x, weight, gate_up, bias)
    return act_mul_interleaved(gate_up, out, activation)


def linear(x, weight, out, bias=None, residual=None):
    """The product alone: a norm that is still pending runs first, and the result is never added into `residual`
    here (the caller gets it back as the delta still to be added)."""
    if hasattr(x, "materialise"):
        x = x.materialise()
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias.float()
    if out is None:
        out = torch.empty(y.shape, dtype=x.dtype, device=x.device)
    out.copy_(y.to(out.dtype))
    return out


gemm_simt = linear


def rope_kv_write(qkv, positions, seq_of_token, block_table, k_pool, v_pool, inv_freq, heads, kv_heads,
                  head_dim, rotary_dim, store=True):
    T = qkv.shape[0]
    dtype = qkv.dtype
    page_size = k_pool.shape[2]
    q = qkv[:, :heads * head_dim].float().view(T, heads, head_dim)
    k = qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].float().view(T, kv_heads, head_dim)
    v = qkv[:, (heads + kv_heads) * head_dim:].view(T, kv_heads, head_dim)
    if inv_freq is not None and rotary_dim > 0:
        half = rotary_dim // 2
        angle = positions.float()[:, None] * inv_freq.float()[None, :]
        cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]

        def rot(x):
            a, b = x[..., :half], x[..., half:rotary_dim]
            return torch.cat((a * cos - b * sin, b * cos + a * sin, x[..., rotary_dim:]), dim=-1)

        q, k = rot(q), rot(k)
    qkv[:, :heads * head_dim] = q.reshape(T, -1).to(dtype)
    if not store:
        return
    # Where each token is written: its slot, from the block tables (tokens of padding belong to no sequence).
    real = seq_of_token >= 0
    tables = block_table.tolist()
    seqs, pos = seq_of_token[real].tolist(), positions[real].tolist()
    if all(n == 1 for n in _run_lengths(seqs)):
        slots = addressing.newest_slots([tables[s] for s in seqs], pos, page_size, qkv.device)[0]
    else:
        runs = _runs(seqs, pos)
        slots = addressing.packed_addresses([tables[s] for s, _, _ in runs], [a for _, a, _ in runs],
                                            [n for _, _, n in runs], page_size, qkv.device).slots[0]
    ok = (slots >= 0) & (slots < k_pool.shape[0] * page_size)
    rows = torch.nonzero(real)[:, 0][ok]
    k_pool[slots[ok] // page_size, :, slots[ok] % page_size, :] = k.to(dtype)[rows]
    v_pool[slots[ok] // page_size, :, slots[ok] % page_size, :] = v[rows]


def _run_lengths(seqs):
    lengths, last = [], object()
    for s in seqs:
        if s == last:
            lengths[-1] += 1
        else:
            lengths.append(1)
            last = s
    return lengths


def _runs(seqs, positions):
    """(sequence, first position, count) of each run of consecutive tokens of one sequence."""
    runs = []
    for s, p in zip(seqs, positions):
        if runs and runs[-1][0] == s and runs[-1][1] + runs[-1][2] == p:
            runs[-1][2] += 1
        else:
            runs.append([s, p, 1])
    return runs


def paged_attention(q, q_row_stride, out, k_pool, v_pool, block_table, query_start_loc, context_lens, num_seqs,
                    max_q_len, heads, kv_heads, head_dim, scale, window=0, plan=None, decode_splits=None):
    dtype = out.dtype
    page_size = k_pool.shape[2]
    groups = heads // kv_heads
    qsl = query_start_loc.tolist()
    ctx = context_lens.tolist()
    qmat = q[:, :heads * head_dim].float().view(-1, heads, head_dim)
    # What each sequence reads: the slots of its whole context, from the block tables.
    slots_of = addressing.slot_table(block_table.tolist()[:num_seqs], [max(c, 0) for c in ctx[:num_seqs]], page_size,
                                     q.device)
    k_flat = k_pool.permute(0, 2, 1, 3).reshape(-1, kv_heads, head_dim)      # [slot, kv_heads, head_dim]
    v_flat = v_pool.permute(0, 2, 1, 3).reshape(-1, kv_heads, head_dim)
    for s in range(num_seqs):
        q0, q1 = qsl[s], qsl[s + 1]
        n, c = q1 - q0, ctx[s]
        if n == 0:
            continue
        first = 0 if window <= 0 else max(0, (c - n) - window + 1)
        kpos = torch.arange(first, c, device=q.device)
        slots = slots_of[s, first:c]
        pages = torch.where(slots >= 0, slots // page_size, slots)
        keys = k_flat[slots.clamp(min=0)].float()
        vals = v_flat[slots.clamp(min=0)].float()
        keys = keys.repeat_interleave(groups, dim=1)
        vals = vals.repeat_interleave(groups, dim=1)
        scores = torch.einsum("qhd,khd->hqk", qmat[q0:q1], keys) * scale
        qpos = torch.arange(c - n, c, device=q.device)
        hidden = kpos[None, :] > qpos[:, None]
        if window > 0:
            hidden = hidden | (kpos[None, :] <= qpos[:, None] - window)
        hidden = hidden | (pages < 0)[None, :]
        scores = scores.masked_fill(hidden[None], float("-inf"))
        m = scores.amax(-1, keepdim=True)
        p = torch.exp(scores - m)
        denom = p.sum(-1, keepdim=True)
        o = torch.einsum("hqk,khd->qhd", _r(p, dtype), vals) / denom.permute(1, 0, 2)
        out[q0:q1] = o.reshape(n, heads * head_dim).to(dtype)
    return out


def gemm_error_flag(device):
    return 0


def error_flags(device):
    return (0, 0)


def token_error_flag(device):
    return None


def argmax(logits, out):
    out.copy_(torch.argmax(logits.float(), dim=-1).to(torch.int32))
    return out


def sample_row(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, uniform: float) -> int:
    """The sampling kernel's rule for one row (liteinfer/sampling/sampler.py:50-97), in float64 where it sums."""
    logits = logits.float()
    if not temperature > 0 or top_k == 1:
        return int(torch.argmax(logits))
    x = logits / temperature
    n = x.numel()
    order = sorted(range(n), key=lambda i: (-float(x[i]), i))   # descending, equal values by index
    keep = order[:top_k] if 0 < top_k < n else order
    w = torch.exp(x - x.max()).double()
    if 0.0 < top_p < 1.0:
        total = float(sum(w[i] for i in keep))
        kept, before = [], 0.0
        for i in keep:
            if before > top_p * total:
                break
            kept.append(i)
            before += float(w[i])
        keep = kept
    keep = sorted(keep)
    total = float(sum(w[i] for i in keep))
    target, run = uniform * total, 0.0
    for i in keep:
        run += float(w[i])
        if run > target:
            return i
    return keep[-1]


def sample(logits, temperature, top_k, top_p, uniform, out):
    for r in range(logits.shape[0]):
        out[r] = sample_row(logits[r], float(temperature[r]), int(top_k[r]), float(top_p[r]), float(uniform[r]))
    return out


def fused_decode_supports(*args) -> bool:
    return False      # the stand-ins rotate and store in `rope_kv_write`, never inside the attention


ALL = ("fused_decode_supports", "scatter_tokens", "embedding", "rmsnorm", "add_", "add_bias_", "act_mul", "act_mul_interleaved", "gated_linear_supported",
       "gated_linear", "gemm_error_flag", "error_flags", "token_error_flag", "linear", "gemm_simt", "rope_kv_write", "paged_attention", "argmax", "sample")
