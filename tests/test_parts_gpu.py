"""Each part alone against the plain implementation, and parts the framework does not have, defined here:
a toy mixer that keeps a state of its own per request, a windowed attention layer, a layer without position
encoding, a layer that runs twice and a layer that reads another layer's cache — registered, built from a
random-weights folder, and stepped through the ordinary step function without touching the framework."""

from __future__ import annotations

import json
from dataclasses import dataclass

import pytest
import torch

import plain_llama
import tiny_configs

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2 ** -6, atol=2 ** -6)


def _randn(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from liteinfer_b200.parts.norm import RMSNorm

    part = RMSNorm(size=100, eps=1e-4, dtype=dtype, device=torch.device(DEV))
    assert part.tensor_specs()["weight"].shape == (100,)
    w = (1 + 0.1 * _randn(100, seed=1)).to(dtype)
    part.bind({"weight": w})
    x, delta = _randn(7, 100, seed=2, dtype=dtype), _randn(7, 100, seed=3, dtype=dtype)
    torch.testing.assert_close(part.forward(x.clone()).float(), plain_llama.rms_norm(x, w, 1e-4).float(), **_tol(dtype))
    stream = x.clone()
    out = part.forward(stream, delta)
    torch.testing.assert_close(stream.float(), (x + delta).float(), **_tol(dtype))      # the stream moved on
    torch.testing.assert_close(out.float(), plain_llama.rms_norm(x + delta, w, 1e-4).float(), **_tol(dtype))
    rows = torch.tensor([6, 2], dtype=torch.int32, device=DEV)
    stream = x.clone()
    picked = part.forward(stream, delta, rows=rows)
    assert torch.equal(stream, x)                                                      # gathered rows: stream untouched
    torch.testing.assert_close(picked.float(), plain_llama.rms_norm(x + delta, w, 1e-4)[[6, 2]].float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens", [3, 100])
@pytest.mark.parametrize("act,bias", [("silu", False), ("gelu_pytorch_tanh", True)])
def test_gated_mlp_part(dtype, tokens, act, bias):
    from liteinfer_b200.parts.feed_forward import GatedMLP

    part = GatedMLP(hidden_size=96, intermediate_size=176, activation=act, dtype=dtype, device=torch.device(DEV), bias=bias)
    specs = part.tensor_specs()
    tensors = {n: _randn(*s.shape, seed=i, scale=0.1, dtype=dtype) for i, (n, s) in enumerate(specs.items())}
    part.bind(tensors)
    x = _randn(tokens, 96, seed=50, dtype=dtype)
    want = plain_llama.gated_mlp(x.float(), tensors["gate_proj.weight"].float(), tensors["up_proj.weight"].float(),
                                 tensors["down_proj.weight"].float(), act,
                                 *(tensors[n].float() if bias else None for n in ("gate_proj.bias", "up_proj.bias", "down_proj.bias")))
    torch.testing.assert_close(part.forward(x, None).float(), want, **_tol(dtype))


def test_embedding_and_head_parts():
    from liteinfer_b200.parts.embedding import LinearHead, TokenEmbedding

    emb = TokenEmbedding(vocab_size=300, hidden_size=48, dtype=torch.bfloat16, device=torch.device(DEV))
    table = _randn(300, 48, dtype=torch.bfloat16)
    emb.bind({"weight": table})
    ids = torch.tensor([0, 299, 7], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids), table[ids.long()])
    head = LinearHead(vocab_size=300, hidden_size=48, dtype=torch.bfloat16, device=torch.device(DEV))
    head.bind({"weight": table})
    x = _randn(5, 48, seed=2, dtype=torch.bfloat16)
    torch.testing.assert_close(head.forward(x).float(), x.float() @ table.float().t(), rtol=2 ** -6, atol=2 ** -6)


def test_rotary_part_frequencies_are_the_plain_ones():
    from liteinfer_b200.parts.position import RotaryEmbedding

    for cfg in (tiny_configs.TINY_A, tiny_configs.TINY_B, tiny_configs.TINY_C, tiny_configs.TINY_D):
        scaling = cfg.get("rope_scaling") or {}
        part = RotaryEmbedding(head_dim=cfg["head_dim"], theta=cfg["rope_theta"], dtype=torch.float32,
                               device=torch.device(DEV), **{k: v for k, v in scaling.items()})
        assert torch.equal(part.rotary().inv_freq.cpu(), plain_llama.rope_inverse_frequencies(cfg))


# ------------------------------------------------------------------ toy parts, defined by the test
class EmaMixer:
    """y_t = (s_t) W, s_t = decay * s_{t-1} + x_t: a recurrence whose state lives in the request's state slot."""

    graph_safe = False      # forward reads the slots on the host, so steps are not captured into CUDA graphs

    def __init__(self, hidden_size: int, decay: float, dtype, device):
        self.hidden_size, self.decay, self.dtype, self.device = hidden_size, decay, dtype, device
        self.weight = None

    def tensor_specs(self):
        from liteinfer_b200.parts.spec import TensorSpec
        return {"mix.weight": TensorSpec((self.hidden_size, self.hidden_size))}

    def bind(self, tensors):
        self.weight = tensors["mix.weight"]

    def cache_needs(self):
        from liteinfer_b200.parts.context import StateNeed
        return (StateNeed((self.hidden_size,), "f32"),)

    def forward(self, x, ctx, cache):
        out = torch.empty_like(x)
        at = 0
        slots = ctx.state_slots.tolist()
        for seq, n in enumerate(ctx.query_lens):
            state = cache.state[slots[seq]]
            rows = []
            for t in range(n):
                state.mul_(self.decay).add_(x[at + t].float())
                rows.append(state.clone())
            out[at:at + n] = (torch.stack(rows) @ self.weight.float().t()).to(x.dtype)
            at += n
        return out


class ScalePositions:
    """A position encoding that is no rotation: q and k are scaled by 1 / (1 + position / 64)."""

    def __init__(self, dtype, device):
        pass

    def tensor_specs(self):
        return {}

    def bind(self, tensors):
        pass

    def rotary(self):
        return None

    def apply(self, q, k, ctx):
        scale = (1.0 / (1.0 + ctx.positions.float() / 64.0)).to(q.dtype)[:, None, None]
        q.mul_(scale)
        k.mul_(scale)


class RoutedFeedForward:
    """A feed-forward with routing: every token goes through its `top_k` best of `experts` small two-layer
    networks, weighted by the router's renormalised probabilities.  The router's weight stays 32-bit."""

    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top_k: int, dtype, device):
        self.h, self.i, self.experts, self.top_k = hidden_size, intermediate_size, experts, top_k
        self.router = self.up = self.down = None

    def tensor_specs(self):
        from liteinfer_b200.parts.spec import TensorSpec
        specs = {"router.weight": TensorSpec((self.experts, self.h), kind="f32")}
        for e in range(self.experts):
            specs[f"experts.{e}.up.weight"] = TensorSpec((self.i, self.h))
            specs[f"experts.{e}.down.weight"] = TensorSpec((self.h, self.i))
        return specs

    def bind(self, tensors):
        self.router = tensors["router.weight"]
        assert self.router.dtype == torch.float32
        self.up = [tensors[f"experts.{e}.up.weight"] for e in range(self.experts)]
        self.down = [tensors[f"experts.{e}.down.weight"] for e in range(self.experts)]

    def forward(self, x, ctx):
        probs = torch.softmax(x.float() @ self.router.t(), dim=-1)
        best, chosen = probs.topk(self.top_k, dim=-1)
        gate = torch.zeros_like(probs).scatter_(1, chosen, best / best.sum(-1, keepdim=True))
        out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
        for e in range(self.experts):
            hidden = torch.relu(x.float() @ self.up[e].float().t())
            out += gate[:, e:e + 1] * (hidden @ self.down[e].float().t())
        return out.to(x.dtype)


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    hidden_size: int
    window: int

    @classmethod
    def from_dict(cls, raw):
        return cls(raw["vocab_size"], raw["hidden_size"], raw["window"])

    def to_dict(self):
        return {"architectures": ["ToyStateLM"], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "window": self.window}


def toy_spec(cfg: ToyConfig):
    from liteinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    h = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"size": h, "eps": 1e-5})
    ffn = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": 2 * h, "activation": "silu"})

    def layer(i, mixer, feed_forward=ffn):
        return LayerSpec("prenorm_residual",
                         {"mixer_norm": norm, "mixer": mixer, "feed_forward_norm": norm, "feed_forward": feed_forward},
                         {"mixer_norm": f"l{i}.n1.", "mixer": f"l{i}.mixer.", "feed_forward_norm": f"l{i}.n2.",
                          "feed_forward": f"l{i}.ffn."})

    attention = lambda position, window=None: PartSpec("attention", {
        "hidden_size": h, "heads": 4, "kv_heads": 2, "head_dim": 16, "position": position, "window": window})
    routed = PartSpec("toy_routed", {"hidden_size": h, "intermediate_size": 24, "experts": 3, "top_k": 2})
    layers = (
        layer(0, PartSpec("toy_ema", {"hidden_size": h, "decay": 0.5})),                      # a state of its own
        layer(1, attention(PartSpec("toy_scale_positions", {}), cfg.window), routed),         # a window, odd positions, routing
        layer(2, attention(PartSpec("rotary", {"head_dim": 16, "theta": 100.0, "rotary_dim": 8}))),   # partial rotary
    )
    sizes = {"vocab_size": cfg.vocab_size, "hidden_size": h}
    # layer 2 runs twice; its second stop reads the cache its first stop wrote
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(2, cache_of=2))
    return ModelSpec(cfg.vocab_size, h, PartSpec("token_embedding", sizes), "emb.", layers, schedule, norm, "final.",
                     PartSpec("linear", sizes), "head.", tied={"head.weight": "emb.weight"})


def _plain_toy(weights, cfg: ToyConfig, tokens):
    """The same model, whole sequence, no cache, stock torch ops."""
    w = {k: v.float() for k, v in weights.items()}
    x = w["emb.weight"][torch.tensor(tokens)]
    T = len(tokens)
    pos = torch.arange(T)

    def attn(x, p, rope, window, kv_override=None):
        q = (x @ w[p + "q_proj.weight"].t()).view(T, 4, 16)
        k = (x @ w[p + "k_proj.weight"].t()).view(T, 2, 16)
        v = (x @ w[p + "v_proj.weight"].t()).view(T, 2, 16)
        if rope:
            inv = 1.0 / (100.0 ** (torch.arange(0, 8, 2).float() / 8))
            cos, sin = plain_llama.rope_tables(inv, pos, torch.float32)
            q = torch.cat([plain_llama.apply_rope(q[..., :8], cos, sin), q[..., 8:]], -1)
            k = torch.cat([plain_llama.apply_rope(k[..., :8], cos, sin), k[..., 8:]], -1)
        else:
            scale = (1.0 / (1.0 + pos.float() / 64.0))[:, None, None]
            q, k = q * scale, k * scale
        if kv_override is not None:
            k, v = kv_override
        o = plain_llama.causal_attention(q, k, v, 16 ** -0.5, window)
        return o.reshape(T, 64) @ w[p + "o_proj.weight"].t(), (k, v)

    def routed(h, f):
        probs = torch.softmax(h @ w[f + "router.weight"].t(), dim=-1)
        out = torch.zeros_like(h)
        for t in range(T):
            best = sorted(range(3), key=lambda e: -float(probs[t, e]))[:2]
            total = sum(probs[t, e] for e in best)
            for e in best:
                hidden = torch.relu(w[f + f"experts.{e}.up.weight"] @ h[t])
                out[t] += probs[t, e] / total * (w[f + f"experts.{e}.down.weight"] @ hidden)
        return out

    def block(x, i, mix):
        x = x + mix(plain_llama.rms_norm(x, w[f"l{i}.n1.weight"], 1e-5))
        f = f"l{i}.ffn."
        if f + "router.weight" in w:
            return x + routed(plain_llama.rms_norm(x, w[f"l{i}.n2.weight"], 1e-5), f)
        return x + plain_llama.gated_mlp(plain_llama.rms_norm(x, w[f"l{i}.n2.weight"], 1e-5), w[f + "gate_proj.weight"],
                                         w[f + "up_proj.weight"], w[f + "down_proj.weight"], "silu")

    def ema(h):
        state, rows = torch.zeros(cfg.hidden_size), []
        for t in range(T):
            state = 0.5 * state + h[t]
            rows.append(state)
        return torch.stack(rows) @ w["l0.mixer.mix.weight"].t()

    x = block(x, 0, ema)
    x = block(x, 1, lambda h: attn(h, "l1.mixer.", False, cfg.window)[0])
    kept = {}

    def first(h):
        out, kept["kv"] = attn(h, "l2.mixer.", True, None)
        return out

    x = block(x, 2, first)
    x = block(x, 2, lambda h: attn(h, "l2.mixer.", True, None, kept["kv"])[0])
    return plain_llama.rms_norm(x, w["final.weight"], 1e-5) @ w["emb.weight"].t()


@pytest.fixture(scope="module")
def toy_model(tmp_path_factory):
    from liteinfer_b200.config.registry import register_architecture
    from liteinfer_b200.parts.registry import register_feed_forward, register_mixer, register_position_encoding
    from liteinfer_b200.weights.random_init import write_random_model

    register_mixer("toy_ema", EmaMixer, replace=True)
    register_feed_forward("toy_routed", RoutedFeedForward, replace=True)
    register_position_encoding("toy_scale_positions", ScalePositions, replace=True)
    register_architecture("ToyStateLM", ToyConfig, toy_spec, replace=True)
    cfg = ToyConfig(vocab_size=211, hidden_size=64, window=9)
    folder = write_random_model(cfg.to_dict(), tmp_path_factory.mktemp("toy") / "toy", seed=5, dtype=torch.float32)
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyStateLM"]
    return cfg, folder


def test_toy_parts_are_registered_built_and_stepped(toy_model):
    from safetensors.torch import load_file

    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    cfg, folder = toy_model
    weights = load_file(str(folder / "model.safetensors"))
    tokens = {"a": tiny_configs.prompt(cfg.vocab_size, 45, 0), "b": tiny_configs.prompt(cfg.vocab_size, 23, 1)}
    want = {k: _plain_toy(weights, cfg, v) for k, v in tokens.items()}

    runner = build_runner(folder, torch.float32, DEV, page_size=4, num_pages=24, max_requests=2)
    cache = runner.cache
    assert len(cache.groups) == 2                                    # windowed pages apart from the full ones
    assert {g.need.window for g in cache.groups} == {9, None}
    assert [c.read_only for c in runner.layer_caches] == [False, False, False, True]
    assert runner.layer_caches[0].state is not None and runner.layer_caches[0].kv is None

    # whole, then in portions (the state and the window's pages carry over), then b in the slot a left
    got = runner.step([StepEntry("a", tokens["a"], range(45))]).cpu()
    torch.testing.assert_close(got, want["a"], rtol=1e-4, atol=1e-4)
    runner.release("a")
    rows, at = [], 0
    for n in (7, 2, 20, 1, 1, 14):
        rows.append(runner.step([StepEntry("a", tokens["a"][at:at + n], range(n))]).cpu())
        at += n
        window_group = next(g for g in cache.groups if g.need.window == 9)
        assert window_group.allocator.num_held <= 4 + -(-n // 4)      # pages the window has passed came back
        cache.check_invariants()
    torch.testing.assert_close(torch.cat(rows), want["a"], rtol=1e-4, atol=1e-4)
    # mixed: a decodes on while b's prompt arrives in portions beside it
    mixed_b = [runner.step([StepEntry("b", tokens["b"][:10], range(10))]).cpu()]
    runner.release("a")
    mixed_b.append(runner.step([StepEntry("b", tokens["b"][10:], range(13))]).cpu())
    torch.testing.assert_close(torch.cat(mixed_b), want["b"], rtol=1e-4, atol=1e-4)
    runner.release("b")
    assert all(g.allocator.num_held == 0 for g in cache.groups) and cache.slots.num_held == 0


def test_toy_model_generates_through_the_entry_point(toy_model):
    from safetensors.torch import load_file

    from liteinfer_b200 import LLM, SamplingParams

    cfg, folder = toy_model
    weights = load_file(str(folder / "model.safetensors"))
    prompt = tiny_configs.prompt(cfg.vocab_size, 12, 3)
    tokens = list(prompt)
    for _ in range(6):
        tokens.append(int(torch.argmax(_plain_toy(weights, cfg, tokens)[-1])))
    with LLM(str(folder), dtype="float32", device=DEV, block_size=4, max_num_seqs=2, max_model_len=64,
             max_num_batched_tokens=5) as llm:
        out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    assert out[0].token_ids == tokens[12:]


def _context_for(cache, entries):
    """A StepContext for `entries` = [(request id, number of new tokens)], the way the step function builds it."""
    from liteinfer_b200.engine.runner import StepEntry, _Batch, _context, _fill

    step = [StepEntry(r, [0] * n, ()) for r, n in entries]
    starts = [cache.length(r) for r, _ in entries]
    counts = [n for _, n in entries]
    totals = [s + n for s, n in zip(starts, counts)]
    cache.reserve([r for r, _ in entries], totals)
    widths = [max(len(cache.block_table(g, r)) for r, _ in entries) for g in range(len(cache.groups))]
    n_dec = sum(1 for n in counts if n == 1)
    batch = _Batch(len(entries), sum(counts), 0, widths, n_dec, len(entries) - n_dec)
    host = torch.empty(batch.total, dtype=torch.int32)
    _fill(batch, host.numpy(), step, cache, starts)
    ctx = _context(batch, host.to(DEV), torch.device(DEV), counts, totals, None,
                   max((t for t, n in zip(totals, counts) if n == 1), default=0))
    for (r, _), total in zip(entries, totals):
        cache.commit(r, total)
    return ctx


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(4, 2, 16, 8), (8, 2, 64, 16), (6, 6, 48, 4)])
def test_attention_part_alone(dtype, heads, kv_heads, head_dim, page):
    """The attention mixer by itself (projections, rotary, cache write, attention over pages, output projection):
    a sequence fed whole, and the same sequence fed in portions beside another request, against the plain block."""
    from liteinfer_b200.cache.manager import CacheManager
    from liteinfer_b200.parts.attention import Attention
    from liteinfer_b200.parts.spec import PartSpec, ScheduleEntry

    hidden = 96
    config = {"num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim,
              "hidden_size": hidden, "rope_theta": 10000.0}
    part = Attention(hidden_size=hidden, heads=heads, kv_heads=kv_heads, head_dim=head_dim, dtype=dtype,
                     device=torch.device(DEV), position=PartSpec("rotary", {"head_dim": head_dim, "theta": 10000.0}))
    tensors = {n: _randn(*s.shape, seed=i, scale=0.08, dtype=dtype) for i, (n, s) in enumerate(part.tensor_specs().items())}
    part.bind(dict(tensors))
    x = _randn(70, hidden, seed=40, dtype=dtype)
    other = _randn(9, hidden, seed=41, dtype=dtype)
    cos, sin = plain_llama.rope_tables(plain_llama.rope_inverse_frequencies(config), torch.arange(70, device=DEV), torch.float32)
    w32 = {"p." + n: t.float() for n, t in tensors.items()}
    want = plain_llama.attention_block(x.float(), w32, "p.", config, cos, sin)

    cache = CacheManager([part.cache_needs()], (ScheduleEntry(0),), page, 40, 4, dtype, DEV)
    view = cache.layer_caches()[0]
    whole = part.forward(x, _context_for(cache, [("a", 70)]), view)
    torch.testing.assert_close(whole.float(), want, **_tol(dtype))
    cache.release("a")
    rows, at = [], 0
    for n, m in ((33, 4), (1, 1), (2, 3), (34, 1)):      # request a in portions; request b beside it, also growing
        ctx = _context_for(cache, [("b", m), ("a", n)])
        out = part.forward(torch.cat([other[:m], x[at:at + n]]), ctx, view)
        rows.append(out[m:])
        at += n
    torch.testing.assert_close(torch.cat(rows).float(), want, **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prenorm_block_alone(dtype):
    """The block arrangement with real parts against the plain decoder layer; the residual stream travels as
    (hidden, pending delta)."""
    from liteinfer_b200.cache.manager import CacheManager
    from liteinfer_b200.parts.model import Layer
    from liteinfer_b200.parts.spec import LayerSpec, PartSpec, ScheduleEntry

    config = dict(tiny_configs.TINY_B)
    h, heads, kvh, d = config["hidden_size"], config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    norm = PartSpec("rmsnorm", {"size": h, "eps": config["rms_norm_eps"]})
    scaling = config["rope_scaling"]
    spec = LayerSpec("prenorm_residual", {
        "mixer_norm": norm,
        "mixer": PartSpec("attention", {"hidden_size": h, "heads": heads, "kv_heads": kvh, "head_dim": d,
                                        "position": PartSpec("rotary", {"head_dim": d, "theta": config["rope_theta"], **scaling})}),
        "feed_forward_norm": norm,
        "feed_forward": PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": config["intermediate_size"],
                                               "activation": "silu"}),
    }, {"mixer_norm": "model.layers.0.input_layernorm.", "mixer": "model.layers.0.self_attn.",
        "feed_forward_norm": "model.layers.0.post_attention_layernorm.", "feed_forward": "model.layers.0.mlp."})
    layer = Layer(spec, dtype, torch.device(DEV))
    weights = {}
    for role, part in layer.parts.items():
        local = {n: (1 + 0.1 * _randn(*s.shape, seed=len(weights) + i)).to(dtype) if s.init == "ones_normal"
                 else _randn(*s.shape, seed=len(weights) + i, scale=0.08, dtype=dtype)
                 for i, (n, s) in enumerate(part.tensor_specs().items())}
        part.bind(dict(local))
        weights.update({spec.prefixes[role] + n: t.float() for n, t in local.items()})
    x = _randn(40, h, seed=90, dtype=dtype)
    delta = _randn(40, h, seed=91, dtype=dtype)
    cos, sin = plain_llama.rope_tables(plain_llama.rope_inverse_frequencies(config), torch.arange(40, device=DEV), torch.float32)
    want = plain_llama.decoder_layer((x + delta).float(), weights, 0, config, cos, sin)
    cache = CacheManager([layer.cache_needs()], (ScheduleEntry(0),), 8, 16, 2, dtype, DEV)
    hidden, pending = layer.block.forward(x.clone(), delta, _context_for(cache, [("a", 40)]), cache.layer_caches()[0])
    torch.testing.assert_close((hidden.float() + pending.float()), want, **_tol(dtype))


@dataclass(frozen=True)
class WindowConfig:
    vocab_size: int
    window: int

    @classmethod
    def from_dict(cls, raw):
        return cls(raw["vocab_size"], raw["window"])

    def to_dict(self):
        return {"architectures": ["ToyWindowLM"], "vocab_size": self.vocab_size, "window": self.window}


def window_spec(cfg: WindowConfig):
    """Two attention layers of head size 64, one behind a window, nothing that works on the host: the decode
    steps of this model run the tensor-core kernels and replay from graphs."""
    from liteinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    h = 128
    norm = PartSpec("rmsnorm", {"size": h, "eps": 1e-5})
    ffn = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": 192, "activation": "silu"})

    def layer(i, window):
        mixer = PartSpec("attention", {"hidden_size": h, "heads": 4, "kv_heads": 2, "head_dim": 64, "window": window,
                                       "position": PartSpec("rotary", {"head_dim": 64, "theta": 10000.0})})
        return LayerSpec("prenorm_residual",
                         {"mixer_norm": norm, "mixer": mixer, "feed_forward_norm": norm, "feed_forward": ffn},
                         {"mixer_norm": f"l{i}.n1.", "mixer": f"l{i}.mixer.", "feed_forward_norm": f"l{i}.n2.",
                          "feed_forward": f"l{i}.ffn."})

    sizes = {"vocab_size": cfg.vocab_size, "hidden_size": h}
    return ModelSpec(cfg.vocab_size, h, PartSpec("token_embedding", sizes), "emb.", (layer(0, cfg.window), layer(1, None)),
                     (ScheduleEntry(0), ScheduleEntry(1)), norm, "final.", PartSpec("linear", sizes), "head.",
                     tied={"head.weight": "emb.weight"})


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_window_pages_come_back_under_graphs(tmp_path, dtype):
    """Long decoding behind a window, replayed from graphs: the window's pages are given back as it moves (the
    staged block tables must follow), and every token's logits equal those of the same tokens fed whole."""
    from liteinfer_b200.config.registry import register_architecture
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry
    from liteinfer_b200.weights.random_init import write_random_model

    register_architecture("ToyWindowLM", WindowConfig, window_spec, replace=True)
    cfg = WindowConfig(vocab_size=300, window=40)
    folder = write_random_model(cfg.to_dict(), tmp_path / "window", seed=5)
    tokens = {"a": tiny_configs.prompt(300, 230, 1), "b": tiny_configs.prompt(300, 150, 2)}
    heads = {"a": 70, "b": 3}

    whole = build_runner(folder, dtype, DEV, 16, 40, 2)
    want = {r: whole.step([StepEntry(r, t, tuple(range(len(t))))]) for r, t in tokens.items()}

    runner = build_runner(folder, dtype, DEV, 16, 40, 2)
    runner.enable_decode_graphs(2, 256)
    got = {r: [runner.step([StepEntry(r, tokens[r][:heads[r]], (heads[r] - 1,))])] for r in tokens}
    for step in range(147):                       # b ends with this loop, a goes on alone in a narrower graph
        live = [r for r in tokens if heads[r] + step < len(tokens[r])]
        rows = runner.step([StepEntry(r, [tokens[r][heads[r] + step]], (0,)) for r in live])
        for i, r in enumerate(live):
            got[r].append(rows[i:i + 1])
    assert runner.graph_replays == 147 + 2          # the two prompts went through padded graphs
    windowed = next(g for g in runner.cache.groups if g.need.window == 40)
    assert windowed.allocator.num_held <= 2 * 4                  # what the window has passed came back
    for r in tokens:
        have = torch.cat(got[r]).float()
        ref = want[r][heads[r] - 1:heads[r] - 1 + have.shape[0]].float()
        if dtype == torch.float32:
            torch.testing.assert_close(have, ref, rtol=1e-4, atol=1e-5)
        else:
            torch.testing.assert_close(have, ref, rtol=2 ** -5, atol=2 ** -5)
