"""A second toy architecture, defined here and registered from here: a block with two mixers side by side (an
attention and a running-mean memory), the memory keeping two states of different shapes per request, a weight
drawn by the part's own init function, and every kernel launch of the memory mixer safe to capture in a CUDA
graph.  Nothing under liteinfer_b200/ knows of it.  It is stepped whole, in portions and beside another request
against a plain twin, and with CUDA graphs against without them from the very first step of every shape (a
capture that ran a live batch more than once would add that batch to the state more than once).
"""

from __future__ import annotations

from dataclasses import dataclass

import pytest
import torch

import plain_llama
import tiny_configs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class RunningMeanMixer:
    """y_t = mean(x_0 .. x_t) W.  Per request it keeps the sum of what it has seen and how many tokens that was:
    two states, found in the layer's cache under their names.  Only tensor operations on the device: steps of a
    model with this mixer are captured into CUDA graphs like any other."""

    def __init__(self, hidden_size: int, dtype, device):
        self.hidden_size = hidden_size
        self.weight = None

    def tensor_specs(self):
        from liteinfer_b200.parts.spec import TensorSpec
        positive = lambda shape, generator: 0.05 * torch.rand(shape, generator=generator)      # its own distribution
        return {"mix.weight": TensorSpec((self.hidden_size, self.hidden_size), init=positive)}

    def bind(self, tensors):
        self.weight = tensors["mix.weight"]

    def cache_needs(self):
        from liteinfer_b200.parts.context import StateNeed
        return (StateNeed((self.hidden_size,), "f32", name="sum"), StateNeed((1,), "f32", name="count"))

    def forward(self, x, ctx, cache):
        seq = ctx.seq_of_token.long()
        real = seq >= 0                                     # tokens of padding belong to no sequence
        seq = seq.clamp(min=0)
        slot = ctx.state_slots.long()[seq]
        xf = x.float() * real[:, None]
        order = torch.arange(x.shape[0], device=x.device)
        earlier = ((seq[:, None] == seq[None, :]) & real[:, None] & real[None, :] & (order[None, :] <= order[:, None])).float()
        total = cache.states["sum"][slot] + earlier @ xf
        count = cache.states["count"][slot] + earlier.sum(-1, keepdim=True)
        if not cache.read_only:
            cache.states["sum"].index_add_(0, slot, xf)
            cache.states["count"].index_add_(0, slot, real.float()[:, None])
        return ((total / count.clamp(min=1.0)) @ self.weight.float().t()).to(x.dtype)


class TwoMixerBlock:
    """h += attention(norm(h)) + memory(norm(h)); h += feed_forward(norm(h)): roles beyond a mixer and its norms."""

    roles = {"norm": "norm", "attention": "mixer", "memory": "mixer", "feed_forward_norm": "norm",
             "feed_forward": "feed_forward"}

    def __init__(self, parts):
        self.parts = parts

    def forward(self, hidden, delta, ctx, cache):
        from liteinfer_b200 import ops
        p = self.parts
        normed = p["norm"].forward(hidden, delta)
        mixed = ops.add_(p["attention"].forward(normed, ctx, cache), p["memory"].forward(normed, ctx, cache))
        normed = p["feed_forward_norm"].forward(hidden, mixed)
        return hidden, p["feed_forward"].forward(normed, ctx)


@dataclass(frozen=True)
class TwoConfig:
    vocab_size: int
    hidden_size: int

    @classmethod
    def from_dict(cls, raw):
        return cls(raw["vocab_size"], raw["hidden_size"])

    def to_dict(self):
        return {"architectures": ["ToyTwoMixerLM"], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size}


def two_spec(cfg: TwoConfig):
    from liteinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    h = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"size": h, "eps": 1e-5})
    ffn = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": 2 * h, "activation": "silu"})
    attention = PartSpec("attention", {"hidden_size": h, "heads": 4, "kv_heads": 2, "head_dim": 16,
                                       "position": PartSpec("rotary", {"head_dim": 16, "theta": 100.0})})
    both = LayerSpec("toy_two_mixers",
                     {"norm": norm, "attention": attention, "memory": PartSpec("toy_running_mean", {"hidden_size": h}),
                      "feed_forward_norm": norm, "feed_forward": ffn},
                     {"norm": "l0.n1.", "attention": "l0.attn.", "memory": "l0.mem.", "feed_forward_norm": "l0.n2.",
                      "feed_forward": "l0.ffn."})
    plain = LayerSpec("prenorm_residual",
                      {"mixer_norm": norm, "mixer": attention, "feed_forward_norm": norm, "feed_forward": ffn},
                      {"mixer_norm": "l1.n1.", "mixer": "l1.attn.", "feed_forward_norm": "l1.n2.", "feed_forward": "l1.ffn."})
    sizes = {"vocab_size": cfg.vocab_size, "hidden_size": h}
    return ModelSpec(cfg.vocab_size, h, PartSpec("token_embedding", sizes), "emb.", (both, plain),
                     (ScheduleEntry(0), ScheduleEntry(1)), norm, "final.", PartSpec("linear", sizes), "head.",
                     tied={"head.weight": "emb.weight"})


def _plain(weights, tokens):
    """The same model on one whole sequence with stock torch ops."""
    w = {k: v.float() for k, v in weights.items()}
    T = len(tokens)
    x = w["emb.weight"][torch.tensor(tokens)]
    config = {"num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "hidden_size": x.shape[1]}
    inv = 1.0 / (100.0 ** (torch.arange(0, 16, 2).float() / 16))
    cos, sin = plain_llama.rope_tables(inv, torch.arange(T), torch.float32)

    def ffn(h, p):
        return plain_llama.gated_mlp(h, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"], "silu")

    h = plain_llama.rms_norm(x, w["l0.n1.weight"], 1e-5)
    mean = h.cumsum(0) / torch.arange(1, T + 1)[:, None]
    x = x + plain_llama.attention_block(h, w, "l0.attn.", config, cos, sin) + mean @ w["l0.mem.mix.weight"].t()
    x = x + ffn(plain_llama.rms_norm(x, w["l0.n2.weight"], 1e-5), "l0.ffn.")
    x = x + plain_llama.attention_block(plain_llama.rms_norm(x, w["l1.n1.weight"], 1e-5), w, "l1.attn.", config, cos, sin)
    x = x + ffn(plain_llama.rms_norm(x, w["l1.n2.weight"], 1e-5), "l1.ffn.")
    return plain_llama.rms_norm(x, w["final.weight"], 1e-5) @ w["emb.weight"].t()


@pytest.fixture(scope="module")
def two_model(tmp_path_factory):
    from liteinfer_b200.config.registry import register_architecture
    from liteinfer_b200.parts.registry import register_block, register_mixer
    from liteinfer_b200.weights.random_init import write_random_model

    register_mixer("toy_running_mean", RunningMeanMixer, replace=True)
    register_block("toy_two_mixers", TwoMixerBlock, replace=True)
    register_architecture("ToyTwoMixerLM", TwoConfig, two_spec, replace=True)
    cfg = TwoConfig(vocab_size=157, hidden_size=64)
    folder = write_random_model(cfg.to_dict(), tmp_path_factory.mktemp("two") / "two", seed=8, dtype=torch.float32)
    return cfg, folder


def test_two_mixers_and_two_states_in_one_layer(two_model):
    from safetensors.torch import load_file

    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    cfg, folder = two_model
    weights = load_file(str(folder / "model.safetensors"))
    assert float(weights["l0.mem.mix.weight"].min()) >= 0.0            # drawn by the part's own init function
    tokens = {"a": tiny_configs.prompt(cfg.vocab_size, 41, 0), "b": tiny_configs.prompt(cfg.vocab_size, 19, 1)}
    want = {k: _plain(weights, v) for k, v in tokens.items()}
    runner = build_runner(folder, torch.float32, DEV, page_size=4, num_pages=40, max_requests=2)
    first = runner.layer_caches[0]
    assert set(first.states) == {"sum", "count"} and first.states["count"].shape == (2, 1) and set(first.kvs) == {"kv"}
    assert len(runner.cache.groups) == 1 and runner.cache.groups[0].stops == [0, 1]
    got = runner.step([StepEntry("a", tokens["a"], range(41))]).cpu()
    torch.testing.assert_close(got, want["a"], rtol=1e-4, atol=1e-4)
    runner.release("a")
    rows = {"a": [], "b": []}
    at = {"a": 0, "b": 0}
    for na, nb in ((7, 1), (2, 5), (1, 1), (20, 0), (1, 12), (10, 0)):      # both in portions and single tokens, side by side
        entries = []
        for r, n in (("a", na), ("b", nb)):
            if n:
                entries.append(StepEntry(r, tokens[r][at[r]:at[r] + n], range(n)))
        out = runner.step(entries).cpu()
        for e in entries:
            n = len(e.tokens)
            rows[e.request_id].append(out[:n])
            out = out[n:]
            at[e.request_id] += n
    for r in ("a", "b"):
        torch.testing.assert_close(torch.cat(rows[r]), want[r], rtol=1e-4, atol=1e-4)
    runner.release("a"); runner.release("b")
    # the slots come back zeroed: b again, in a's old slot, starts from nothing
    got = runner.step([StepEntry("b", tokens["b"], range(19))]).cpu()
    torch.testing.assert_close(got, want["b"], rtol=1e-4, atol=1e-4)


def test_graphs_agree_with_eager_from_the_first_step_of_every_shape(two_model):
    """Every step here is the first of its width or padded shape, so each one captures its graph."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    cfg, folder = two_model
    tokens = {r: tiny_configs.prompt(cfg.vocab_size, 60, 10 + i) for i, r in enumerate("abc")}
    runs = []
    for graphs in (False, True):
        runner = build_runner(folder, torch.float32, DEV, page_size=4, num_pages=60, max_requests=4)
        if graphs:
            assert runner.model.graph_safe
            runner.enable_decode_graphs(4, 128)
        at = {r: 0 for r in tokens}
        rows = []
        plan = [[("a", 5)], [("a", 1)], [("a", 1), ("b", 9)], [("a", 1), ("b", 1)], [("a", 1), ("b", 1), ("c", 17)],
                [("a", 1), ("b", 1), ("c", 1)], [("a", 33), ("b", 1)], [("c", 1)]]
        for step in plan:
            entries = []
            for r, n in step:
                entries.append(StepEntry(r, tokens[r][at[r]:at[r] + n], (n - 1,)))
                at[r] += n
            rows.append(runner.step(entries))
        if graphs:
            assert runner.graph_replays == len(plan) and len(runner._graphs) == 3
        runs.append(rows)
    for eager, replayed in zip(*runs):
        torch.testing.assert_close(eager, replayed, rtol=1e-5, atol=1e-5)
