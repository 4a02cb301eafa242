"""A plain, slow Llama: whole sequences, no cache, one function for each part.

Written from the reference's formulas (each function cites file:line of
ValeGian/liteinfer); it shares no code with `liteinfer_b200`: it parses
config.json with `json`, reads tensors with `safetensors`, and computes with
stock torch ops on whatever device and dtype it is given.  `tests/golden/`
holds logits of the reference's own `LlamaForCausalLM` on a tiny random model,
and `test_plain_matches_reference_golden` compares this file with them.

In bfloat16 the functions round where the reference rounds (norm output before
the weight multiply, cos/sin tables, every elementwise result), so that
`forward(..., dtype=torch.bfloat16)` shows what a stock bfloat16 run gives.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors.torch import load_file


def read_model(model_dir: str | Path) -> tuple[dict, dict[str, torch.Tensor]]:
    """(config.json as a dict, tensors by name in float32)."""
    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    tensors: dict[str, torch.Tensor] = {}
    for shard in sorted(model_dir.glob("*.safetensors")):
        tensors.update(load_file(str(shard)))
    return config, {name: t.float() for name, t in tensors.items()}


def head_dim_of(config: dict) -> int:
    # liteinfer/models/llama.py:130 — head_dim, else hidden_size // num_attention_heads.
    return int(config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"])


def rope_inverse_frequencies(config: dict) -> torch.Tensor:
    """inv_freq [head_dim/2], float32.

    default: liteinfer/models/llama.py:66-71, inv_freq_i = theta^(-2i/d).
    llama3 / linear: llama.py:73-74 hands over to the rope registry; the rule is
    restated here: wavelength = 2*pi/inv_freq; shorter than original/high keeps its
    frequency, longer than original/low is divided by factor, the band between is
    blended with weight s = (original/wavelength - low) / (high - low).
    """
    d = head_dim_of(config)
    scaling = dict(config.get("rope_scaling") or {})
    scaling.update(config.get("rope_parameters") or {})
    theta = float(scaling.get("rope_theta", config.get("rope_theta")))
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind == "default":
        return inv_freq
    factor = float(scaling["factor"])
    if kind == "linear":
        return inv_freq / factor
    assert kind == "llama3", kind
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    low_freq_wavelen = original / low
    high_freq_wavelen = original / high
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_freq_wavelen, inv_freq / factor, inv_freq)
    smooth = (original / wavelen - low) / (high - low)
    blended = (1 - smooth) * scaled / factor + smooth * scaled
    is_medium = ~(wavelen < high_freq_wavelen) & ~(wavelen > low_freq_wavelen)
    return torch.where(is_medium, blended, scaled)


def rope_tables(inv_freq: torch.Tensor, positions: torch.Tensor, dtype: torch.dtype):
    """cos, sin [T, head_dim] — liteinfer/models/llama.py:78-86: angles in float32,
    `cat(freqs, freqs)`, tables rounded to the model dtype."""
    freqs = positions.float()[:, None] * inv_freq.float()[None, :].to(positions.device)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    # liteinfer/models/llama.py:89-92
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, heads, d]; liteinfer/models/llama.py:95-102 (tables broadcast over heads)."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    # liteinfer/models/llama.py:43-48 — statistics in float32, cast, then the weight.
    dtype = x.dtype
    x32 = x.float()
    variance = x32.pow(2).mean(-1, keepdim=True)
    x32 = x32 * torch.rsqrt(variance + eps)
    return weight * x32.to(dtype)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    # nn.Linear (liteinfer/models/llama.py:108-110,137-140): y = x W^T (+ b).
    y = x @ weight.t()
    return y if bias is None else y + bias


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scaling: float,
                     window: int | None = None) -> torch.Tensor:
    """q [T, heads, d], k/v [T, kv_heads, d] of one whole sequence -> [T, heads, d].

    liteinfer/models/attention.py:69-78 (query head h reads KV head h // groups),
    146-164 (scores * scaling, future keys masked, softmax in float32 cast back,
    P @ V).  `window` keeps only the newest `window` keys of each query; the
    reference's Llama has no window (None).
    """
    T, heads, _ = q.shape
    groups = heads // k.shape[1]
    k = k.repeat_interleave(groups, dim=1)
    v = v.repeat_interleave(groups, dim=1)
    scores = torch.einsum("thd,shd->hts", q, k) * scaling
    pos = torch.arange(T, device=q.device)
    hidden = pos[None, :] > pos[:, None]
    if window is not None:
        hidden = hidden | (pos[None, :] <= pos[:, None] - window)
    scores = scores.masked_fill(hidden[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
    return torch.einsum("hts,shd->thd", probs, v)


_ACT = {
    "silu": torch.nn.functional.silu,
    "gelu": torch.nn.functional.gelu,
    "gelu_pytorch_tanh": lambda x: torch.nn.functional.gelu(x, approximate="tanh"),
    "relu": torch.nn.functional.relu,
}


def gated_mlp(x, gate_w, up_w, down_w, act: str, gate_b=None, up_b=None, down_b=None):
    # liteinfer/models/llama.py:114 — down(act(gate(x)) * up(x)).
    return linear(_ACT[act](linear(x, gate_w, gate_b)) * linear(x, up_w, up_b), down_w, down_b)


def attention_block(x, w: dict, prefix: str, config: dict, cos, sin, window=None):
    """liteinfer/models/llama.py:142-163: q/k/v projections, rope on q and k, attention, o_proj."""
    heads, kv_heads = config["num_attention_heads"], config.get("num_key_value_heads") or config["num_attention_heads"]
    d = head_dim_of(config)
    T = x.shape[0]
    b = (lambda n: w.get(prefix + n + ".bias"))
    q = linear(x, w[prefix + "q_proj.weight"], b("q_proj")).view(T, heads, d)
    k = linear(x, w[prefix + "k_proj.weight"], b("k_proj")).view(T, kv_heads, d)
    v = linear(x, w[prefix + "v_proj.weight"], b("v_proj")).view(T, kv_heads, d)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    out = causal_attention(q, k, v, d ** -0.5, window)  # llama.py:134 scaling = head_dim^-0.5
    return linear(out.reshape(T, heads * d), w[prefix + "o_proj.weight"], b("o_proj"))


def decoder_layer(x, w: dict, layer: int, config: dict, cos, sin):
    """liteinfer/models/llama.py:174-192: pre-norm residual block."""
    p = f"model.layers.{layer}."
    eps = float(config["rms_norm_eps"])
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    x = x + attention_block(h, w, p + "self_attn.", config, cos, sin)
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    m = p + "mlp."
    return x + gated_mlp(h, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"],
                         config.get("hidden_act", "silu"), w.get(m + "gate_proj.bias"),
                         w.get(m + "up_proj.bias"), w.get(m + "down_proj.bias"))


def hidden_states(config: dict, weights: dict[str, torch.Tensor], tokens, dtype=torch.float32,
                  device="cpu") -> torch.Tensor:
    """Final-norm output [T, hidden] of one whole sequence (liteinfer/models/llama.py:211-229)."""
    w = {n: t.to(device=device, dtype=dtype) for n, t in weights.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long, device=device)
    x = w["model.embed_tokens.weight"][ids]
    positions = torch.arange(len(ids), device=device)
    cos, sin = rope_tables(rope_inverse_frequencies(config), positions, dtype)
    for layer in range(config["num_hidden_layers"]):
        x = decoder_layer(x, w, layer, config, cos, sin)
    return rms_norm(x, w["model.norm.weight"], float(config["rms_norm_eps"]))


def forward(config: dict, weights: dict[str, torch.Tensor], tokens, dtype=torch.float32,
            device="cpu") -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence, as float32.

    liteinfer/models/llama.py:269-278; a tied head reads the embedding (246-247).
    """
    h = hidden_states(config, weights, tokens, dtype, device)
    head = weights.get("lm_head.weight")
    if config.get("tie_word_embeddings", False) or head is None:
        head = weights["model.embed_tokens.weight"]
    return linear(h, head.to(device=device, dtype=dtype)).float()


def greedy(config: dict, weights: dict[str, torch.Tensor], prompt, num_new: int, dtype=torch.float32,
           device="cpu") -> list[int]:
    """`num_new` greedy tokens after `prompt`, recomputing the whole sequence each time."""
    tokens = list(prompt)
    for _ in range(num_new):
        logits = forward(config, weights, tokens, dtype, device)
        tokens.append(int(torch.argmax(logits[-1]).item()))
    return tokens[len(prompt):]
