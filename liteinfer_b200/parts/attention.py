"""The attention mixer.  Interface of a mixer:

    tensor_specs() / bind(tensors)
    cache_needs() -> tuple of KVNeed / StateNeed     # what the cache manager must keep for this layer
    forward(x, ctx, cache) -> Tensor [tokens, hidden]

`x` holds the step's tokens of every sequence end to end; `ctx` (StepContext)
says which token belongs to which sequence and position; `cache` (LayerCache) is
this layer's pages or state.  A mixer writes what it must remember into `cache`
and reads earlier tokens from there only, so a sequence may arrive whole, in
portions, or one token at a time.
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.context import KVNeed, LayerCache, StepContext
from liteinfer_b200.parts.registry import build_part, register_mixer
from liteinfer_b200.parts.spec import PartSpec, TensorSpec


class Attention:
    """Causal grouped-query attention over a paged cache.

    liteinfer/models/llama.py:117-163: q/k/v projections, the position encoding
    on q and k, keys and values stored, attention of the new queries over
    everything stored, output projection.  Query head h reads KV head
    h // (heads // kv_heads); scores are scaled by `scale` (head_dim^-0.5 unless
    given).  `window` keeps only the newest `window` keys visible.  The three
    projections are one product against the concatenated weights.
    """

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, head_dim: int, position: PartSpec,
                 dtype: torch.dtype, device: torch.device, bias: bool = False, out_bias: bool | None = None,
                 window: int | None = None, scale: float | None = None, cache_name: str = "kv") -> None:
        if heads % kv_heads:
            raise ValueError(f"heads={heads} is not a multiple of kv_heads={kv_heads}")
        self.hidden_size, self.heads, self.kv_heads, self.head_dim = hidden_size, heads, kv_heads, head_dim
        self.bias = bias
        self.out_bias = bias if out_bias is None else out_bias
        self.window = window
        self.cache_name = cache_name    # under which name this mixer's pages lie in its layer's cache
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.dtype, self.device = dtype, device
        self.position = build_part("position", position, dtype=dtype, device=device)
        self.qkv_weight: torch.Tensor | None = None
        self.qkv_bias: torch.Tensor | None = None
        self.o_weight: torch.Tensor | None = None
        self.o_bias: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        q, kv = self.heads * self.head_dim, self.kv_heads * self.head_dim
        specs = {
            "q_proj.weight": TensorSpec((q, self.hidden_size)),
            "k_proj.weight": TensorSpec((kv, self.hidden_size)),
            "v_proj.weight": TensorSpec((kv, self.hidden_size)),
            "o_proj.weight": TensorSpec((self.hidden_size, q)),
        }
        if self.bias:
            specs.update({"q_proj.bias": TensorSpec((q,), init="zeros"), "k_proj.bias": TensorSpec((kv,), init="zeros"),
                          "v_proj.bias": TensorSpec((kv,), init="zeros")})
        if self.out_bias:
            specs["o_proj.bias"] = TensorSpec((self.hidden_size,), init="zeros")
        for name, spec in self.position.tensor_specs().items():
            specs["position." + name] = spec
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.qkv_weight = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]])
        if self.bias:
            self.qkv_bias = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]])
        self.o_weight = tensors["o_proj.weight"]
        self.o_bias = tensors.get("o_proj.bias") if self.out_bias else None
        self.position.bind({n[len("position."):]: t for n, t in tensors.items() if n.startswith("position.")})

    def cache_needs(self) -> tuple:
        return (KVNeed(self.kv_heads, self.head_dim, self.window, name=self.cache_name),)

    takes_pending_norm = True       # x may be an ops.PendingNorm: the qkv product folds the norm in
    adds_to_residual = True         # the output projection adds into the residual stream where its kernel can

    def forward(self, x, ctx: StepContext, cache: LayerCache, residual: torch.Tensor | None = None):
        kv = cache.kvs[self.cache_name]
        tokens = x.shape[0]
        q_width = self.heads * self.head_dim
        qkv = torch.empty((tokens, q_width + 2 * self.kv_heads * self.head_dim), dtype=x.dtype, device=x.device)
        ops.linear(x, self.qkv_weight, qkv, self.qkv_bias)
        table = ctx.block_tables[kv.group]
        rotary = self.position.rotary()
        attended = torch.empty((tokens, q_width), dtype=x.dtype, device=x.device)
        if rotary is not None and ops.fused_decode_supports(x.dtype, self.heads, self.kv_heads, self.head_dim,
                                                            rotary.rotary_dim, ctx.plan):
            # Every sequence brings one token: one launch rotates q and k, stores k and v and attends.
            kv_width = self.kv_heads * self.head_dim
            newest = ops.NewestToken(rotary.inv_freq, qkv[:, q_width:], qkv[:, q_width + kv_width:],
                                     store=not cache.read_only)
            ops.paged_attention(qkv, qkv.shape[1], attended, kv.k_pool, kv.v_pool, table, ctx.query_start_loc,
                                ctx.context_lens, ctx.num_seqs, ctx.max_query_len, self.heads, self.kv_heads,
                                self.head_dim, self.scale, self.window or 0, plan=ctx.plan,
                                decode_splits=ctx.decode_splits, newest=newest)
            return ops.linear(attended, self.o_weight, None, self.o_bias, residual=residual)
        if rotary is None:
            kv_width = self.kv_heads * self.head_dim
            self.position.apply(qkv[:, :q_width].unflatten(1, (self.heads, self.head_dim)),
                                qkv[:, q_width:q_width + kv_width].unflatten(1, (self.kv_heads, self.head_dim)), ctx)
        ops.rope_kv_write(qkv, ctx.positions, ctx.seq_of_token, table, kv.k_pool, kv.v_pool,
                          rotary.inv_freq if rotary else None, self.heads, self.kv_heads, self.head_dim,
                          rotary.rotary_dim if rotary else 0, store=not cache.read_only)
        ops.paged_attention(qkv, qkv.shape[1], attended, kv.k_pool, kv.v_pool, table, ctx.query_start_loc,
                            ctx.context_lens, ctx.num_seqs, ctx.max_query_len, self.heads, self.kv_heads,
                            self.head_dim, self.scale, self.window or 0, plan=ctx.plan,
                            decode_splits=ctx.decode_splits)
        return ops.linear(attended, self.o_weight, None, self.o_bias, residual=residual)


register_mixer("attention", Attention)
