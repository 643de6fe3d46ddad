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
    given).  `window` keeps only the newest `window` keys visible, and beside
    them the first `keep_first` of the sequence.  `v_head_dim`: values of another
    size than keys.  `softcap` > 0: a scaled score s becomes softcap * tanh(s / softcap).
    `qk_norm` "projection": q and k are each divided by their root mean square over the
    whole projection (all heads at once; eps `qk_norm_eps`) and multiplied by the weights
    `q_norm.weight` / `k_norm.weight`, before the position encoding; "head": each head of q and of k is divided
    by its own root mean square and multiplied by a weight of `head_dim` entries that the heads share
    (`qk_norm_weight` False: by no weight; `qk_norm_after_rotation`: the norm comes behind the position encoding).
    `sink`: a learned number per head (`sink`, 32-bit) whose exponential joins the denominator of that head's
    softmax; it has no key and no value and is not scaled.  `output_gate`: the concatenated heads are multiplied
    element by element by sigmoid(`gate_proj.weight` x) before the output projection.
    `head_gate`: head h of the attention's output is multiplied by sigmoid(g_h), g = `g_proj.weight` x, one number
    per head, before the output projection.  `value_mix`: "source" leaves this layer's values of the step's tokens
    in `ctx.extras[value_mix_key]` for later layers; "mixed" stores (1 - l) v + l v_source instead of v, l the
    scalar tensor `value_mix` and v_source what the source layer left for the same tokens.  Everything that reads
    x is one product against the concatenated weights.
    """

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, head_dim: int, position: PartSpec,
                 dtype: torch.dtype, device: torch.device, bias: bool = False, out_bias: bool | None = None,
                 window: int | None = None, scale: float | None = None, cache_name: str = "kv",
                 v_head_dim: int | None = None, keep_first: int = 0, softcap: float = 0.0,
                 qk_norm: str | None = None, qk_norm_eps: float = 1e-6, head_gate: bool = False,
                 value_mix: str | None = None, value_mix_key: str = "value_mix", qk_norm_weight: bool = True,
                 qk_norm_after_rotation: bool = False, sink: bool = False, output_gate: bool = False) -> None:
        if heads % kv_heads:
            raise ValueError(f"heads={heads} is not a multiple of kv_heads={kv_heads}")
        if qk_norm not in (None, "projection", "head"):
            raise ValueError(f"qk_norm {qk_norm!r} is not supported; known: None, 'projection', 'head'")
        if value_mix not in (None, "source", "mixed"):
            raise ValueError(f"value_mix {value_mix!r} is not supported; known: None, 'source', 'mixed'")
        if (not qk_norm_weight or qk_norm_after_rotation) and qk_norm != "head":
            raise ValueError("a norm without a weight, or behind the rotation, is an option of qk_norm='head'")
        if head_gate and output_gate:
            raise ValueError("an attention has one gate: per head (head_gate) or per element (output_gate)")
        self.qk_norm_weight, self.qk_norm_after_rotation = bool(qk_norm_weight), bool(qk_norm_after_rotation)
        self.has_sink, self.output_gate = bool(sink), bool(output_gate)
        self.sink: torch.Tensor | None = None
        self.head_gate, self.value_mix, self.value_mix_key = bool(head_gate), value_mix, value_mix_key
        self.blend: torch.Tensor | None = None
        self.hidden_size, self.heads, self.kv_heads, self.head_dim = hidden_size, heads, kv_heads, head_dim
        self.v_head_dim = head_dim if v_head_dim is None else v_head_dim
        self.keep_first = int(keep_first) if window is not None else 0
        self.softcap = float(softcap or 0.0)
        self.qk_norm, self.qk_norm_eps = qk_norm, float(qk_norm_eps)
        self.q_norm_weight = self.k_norm_weight = None
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
        q, kv, v = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.kv_heads * self.v_head_dim
        specs = {
            "q_proj.weight": TensorSpec((q, self.hidden_size)),
            "k_proj.weight": TensorSpec((kv, self.hidden_size)),
            "v_proj.weight": TensorSpec((v, self.hidden_size)),
            "o_proj.weight": TensorSpec((self.hidden_size, self.heads * self.v_head_dim)),
        }
        if self.qk_norm == "head":
            if self.qk_norm_weight:
                specs.update({"q_norm.weight": TensorSpec((self.head_dim,), init="ones_normal"),
                              "k_norm.weight": TensorSpec((self.head_dim,), init="ones_normal")})
        elif self.qk_norm:
            specs.update({"q_norm.weight": TensorSpec((q,), init="ones_normal"),
                          "k_norm.weight": TensorSpec((kv,), init="ones_normal")})
        if self.head_gate:
            specs["g_proj.weight"] = TensorSpec((self.heads, self.hidden_size))
        if self.output_gate:
            specs["gate_proj.weight"] = TensorSpec((self.heads * self.v_head_dim, self.hidden_size))
        if self.has_sink:
            specs["sink"] = TensorSpec((self.heads,), kind="f32", init=_sink_init)
        if self.value_mix == "mixed":
            specs["value_mix"] = TensorSpec((), kind="f32", init=_blend_init)
        if self.bias:
            specs.update({"q_proj.bias": TensorSpec((q,), init="zeros"), "k_proj.bias": TensorSpec((kv,), init="zeros"),
                          "v_proj.bias": TensorSpec((v,), init="zeros")})
        if self.out_bias:
            specs["o_proj.bias"] = TensorSpec((self.hidden_size,), init="zeros")
        for name, spec in self.position.tensor_specs().items():
            specs["position." + name] = spec
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        weights = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        biases = [tensors[n] for n in ("q_proj.bias", "k_proj.bias", "v_proj.bias")] if self.bias else []
        order = self.position.pair_order() if hasattr(self.position, "pair_order") else None
        if order is not None:
            # The checkpoint pairs neighbouring dimensions: every head's rows of q and k (and what belongs to those
            # dimensions) are brought into the order whose pairs are half a rotary width apart.
            at = torch.tensor(order, device=weights[0].device)
            per_head = lambda t: t.unflatten(0, (-1, self.head_dim))[:, at].flatten(0, 1)
            weights[0], weights[1] = per_head(weights[0]), per_head(weights[1])
            if self.bias:
                biases[0], biases[1] = per_head(biases[0]), per_head(biases[1])
        if self.head_gate or self.output_gate:
            # The gate's rows ride behind v, filled up to a multiple of 16 rows (what the products' tiles like).
            gate = tensors["g_proj.weight" if self.head_gate else "gate_proj.weight"]
            pad = -(sum(w.shape[0] for w in weights) + gate.shape[0]) % 16
            weights += [gate, gate.new_zeros((pad, self.hidden_size))]
            if self.bias:
                biases.append(biases[0].new_zeros(gate.shape[0] + pad))
        self.qkv_weight = torch.cat(weights).contiguous()
        if self.bias:
            self.qkv_bias = torch.cat(biases).contiguous()
        if self.value_mix == "mixed":
            self.blend = tensors["value_mix"].to(torch.float32).reshape(1).contiguous()
        self.o_weight = tensors["o_proj.weight"]
        if self.qk_norm and self.qk_norm_weight:
            self.q_norm_weight, self.k_norm_weight = tensors["q_norm.weight"], tensors["k_norm.weight"]
            if order is not None and self.qk_norm == "head":
                self.q_norm_weight, self.k_norm_weight = self.q_norm_weight[at].contiguous(), self.k_norm_weight[at].contiguous()
            elif order is not None:
                self.q_norm_weight, self.k_norm_weight = per_head(self.q_norm_weight), per_head(self.k_norm_weight)
        if self.has_sink:
            self.sink = tensors["sink"].to(torch.float32).contiguous()
        self.o_bias = tensors.get("o_proj.bias") if self.out_bias else None
        self.position.bind({n[len("position."):]: t for n, t in tensors.items() if n.startswith("position.")})

    def cache_needs(self) -> tuple:
        return (KVNeed(self.kv_heads, self.head_dim, self.window, name=self.cache_name,
                       v_head_dim=None if self.v_head_dim == self.head_dim else self.v_head_dim,
                       keep_first=self.keep_first),)

    takes_pending_norm = True       # x may be an ops.PendingNorm: the qkv product folds the norm in
    adds_to_residual = True         # the output projection adds into the residual stream where its kernel can

    def forward(self, x, ctx: StepContext, cache: LayerCache, residual: torch.Tensor | None = None):
        kv = cache.kvs[self.cache_name]
        tokens = x.shape[0]
        q_width, kv_width = self.heads * self.head_dim, self.kv_heads * self.head_dim
        v_width = self.kv_heads * self.v_head_dim
        qkv = torch.empty((tokens, self.qkv_weight.shape[0]), dtype=x.dtype, device=x.device)
        ops.linear(x, self.qkv_weight, qkv, self.qkv_bias)
        if self.qk_norm == "head" or self.head_gate or self.output_gate or self.value_mix:
            return self._forward_prepared(qkv, ctx, cache, residual)
        if self.qk_norm:
            ops.qk_projection_rmsnorm_(qkv[:, :q_width], self.q_norm_weight, qkv[:, q_width:q_width + kv_width],
                                       self.k_norm_weight, self.qk_norm_eps)
        table = ctx.block_tables[kv.group]
        rotary = self.position.rotary()
        attended = torch.empty((tokens, self.heads * self.v_head_dim), dtype=x.dtype, device=x.device)
        masked = dict(keep_first=self.keep_first, softcap=self.softcap) if (self.keep_first or self.softcap) else {}
        if self.sink is not None:
            masked["sink"] = self.sink
        plain = not masked and self.v_head_dim == self.head_dim and (rotary is None or rotary.attention_scaling == 1.0)
        if plain and rotary is not None and ops.fused_decode_supports(x.dtype, self.heads, self.kv_heads, self.head_dim,
                                                                      rotary.rotary_dim, ctx.plan):
            # Every sequence brings one token: one launch rotates q and k, stores k and v and attends.
            newest = ops.NewestToken(rotary.inv_freq, qkv[:, q_width:], qkv[:, q_width + kv_width:],
                                     store=not cache.read_only)
            ops.paged_attention(qkv, qkv.shape[1], attended, kv.k_pool, kv.v_pool, table, ctx.query_start_loc,
                                ctx.context_lens, ctx.num_seqs, ctx.max_query_len, self.heads, self.kv_heads,
                                self.head_dim, self.scale, self.window or 0, plan=ctx.plan,
                                decode_splits=ctx.decode_splits, newest=newest)
            return ops.linear(attended, self.o_weight, None, self.o_bias, residual=residual)
        if rotary is None:
            self.position.apply(qkv[:, :q_width].unflatten(1, (self.heads, self.head_dim)),
                                qkv[:, q_width:q_width + kv_width].unflatten(1, (self.kv_heads, self.head_dim)), ctx)
        wide = {} if plain else dict(v_head_dim=self.v_head_dim,
                                     cos_sin_scale=rotary.attention_scaling if rotary else 1.0)
        ops.rope_kv_write(qkv, ctx.positions, ctx.seq_of_token, table, kv.k_pool, kv.v_pool,
                          rotary.inv_freq if rotary else None, self.heads, self.kv_heads, self.head_dim,
                          rotary.rotary_dim if rotary else 0, store=not cache.read_only, **wide)
        ops.paged_attention(qkv, qkv.shape[1], attended, kv.k_pool, kv.v_pool, table, ctx.query_start_loc,
                            ctx.context_lens, ctx.num_seqs, ctx.max_query_len, self.heads, self.kv_heads,
                            self.head_dim, self.scale, self.window or 0, plan=ctx.plan,
                            decode_splits=ctx.decode_splits, **masked)
        return ops.linear(attended, self.o_weight, None, self.o_bias, residual=residual)


    def _forward_prepared(self, qkv: torch.Tensor, ctx: StepContext, cache: LayerCache, residual):
        """The path of an attention with per-head q/k norms, mixed values or a head gate: one kernel normalises
        and rotates q and k, blends v and stores k and v; the attention reads q from the projection's rows; the
        gate multiplies the heads' outputs in place."""
        kv = cache.kvs[self.cache_name]
        tokens = qkv.shape[0]
        q_width, kv_width = self.heads * self.head_dim, self.kv_heads * self.head_dim
        v_width = self.kv_heads * self.v_head_dim
        table = ctx.block_tables[kv.group]
        rotary = self.position.rotary()
        if rotary is None:
            self.position.apply(qkv[:, :q_width].unflatten(1, (self.heads, self.head_dim)),
                                qkv[:, q_width:q_width + kv_width].unflatten(1, (self.kv_heads, self.head_dim)), ctx)
        values = qkv[:, q_width + kv_width:q_width + kv_width + v_width]
        other = None
        if self.value_mix == "source":
            ctx.extras[self.value_mix_key] = values
        elif self.value_mix == "mixed":
            other = ctx.extras.get(self.value_mix_key)
            if other is None or other.shape != values.shape:
                raise ValueError("a layer that mixes values runs behind the layer whose values it mixes in, "
                                 "with values of the same shape")
        per_head = self.qk_norm == "head"
        options = {}
        if per_head and (not self.qk_norm_weight or self.qk_norm_after_rotation):
            options = dict(unit_norm=not self.qk_norm_weight, norm_after_rotation=self.qk_norm_after_rotation)
        if rotary is not None and rotary.attention_scaling != 1.0:
            options["cos_sin_scale"] = rotary.attention_scaling
        ops.head_norm_rope_kv_write(qkv, ctx.positions, ctx.seq_of_token, table, kv.k_pool, kv.v_pool,
                                    rotary.inv_freq if rotary else None, self.heads, self.kv_heads, self.head_dim,
                                    rotary.rotary_dim if rotary else 0,
                                    self.q_norm_weight if per_head else None, self.k_norm_weight if per_head else None,
                                    self.qk_norm_eps, store=not cache.read_only, v_other=other,
                                    blend=self.blend if other is not None else None, **options)
        attended = torch.empty((tokens, self.heads * self.v_head_dim), dtype=qkv.dtype, device=qkv.device)
        masked = dict(keep_first=self.keep_first, softcap=self.softcap) if (self.keep_first or self.softcap) else {}
        if self.sink is not None:
            masked["sink"] = self.sink
        ops.paged_attention(qkv, qkv.shape[1], attended, kv.k_pool, kv.v_pool, table, ctx.query_start_loc,
                            ctx.context_lens, ctx.num_seqs, ctx.max_query_len, self.heads, self.kv_heads,
                            self.head_dim, self.scale, self.window or 0, plan=ctx.plan,
                            decode_splits=ctx.decode_splits, **masked)
        if self.head_gate:
            gate_at = q_width + kv_width + v_width
            ops.sigmoid_gate_heads_(attended, qkv[:, gate_at:gate_at + self.heads], self.heads)
        elif self.output_gate:
            gate_at = q_width + kv_width + v_width
            ops.sigmoid_gate_(attended, qkv[:, gate_at:gate_at + self.heads * self.v_head_dim])
        return ops.linear(attended, self.o_weight, None, self.o_bias, residual=residual)


def _sink_init(shape, generator):
    return torch.randn(shape, generator=generator)


def _blend_init(shape, generator):
    """A blending weight in [0.2, 0.8]."""
    return 0.2 + 0.6 * torch.rand(shape, generator=generator)


register_mixer("attention", Attention)
