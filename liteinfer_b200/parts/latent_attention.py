"""The latent attention mixer: queries through a low-rank latent, keys and values expanded per head from one
shared latent per token, one rotated key part shared by all heads.

Per token, with h the mixer's input, H heads, per head d unrotated and r rotated query/key numbers, e value
numbers, latent sizes c_q (queries) and c (keys and values):

    c_q  = rmsnorm(W_dq h) * w_dq;   q_i = W_uq,i c_q = [q_i,plain (d) | q_i,rot (r)]        per head i
    [l | s] = W_dkv h;   latent = rmsnorm(l) * w_dkv (c numbers);   shared = rotate(s) (r numbers)
    k_i(j) = [W_uk,i latent(j) | shared(j)];   v_i(j) = W_uv,i latent(j)
    score_i(t, j) = (q_i,plain(t) . W_uk,i latent(j) + rotate(q_i,rot(t)) . shared(j)) * scale,   j <= t
    p_i(t, .) = softmax over the visible j, with exp(sink_i) as one more term of the denominator (optional)
    y = W_o ( [sum_j p_i(t, j) v_i(j)]_i * sigmoid(W_g h) )                                  (gate optional)

A token's cache entry is [latent | shared]: c + r numbers for all heads together (a `KVNeed` of one key head and
no values).  The products with W_uk and W_uv are moved to the query's side, q'_i = W_uk,i^T q_i,plain and
out_i = W_uv,i (sum_j p_i(t, j) latent(j)), so the attention kernel reads the entries as they are stored
(`ops.latent_attention`).  `own_kv` False: the layer makes no entries; it reads those of the stop that its
schedule entry names (`cache_of`) with its own W_uk, W_uv and queries.  Rotation: half-split pairs over the first
`rot.rotary_dim` numbers of the r-part; a position encoding whose checkpoint pairs neighbours has the rows of the
rotated parts reordered when the tensors are bound, and one that stretches cosines and sines (YaRN) has its factor
passed to the kernels.  `q_rank` None: no query latent, q = W_q h straight from the mixer's input.  `window`: the
query at position p reads the keys at p - window + 1 ... p, and the cache gives back the pages the window has
passed.  Norms, angles, scores, softmax and the gate's sigmoid are 32-bit.
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.context import KVNeed, LayerCache, StepContext
from liteinfer_b200.parts.registry import build_part, register_mixer
from liteinfer_b200.parts.spec import PartSpec, TensorSpec


def _sink_init(shape, generator):
    return torch.randn(shape, generator=generator)


class LatentAttention:
    def __init__(self, hidden_size: int, heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int | None,
                 kv_rank: int, scale: float, norm_eps: float, position: PartSpec, dtype: torch.dtype,
                 device: torch.device, sink: bool = True, gate: bool = True, own_kv: bool = True,
                 cache_name: str = "latent", window: int | None = None) -> None:
        self.hidden_size, self.heads, self.dim, self.rot_dim, self.vdim = hidden_size, heads, dim, rot_dim, vdim
        self.q_rank, self.kv_rank, self.scale, self.norm_eps = q_rank, kv_rank, float(scale), float(norm_eps)
        self.has_sink, self.has_gate, self.own_kv, self.cache_name = sink, gate, own_kv, cache_name
        self.dtype, self.device = dtype, device
        self.position = build_part("position", position, dtype=dtype, device=device)
        table = self.position.rotary()
        if table is None:       # no rotation: a table of no pairs
            from liteinfer_b200.parts.position import RotaryTable
            table = RotaryTable(torch.zeros(0, dtype=torch.float32, device=device), 0)
        if table.rotary_dim > rot_dim:
            raise ValueError("latent attention rotates (a part of) its shared key part")
        if window is not None and not own_kv:
            raise ValueError("a latent attention with a window keeps its own entries")
        self.rotary, self.window = table, window
        # Columns of the one product that reads h: [queries or their latent | key/value latent, shared key part | gate].
        self.q_width = q_rank if q_rank is not None else heads * (dim + rot_dim)
        self.kv_off = self.q_width if own_kv else None
        self.gate_off = self.q_width + (kv_rank + rot_dim if own_kv else 0)
        self.in_weight = self.q_norm = self.kv_norm = self.uq_weight = self.uk_t = self.uv = None
        self.sink = self.o_weight = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        d, H = self.hidden_size, self.heads
        if self.q_rank is not None:
            specs = {"dq.weight": TensorSpec((self.q_rank, d)),
                     "dq_norm.weight": TensorSpec((self.q_rank,), kind="f32", init="ones_normal"),
                     "uq.weight": TensorSpec((H * (self.dim + self.rot_dim), self.q_rank))}
        else:
            specs = {"q.weight": TensorSpec((H * (self.dim + self.rot_dim), d))}
        specs |= {
            "uk.weight": TensorSpec((H * self.dim, self.kv_rank)),
            "uv.weight": TensorSpec((H * self.vdim, self.kv_rank)),
            "o.weight": TensorSpec((d, H * self.vdim)),
        }
        if self.own_kv:
            specs["dkv.weight"] = TensorSpec((self.kv_rank + self.rot_dim, d))
            specs["dkv_norm.weight"] = TensorSpec((self.kv_rank,), kind="f32", init="ones_normal")
        if self.has_sink:
            specs["sink"] = TensorSpec((H,), kind="f32", init=_sink_init)
        if self.has_gate:
            specs["g.weight"] = TensorSpec((H * self.vdim, d))
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        H = self.heads
        # One product for everything that reads h: [query latent | key/value latent and shared key part | gate],
        # padded to a multiple of 16 rows.
        order = self.position.pair_order() if hasattr(self.position, "pair_order") else None
        at = None if order is None else torch.tensor(order, device=tensors["o.weight"].device)
        per = self.dim + self.rot_dim

        def queries(w: torch.Tensor) -> torch.Tensor:
            """The rows of the query projection with every head's rotated part in the kernels' order of pairs."""
            if at is None:
                return w
            heads = w.unflatten(0, (H, per))
            return torch.cat([heads[:, :self.dim], heads[:, self.dim:][:, at]], dim=1).flatten(0, 1)

        parts = [tensors["dq.weight"] if self.q_rank is not None else queries(tensors["q.weight"])]
        if self.own_kv:
            dkv = tensors["dkv.weight"]
            parts.append(dkv if at is None else torch.cat([dkv[:self.kv_rank], dkv[self.kv_rank:][at]]))
            self.kv_norm = tensors["dkv_norm.weight"].to(torch.float32).contiguous()
        if self.has_gate:
            parts.append(tensors["g.weight"])
        rows = sum(p.shape[0] for p in parts)
        if -rows % 16:
            parts.append(torch.zeros((-rows % 16, self.hidden_size), dtype=parts[0].dtype, device=parts[0].device))
        self.in_weight = torch.cat(parts).contiguous()
        if self.q_rank is not None:
            self.q_norm = tensors["dq_norm.weight"].contiguous()
            self.uq_weight = queries(tensors["uq.weight"])
        # W_uk per head, transposed: q'_i = W_uk,i^T q_i,plain is a product against [c, d] rows.
        self.uk_t = tensors["uk.weight"].view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv = tensors["uv.weight"].view(H, self.vdim, self.kv_rank).contiguous()
        self.sink = tensors["sink"].contiguous() if self.has_sink else None
        self.o_weight = tensors["o.weight"]

    def cache_needs(self) -> tuple:
        return (KVNeed(1, self.kv_rank + self.rot_dim, self.window, name=self.cache_name, v_head_dim=0),)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        if self.own_kv == cache.read_only:
            raise ValueError("a latent attention that makes its own entries needs a cache of its own; one that "
                             "makes none needs another stop's (ScheduleEntry.cache_of)")
        kv = cache.kvs[self.cache_name]
        table = ctx.block_tables[kv.group]
        tokens, H, c = x.shape[0], self.heads, self.kv_rank
        rot = self.rotary
        proj = ops.linear(x, self.in_weight, None)
        stretch = {} if rot.attention_scaling == 1.0 else {"cos_sin_scale": rot.attention_scaling}
        if self.q_rank is not None:
            q_latent = torch.empty((tokens, self.q_rank), dtype=x.dtype, device=x.device)
            ops.latent_prep(proj, 0, self.q_rank, self.kv_off, c, self.rot_dim, rot.rotary_dim, self.q_norm,
                            self.kv_norm, self.norm_eps, rot.inv_freq, ctx.positions, ctx.seq_of_token, table,
                            kv.k_pool, q_latent, store=self.own_kv, **stretch)
            q = ops.linear(q_latent, self.uq_weight, None)                  # [tokens, H * (d + r)]
        else:
            ops.latent_prep(proj, 0, 0, self.kv_off, c, self.rot_dim, rot.rotary_dim, None, self.kv_norm,
                            self.norm_eps, rot.inv_freq, ctx.positions, ctx.seq_of_token, table, kv.k_pool, None,
                            store=self.own_kv, **stretch)
            q = proj[:, :self.q_width]                                      # the queries' columns of the one product
        per_head = self.dim + self.rot_dim
        absorbed = torch.empty((H, tokens, c), dtype=x.dtype, device=x.device)
        ops.batched_linear(q.unflatten(1, (H, per_head))[:, :, :self.dim].transpose(0, 1), self.uk_t, absorbed)
        attended = torch.empty_like(absorbed)
        ops.latent_attention(absorbed, q, per_head, self.dim, attended, kv.k_pool, table, ctx.query_start_loc,
                             ctx.context_lens, rot.inv_freq, self.sink, ctx.num_seqs, ctx.max_query_len, H, c,
                             self.rot_dim, rot.rotary_dim, self.scale, plan=ctx.plan,
                             **({"window": self.window} if self.window else {}), **stretch)
        values = torch.empty((H, tokens, self.vdim), dtype=x.dtype, device=x.device)
        ops.batched_linear(attended, self.uv, values)
        joined = torch.empty((tokens, H * self.vdim), dtype=x.dtype, device=x.device)
        if self.has_gate:
            ops.gate_heads(values, proj[:, self.gate_off:self.gate_off + H * self.vdim], joined)
        else:
            ops.gate_heads(values, None, joined)
        return ops.linear(joined, self.o_weight, None)


register_mixer("latent_attention", LatentAttention)
