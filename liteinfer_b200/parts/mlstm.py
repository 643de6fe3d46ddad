"""The mLSTM mixer: a matrix memory per head with exponential gates, kept stable by a running maximum.

Per token, with h the mixer's input and per head (dim, vdim the sizes of keys and values):

    q = W_q h * dim^-0.5;  k = W_k h;  v = W_v h
    i = cap * tanh((W_i h + b_i) / cap);  f = logsigmoid(cap * tanh((W_f h + b_f) / cap))     # logarithms of the gates
    m' = max(f + m, i)                                                                       # m starts at 0
    S <- exp(f + m - m') S + exp(i - m') k v^T;  n <- exp(f + m - m') n + exp(i - m') k;  m <- m'
    o = S^T q / (max(|n . q|, exp(-m)) + 1e-6)
    y = W_o (norm_weight * [o / rms(o) per head] * sigmoid(W_g h))                           # norm_weight: all heads' size

What a request keeps between steps is S, n and m, all 32-bit and zero at its start: two `StateNeed`s (n lies
beside S as one more column; m beside them, a copy per column, as the kernel wants it), so a sequence may arrive
whole, in portions or one token at a time.  Everything besides the projections is computed in 32-bit.
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.context import LayerCache, StateNeed, StepContext
from liteinfer_b200.parts.registry import register_mixer
from liteinfer_b200.parts.spec import TensorSpec


def _forget_bias_init(shape, generator):
    """Forget gates that start between 0.88 and 0.998."""
    return 2.0 + 4.0 * torch.rand(shape, generator=generator)


def _gate_weight_init(shape, generator):
    return 0.3 * torch.randn(shape, generator=generator)


class MLSTM:
    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, gate_cap: float, norm_eps: float,
                 dtype: torch.dtype, device: torch.device, state_name: str = "mlstm",
                 max_name: str = "mlstm_max") -> None:
        if not gate_cap > 0:
            raise ValueError("the gates' cap must be > 0")
        self.hidden_size, self.heads, self.dim, self.vdim = hidden_size, heads, dim, vdim
        self.gate_cap, self.norm_eps = float(gate_cap), float(norm_eps)
        self.state_name, self.max_name = state_name, max_name
        self.qk_width, self.v_width = heads * dim, heads * vdim
        # Columns of the fused projection: [q | k | v | g | i | f].
        self.k_at, self.v_at = self.qk_width, 2 * self.qk_width
        self.g_at = self.v_at + self.v_width
        self.i_at = self.g_at + self.v_width
        self.f_at = self.i_at + heads
        self.in_weight = self.i_bias = self.f_bias = self.norm_weight = self.o_weight = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        d, qk, v, h = self.hidden_size, self.qk_width, self.v_width, self.heads
        return {
            "q_proj.weight": TensorSpec((qk, d)), "k_proj.weight": TensorSpec((qk, d)),
            "v_proj.weight": TensorSpec((v, d)), "g_proj.weight": TensorSpec((v, d)),
            "o_proj.weight": TensorSpec((d, v)), "norm.weight": TensorSpec((v,), kind="f32", init="ones_normal"),
            "i_proj.weight": TensorSpec((h, d), init=_gate_weight_init), "i_proj.bias": TensorSpec((h,), kind="f32"),
            "f_proj.weight": TensorSpec((h, d), init=_gate_weight_init),
            "f_proj.bias": TensorSpec((h,), kind="f32", init=_forget_bias_init),
        }

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        # One product for everything that reads h, filled up to a multiple of 16 rows.
        parts = [tensors[n + "_proj.weight"] for n in ("q", "k", "v", "g", "i", "f")]
        pad = -sum(p.shape[0] for p in parts) % 16
        if pad:
            parts.append(parts[0].new_zeros((pad, self.hidden_size)))
        self.in_weight = torch.cat(parts).contiguous()
        self.i_bias, self.f_bias = tensors["i_proj.bias"].contiguous(), tensors["f_proj.bias"].contiguous()
        self.norm_weight, self.o_weight = tensors["norm.weight"].contiguous(), tensors["o_proj.weight"]

    def cache_needs(self) -> tuple:
        return (StateNeed((self.heads, self.vdim + 1, self.dim), "f32", name=self.state_name),   # S^T, then n
                StateNeed((self.heads, self.vdim + 1), "f32", name=self.max_name))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        if cache.read_only:
            raise ValueError("an mLSTM mixer cannot read another stop's state: its state moves with every token")
        tokens = x.shape[0]
        state, maxima = cache.states[self.state_name], cache.states[self.max_name]
        proj = ops.linear(x, self.in_weight, None)
        read = torch.empty((tokens, self.v_width), dtype=torch.float32, device=x.device)
        den = torch.empty((tokens, self.heads), dtype=torch.float32, device=x.device)
        ops.mlstm(proj, (0, self.k_at, self.v_at, self.i_at, self.f_at), self.i_bias, self.f_bias, self.gate_cap, state,
                  maxima, ctx.query_start_loc, ctx.state_slots, ctx.num_seqs, self.heads, self.dim, self.vdim, read, den,
                  ctx.max_query_len)
        gated = torch.empty((tokens, self.v_width), dtype=x.dtype, device=x.device)
        ops.gated_rmsnorm(read, proj[:, self.g_at:self.g_at + self.v_width], self.norm_weight, self.norm_eps, gated,
                          self.heads, gate_activation="sigmoid", den=den)
        return ops.linear(gated, self.o_weight, None)


register_mixer("mlstm", MLSTM)
