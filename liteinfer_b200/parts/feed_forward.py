"""Feed-forward parts.  Interface of a feed-forward:

    tensor_specs() / bind(tensors)
    forward(x, ctx) -> Tensor [tokens, hidden]
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.context import StepContext
from liteinfer_b200.parts.registry import register_feed_forward
from liteinfer_b200.parts.spec import TensorSpec


class GatedMLP:
    """down(act(gate(x)) * up(x)) — liteinfer/models/llama.py:105-114.

    gate and up are one product against the concatenated weights; the activation
    and the multiply are one kernel.
    """

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str, dtype: torch.dtype,
                 device: torch.device, bias: bool = False) -> None:
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} has no kernel; known: {sorted(ops.ACTIVATIONS)}")
        self.hidden_size, self.intermediate_size, self.activation, self.bias = (
            hidden_size, intermediate_size, activation, bias)
        self.gate_up_weight = self.gate_up_bias = self.down_weight = self.down_bias = None
        self.interleaved = False

    def tensor_specs(self) -> dict[str, TensorSpec]:
        i, h = self.intermediate_size, self.hidden_size
        specs = {"gate_proj.weight": TensorSpec((i, h)), "up_proj.weight": TensorSpec((i, h)),
                 "down_proj.weight": TensorSpec((h, i))}
        if self.bias:
            specs.update({"gate_proj.bias": TensorSpec((i,), init="zeros"), "up_proj.bias": TensorSpec((i,), init="zeros"),
                          "down_proj.bias": TensorSpec((h,), init="zeros")})
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        # bfloat16: gate and up rows interleaved in eights, the layout whose product, activation and
        # multiply one decode kernel can do together; otherwise gate rows first, then up rows.
        self.interleaved = gate.dtype == torch.bfloat16 and self.intermediate_size % 8 == 0
        self.gate_up_weight = self._pair(gate, up)
        self.down_weight = tensors["down_proj.weight"]
        if self.bias:
            self.gate_up_bias = self._pair(tensors["gate_proj.bias"], tensors["up_proj.bias"])
            self.down_bias = tensors["down_proj.bias"]

    def _pair(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        if not self.interleaved:
            return torch.cat([gate, up])
        rest = gate.shape[1:]
        stacked = torch.stack([gate.reshape(-1, 8, *rest), up.reshape(-1, 8, *rest)], dim=1)
        return stacked.reshape(2 * gate.shape[0], *rest).contiguous()

    takes_pending_norm = True       # x may be an ops.PendingNorm: the gate_up product folds the norm in
    adds_to_residual = True         # the down projection adds into the residual stream where its kernel can

    def forward(self, x, ctx: StepContext, residual: torch.Tensor | None = None):
        tokens = x.shape[0]
        hidden = torch.empty((tokens, self.intermediate_size), dtype=x.dtype, device=x.device)
        if self.interleaved and ops.gated_linear_supported(x, self.gate_up_weight):
            ops.gated_linear(x, self.gate_up_weight, hidden, self.activation, self.gate_up_bias)
        else:
            gate_up = torch.empty((tokens, 2 * self.intermediate_size), dtype=x.dtype, device=x.device)
            ops.linear(x, self.gate_up_weight, gate_up, self.gate_up_bias)
            if self.interleaved:
                ops.act_mul_interleaved(gate_up, hidden, self.activation)
            else:
                ops.act_mul(gate_up, hidden, self.activation)
        return ops.linear(hidden, self.down_weight, None, self.down_bias, residual=residual)


class DenseMLP:
    """down(act(up(x))): a feed-forward without a gate; `activation` from `ops.UNARY_ACTIVATIONS`
    ("relu_squared": the square of relu)."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str, dtype: torch.dtype,
                 device: torch.device) -> None:
        if activation not in ops.UNARY_ACTIVATIONS:
            raise ValueError(f"activation {activation!r} has no kernel; known: {sorted(ops.UNARY_ACTIVATIONS)}")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.up_weight = self.down_weight = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        i, h = self.intermediate_size, self.hidden_size
        return {"up_proj.weight": TensorSpec((i, h)), "down_proj.weight": TensorSpec((h, i))}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.up_weight, self.down_weight = tensors["up_proj.weight"], tensors["down_proj.weight"]

    def forward(self, x, ctx: StepContext):
        hidden = ops.linear(x, self.up_weight, None, activation=self.activation)      # one kernel for a few rows of x
        return ops.linear(hidden, self.down_weight, None)


class RoutedExperts:
    """A mixture of experts: every token runs `top` of `experts` small gated feed-forwards and adds up their
    outputs, weighted by the router's scores.

    Router: logits = `router.weight` x in 32-bit; scores = softmax over all experts.  With `groups` > 1 the experts
    form that many equal groups of neighbours; a group's score is its largest score, and only experts of the best
    `groups_keep` groups can be chosen.  The `top` largest scores among those are chosen; the weights are those
    scores themselves (`renormalise`: divided by their sum).  Expert e: down_e(act(gate_e x, up_e x)), without
    biases, `activation` of `ops.EXPERT_ACTIVATIONS` ("swiglu": silu(g) * u; "capped_swiglu": g' = min(g, limit),
    u' = clamp(u, -limit, limit), g' * sigmoid(alpha * g') * (u' + 1)).  The step's (token, slot) pairs are ordered
    by expert on the device, and both products run tile by tile over each expert's rows, so an expert's weights are
    read once per tile of its tokens and nothing is read on the host.
    """

    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int, dtype: torch.dtype,
                 device: torch.device, groups: int = 1, groups_keep: int = 1, activation: str = "swiglu",
                 limit: float = 0.0, alpha: float = 1.0, renormalise: bool = False) -> None:
        if activation not in ops.EXPERT_ACTIVATIONS:
            raise ValueError(f"activation {activation!r} has no kernel; known: {sorted(ops.EXPERT_ACTIVATIONS)}")
        if not 1 <= top <= experts or groups < 1 or experts % groups or not 1 <= groups_keep <= groups:
            raise ValueError("a mixture of experts needs 1 <= top <= experts, groups that divide experts, and "
                             "1 <= groups_keep <= groups")
        if groups_keep * (experts // groups) < top:
            raise ValueError("the kept groups hold fewer experts than `top`")
        self.hidden_size, self.intermediate_size, self.experts, self.top = hidden_size, intermediate_size, experts, top
        self.groups, self.groups_keep, self.activation = groups, groups_keep, activation
        self.limit, self.alpha, self.renormalise = float(limit), float(alpha), bool(renormalise)
        self.dtype, self.device = dtype, device
        self.router = self.gate_up = self.down = None
        self.eights = False

    def tensor_specs(self) -> dict[str, TensorSpec]:
        f, h = self.intermediate_size, self.hidden_size
        specs = {"router.weight": TensorSpec((self.experts, h), kind="f32")}
        for e in range(self.experts):
            specs.update({f"experts.{e}.gate_proj.weight": TensorSpec((f, h)),
                          f"experts.{e}.up_proj.weight": TensorSpec((f, h)),
                          f"experts.{e}.down_proj.weight": TensorSpec((h, f))})
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.router = tensors["router.weight"].to(torch.float32).contiguous()
        # [experts, 2 * ff, hidden]: an expert's gate rows, then its up rows; in bfloat16 with a width in eights both
        # interleaved in eights (eight gate rows, then their eight up rows), the layout whose product and activation
        # the tensor-core kernels do together.  [experts, hidden, ff].
        gates = [tensors[f"experts.{e}.gate_proj.weight"] for e in range(self.experts)]
        ups = [tensors[f"experts.{e}.up_proj.weight"] for e in range(self.experts)]
        self.eights = gates[0].dtype == torch.bfloat16 and self.intermediate_size % 8 == 0
        if self.eights:
            pair = lambda g, u: torch.stack([g.unflatten(0, (-1, 8)), u.unflatten(0, (-1, 8))], dim=1).flatten(0, 2)
        else:
            pair = lambda g, u: torch.cat([g, u])
        self.gate_up = torch.stack([pair(g, u) for g, u in zip(gates, ups)]).contiguous()
        self.down = torch.stack([tensors[f"experts.{e}.down_proj.weight"] for e in range(self.experts)]).contiguous()

    def route(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """(chosen experts [tokens, top] int32, their weights [tokens, top] float32)."""
        tokens = x.shape[0]
        ids = torch.empty((tokens, self.top), dtype=torch.int32, device=x.device)
        weights = torch.empty((tokens, self.top), dtype=torch.float32, device=x.device)
        ops.moe_router(x, self.router, self.top, self.groups, self.groups_keep, self.renormalise, ids, weights)
        return ids, weights

    def forward(self, x, ctx: StepContext):
        ids, weights = self.route(x)
        out = torch.empty((x.shape[0], self.hidden_size), dtype=x.dtype, device=x.device)
        return ops.moe_experts(x, self.gate_up, self.down, ids, weights, self.activation, self.limit, self.alpha,
                               self.eights, out)


register_feed_forward("gated_mlp", GatedMLP)
register_feed_forward("routed_experts", RoutedExperts)
register_feed_forward("dense_mlp", DenseMLP)
