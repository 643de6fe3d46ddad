"""Norm parts.  Interface of a norm:

    tensor_specs() -> {local name: TensorSpec}
    bind(tensors)                      # {local name: device tensor}
    forward(x, delta=None, rows=None, out=None) -> Tensor

`forward` normalises `x` [tokens, size].  With `delta` the sum x + delta is
what is normalised, and it is stored back into `x` (the residual stream moves on
in place) unless `rows` is given.  With `rows` (int32 indices) only those rows are
produced: the final norm computes just the rows whose logits are wanted.

Two optional abilities, which a block asks for only of a norm that declares them
(`apply_norm` in parts/block.py): `reads_row_stats`: `delta` may be an
`ops.RowStats` (the part before has already added its result into `x` and hands
on the new rows' sums of squares); `defers`: with `lazy=True` and such statistics
the norm does not run but returns an `ops.PendingNorm`, which the next part's
first product folds in.
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.registry import register_norm
from liteinfer_b200.parts.spec import TensorSpec


class RMSNorm:
    """y = weight * round(x * rsqrt(mean(x^2) + eps)), statistics in 32-bit.

    liteinfer/models/llama.py:35-48.
    """

    def __init__(self, size: int, eps: float, dtype: torch.dtype, device: torch.device) -> None:
        self.size, self.eps, self.dtype, self.device = size, float(eps), dtype, device
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), init="ones_normal")}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    reads_row_stats = True
    defers = True

    def forward(self, x: torch.Tensor, delta: "torch.Tensor | ops.RowStats | None" = None,
                rows: torch.Tensor | None = None, out: torch.Tensor | None = None, lazy: bool = False):
        if isinstance(delta, ops.RowStats):
            if lazy and out is None:
                return ops.PendingNorm(x, self.weight, self.eps, delta, rows)
            delta = None            # x holds the sum already
        n = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty((n, self.size), dtype=x.dtype, device=x.device)
        return ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows,
                           write_residual=delta is not None and rows is None)


class LayerNorm:
    """y = weight * (x - mean) / sqrt(var + eps), var the mean of the squared deviations; no bias.

    The stream `x` may be 32-bit whatever the engine's dtype: the norm reads it as it is and writes its result
    in the engine's dtype.  `delta` may be an `ops.NormedDelta` (the sublayer before is itself normalised before
    it is added): one kernel normalises the delta, adds it into the stream and normalises the sum."""

    def __init__(self, size: int, eps: float, dtype: torch.dtype, device: torch.device) -> None:
        self.size, self.eps, self.dtype, self.device = size, float(eps), dtype, device
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), init="ones_normal")}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def forward(self, x: torch.Tensor, delta: "torch.Tensor | ops.NormedDelta | None" = None,
                rows: torch.Tensor | None = None, out: torch.Tensor | None = None):
        if isinstance(delta, torch.Tensor):     # a plain delta: the sum first, then the norm
            ops.add_(x, delta)
            delta = None
        n = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty((n, self.size), dtype=self.weight.dtype, device=x.device)
        return ops.layernorm(x, self.weight, self.eps, out, delta=delta, rows=rows,
                             write_stream=delta is not None and rows is None)

    def normed_delta(self, value: torch.Tensor) -> "ops.NormedDelta":
        """What a sublayer's output becomes when this norm stands between it and the stream."""
        return ops.NormedDelta(value, self.weight, self.eps)


def _around_zero(shape, generator):
    return 0.05 * torch.randn(shape, generator=generator)


class AffineRMSNorm:
    """y = x / sqrt(mean(x^2) + eps) * (offset + weight) * mult: a root-mean-square norm whose stored weight is
    shifted by `offset` (0: the weight itself; 1: a stored weight that lies around zero) and whose result is
    multiplied by the constant `mult` (a model that scales what a sublayer adds to its residual stream).

    (offset + weight) * mult is formed once, in 32-bit, when the tensors are bound.  Like `LayerNorm` it reads a
    stream that may be 32-bit whatever the engine's dtype, writes the engine's dtype, and takes a pending
    `ops.NormedDelta`; `normed_delta` makes one of a sublayer's output, for a block that normalises what a sublayer
    gives back."""

    def __init__(self, size: int, eps: float, dtype: torch.dtype, device: torch.device, offset: float = 0.0,
                 mult: float = 1.0) -> None:
        self.size, self.eps, self.dtype, self.device = size, float(eps), dtype, device
        self.offset, self.mult = float(offset), float(mult)
        self.weight: torch.Tensor | None = None         # (offset + the stored weight) * mult, float32

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), kind="f32", init=_around_zero if self.offset else "ones_normal")}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = ((self.offset + tensors["weight"].to(torch.float32)) * self.mult).contiguous()

    def forward(self, x: torch.Tensor, delta: "torch.Tensor | ops.NormedDelta | None" = None,
                rows: torch.Tensor | None = None, out: torch.Tensor | None = None):
        if isinstance(delta, torch.Tensor):     # a plain delta: the sum first, then the norm
            ops.add_(x, delta)
            delta = None
        n = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty((n, self.size), dtype=self.dtype, device=x.device)
        return ops.layernorm(x, self.weight, self.eps, out, delta=delta, rows=rows,
                             write_stream=delta is not None and rows is None, centre=False)

    def normed_delta(self, value: torch.Tensor) -> "ops.NormedDelta":
        """What a sublayer's output becomes when this norm stands between it and the stream."""
        return ops.NormedDelta(value, self.weight, self.eps, centred=False)


class UnitOffsetRMSNorm(AffineRMSNorm):
    """y = x / sqrt(mean(x^2) + eps) * (1 + weight): `AffineRMSNorm` whose stored weight lies around zero."""

    def __init__(self, size: int, eps: float, dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(size, eps, dtype, device, offset=1.0)


class StreamRMSNorm:
    """y = u / sqrt(mean(u^2) + eps) * weight * out_scale, all in 32-bit, of a residual kept as `streams` 32-bit
    copies side by side in a row: u = sum_s read[s] * stream s (`read` None: the plain sum; with one stream, the
    stream).  `delta` may be an `ops.StreamUpdate`, the rewrite of the streams that the sublayer before left
    pending: the same kernel does it on its way (and stores it, unless only `rows` are asked for).  The result has
    the engine's dtype; the weight is kept 32-bit.  `out_scale`: a constant folded into the result (a model that
    scales its logits gives it to its last norm)."""

    def __init__(self, size: int, eps: float, dtype: torch.dtype, device: torch.device, streams: int = 1,
                 out_scale: float = 1.0) -> None:
        self.size, self.eps, self.dtype, self.device = size, float(eps), dtype, device
        self.streams, self.out_scale = int(streams), float(out_scale)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), kind="f32", init="ones_normal")}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, x: torch.Tensor, delta: "ops.StreamUpdate | None" = None, rows: torch.Tensor | None = None,
                out: torch.Tensor | None = None, read: torch.Tensor | None = None) -> torch.Tensor:
        if delta is not None and not isinstance(delta, ops.StreamUpdate):
            raise TypeError("a norm over residual streams takes a pending ops.StreamUpdate, not a plain delta")
        n = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty((n, self.size), dtype=self.dtype, device=x.device)
        return ops.stream_rmsnorm(x, self.weight, self.eps, out, read=read, update=delta, rows=rows,
                                  out_scale=self.out_scale)


register_norm("rmsnorm", RMSNorm)
register_norm("stream_rmsnorm", StreamRMSNorm)
register_norm("layernorm", LayerNorm)
register_norm("rmsnorm_unit_offset", UnitOffsetRMSNorm)
register_norm("rmsnorm_affine", AffineRMSNorm)
