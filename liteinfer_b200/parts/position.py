"""Position-encoding parts.  Interface of a position encoding:

    tensor_specs() / bind(tensors)     # most have no tensors
    rotary() -> RotaryTable | None     # the fused path: the mixer's kernel rotates q and k itself
    apply(q, k, ctx) -> None           # otherwise: change q and k in place before k is stored

A mixer asks `rotary()` first.  An encoding that is not a rotation of pairs
returns None there and does its work in `apply`.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from liteinfer_b200.parts.registry import register_position_encoding
from liteinfer_b200.parts.spec import TensorSpec


@dataclass
class RotaryTable:
    inv_freq: torch.Tensor   # [rotary_dim / 2] float32 on the device
    rotary_dim: int
    attention_scaling: float = 1.0


def rotary_inverse_frequencies(head_dim: int, theta: float, rope_type: str = "default", factor: float = 1.0,
                               low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                               original_max_position_embeddings: int = 0) -> torch.Tensor:
    """inv_freq [head_dim / 2] in float32 (CPU).

    default: theta^(-2i/d) (liteinfer/models/llama.py:66-71).  linear: divided by
    `factor`.  llama3 (llama.py:73-74 takes it from the rope registry): a
    wavelength 2*pi/f longer than original/low is divided by factor, shorter than
    original/high is kept, between them the two are blended with weight
    (original/wavelength - low) / (high - low).
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    if rope_type == "default":
        return inv_freq
    if rope_type == "linear":
        return inv_freq / factor
    if rope_type != "llama3":
        raise ValueError(f"rope_type {rope_type!r} is not supported")
    original = float(original_max_position_embeddings)
    wavelen = 2 * math.pi / inv_freq
    long_wave = wavelen > original / low_freq_factor
    short_wave = wavelen < original / high_freq_factor
    scaled = torch.where(long_wave, inv_freq / factor, inv_freq)
    smooth = (original / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    blended = (1 - smooth) * scaled / factor + smooth * scaled
    return torch.where(~long_wave & ~short_wave, blended, scaled)


def yarn_inverse_frequencies(dims: int, theta: float, factor: float, original: float, fast: float,
                             slow: float) -> tuple[torch.Tensor, float]:
    """(inv_freq [dims / 2] float32, the factor that multiplies every cosine and sine) of YaRN scaling.

    A pair that turns `t` times within `original` positions has the (fractional) index
    n(t) = dims * ln(original / (2 pi t)) / (2 ln theta).  Pairs up to lo = floor(n(fast)) keep their frequency
    f_i = theta^(-2i/dims), pairs from hi = ceil(n(slow)) on have it divided by `factor`, and between them the two
    are blended linearly in i (lo and hi clamped to [0, dims - 1], a span of at least 0.001).  Cosines and sines
    are stretched by 0.1 ln(factor) + 1.  Computed in 64-bit, rounded once.
    """
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = float(theta) ** (-2.0 * i / dims)

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(theta))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    blended = freq / factor * ramp + freq * (1.0 - ramp)
    return blended.to(torch.float32), 0.1 * math.log(factor) + 1.0


class RotaryEmbedding:
    """Half-split rotary embedding: dimension j pairs with j + rotary_dim/2 (llama.py:89-102).  `rope_type`
    "yarn" takes `factor`, `original_max_position_embeddings`, `fast` and `slow` (`yarn_inverse_frequencies`).
    `exact`: the plain frequencies computed in 64-bit and rounded once, instead of in 32-bit as the reference does.
    `pairs` "interleaved": the checkpoint pairs dimension 2i with 2i + 1.  The kernels rotate half-split pairs, so a
    mixer brings the rows of its query and key projections into the order `pair_order()` when it binds them:
    every score is a sum over the same products, in another order."""

    def __init__(self, head_dim: int, theta: float, dtype: torch.dtype, device: torch.device,
                 rotary_dim: int | None = None, rope_type: str = "default", factor: float = 1.0,
                 low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                 original_max_position_embeddings: float = 0, fast: float | None = None,
                 slow: float | None = None, exact: bool = False, pairs: str = "half") -> None:
        if pairs not in ("half", "interleaved"):
            raise ValueError(f"pairs {pairs!r} is not supported; known: 'half', 'interleaved'")
        self.head_dim, self.pairs = head_dim, pairs
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        scale = 1.0
        if exact:
            # theta^(-2i/d) in 64-bit, rounded once (the plain frequencies only).
            if rope_type != "default":
                raise ValueError("exact frequencies are the plain ones (rope_type 'default')")
            i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
            inv_freq = (float(theta) ** (-2.0 * i / self.rotary_dim)).to(torch.float32)
        elif rope_type == "yarn":
            if fast is None or slow is None or not original_max_position_embeddings > 0:
                raise ValueError("yarn scaling needs factor, original_max_position_embeddings, fast and slow")
            inv_freq, scale = yarn_inverse_frequencies(self.rotary_dim, theta, factor,
                                                       float(original_max_position_embeddings), fast, slow)
        else:
            inv_freq = rotary_inverse_frequencies(self.rotary_dim, theta, rope_type, factor, low_freq_factor,
                                                  high_freq_factor, int(original_max_position_embeddings))
        self.table = RotaryTable(inv_freq.to(device), self.rotary_dim, scale)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        pass

    def rotary(self) -> RotaryTable | None:
        return self.table

    def pair_order(self) -> list[int] | None:
        """None where the checkpoint's pairs are half-split already; else, for a head (or rotated part) of
        `head_dim` numbers, which stored dimension comes to stand at each place: the even ones of the first
        `rotary_dim`, then the odd ones, then the rest as they are."""
        if self.pairs == "half":
            return None
        r = self.rotary_dim
        return list(range(0, r, 2)) + list(range(1, r, 2)) + list(range(r, self.head_dim))

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx) -> None:  # the fused path covers it
        raise NotImplementedError


class NoPositionEncoding:
    """Leaves q and k as they are."""

    def __init__(self, dtype: torch.dtype, device: torch.device) -> None:
        pass

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        pass

    def rotary(self) -> RotaryTable | None:
        return None

    def pair_order(self) -> list[int] | None:
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx) -> None:
        pass


register_position_encoding("rotary", RotaryEmbedding)
register_position_encoding("none", NoPositionEncoding)
