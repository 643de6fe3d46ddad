"""Re-entry parts: what a model does to its residual stream before a stop that its schedule marks `reenter`.

Interface of a re-entry part:

    tensor_specs() / bind(tensors)
    forward(hidden, delta, embedded) -> (hidden, delta)

`hidden` and `delta` are the residual stream and what is still to be added to it (as a block hands them on);
`embedded` is the embedding's output of the step's tokens, in the engine's dtype.  The stream is changed in place.
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.registry import register_reentry
from liteinfer_b200.parts.spec import TensorSpec


class EmbeddingRemix:
    """x <- W [x; e]: the stream and the embedding's output side by side, through one product ([hidden, 2 hidden],
    the stream's columns first).  A model that runs a group of layers several times feeds the tokens in again
    this way at the start of every pass."""

    def __init__(self, hidden_size: int, dtype: torch.dtype, device: torch.device) -> None:
        self.hidden_size, self.dtype, self.device = hidden_size, dtype, device
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h = self.hidden_size
        return {"weight": TensorSpec((h, 2 * h), init=_remix_init)}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def forward(self, hidden: torch.Tensor, delta, embedded: torch.Tensor):
        if isinstance(delta, ops.NormedDelta):
            ops.layernorm_add(hidden, delta.value, delta.weight, delta.eps, centred=delta.centred)
        elif isinstance(delta, torch.Tensor):
            ops.add_(hidden, delta)
        h = self.hidden_size
        both = torch.empty((hidden.shape[0], 2 * h), dtype=embedded.dtype, device=hidden.device)
        ops.convert(hidden, both[:, :h])
        ops.convert(embedded, both[:, h:])
        mixed = ops.linear(both, self.weight, None)
        ops.convert(mixed, hidden)
        return hidden, None


def _remix_init(shape, generator):
    """Near [I, 0] + noise: a random model's stream keeps its size from pass to pass."""
    h = shape[0]
    return torch.cat([torch.eye(h), torch.zeros(h, h)], dim=1) * 0.7 + 0.02 * torch.randn(shape, generator=generator)


register_reentry("embedding_remix", EmbeddingRemix)
