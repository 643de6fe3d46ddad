"""Token embedding and output head.

Interface of an embedding: tensor_specs() / bind(tensors) / forward(token_ids) -> [tokens, hidden].
Interface of a head: tensor_specs() / bind(tensors) / forward(x [rows, hidden]) -> logits [rows, vocab].
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.registry import register_embedding, register_head
from liteinfer_b200.parts.spec import TensorSpec


class TokenEmbedding:
    """h[t] = table[token[t]] — liteinfer/models/llama.py:204,217.  `scale` multiplies every row; a model whose
    residual is 32-bit streams starts them with `forward_streams`, where the row is widened before the multiply."""

    def __init__(self, vocab_size: int, hidden_size: int, dtype: torch.dtype, device: torch.device,
                 scale: float = 1.0) -> None:
        self.vocab_size, self.hidden_size, self.dtype, self.device = vocab_size, hidden_size, dtype, device
        self.scale = float(scale)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = torch.empty((token_ids.numel(), self.hidden_size), dtype=self.weight.dtype, device=token_ids.device)
        # An id outside the table gives a zero row and raises the device's token flag, which
        # `ModelRunner.check_kernels` reports (the step function refuses such ids on the host before that).
        if self.scale != 1.0:
            if self.weight.dtype == torch.float32:
                return self.forward_streams(token_ids, 1)
            raise ValueError("a scaled embedding starts a 32-bit stream (forward_streams); it has no output of the engine's dtype")
        return ops.embedding(token_ids, self.weight, out, ops.token_error_flag(token_ids.device))

    def forward_streams(self, token_ids: torch.Tensor, copies: int) -> torch.Tensor:
        """[tokens, copies * hidden] float32: `copies` equal streams, each table[token] * scale."""
        out = torch.empty((token_ids.numel(), copies * self.hidden_size), dtype=torch.float32, device=token_ids.device)
        return ops.embedding_streams(token_ids, self.weight, out, self.scale, ops.token_error_flag(token_ids.device))


class LinearHead:
    """logits = x @ weight^T, no bias — liteinfer/models/llama.py:245,277.  A tied head
    is bound to the embedding's tensor by the loader (llama.py:246-247).  `softcap` c > 0: the logits become
    c * tanh(logits / c)."""

    def __init__(self, vocab_size: int, hidden_size: int, dtype: torch.dtype, device: torch.device,
                 softcap: float | None = None) -> None:
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.softcap = float(softcap) if softcap else 0.0
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    takes_pending_norm = True       # x may be an ops.PendingNorm: the product folds the final norm in

    def forward(self, x) -> torch.Tensor:
        logits = ops.linear(x, self.weight, None)
        if self.softcap > 0:
            ops.softcap_(logits, self.softcap)
        return logits


register_embedding("token_embedding", TokenEmbedding)
register_head("linear", LinearHead)
