"""Block arrangements: how a layer's mixer, feed-forward and norms are wired.

Interface of a block:

    roles = {role: registry}                # its parts by role, and the registry each is built from
                                            # ("mixer", "feed_forward", "norm", "position")
    __init__(parts: {role: built part})
    forward(hidden, delta, ctx, cache) -> (hidden, delta)

A block may have any roles (two mixers side by side, a third norm); it hands
each part what it needs of `cache`, where every part finds its own pages or
state under the name its need declared.

The residual stream travels as a pair: `hidden` [tokens, hidden_size] and a
`delta` not yet added to it (None at the first layer).  A block's first norm
adds the pending delta while it normalises, so the sum costs no pass of its own;
what the block returns is again (hidden, pending delta).  Where a part's last
product can add into the stream itself (`adds_to_residual`), the pending delta
is instead an `ops.RowStats`: the sum is made, and the next norm gets the rows'
statistics for nothing (`apply_norm`, `run_part`).
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.context import LayerCache, StepContext
from liteinfer_b200.parts.registry import register_block


def apply_norm(norm, hidden: torch.Tensor, delta, consumer=None, rows: torch.Tensor | None = None):
    """Runs `norm` on the residual stream, whatever form the pending `delta` has (None, a tensor still to be
    added, or `ops.RowStats` of a sum already made), using what the norm and the part that reads its result say
    they can do: a norm that `defers` hands a consumer that `takes_pending_norm` the unfinished norm."""
    if isinstance(delta, (ops.NormedDelta, ops.StreamUpdate)):
        return norm.forward(hidden, delta) if rows is None else norm.forward(hidden, delta, rows=rows)
    if isinstance(delta, ops.RowStats) and not getattr(norm, "reads_row_stats", False):
        delta = None                # the sum is in `hidden` already; a plain norm needs no more
    lazy = (isinstance(delta, ops.RowStats) and getattr(norm, "defers", False)
            and getattr(consumer, "takes_pending_norm", False))
    if lazy:
        return norm.forward(hidden, delta, rows=rows, lazy=True)
    return norm.forward(hidden, delta) if rows is None else norm.forward(hidden, delta, rows=rows)


def run_part(part, normed, hidden: torch.Tensor, *args):
    """A mixer's or feed-forward's contribution to the residual stream: a part that `adds_to_residual` is given
    the stream and may add to it itself (it then returns `ops.RowStats`); what any part returns is the pending
    delta of the next norm."""
    if getattr(part, "adds_to_residual", False):
        return part.forward(normed, *args, residual=hidden)
    return part.forward(normed, *args)


class PreNormResidualBlock:
    """h = h + mixer(norm(h)); h = h + feed_forward(norm(h)) — liteinfer/models/llama.py:174-192."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, parts: dict) -> None:
        self.mixer_norm = parts["mixer_norm"]
        self.mixer = parts["mixer"]
        self.feed_forward_norm = parts["feed_forward_norm"]
        self.feed_forward = parts["feed_forward"]

    def forward(self, hidden: torch.Tensor, delta: torch.Tensor | None, ctx: StepContext,
                cache: LayerCache) -> tuple[torch.Tensor, torch.Tensor]:
        normed = apply_norm(self.mixer_norm, hidden, delta, self.mixer)
        mixed = run_part(self.mixer, normed, hidden, ctx, cache)
        normed = apply_norm(self.feed_forward_norm, hidden, mixed, self.feed_forward)
        return hidden, run_part(self.feed_forward, normed, hidden, ctx)


class SandwichNormBlock:
    """h = h + post(mixer(pre(h))); h = h + post'(feed_forward(pre'(h))): every sublayer is normalised on its way
    in and on its way out.  The sublayer's normalised output travels as an `ops.NormedDelta`, so the norm that
    reads the stream next (of this block, the next block, the re-entry part or the model's final norm) does the
    outgoing norm, the sum and its own norm in one kernel."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm", "feed_forward_norm": "norm",
             "feed_forward": "feed_forward", "feed_forward_post_norm": "norm"}

    def __init__(self, parts: dict) -> None:
        self.mixer_norm, self.mixer, self.mixer_post_norm = parts["mixer_norm"], parts["mixer"], parts["mixer_post_norm"]
        self.feed_forward_norm = parts.get("feed_forward_norm")
        self.feed_forward = parts.get("feed_forward")
        self.feed_forward_post_norm = parts.get("feed_forward_post_norm")

    def forward(self, hidden: torch.Tensor, delta, ctx: StepContext, cache: LayerCache):
        normed = apply_norm(self.mixer_norm, hidden, delta)
        delta = self.mixer_post_norm.normed_delta(self.mixer.forward(normed, ctx, cache))
        if self.feed_forward is None:
            return hidden, delta
        normed = apply_norm(self.feed_forward_norm, hidden, delta)
        return hidden, self.feed_forward_post_norm.normed_delta(self.feed_forward.forward(normed, ctx))


class SandwichNormMixerBlock(SandwichNormBlock):
    """`SandwichNormBlock` of a layer that has no feed-forward."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm"}


class OutputNormBlock:
    """h = h + norm(mixer(h)); h = h + norm'(feed_forward(h)): the sublayers read the stream as it is, and only
    what they give back is normalised.  The normalised output travels as an `ops.NormedDelta`; whoever reads the
    stream next adds it: this block's `_read` (one kernel: the outgoing norm, the 32-bit sum, and the sum rounded
    to the engine's dtype for the sublayer's products) or the model's final norm."""

    roles = {"mixer": "mixer", "mixer_out_norm": "norm", "feed_forward": "feed_forward",
             "feed_forward_out_norm": "norm"}

    def __init__(self, parts: dict) -> None:
        self.mixer, self.mixer_out_norm = parts["mixer"], parts["mixer_out_norm"]
        self.feed_forward = parts.get("feed_forward")
        self.feed_forward_out_norm = parts.get("feed_forward_out_norm")
        self.dtype = self.mixer_out_norm.dtype

    def _read(self, hidden: torch.Tensor, delta) -> torch.Tensor:
        """Adds the pending delta into the stream and returns the stream in the engine's dtype."""
        narrow = hidden.dtype != self.dtype
        out = torch.empty(hidden.shape, dtype=self.dtype, device=hidden.device) if narrow else None
        if isinstance(delta, ops.NormedDelta):
            ops.layernorm_add(hidden, delta.value, delta.weight, delta.eps, centred=delta.centred, out=out)
            return out if narrow else hidden
        if isinstance(delta, torch.Tensor):
            ops.add_(hidden, delta)
        return ops.convert(hidden, out) if narrow else hidden

    def forward(self, hidden: torch.Tensor, delta, ctx: StepContext, cache: LayerCache):
        delta = self.mixer_out_norm.normed_delta(self.mixer.forward(self._read(hidden, delta), ctx, cache))
        if self.feed_forward is None:
            return hidden, delta
        return hidden, self.feed_forward_out_norm.normed_delta(self.feed_forward.forward(self._read(hidden, delta), ctx))


class OutputNormMixerBlock(OutputNormBlock):
    """`OutputNormBlock` of a layer that has no feed-forward."""

    roles = {"mixer": "mixer", "mixer_out_norm": "norm"}


class StreamMixedBlock:
    """A pre-norm block whose residual is one or several 32-bit streams (parts/connection.py): every sublayer
    reads the streams through its connection's coefficients, and its output, scaled per channel, rewrites all
    streams through the connection's small matrix:

        u = sum_s read[s] x_s;  y = sublayer(norm(u));  x_t <- sum_s mix[s, t] x_s + write[t] * gain * y

    The rewrite travels as an `ops.StreamUpdate`; the norm that reads the streams next (this block's second, the
    next block's first, the model's last) does it on its way, so the streams are read and written once per
    sublayer.  A layer may have no feed-forward."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_connection": "connection", "feed_forward_norm": "norm",
             "feed_forward": "feed_forward", "feed_forward_connection": "connection"}

    def __init__(self, parts: dict) -> None:
        self.mixer_norm, self.mixer, self.mixer_connection = parts["mixer_norm"], parts["mixer"], parts["mixer_connection"]
        self.feed_forward_norm = parts.get("feed_forward_norm")
        self.feed_forward = parts.get("feed_forward")
        self.feed_forward_connection = parts.get("feed_forward_connection")

    def forward(self, hidden: torch.Tensor, delta, ctx: StepContext, cache: LayerCache):
        normed = self.mixer_norm.forward(hidden, delta, read=self.mixer_connection.read)
        delta = self.mixer_connection.update(self.mixer.forward(normed, ctx, cache))
        if self.feed_forward is None:
            return hidden, delta
        normed = self.feed_forward_norm.forward(hidden, delta, read=self.feed_forward_connection.read)
        return hidden, self.feed_forward_connection.update(self.feed_forward.forward(normed, ctx))


class StreamMixedMixerBlock(StreamMixedBlock):
    """`StreamMixedBlock` of a layer that has no feed-forward."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_connection": "connection"}


register_block("prenorm_residual", PreNormResidualBlock)
register_block("stream_mixed", StreamMixedBlock)
register_block("stream_mixed_mixer_only", StreamMixedMixerBlock)
register_block("output_norm", OutputNormBlock)
register_block("output_norm_mixer_only", OutputNormMixerBlock)
register_block("sandwich_norm", SandwichNormBlock)
register_block("sandwich_norm_mixer_only", SandwichNormMixerBlock)
