"""Python faces of the CUDA kernels in `liteinfer_b200/csrc`.

Every function checks its tensors (device, dtype, contiguity, shapes), launches
on torch's current stream and raises when the launch is refused.  None of them
has a CPU or library path: a tensor that is not on a CUDA device raises
`KernelLibraryError`.  The parts of a model call these functions through the
module (`from liteinfer_b200 import ops` then `ops.rmsnorm(...)`), never by a
bound name, so tests can stand in for a single kernel.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_size_t, c_void_p

from dataclasses import dataclass

import torch

from liteinfer_b200.ops.library import KernelLibraryError, load

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
ACTIVATIONS = {"silu": 0, "gelu": 1, "gelu_pytorch_tanh": 2, "gelu_tanh": 2, "relu": 3}
# Activations of a feed-forward without a gate (`activation`): the above, and the square of relu.
UNARY_ACTIVATIONS = {**ACTIVATIONS, "relu_squared": 4}
# A weight-streaming product takes an activation of one argument as this base plus its code (csrc/gemm_skinny.cuh).
UNARY_ACT_BASE = 16

_ERRORS = {
    100001: "the kernel refuses these sizes (unsupported shape or option)",
    100002: "the kernel needs 16-byte aligned rows",
}

_functions: dict[str, ctypes._CFuncPtr] = {}

_SIGNATURES = {
    "li_embedding": ("elementwise", [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "li_scatter_tokens": ("elementwise", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "li_stage_batch": ("elementwise", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "li_rmsnorm": ("elementwise", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                                   c_int, c_void_p]),
    "li_add": ("elementwise", [c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
    "li_add_bias": ("elementwise", [c_int, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "li_act_mul": ("elementwise", [c_int, c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p]),
    "li_act_mul_interleaved": ("elementwise", [c_int, c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p]),
    "li_rope_kv_write": ("rope_cache", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                        c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                        c_void_p]),
    "li_head_norm_rope_kv_write": ("rope_cache", [c_int, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_int,
                                                  c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                  c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
                                                  c_size_t, c_void_p, c_int, c_float, c_void_p]),
    "li_sigmoid_gate": ("rope_cache", [c_int, c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p]),
    "li_softcap": ("elementwise", [c_int, c_void_p, c_size_t, c_float, c_void_p]),
    "li_moe_route": ("moe", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "li_moe_tile_rows": ("moe", [c_int, c_int, c_int]),
    "li_moe_sort": ("moe", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                            c_void_p]),
    "li_moe_router": ("moe", [c_int, c_void_p, c_size_t, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_void_p, c_void_p, c_void_p]),
    "li_moe_gather": ("moe", [c_int, c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]),
    "li_gemm_tcgen05_grouped": ("gemm_tcgen05", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                                 c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                 c_void_p, c_void_p]),
    "li_moe_grouped": ("moe", [c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_int,
                               c_int, c_int, c_void_p]),
    "li_moe_combine": ("moe", [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "li_sigmoid_gate_heads": ("rope_cache", [c_int, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_void_p]),
    "li_mlstm": ("mlstm", [c_int, c_void_p, c_size_t, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                           c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                           c_int, c_int, c_void_p]),
    "li_paged_attention_generic": ("attention_generic", [
        c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_float, c_void_p, c_void_p]),
    "li_convert": ("layernorm", [c_int, c_void_p, c_size_t, c_int, c_void_p, c_size_t, c_int, c_int, c_void_p]),
    "li_layernorm": ("layernorm", [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_int, c_int, c_float, c_float, c_int, c_int, c_void_p]),
    "li_projection_rmsnorm": ("layernorm", [c_int, c_void_p, c_size_t, c_int, c_int, c_void_p, c_int, c_void_p,
                                            c_float, c_void_p]),
    "li_gated_rmsnorm": ("layernorm", [c_int, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p, c_int, c_int, c_int,
                                       c_float, c_int, c_int, c_void_p, c_void_p]),
    "li_short_conv": ("delta_rule", [c_int, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "li_short_conv_update": ("delta_rule", [c_int, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                            c_int, c_void_p]),
    "li_gated_delta_rule": ("delta_rule", [c_int, c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                           c_void_p, c_void_p]),
    "li_paged_attention_mma": ("attention_mma", [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p]),
    "li_paged_attention_stream": ("attention_stream", [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "li_paged_attention_stream_supports": ("attention_stream", [c_int, c_int, c_int, c_int]),
    "li_paged_attention_stream_capacity": ("attention_stream", [c_int]),
    "li_paged_attention_stream_cluster_capacity": ("attention_stream", [c_int, c_int]),
    "li_paged_attention_mma_counters": ("attention_mma", [c_int, c_int, c_int, c_int]),
    "li_paged_attention_mma_decode_capacity": ("attention_mma", [c_int]),
    "li_paged_attention_tcgen05": ("attention_tcgen05", [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_float, c_void_p, c_void_p]),
    "li_paged_attention_tcgen05_supports": ("attention_tcgen05", [c_int, c_int, c_int, c_int]),
    "li_gemm_skinny": ("gemm_skinny", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                       c_void_p, c_size_t, c_void_p, c_int, c_void_p]),
    "li_gemm_skinny_fused": ("gemm_skinny", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                             c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                             c_float, c_void_p, c_void_p, c_int, c_void_p]),
    "li_gemm_skinny_plan": ("gemm_skinny", [c_int, c_int, c_void_p, c_void_p]),
    "li_gemm_stream": ("gemm_stream", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                       c_int, c_void_p, c_void_p]),
    "li_gemm_stream_supports": ("gemm_stream", [c_int, c_int, c_int]),
    "li_gemm_tcgen05": ("gemm_tcgen05", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                         c_void_p]),
    "li_gemm_simt": ("gemm_simt", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "li_gemm_simt_batched": ("gemm_simt", [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                           c_int, c_long, c_long, c_long, c_void_p]),
    "li_activation": ("elementwise", [c_int, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "li_embedding_streams": ("stream_mix", [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int,
                                            c_void_p, c_void_p]),
    "li_stream_rmsnorm": ("stream_mix", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p]),
    "li_latent_prep": ("attention_latent", [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                            c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                            c_int, c_int, c_void_p, c_int, c_float, c_void_p]),
    "li_latent_attention": ("attention_latent", [c_int, c_void_p, c_long, c_int, c_void_p, c_int, c_int, c_int,
                                                 c_void_p, c_long, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                 c_int, c_float, c_int, c_float, c_void_p]),
    "li_latent_attention_mma": ("attention_latent_mma", [
        c_void_p, c_long, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_long, c_int, c_void_p, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
        c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_float, c_void_p]),
    "li_latent_attention_mma_supports": ("attention_latent_mma", [c_int, c_int, c_int]),
    "li_gate_heads": ("attention_latent", [c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]),
    "li_argmax": ("sampling", [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                               c_void_p]),
    "li_sample": ("sampling", [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p]),
}


def _fn(name: str):
    fn = _functions.get(name)
    if fn is None:
        library, argtypes = _SIGNATURES[name]
        fn = getattr(load(library), name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _functions[name] = fn
    return fn


# Launches of this package's own kernels since import (library products are not counted).
launch_count = 0


def _check(code: int, name: str) -> None:
    global launch_count
    if code == 0:
        launch_count += 1
        return
    if code in _ERRORS:
        raise KernelLibraryError(f"{name}: {_ERRORS[code]}")
    raise KernelLibraryError(f"{name}: CUDA error {code} at launch")


_pinned_stream: int | None = None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream if _pinned_stream is None else _pinned_stream


class on_current_stream:
    """Within this context every kernel of this module goes to the stream that was current when it was entered,
    without asking for it again at every launch (a step of a model launches a few hundred kernels; the lookup
    was a noticeable part of a step's host time).  Contexts nest; leave the stream alone inside."""

    def __enter__(self):
        global _pinned_stream
        self.before = _pinned_stream
        _pinned_stream = torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else None
        return self

    def __exit__(self, *exc):
        global _pinned_stream
        _pinned_stream = self.before
        return False


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelLibraryError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _on_gpu(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelLibraryError(
                "liteinfer_b200 kernels run on a CUDA device only; there is no CPU path "
                f"(got a tensor on {t.device})")
        if not t.is_contiguous():
            raise KernelLibraryError("kernels take contiguous tensors")


class _Scratch:
    """Per-device scratch that split kernels leave partial results in, and their arrival counters.

    The counters are zero between launches (the kernels reset them); the buffers live as long as the
    process, so CUDA graphs may hold their addresses."""

    GEMM_FLOATS = 1 << 21
    GEMM_COUNTERS = 1 << 12
    ATTENTION_COUNTERS = 1 << 16
    ARGMAX_ROWS = 4096

    def __init__(self, device: torch.device) -> None:
        self.gemm = torch.empty(self.GEMM_FLOATS, dtype=torch.float32, device=device)
        self.gemm_counters = torch.zeros(self.GEMM_COUNTERS, dtype=torch.int32, device=device)
        self.attention_counters = torch.zeros(self.ATTENTION_COUNTERS, dtype=torch.int32, device=device)
        self.argmax_value = torch.empty(self.ARGMAX_ROWS * 32, dtype=torch.float32, device=device)
        self.argmax_index = torch.empty(self.ARGMAX_ROWS * 32, dtype=torch.int32, device=device)
        self.argmax_counters = torch.zeros(self.ARGMAX_ROWS, dtype=torch.int32, device=device)
        # Error flags that kernels raise and the engine reads where it synchronises anyway: [0] the number of a
        # bounded wait that gave up (tcgen05 and TMA kernels), [1] a token id outside the embedding table.
        self.errors = torch.zeros(2, dtype=torch.int32, device=device)
        self.gemm_error = self.errors[0:1]
        self.token_error = self.errors[1:2]


_scratch: dict[torch.device, _Scratch] = {}


def normalise_device(device: torch.device | str) -> torch.device:
    """`cuda` and `cuda:0` are one device (torch compares and hashes them apart): the index is filled in with the
    current device's."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device() if torch.cuda.is_available() else 0)
    return device


def scratch_for(device: torch.device | str) -> _Scratch:
    device = normalise_device(device)
    found = _scratch.get(device)
    if found is None:
        found = _scratch[device] = _Scratch(device)
    return found


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _int32(t: torch.Tensor | None, what: str) -> None:
    if t is not None and t.dtype != torch.int32:
        raise KernelLibraryError(f"{what} must be int32, got {t.dtype}")


# ------------------------------------------------------------------ row-wise
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
              error_flag: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[ids[t]].  An id outside the table sets `error_flag[0]` and gives a zero row."""
    _on_gpu(ids, table, out, error_flag)
    _int32(ids, "ids")
    _int32(error_flag, "error_flag")
    tokens, width = out.shape
    assert ids.numel() == tokens and table.shape[1] == width and table.dtype == out.dtype
    _check(_fn("li_embedding")(_code(out), ids.data_ptr(), table.data_ptr(), out.data_ptr(), tokens, width,
                               table.shape[0], _ptr(error_flag), _stream()), "embedding")
    return out


def scatter_tokens(tokens: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, source: torch.Tensor) -> torch.Tensor:
    """tokens[dst[i]] = source[src[i]] wherever dst[i] >= 0 (all int32): sampled token ids that never left the
    device take their places in the next step's batch."""
    _on_gpu(tokens, dst, src, source)
    for t, what in ((tokens, "tokens"), (dst, "dst"), (src, "src"), (source, "source")):
        _int32(t, what)
    assert dst.numel() == src.numel()
    _check(_fn("li_scatter_tokens")(tokens.data_ptr(), dst.data_ptr(), src.data_ptr(), source.data_ptr(), dst.numel(),
                                    _stream()), "scatter_tokens")
    return tokens


# Batches up to this many 32-bit words are brought to the device by a kernel that reads the pinned buffer in place
# (one block; a copy engine's latency is longer than that for a few kilobytes, shorter for many).
STAGE_KERNEL_MAX_WORDS = 16384


def stage_batch(device: torch.Tensor, host: torch.Tensor, tokens: torch.Tensor, dst: torch.Tensor, src: torch.Tensor,
                source: torch.Tensor | None) -> bool:
    """device[:] = host[:] (int32; `host` pinned), then tokens[dst[i]] = source[src[i]] wherever dst[i] >= 0, in one
    launch.  False (and nothing done) where the buffer is too large for that or the device cannot read `host` in
    place: the caller then copies and scatters."""
    _on_gpu(device, tokens, dst, src, source)
    for t, what in ((device, "device"), (host, "host"), (tokens, "tokens"), (dst, "dst"), (src, "src")):
        _int32(t, what)
    words = device.numel()
    if words > STAGE_KERNEL_MAX_WORDS or host.numel() != words or not host.is_pinned():
        return False
    code = _fn("li_stage_batch")(device.data_ptr(), host.data_ptr(), words, tokens.data_ptr(), dst.data_ptr(),
                                 src.data_ptr(), _ptr(source), dst.numel() if source is not None else 0, _stream())
    if code == 100001:        # LI_ERR_UNSUPPORTED: the device cannot read this host memory in place
        return False
    _check(code, "stage_batch")
    return True


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            delta: torch.Tensor | None = None, rows: torch.Tensor | None = None,
            write_residual: bool = False) -> torch.Tensor:
    """out[r] = weight * rmsnorm(x[row] (+ delta[row])), row = rows[r] if rows is given else r.

    With `write_residual` the sum x + delta is stored back into x (the residual
    stream moves on in place); statistics and the sum are 32-bit.
    """
    _on_gpu(x, weight, out, delta, rows)
    _int32(rows, "rows")
    width = x.shape[-1]
    out_rows = out.shape[0]
    assert weight.numel() == width and out.shape[-1] == width and x.dtype == out.dtype == weight.dtype
    assert delta is None or (delta.shape == x.shape and delta.dtype == x.dtype)
    assert rows is not None or out_rows == x.shape[0]
    assert rows is None or rows.numel() == out_rows
    assert not (write_residual and delta is None)
    _check(_fn("li_rmsnorm")(_code(x), x.data_ptr(), _ptr(delta), weight.data_ptr(), out.data_ptr(), _ptr(rows),
                             out_rows, width, float(eps), int(write_residual), _stream()), "rmsnorm")
    return out


def add_(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += delta, summed in 32-bit."""
    _on_gpu(x, delta)
    assert x.shape == delta.shape and x.dtype == delta.dtype
    _check(_fn("li_add")(_code(x), x.data_ptr(), delta.data_ptr(), x.numel(), _stream()), "add")
    return x


def add_bias_(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    _on_gpu(out, bias)
    assert out.shape[-1] == bias.numel() and out.dtype == bias.dtype
    _check(_fn("li_add_bias")(_code(out), out.data_ptr(), bias.data_ptr(), out.numel() // bias.numel(),
                              bias.numel(), _stream()), "add_bias")
    return out


def act_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str) -> torch.Tensor:
    """out = act(gate_up[:, :w]) * gate_up[:, w:], w = out.shape[1]."""
    _on_gpu(gate_up, out)
    rows, width = out.shape
    assert gate_up.shape == (rows, 2 * width) and gate_up.dtype == out.dtype
    if activation not in ACTIVATIONS:
        raise KernelLibraryError(f"activation {activation!r} has no kernel; known: {sorted(ACTIVATIONS)}")
    _check(_fn("li_act_mul")(_code(out), gate_up.data_ptr(), out.data_ptr(), rows, width, ACTIVATIONS[activation],
                             _stream()), "act_mul")
    return out


# ------------------------------------------------------------- matrix product
@dataclass
class RowStats:
    """What a product leaves behind when it has added its result into the residual stream itself: the sums of
    squares of the stream's new rows, in parts (one per 16 columns the product wrote), [parts, rows] float32.
    The norm that follows needs nothing else of the rows' statistics."""

    sumsq: torch.Tensor


@dataclass
class PendingNorm:
    """A root-mean-square norm that has not run yet: `x` (the residual stream, sums done), the norm's weight and
    eps, the rows' statistics, and optionally the rows that are wanted (int32 indices).  `linear` and
    `gated_linear` take one in place of x and fold the norm into the product where their kernel can; anything
    else calls `materialise()`."""

    x: torch.Tensor
    weight: torch.Tensor
    eps: float
    stats: RowStats
    rows: torch.Tensor | None = None

    @property
    def shape(self) -> tuple[int, int]:
        return ((self.x.shape[0] if self.rows is None else self.rows.numel()), self.x.shape[1])

    @property
    def dtype(self) -> torch.dtype:
        return self.x.dtype

    @property
    def device(self) -> torch.device:
        return self.x.device

    def materialise(self) -> torch.Tensor:
        from liteinfer_b200 import ops      # through the module, so that a stand-in kernel is found
        out = torch.empty(self.shape, dtype=self.x.dtype, device=self.x.device)
        return ops.rmsnorm(self.x, self.weight, self.eps, out, rows=self.rows)


# LITEINFER_FUSED_NORM=1: the weight-streaming products add into the residual stream themselves and fold the norm
# after it into the next product, which takes 32 launches out of a decode step of 16 layers.  Off by default: measured
# on B200 at the 1B shape, a norm launched early costs 1.3 us between two products (its launch hides behind the
# product's weights, which are asked for before the wait), while multiplying x by the norm's weight inside the
# product's loop costs more (gate_up at 8 rows 20.9 against 15.2 us, the head 130 against 91): 1.17 against 1.06 ms
# per decode step at batch 8.
FUSED_NORM = os.environ.get("LITEINFER_FUSED_NORM", "0") == "1"


# LITEINFER_GEMM_STREAM=0: products of at most 16 rows run on the kernel that loads its weights through registers
# (gemm_skinny) instead of the persistent kernel with per-warp TMA rings (gemm_stream).
GEMM_STREAM = os.environ.get("LITEINFER_GEMM_STREAM", "1") != "0"


def _streams(M: int, N: int, K: int) -> bool:
    """Whether the weight-streaming kernel runs a bfloat16 product of these sizes."""
    if K % 8 or K < 8 or M <= 0:
        return False
    return M <= SKINNY_MAX_ROWS or (M <= SKINNY_MAX_ROWS_SMALL and N <= SKINNY_SMALL_WEIGHT_ROWS)


def linear(x: "torch.Tensor | PendingNorm", weight: torch.Tensor, out: torch.Tensor | None,
           bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
           activation: str | None = None) -> "torch.Tensor | RowStats":
    """out[M, N] = x[M, K] @ weight[N, K]^T (+ bias).

    float32 runs the FFMA kernel (a true 32-bit product: tensor cores have no such
    mode).  bfloat16 hands the product to the library GEMM, as the reference's
    `nn.Linear` does (liteinfer/models/llama.py:108-110,137-140), with 32-bit
    accumulation, except for a handful of rows, which the weight-streaming kernel takes.

    `x` may be a `PendingNorm`: the weight-streaming kernel then normalises on its way in; any other path runs
    the norm first.  With `residual` [M, N] the weight-streaming kernel adds its result into it
    (residual = round(residual + round(product))) and returns the new rows' `RowStats`, `out` being unused; any
    other path returns the product in `out`, for the caller to add.

    `activation` (a name of `UNARY_ACTIVATIONS`; not with `residual`): out = act(product), the product rounded to
    the engine's dtype first; the weight-streaming kernel does it on its way out, any other path by the
    elementwise kernel.
    """
    if activation is not None:
        assert residual is None
        if activation not in UNARY_ACTIVATIONS:
            raise KernelLibraryError(f"activation {activation!r} has no kernel; known: {sorted(UNARY_ACTIVATIONS)}")
    pending = x if isinstance(x, PendingNorm) else None
    M, K = x.shape
    N = weight.shape[0]
    fused = x.dtype == torch.bfloat16 and _streams(M, N, K)
    if pending is not None and not fused:
        x, pending = pending.materialise(), None
    if residual is not None and not (fused and FUSED_NORM):
        residual = None
    if out is None and residual is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    _on_gpu(x if pending is None else pending.x, weight, out, bias, residual)
    assert weight.shape[1] == K and x.dtype == weight.dtype
    assert residual is None or (residual.shape == (M, N) and residual.dtype == x.dtype)
    assert out is None or (out.shape == (M, N) and out.dtype == x.dtype)
    if x.dtype == torch.float32:
        _check(_fn("li_gemm_simt")(0, x.data_ptr(), weight.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K,
                                   _stream()), "gemm_simt")
        return out if activation is None else _unary(out, out, activation)
    if fused:
        return _skinny(x, weight, out, bias, -1 if activation is None else UNARY_ACT_BASE + UNARY_ACTIVATIONS[activation],
                       residual)
    if M > 0:
        torch.mm(x, weight.t(), out=out)
        if bias is not None:
            add_bias_(out, bias)
        if activation is not None:
            _unary(out, out, activation)
    return out


# Rows of x up to which the weight-streaming kernel runs the bfloat16 product (measured on B200: beyond
# eight rows the library product streams the weights faster).
SKINNY_MAX_ROWS = 8
# ...except for weights of few rows (the projections around the attention, the down projection), where the kernel
# still wins at 9 to 16 rows of x: 5.4 against 5.8 us (3072 x 2048), 4.7 against 5.6 (2048 x 2048), 11.3 against
# 13.2 (2048 x 8192); inside a step of 12 sequences 1.219 against 1.245 ms, of 16 sequences 1.315 against 1.330.
SKINNY_MAX_ROWS_SMALL = 16
SKINNY_SMALL_WEIGHT_ROWS = 4096
NUM_SMS = 148


def _skinny(x, weight, out, bias, gated_act: int, residual: torch.Tensor | None = None, rings: bool = True):
    """A weight-streaming kernel, with what `x` (a tensor or a PendingNorm) and `residual` ask to be fused in:
    the persistent kernel with TMA rings where it takes the sizes (and `rings`), else the one that loads through
    registers."""
    M, K = x.shape
    N = weight.shape[0]
    pending = x if isinstance(x, PendingNorm) else None
    ws = scratch_for(weight.device)
    if pending is None and rings and GEMM_STREAM and M <= 16:
        # The persistent kernel that streams the weights through per-warp TMA rings.
        stats = None
        if residual is not None:
            stats = RowStats(torch.empty((-(-N // 16), M), dtype=torch.float32, device=weight.device))
        code = _fn("li_gemm_stream")(x.data_ptr(), weight.data_ptr(), _ptr(bias),
                                     (residual if residual is not None else out).data_ptr(), M, N, K, gated_act,
                                     _ptr(stats.sumsq if stats is not None else None), M if stats is not None else 0,
                                     ws.gemm_error.data_ptr(), _stream())
        if code != 100001:          # sizes it refuses go to the kernel below
            _check(code, "gemm_stream")
            return stats if stats is not None else out
    if pending is None and residual is None:
        _check(_fn("li_gemm_skinny")(x.data_ptr(), weight.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, gated_act,
                                     ws.gemm.data_ptr(), ws.gemm.numel(), ws.gemm_counters.data_ptr(),
                                     ws.gemm_counters.numel(), _stream()), "gemm_skinny")
        return out
    stats = None
    if residual is not None:
        stats = RowStats(torch.empty((-(-N // 16), M), dtype=torch.float32, device=weight.device))
    source = pending.x if pending is not None else x
    _int32(pending.rows if pending is not None else None, "rows")
    _check(_fn("li_gemm_skinny_fused")(
        source.data_ptr(), weight.data_ptr(), _ptr(bias), (residual if residual is not None else out).data_ptr(),
        M, N, K, gated_act, ws.gemm.data_ptr(), ws.gemm.numel(), ws.gemm_counters.data_ptr(),
        ws.gemm_counters.numel(),
        _ptr(pending.weight if pending is not None else None),
        _ptr(pending.stats.sumsq if pending is not None else None),
        pending.stats.sumsq.shape[0] if pending is not None else 0,
        pending.stats.sumsq.shape[1] if pending is not None else 0,
        float(pending.eps) if pending is not None else 0.0,
        _ptr(pending.rows if pending is not None else None),
        _ptr(stats.sumsq if stats is not None else None), M if stats is not None else 0, _stream()), "gemm_skinny_fused")
    return stats if stats is not None else out


def gemm_skinny(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """The weight-streaming bfloat16 product for at most 64 rows of x."""
    _on_gpu(x, weight, out, bias)
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and out.shape == (M, N) and x.dtype == weight.dtype == out.dtype == torch.bfloat16
    return _skinny(x, weight, out, bias, -1, rings=False)


def gemm_stream(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
                gated_activation: str | None = None, residual: torch.Tensor | None = None):
    """The persistent weight-streaming product (per-warp TMA rings) for at most 16 rows of x: out = x @ weight^T
    (+ bias); with `gated_activation`, act(gate) * up on a weight interleaved in eights (out is [M, N/2]); with
    `residual` [M, N] the result is added into it and the new rows' `RowStats` are returned (`out` unused)."""
    _on_gpu(x, weight, out, bias, residual)
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and x.dtype == weight.dtype == torch.bfloat16
    act = -1 if gated_activation is None else ACTIVATIONS[gated_activation]
    stats = None
    if residual is not None:
        stats = RowStats(torch.empty((-(-N // 16), M), dtype=torch.float32, device=weight.device))
    _check(_fn("li_gemm_stream")(x.data_ptr(), weight.data_ptr(), _ptr(bias),
                                 (residual if residual is not None else out).data_ptr(), M, N, K, act,
                                 _ptr(stats.sumsq if stats is not None else None), M if stats is not None else 0,
                                 scratch_for(x.device).gemm_error.data_ptr(), _stream()), "gemm_stream")
    return stats if stats is not None else out


def gemm_tcgen05(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
                 gated_activation: str | None = None) -> torch.Tensor:
    """The tcgen05 / TMA / tensor-memory product for bfloat16: out = x @ weight^T (+ bias), or with
    `gated_activation` act(gate) * up on a weight whose rows are interleaved in eights (out is [M, N/2]).

    `gemm_error_flag(device)` tells afterwards whether a wait inside the kernel ever gave up."""
    _on_gpu(x, weight, out, bias)
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and x.dtype == weight.dtype == out.dtype == torch.bfloat16
    assert out.shape == ((M, N) if gated_activation is None else (M, N // 2))
    act = -1 if gated_activation is None else ACTIVATIONS[gated_activation]
    _check(_fn("li_gemm_tcgen05")(x.data_ptr(), weight.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, act,
                                  scratch_for(x.device).gemm_error.data_ptr(), _stream()), "gemm_tcgen05")
    return out


def gemm_error_flag(device: torch.device | str) -> int:
    """0, or the number of the wait that gave up in a tcgen05 or TMA kernel since the flag was last cleared
    (synchronises the device)."""
    return error_flags(device)[0]


def token_error_flag(device: torch.device | str) -> torch.Tensor:
    """The device's flag that the embedding kernel raises for a token id outside its table."""
    return scratch_for(device).token_error


def error_flags(device: torch.device | str) -> tuple[int, int]:
    """(the number of a bounded wait that gave up, whether a token id lay outside an embedding table) since the
    flags were last read; reading clears them (one small copy that synchronises the device)."""
    flags = scratch_for(device).errors
    wait, token = flags.tolist()
    if wait or token:
        flags.zero_()
    return int(wait), int(token)


def gemm_simt(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """The FFMA product for either dtype (32-bit accumulation, fixed summation order)."""
    _on_gpu(x, weight, out, bias)
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and out.shape == (M, N) and x.dtype == weight.dtype == out.dtype
    _check(_fn("li_gemm_simt")(_code(x), x.data_ptr(), weight.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K,
                               _stream()), "gemm_simt")
    return out


def gemm_skinny_plan(N: int, K: int) -> tuple[int, int]:
    """(warps per block, slices of k) with which the weight-streaming kernel runs a weight [N, K]."""
    warps = ctypes.c_int(0)
    slices = int(_fn("li_gemm_skinny_plan")(N, K, ctypes.byref(warps), None))
    return warps.value, slices


def gemm_skinny_slices(N: int, K: int) -> int:
    """Into how many slices the weight-streaming kernel cuts k for a weight of [N, K]."""
    return gemm_skinny_plan(N, K)[1]


# Rows of x from which the gated product runs on the tcgen05 kernel (pairs of CTAs on 256 x 256 tiles) with the
# activation in its epilogue.  Measured on B200 at 2,048 rows x 16,384 x 2,048: 100 us, against 95 us for the
# library product plus 25 us for the activation kernel inside a step.  LITEINFER_TCGEN05_GATED=0 turns it off.
TCGEN05_MIN_ROWS = 256 if os.environ.get("LITEINFER_TCGEN05_GATED", "1") != "0" else 1 << 30


def gated_linear_supported(x: "torch.Tensor | PendingNorm", weight: torch.Tensor) -> bool:
    """Whether product, activation and multiply can be one kernel for this x: at most 8 rows (the
    weight-streaming kernel) or at least `TCGEN05_MIN_ROWS` (the tcgen05 kernel)."""
    M, K = x.shape
    return (x.dtype == torch.bfloat16 and K % 8 == 0 and K >= 8 and weight.shape[0] % 16 == 0
            and (0 < M <= SKINNY_MAX_ROWS or M >= TCGEN05_MIN_ROWS))


def gated_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, activation: str,
                 bias: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N/2] = act(gate) * up, where `weight` [N, K] holds gate and up rows interleaved in eights
    (rows 16b..16b+7 are gate rows 8b..8b+7, rows 16b+8..16b+15 their up rows): product, activation and
    multiply in one kernel (bfloat16)."""
    M, K = x.shape
    N = weight.shape[0]
    if isinstance(x, PendingNorm) and M > SKINNY_MAX_ROWS:
        x = x.materialise()
    _on_gpu(x.x if isinstance(x, PendingNorm) else x, weight, out, bias)
    assert weight.shape[1] == K and out.shape == (M, N // 2) and gated_linear_supported(x, weight)
    if M <= SKINNY_MAX_ROWS:
        return _skinny(x, weight, out, bias, ACTIVATIONS[activation])
    return gemm_tcgen05(x, weight, out, bias, activation)


def act_mul_interleaved(gate_up: torch.Tensor, out: torch.Tensor, activation: str) -> torch.Tensor:
    """`act_mul` for a gate_up whose columns are interleaved in eights like `gated_linear`'s weight rows."""
    _on_gpu(gate_up, out)
    rows, width = out.shape
    assert gate_up.shape == (rows, 2 * width) and gate_up.dtype == out.dtype and width % 8 == 0
    _check(_fn("li_act_mul_interleaved")(_code(out), gate_up.data_ptr(), out.data_ptr(), rows, width,
                                         ACTIVATIONS[activation], _stream()), "act_mul_interleaved")
    return out


# ------------------------------------------------------------ cache and mixer
def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                  block_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                  inv_freq: torch.Tensor | None, heads: int, kv_heads: int, head_dim: int,
                  rotary_dim: int, store: bool = True, v_head_dim: int | None = None,
                  cos_sin_scale: float = 1.0) -> None:
    """Rotates q (in place) and k, and stores k and v of every token into its page
    (with `store` False only q is rotated; the pages are left alone).

    qkv: [tokens, (heads + kv_heads) * head_dim + kv_heads * v_head_dim].  k_pool:
    [pages, kv_heads, page_size, head_dim], v_pool likewise with `v_head_dim` (None: head_dim).
    block_table: [seqs, max_pages] int32.  `cos_sin_scale` multiplies every cosine and sine.
    """
    _on_gpu(qkv, positions, seq_of_token, block_table, k_pool, v_pool, inv_freq)
    _int32(positions, "positions"); _int32(seq_of_token, "seq_of_token"); _int32(block_table, "block_table")
    tokens = qkv.shape[0]
    pages, kvh, page_size, hd = k_pool.shape
    vd = head_dim if v_head_dim is None else v_head_dim
    assert (kvh, hd) == (kv_heads, head_dim) and v_pool.shape == (pages, kv_heads, page_size, vd)
    assert qkv.shape[1] == (heads + kv_heads) * head_dim + kv_heads * vd
    assert k_pool.dtype == qkv.dtype == v_pool.dtype
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rotary_dim)
    _check(_fn("li_rope_kv_write")(_code(qkv), qkv.data_ptr(), positions.data_ptr(), seq_of_token.data_ptr(),
                                   block_table.data_ptr(), block_table.stride(0), k_pool.data_ptr(),
                                   v_pool.data_ptr(), _ptr(inv_freq), tokens, heads, kv_heads, head_dim,
                                   rotary_dim if inv_freq is not None else 0, page_size, pages if store else 0,
                                   vd, float(cos_sin_scale), _stream()),
           "rope_kv_write")


def head_norm_rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                            block_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                            inv_freq: torch.Tensor | None, heads: int, kv_heads: int, head_dim: int, rotary_dim: int,
                            q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, norm_eps: float,
                            store: bool = True, v_other: torch.Tensor | None = None,
                            blend: torch.Tensor | None = None, unit_norm: bool = False,
                            norm_after_rotation: bool = False, cos_sin_scale: float = 1.0) -> None:
    """`rope_kv_write` for an attention whose q and k pass a root-mean-square norm per head first: every q head
    becomes rot(q_norm * q / sqrt(mean(q^2) + eps)) in place, every k head likewise (with k_norm) on its way into
    its page; None leaves that projection unnormalised.  q_norm and k_norm: [head_dim], the dtype of qkv.

    qkv [tokens, >= (heads + kv_heads) * head_dim + kv_heads * v_dim]: q, k, v side by side at the start of each
    row (further columns may follow; v_dim is the value pool's last axis).  `v_other` [tokens, kv_heads * v_dim]
    (a column slice is fine) with `blend` (one float32 on the device): what is stored is
    (1 - blend) * v + blend * v_other, computed in 32-bit and rounded once.  `unit_norm`: q and k are divided by
    their root mean square per head also where no weight is given.  `norm_after_rotation`: the norm (of the rotated
    head, with its weight if any) comes behind the rotation instead of in front of it.  `cos_sin_scale` multiplies
    every cosine and sine."""
    _rows2d(qkv, "qkv")
    _on_gpu(positions, seq_of_token, block_table, k_pool, v_pool, inv_freq, q_norm, k_norm, blend)
    _int32(positions, "positions"); _int32(seq_of_token, "seq_of_token"); _int32(block_table, "block_table")
    tokens = qkv.shape[0]
    pages, kvh, page_size, hd = k_pool.shape
    vd = v_pool.shape[-1]
    assert (kvh, hd) == (kv_heads, head_dim) and v_pool.shape == (pages, kv_heads, page_size, vd)
    assert qkv.shape[1] >= (heads + kv_heads) * head_dim + kv_heads * vd
    assert k_pool.dtype == qkv.dtype == v_pool.dtype
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rotary_dim)
    for w in (q_norm, k_norm):
        assert w is None or (w.numel() == head_dim and w.dtype == qkv.dtype)
    assert (v_other is None) == (blend is None)
    if v_other is not None:
        _rows2d(v_other, "v_other")
        assert v_other.shape == (tokens, kv_heads * vd) and v_other.dtype == qkv.dtype
        assert blend.dtype == torch.float32 and blend.numel() == 1
    _check(_fn("li_head_norm_rope_kv_write")(
        _code(qkv), qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), seq_of_token.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), k_pool.data_ptr(), v_pool.data_ptr(), _ptr(inv_freq), tokens,
        heads, kv_heads, head_dim, rotary_dim if inv_freq is not None else 0, page_size, pages if store else 0, vd,
        _ptr(q_norm), _ptr(k_norm), float(norm_eps), _ptr(v_other), v_other.stride(0) if v_other is not None else 0,
        _ptr(blend), int(unit_norm) | (2 if norm_after_rotation else 0), float(cos_sin_scale), _stream()),
        "head_norm_rope_kv_write")


def sigmoid_gate_(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """x[t, j] *= sigmoid(gate[t, j]) in place, element by element: x [tokens, width] contiguous, gate [tokens,
    width] (a column slice is fine), both in the engine's dtype; the sigmoid and the product are 32-bit."""
    _on_gpu(x)
    _rows2d(gate, "gate")
    assert gate.shape == x.shape and gate.dtype == x.dtype and x.is_contiguous()
    _check(_fn("li_sigmoid_gate")(_code(x), x.data_ptr(), gate.data_ptr(), gate.stride(0), x.shape[0], x.shape[1],
                                  _stream()), "sigmoid_gate")
    return x


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) in place (32-bit inside)."""
    _on_gpu(x)
    assert x.is_contiguous() and cap > 0
    _check(_fn("li_softcap")(_code(x), x.data_ptr(), x.numel(), float(cap), _stream()), "softcap")
    return x


def sigmoid_gate_heads_(x: torch.Tensor, gate: torch.Tensor, heads: int) -> torch.Tensor:
    """x[t, h, :] *= sigmoid(gate[t, h]) in place: x [tokens, heads * size], gate [tokens, heads] (a column
    slice is fine), both in the engine's dtype; the sigmoid and the product are 32-bit."""
    _on_gpu(x)
    _rows2d(gate, "gate")
    tokens, width = x.shape
    assert width % heads == 0 and gate.shape == (tokens, heads) and gate.dtype == x.dtype
    _check(_fn("li_sigmoid_gate_heads")(_code(x), x.data_ptr(), gate.data_ptr(), gate.stride(0), tokens, heads,
                                        width // heads, _stream()), "sigmoid_gate_heads")
    return x


_decode_capacity: dict[tuple[int, bool], int] = {}


def decode_capacity(head_dim: int, streaming: bool = False) -> int:
    """Blocks of the decode attention launch that the device holds at once (asked of the occupancy calculator
    once per head size and kernel); without a device, what a B200 holds."""
    key = (head_dim, streaming)
    if key not in _decode_capacity:
        blocks = 0
        if torch.cuda.is_available():
            name = "li_paged_attention_stream_capacity" if streaming else "li_paged_attention_mma_decode_capacity"
            blocks = int(_fn(name)(head_dim))
        _decode_capacity[key] = blocks or ((3 if streaming else 5) if head_dim <= 64 else 2) * NUM_SMS
    return _decode_capacity[key]


def decode_splits_for(num_decode: int, kv_heads: int, max_context_len: int, head_dim: int = 64,
                      streaming: bool = False) -> int:
    """Blocks that share one sequence's keys in a decode launch: as many as still run as one wave when the
    batch is narrow (a launch a little over one wave takes as long as two), never fewer than two key tiles
    each, at most 32 (liteinfer/engine/model_runner.py:250-272 and paged_kernels.py:645-693 choose likewise)."""
    tiles = -(-max_context_len // 64)
    if tiles < 4:
        return 1
    pairs = max(1, num_decode * kv_heads)
    splits = max(1, min(decode_capacity(head_dim, streaming) // pairs, tiles // 2, 32))
    if streaming and cluster_merge_wanted() and splits > 1:
        # The streaming kernel can merge the splits of a sequence through distributed shared memory when they are
        # one thread-block cluster (16 blocks at most) and every cluster of the launch is resident at once: then a
        # count that allows it is worth more than the last few splits (see attention_stream.cu for the figures).
        for fewer in range(min(splits, 16), max(1, splits // 2) - 1, -1):
            if fewer > 1 and cluster_capacity(head_dim, fewer) >= pairs:
                return fewer
    return splits


def cluster_merge_wanted() -> bool:
    """The switch LITEINFER_ATTN_CLUSTER_MERGE=1 (off by default; the kernel's entry point reads the same variable)."""
    return os.environ.get("LITEINFER_ATTN_CLUSTER_MERGE", "0") == "1"


_cluster_capacity: dict[tuple[int, int], int] = {}


def cluster_capacity(head_dim: int, splits: int) -> int:
    """Clusters of `splits` blocks of the streaming decode kernel that the device holds at once (0: none)."""
    key = (head_dim, splits)
    if key not in _cluster_capacity:
        clusters = 0
        if torch.cuda.is_available():
            clusters = int(_fn("li_paged_attention_stream_cluster_capacity")(head_dim, splits))
        _cluster_capacity[key] = clusters
    return _cluster_capacity[key]


def paged_attention_generic(q, q_row_stride, out, k_pool, v_pool, block_table, query_start_loc, context_lens,
                            num_seqs, max_q_len, heads, kv_heads, head_dim, scale, window=0, keep_first=0,
                            softcap=0.0, sink=None) -> torch.Tensor:
    """The plain SIMT kernel: any dtype, key and value sizes up to 256 (they may differ), any grouping, a window
    that may keep the first `keep_first` keys visible, scores capped by softcap * tanh(score / softcap), a sink."""
    _on_gpu(q, out, k_pool, v_pool, block_table, query_start_loc, context_lens, sink)
    pages, kvh, page_size, hd = k_pool.shape
    _check(_fn("li_paged_attention_generic")(
        _code(q), q.data_ptr(), q_row_stride, out.data_ptr(), out.stride(0), k_pool.data_ptr(), v_pool.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), query_start_loc.data_ptr(), context_lens.data_ptr(),
        num_seqs, max_q_len, heads, kv_heads, head_dim, v_pool.shape[3], page_size, pages, float(scale), int(window),
        int(keep_first), float(softcap), _ptr(sink), _stream()),
        "paged_attention_generic")
    return out


def paged_attention_mma(q, q_row_stride, out, k_pool, v_pool, block_table, query_start_loc, context_lens,
                        seq_index, num_seqs, max_q_len, heads, kv_heads, head_dim, scale, window=0,
                        num_splits=1, newest=None, streaming=False, keep_first=0, softcap=0.0,
                        sink=None) -> torch.Tensor:
    """The tensor-core kernel (bfloat16, head size 64 or 128); `num_splits` > 1 splits every sequence's keys
    over that many blocks, the last of which merges the partial results.  `newest` (NewestToken, single-token
    sequences only): q is unrotated and the newest key and value are not in their pages yet; the kernel
    rotates q and the key and stores key and value itself.  `streaming` (single-token sequences, sizes that
    `stream_attention_supports` allows): the kernel that passes K and V through registers only.  `keep_first`
    (with a window) and `softcap`: as in `paged_attention`; not with `newest` or `streaming`.  `sink`: as in
    `paged_attention`; every form takes it."""
    _on_gpu(q, out, k_pool, v_pool, block_table, query_start_loc, context_lens, seq_index, sink)
    pages, kvh, page_size, hd = k_pool.shape
    partial_out = partial_lse = counters = None
    if num_splits > 1:
        total = q.shape[0] * heads * num_splits
        partial_out = torch.empty((total, head_dim), dtype=torch.float32, device=q.device)
        partial_lse = torch.empty((total,), dtype=torch.float32, device=q.device)
        need = int(_fn("li_paged_attention_mma_counters")(num_seqs, max_q_len, heads, kv_heads))
        counters = scratch_for(q.device).attention_counters
        if need > counters.numel():
            counters = torch.zeros(need, dtype=torch.int32, device=q.device)
    tail = (_ptr(newest.inv_freq if newest else None), _ptr(newest.k if newest else None),
            _ptr(newest.v if newest else None), int(newest.store) if newest else 0)
    if streaming:
        assert max_q_len == 1 and keep_first <= 0 and softcap <= 0
        _check(_fn("li_paged_attention_stream")(
            q.data_ptr(), q_row_stride, out.data_ptr(), out.stride(0), k_pool.data_ptr(), v_pool.data_ptr(),
            block_table.data_ptr(), block_table.stride(0), query_start_loc.data_ptr(), context_lens.data_ptr(),
            _ptr(seq_index), num_seqs, heads, kv_heads, head_dim, page_size, pages, float(scale), int(window),
            int(num_splits), _ptr(partial_out), _ptr(partial_lse), _ptr(counters), *tail,
            scratch_for(q.device).gemm_error.data_ptr(), _ptr(sink), _stream()), "paged_attention_stream")
        return out
    _check(_fn("li_paged_attention_mma")(
        q.data_ptr(), q_row_stride, out.data_ptr(), out.stride(0), k_pool.data_ptr(), v_pool.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), query_start_loc.data_ptr(), context_lens.data_ptr(),
        _ptr(seq_index), num_seqs, max_q_len, heads, kv_heads, head_dim, page_size, pages, float(scale),
        int(window), int(num_splits), _ptr(partial_out), _ptr(partial_lse), _ptr(counters), *tail, int(keep_first),
        float(softcap), _ptr(sink), _stream()),
        "paged_attention_mma")
    return out


@dataclass
class NewestToken:
    """The unrotated key and value projections of each sequence's newest token (views with the row stride of
    q) and the rotary frequencies, for the decode kernel that rotates and stores them itself."""
    inv_freq: torch.Tensor     # [head_dim / 2] float32
    k: torch.Tensor
    v: torch.Tensor
    store: bool = True         # False: the pages are another layer's and already hold the token


def fused_decode_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, rotary_dim: int, plan) -> bool:
    """Whether a step's attention can run as one launch that also rotates q and k and writes the cache: every
    sequence brings one token, all of the head is rotated, and the tensor-core decode kernel takes the sizes."""
    return (plan is not None and plan.num_prefill == 0 and plan.num_decode > 0 and rotary_dim == head_dim
            and mma_attention_supports(dtype, heads, kv_heads, head_dim) and heads // kv_heads <= 16)


def paged_attention_tcgen05(q, q_row_stride, out, k_pool, v_pool, block_table, query_start_loc, context_lens,
                            seq_index, num_seqs, max_q_len, heads, kv_heads, head_dim, scale, window=0, keep_first=0,
                            softcap=0.0, sink=None) -> torch.Tensor:
    """The tcgen05 / TMA / tensor-memory attention kernel for prompts and portions (bfloat16, head size 64 or 128,
    pages of 16, 32 or 64 tokens, groups of at most 128 heads; `keep_first` and `softcap` as in `paged_attention`).
    `gemm_error_flag(device)` tells afterwards whether a wait inside the kernel ever gave up."""
    _on_gpu(q, out, k_pool, v_pool, block_table, query_start_loc, context_lens, seq_index, sink)
    pages, kvh, page_size, hd = k_pool.shape
    _check(_fn("li_paged_attention_tcgen05")(
        q.data_ptr(), q_row_stride, out.data_ptr(), out.stride(0), k_pool.data_ptr(), v_pool.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), query_start_loc.data_ptr(), context_lens.data_ptr(),
        _ptr(seq_index), num_seqs, max_q_len, heads, kv_heads, head_dim, page_size, pages, float(scale),
        int(window), scratch_for(q.device).gemm_error.data_ptr(), int(keep_first), float(softcap), _ptr(sink),
        _stream()),
        "paged_attention_tcgen05")
    return out


def tcgen05_attention_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(
        _fn("li_paged_attention_tcgen05_supports")(heads, kv_heads, head_dim, page_size))


def stream_attention_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether single-token sequences can go through the kernel that streams K and V through registers.
    LITEINFER_DECODE_STREAM=0 keeps them on the shared-memory kernel."""
    return (dtype == torch.bfloat16 and os.environ.get("LITEINFER_DECODE_STREAM", "1") != "0"
            and bool(_fn("li_paged_attention_stream_supports")(heads, kv_heads, head_dim, page_size)))


def mma_attention_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and heads // kv_heads <= 64


# LITEINFER_TCGEN05_ATTN=0: prompts and portions run on the mma.sync kernel (a switch for measurements).
MASKED_ON_MMA = os.environ.get("LITEINFER_TCGEN05_ATTN", "1") == "0"


def paged_attention(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_pool: torch.Tensor,
                    v_pool: torch.Tensor, block_table: torch.Tensor, query_start_loc: torch.Tensor,
                    context_lens: torch.Tensor, num_seqs: int, max_q_len: int, heads: int, kv_heads: int,
                    head_dim: int, scale: float, window: int = 0, plan=None,
                    decode_splits: int | None = None, newest: "NewestToken | None" = None, keep_first: int = 0,
                    softcap: float = 0.0, sink: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of each sequence's newest queries over its pages (any mix of portions and single tokens).

    q: the tensor holding the queries, head h of token t at q[t, h*head_dim:...]
    with `q_row_stride` elements between tokens (the fused qkv buffer is passed as
    it is).  out: [tokens, heads*head_dim].  bfloat16 with head size 64 or 128 runs
    on tensor cores; with a `plan` (AttentionPlan) the sequences that bring one
    token go through a launch that splits their keys over several blocks, the
    others through an unsplit one.  Everything else runs the plain SIMT kernel.
    `newest`: only where `fused_decode_supports` said yes; see `paged_attention_mma`.
    `keep_first` (with a window): the first keys of a sequence stay visible behind the window.  `softcap` > 0:
    a scaled score s becomes softcap * tanh(s / softcap).  Values may have another size than keys
    (`v_pool.shape[3]`); out is then [tokens, heads * value size].  `sink` [heads] float32: exp(sink[h]) is one
    more term of the denominator of head h's softmax; it has no key and no value and is not scaled.
    """
    _on_gpu(q, out, k_pool, v_pool, block_table, query_start_loc, context_lens)
    _int32(block_table, "block_table"); _int32(query_start_loc, "query_start_loc"); _int32(context_lens, "context_lens")
    pages, kvh, page_size, hd = k_pool.shape
    assert (kvh, hd) == (kv_heads, head_dim) and q.dtype == out.dtype == k_pool.dtype == v_pool.dtype
    if newest is not None and not fused_decode_supports(q.dtype, heads, kv_heads, head_dim, head_dim, plan):
        raise ValueError("the decode kernel with the rotary encoding fused in does not take this step")
    masked = softcap > 0 or (keep_first > 0 and window > 0)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == heads)
    if v_pool.shape[3] != head_dim or not mma_attention_supports(q.dtype, heads, kv_heads, head_dim):
        assert newest is None
        return paged_attention_generic(q, q_row_stride, out, k_pool, v_pool, block_table, query_start_loc,
                                       context_lens, num_seqs, max_q_len, heads, kv_heads, head_dim, scale, window,
                                       keep_first, softcap, sink)
    common = (q, q_row_stride, out, k_pool, v_pool, block_table, query_start_loc, context_lens)
    # Kept first keys and capped scores are options of the tcgen05 kernel (prompts) and of the mma.sync kernel
    # (prompts it takes instead, and single tokens); the streaming decode kernel knows neither.
    options = dict(keep_first=keep_first, softcap=softcap) if masked else {}
    if sink is not None:
        options["sink"] = sink
    if plan is None:
        return paged_attention_mma(*common, None, num_seqs, max_q_len, heads, kv_heads, head_dim, scale, window,
                                   **options)
    if plan.num_prefill:
        if tcgen05_attention_supports(q.dtype, heads, kv_heads, head_dim, page_size) and not MASKED_ON_MMA:
            paged_attention_tcgen05(*common, plan.prefill_seqs, plan.num_prefill, plan.max_prefill_query_len, heads,
                                    kv_heads, head_dim, scale, window, **options)
        else:
            paged_attention_mma(*common, plan.prefill_seqs, plan.num_prefill, plan.max_prefill_query_len, heads,
                                kv_heads, head_dim, scale, window, **options)
    if plan.num_decode:
        bound = plan.max_decode_context_len if window <= 0 else min(plan.max_decode_context_len, window + keep_first)
        streaming = not masked and stream_attention_supports(q.dtype, heads, kv_heads, head_dim, page_size)
        splits = decode_splits or decode_splits_for(plan.num_decode, kv_heads, bound, head_dim, streaming)
        paged_attention_mma(*common, plan.decode_seqs, plan.num_decode, 1, heads, kv_heads, head_dim, scale,
                            window, splits, newest, streaming, **options)
    return out


# ------------------------------------------------- 32-bit stream, layer norm, recurrences
@dataclass
class NormedDelta:
    """A delta of the residual stream that has not been computed yet: weight * norm(value), the output of a
    sublayer that is normalised before it is added.  The norm that reads the stream next adds it on its way.
    `centred`: a layer norm (the mean is taken off); otherwise a root-mean-square norm.  The weight has the
    dtype of the value, or float32."""

    value: torch.Tensor
    weight: torch.Tensor
    eps: float
    centred: bool = True


def _rows2d(t: torch.Tensor, what: str) -> None:
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelLibraryError(f"{what} must be two-dimensional with contiguous rows (a column slice is fine)")
    if not t.is_cuda:
        raise KernelLibraryError(f"liteinfer_b200 kernels run on a CUDA device only; there is no CPU path (got {t.device})")


def convert(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """dst[r, c] = src[r, c], between float32 and bfloat16 in either direction (or a copy); both may be column
    slices of wider tensors."""
    _rows2d(src, "src"); _rows2d(dst, "dst")
    assert src.shape == dst.shape
    rows, width = src.shape
    _check(_fn("li_convert")(_code(src), src.data_ptr(), src.stride(0), _code(dst), dst.data_ptr(), dst.stride(0),
                             rows, width, _stream()), "convert")
    return dst


def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
              delta: "NormedDelta | None" = None, rows: torch.Tensor | None = None,
              write_stream: bool = False, centre: bool = True) -> torch.Tensor:
    """out[r] = weight * norm(v), v = x[row] (+ delta.weight * norm(delta.value[row])), row = rows[r] if given else r;
    norm(v) = (v - mean) / sqrt(var + eps) (with `centre` False: v / sqrt(mean(v^2) + eps); the delta's own norm
    likewise by `delta.centred`).  With `write_stream` v is stored back into x.  x may be float32 whatever the
    dtype of out (a 32-bit residual stream), and so may the weights; every statistic and the sum are 32-bit."""
    _on_gpu(x, weight, out, rows, delta.value if delta else None, delta.weight if delta else None)
    _int32(rows, "rows")
    width = x.shape[-1]
    n = out.shape[0]
    assert weight.numel() == width and out.shape[-1] == width and weight.dtype in (out.dtype, torch.float32)
    assert x.dtype in (torch.float32, out.dtype)
    assert rows is None or rows.numel() == n
    assert rows is not None or n == x.shape[0]
    assert delta is None or (delta.value.shape == x.shape and delta.value.dtype == out.dtype
                             and delta.weight.dtype == weight.dtype)
    assert not (write_stream and (delta is None or rows is not None))
    flags = int(write_stream) | (0 if centre else 2) | (0 if delta is None or delta.centred else 4)
    _check(_fn("li_layernorm")(_code(out), x.data_ptr(), _code(x), _ptr(delta.value if delta else None),
                               _ptr(delta.weight if delta else None), weight.data_ptr(), out.data_ptr(), _ptr(rows),
                               n, width, float(eps), float(delta.eps if delta else 0.0), flags, _code(weight),
                               _stream()), "layernorm")
    return out


def layernorm_add(stream: torch.Tensor, value: torch.Tensor, weight: torch.Tensor, eps: float,
                  centred: bool = True, out: torch.Tensor | None = None) -> torch.Tensor:
    """stream += weight * norm(value) (a layer norm, or with `centred` False a root-mean-square norm): `stream`
    float32 or the dtype of value; summed in 32-bit.  `out` (dtype of value) receives the new stream, rounded:
    what a part that reads the stream as it is multiplies with."""
    _on_gpu(stream, value, weight, out)
    assert stream.shape == value.shape and weight.dtype in (value.dtype, torch.float32)
    assert stream.dtype in (torch.float32, value.dtype)
    assert out is None or (out.shape == stream.shape and out.dtype == value.dtype)
    flags = 1 | (0 if centred else 4) | (8 if out is not None else 0)
    _check(_fn("li_layernorm")(_code(value), stream.data_ptr(), _code(stream), value.data_ptr(), weight.data_ptr(),
                               None, _ptr(out), None, stream.shape[0], stream.shape[1], 0.0, float(eps), flags,
                               _code(weight), _stream()), "layernorm_add")
    return stream


def projection_rmsnorm_(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x[r] = weight * x[r] / sqrt(mean(x[r]^2) + eps) in place over whole rows of `x`, which may be a column
    slice of a wider tensor (the q or k part of a fused projection, normalised across all its heads at once)."""
    _rows2d(x, "x")
    _on_gpu(weight)
    rows, width = x.shape
    assert weight.numel() == width and weight.dtype == x.dtype
    _check(_fn("li_projection_rmsnorm")(_code(x), x.data_ptr(), x.stride(0), rows, width, weight.data_ptr(), 0, None,
                                        float(eps), _stream()), "projection_rmsnorm")
    return x


def qk_projection_rmsnorm_(q: torch.Tensor, q_weight: torch.Tensor, k: torch.Tensor, k_weight: torch.Tensor,
                           eps: float) -> None:
    """`projection_rmsnorm_` of two neighbouring column slices of one tensor (q, then k) in one launch."""
    _rows2d(q, "q"); _rows2d(k, "k")
    _on_gpu(q_weight, k_weight)
    assert q.stride(0) == k.stride(0) and q.shape[0] == k.shape[0] and q.dtype == k.dtype == q_weight.dtype
    assert k.data_ptr() == q.data_ptr() + q.shape[1] * q.element_size()
    assert q_weight.numel() == q.shape[1] and k_weight.numel() == k.shape[1]
    _check(_fn("li_projection_rmsnorm")(_code(q), q.data_ptr(), q.stride(0), q.shape[0], q.shape[1],
                                        q_weight.data_ptr(), k.shape[1], k_weight.data_ptr(), float(eps), _stream()),
           "projection_rmsnorm")


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                  heads: int, gate_activation: str = "silu", den: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, h] = weight * x[t, h] / sqrt(mean(x[t, h]^2) + eps) * act(gate[t, h]) per head.  x: float32
    [tokens, heads * size]; weight: float32, `size` entries shared by the heads or `heads * size`, one vector
    per head; gate (a column slice is fine) and out in the engine's dtype.  `gate_activation`: "silu" or
    "sigmoid".  `den` [tokens, heads] float32: x[t, h] is divided by den[t, h] first."""
    _on_gpu(x, weight, out, den)
    _rows2d(gate, "gate")
    tokens, width = out.shape
    size = width // heads
    assert x.dtype == torch.float32 and x.shape == out.shape == gate.shape and width == heads * size
    assert gate.dtype == out.dtype and weight.dtype == torch.float32 and weight.numel() in (size, width)
    assert den is None or (den.dtype == torch.float32 and den.numel() == tokens * heads)
    if gate_activation not in ("silu", "sigmoid"):
        raise KernelLibraryError(f"gated_rmsnorm knows the gates 'silu' and 'sigmoid', not {gate_activation!r}")
    _check(_fn("li_gated_rmsnorm")(_code(out), x.data_ptr(), gate.data_ptr(), gate.stride(0), weight.data_ptr(),
                                   out.data_ptr(), tokens, heads, size, float(eps),
                                   int(weight.numel() == width and heads > 1), int(gate_activation == "sigmoid"),
                                   _ptr(den), _stream()), "gated_rmsnorm")
    return out


def short_conv_step(x: torch.Tensor, taps: torch.Tensor, tail: torch.Tensor, seq_of_token: torch.Tensor,
                    query_start_loc: torch.Tensor, state_slots: torch.Tensor, num_seqs: int, out: torch.Tensor,
                    activation: str = "silu", single_tokens: bool = False) -> torch.Tensor:
    """`short_conv`, then `short_conv_update`: a step's convolution and the tails moved on by it.  With
    `single_tokens` (every sequence of the step brings exactly one token) one launch does both where the kernel
    can."""
    if single_tokens and short_conv(x, taps, tail, seq_of_token, query_start_loc, state_slots, out, activation,
                                    move_tail=True) is not None:
        return out
    short_conv(x, taps, tail, seq_of_token, query_start_loc, state_slots, out, activation)
    short_conv_update(x, tail, query_start_loc, state_slots, num_seqs)
    return out


def short_conv(x: torch.Tensor, taps: torch.Tensor, tail: torch.Tensor, seq_of_token: torch.Tensor,
               query_start_loc: torch.Tensor, state_slots: torch.Tensor, out: torch.Tensor,
               activation: str = "silu", move_tail: bool = False) -> "torch.Tensor | None":
    """A short causal convolution over time per channel, then the activation.

    x [tokens, channels] (a column slice is fine): this step's inputs, every sequence's end to end.  taps
    [K, channels] (tap by tap): row K-1 multiplies the current token, K-2 the one before.  tail [slots, K-1, channels]: the
    last K-1 inputs of each request before this step (zeros at its start), oldest first; it is read, not written
    (`short_conv_update` moves it on).  Tokens whose sequence is -1 give zeros.  `move_tail` (only for steps in
    which every sequence brings exactly one token): the launch also moves the tails on; None is returned, and
    nothing done, where the kernel cannot (sizes that its vector form does not take)."""
    _rows2d(x, "x")
    _on_gpu(taps, tail, seq_of_token, query_start_loc, state_slots, out)
    _int32(seq_of_token, "seq_of_token"); _int32(query_start_loc, "query_start_loc"); _int32(state_slots, "state_slots")
    tokens, channels = x.shape
    K = taps.shape[0]
    assert taps.shape[1] == channels and out.shape == (tokens, channels) and out.dtype == x.dtype == taps.dtype
    assert tail.shape[1:] == (K - 1, channels) and tail.dtype == x.dtype
    if activation not in ("silu", "none"):
        raise KernelLibraryError(f"short_conv knows the activations 'silu' and 'none', not {activation!r}")
    code = _fn("li_short_conv")(_code(x), x.data_ptr(), x.stride(0), taps.data_ptr(), tail.data_ptr() if K > 1 else None,
                                seq_of_token.data_ptr(), query_start_loc.data_ptr(), state_slots.data_ptr(),
                                out.data_ptr(), tokens, channels, K, 1 if activation == "silu" else 0,
                                int(move_tail and K > 1), _stream())
    if move_tail and code == 100001:
        return None
    _check(code, "short_conv")
    return out


def short_conv_update(x: torch.Tensor, tail: torch.Tensor, query_start_loc: torch.Tensor, state_slots: torch.Tensor,
                      num_seqs: int) -> None:
    """Moves every sequence's convolution tail on by this step's inputs: afterwards tail[slot] holds the last K-1
    inputs including this step's (a step shorter than K-1 keeps the newest of the old ones)."""
    _rows2d(x, "x")
    _on_gpu(tail, query_start_loc, state_slots)
    channels = x.shape[1]
    if tail.shape[1] == 0:
        return
    assert tail.shape[2] == channels and tail.dtype == x.dtype
    _check(_fn("li_short_conv_update")(_code(x), x.data_ptr(), x.stride(0), tail.data_ptr(), query_start_loc.data_ptr(),
                                       state_slots.data_ptr(), num_seqs, channels, tail.shape[1] + 1, _stream()),
           "short_conv_update")


def gated_delta_rule(qkv: torch.Tensor, ab: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
                     state: torch.Tensor, query_start_loc: torch.Tensor, state_slots: torch.Tensor, num_seqs: int,
                     heads: int, kv_heads: int, dim: int, vdim: int, out: torch.Tensor,
                     max_query_len: int = 0) -> torch.Tensor:
    """The gated delta rule, token by token, on a 32-bit state per request and head.

    qkv [tokens, 2 * kv_heads * dim + heads * vdim]: q and k (kv_heads heads of dim; head h of the values reads
    q/k head h // (heads / kv_heads)) and v (heads of vdim), after their convolutions.  ab (a column slice is
    fine) [tokens, 2 * heads]: per head the raw write strength (beta = sigmoid) and, behind those, the raw decay
    input (g = exp(-exp(a_log) * softplus(raw + dt_bias))).  q and k are made unit vectors (x / sqrt(sum x^2 +
    1e-6)), q also times dim^-0.5.  Per token: S *= g; u = beta * (v - S^T k); S += k u^T; o = S^T q.
    state [slots, heads, vdim, dim] float32 (S kept column by column) is read and written; out [tokens, heads *
    vdim] float32.  `max_query_len`: the most tokens a sequence brings, if known (1 picks the variant for steps
    of single tokens)."""
    _on_gpu(qkv, a_log, dt_bias, state, query_start_loc, state_slots, out)
    _rows2d(ab, "ab")
    _int32(query_start_loc, "query_start_loc"); _int32(state_slots, "state_slots")
    tokens = qkv.shape[0]
    assert qkv.shape[1] == 2 * kv_heads * dim + heads * vdim and ab.shape == (tokens, 2 * heads) and ab.dtype == qkv.dtype
    assert a_log.dtype == dt_bias.dtype == state.dtype == out.dtype == torch.float32
    assert a_log.numel() == dt_bias.numel() == heads and state.shape[1:] == (heads, vdim, dim)
    assert out.shape == (tokens, heads * vdim) and heads % kv_heads == 0
    # What the kernel in front leaves for the recurrence: per token q and k as unit vectors in 32-bit, and the gates.
    scratch = torch.empty(2 * max(tokens, 1) * (kv_heads * dim + heads) if max_query_len != 1 else 4,
                          dtype=torch.float32, device=qkv.device)
    _check(_fn("li_gated_delta_rule")(_code(qkv), qkv.data_ptr(), ab.data_ptr(), ab.stride(0), tokens, num_seqs,
                                      a_log.data_ptr(), dt_bias.data_ptr(), state.data_ptr(), query_start_loc.data_ptr(),
                                      state_slots.data_ptr(), out.data_ptr(), heads, kv_heads, dim, vdim,
                                      int(max_query_len), scratch.data_ptr(), _stream()), "gated_delta_rule")
    if max_query_len != 1:
        global launch_count
        launch_count += 1   # two kernels
    return out


def mlstm(proj: torch.Tensor, offsets: tuple[int, int, int, int, int], i_bias: torch.Tensor, f_bias: torch.Tensor,
          cap: float, state: torch.Tensor, maxima: torch.Tensor, query_start_loc: torch.Tensor,
          state_slots: torch.Tensor, num_seqs: int, heads: int, dim: int, vdim: int, out: torch.Tensor,
          den: torch.Tensor, max_query_len: int = 0) -> torch.Tensor:
    """The mLSTM matrix memory, token by token, on a 32-bit state per request and head.

    proj [tokens, width] holds, per token, at the columns `offsets` = (q, k, v, i, f): q and k (heads of dim), v
    (heads of vdim) and one raw input gate and one raw forget gate per head.  With x_i, x_f the raw gates plus
    their biases (float32 [heads]):  i = cap tanh(x_i / cap);  f = logsigmoid(cap tanh(x_f / cap));
    m' = max(f + m, i);  S <- exp(f + m - m') S + exp(i - m') k v^T;  n likewise with k alone;  m <- m'.
    out [tokens, heads * vdim] float32 = S^T q dim^-0.5 (not yet divided), den [tokens, heads] float32 =
    max(|n . q dim^-0.5|, exp(-m)) + 1e-6.  state [slots, heads, vdim + 1, dim] float32 (S column by column, n
    as the last column) and maxima [slots, heads, vdim + 1] float32 (m, a copy per column) are read and written.
    `max_query_len`: the most tokens a sequence brings, if known (the kernel then stages no more than that)."""
    _on_gpu(proj, i_bias, f_bias, state, maxima, query_start_loc, state_slots, out, den)
    _int32(query_start_loc, "query_start_loc"); _int32(state_slots, "state_slots")
    tokens, width = proj.shape
    q_off, k_off, v_off, i_off, f_off = offsets
    assert max(q_off, k_off) + heads * dim <= width and v_off + heads * vdim <= width and max(i_off, f_off) + heads <= width
    assert i_bias.dtype == f_bias.dtype == state.dtype == maxima.dtype == out.dtype == den.dtype == torch.float32
    assert i_bias.numel() == f_bias.numel() == heads
    assert state.shape[1:] == (heads, vdim + 1, dim) and maxima.shape[1:] == (heads, vdim + 1)
    assert out.shape == (tokens, heads * vdim) and den.shape == (tokens, heads)
    _check(_fn("li_mlstm")(_code(proj), proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, i_off, f_off,
                           i_bias.data_ptr(), f_bias.data_ptr(), float(cap), state.data_ptr(), maxima.data_ptr(),
                           query_start_loc.data_ptr(), state_slots.data_ptr(), tokens, num_seqs, out.data_ptr(),
                           den.data_ptr(), heads, dim, vdim, int(max_query_len), _stream()), "mlstm")
    return out


# ------------------------------------------- several residual streams, latent attention
@dataclass
class StreamUpdate:
    """A rewrite of the residual streams that has not been done yet: stream t becomes sum_s mix[s, t] * stream s +
    write[t] * gain * value, all from the old streams (`value` [tokens, width] is a sublayer's output in the
    engine's dtype; gain [width], write [S] and mix [S, S], indexed [from, to], are float32; gain None = ones).
    The norm that reads the streams next does the rewrite on its way (`stream_rmsnorm`)."""

    value: torch.Tensor
    gain: torch.Tensor | None
    write: torch.Tensor
    mix: torch.Tensor


def embedding_streams(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0,
                      error_flag: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, s * width:(s + 1) * width] = float32(table[ids[t]]) * scale for every copy s (out float32
    [tokens, copies * width]): the start of a 32-bit residual of one or several streams."""
    _on_gpu(ids, table, out, error_flag)
    _int32(ids, "ids"); _int32(error_flag, "error_flag")
    tokens, width = ids.numel(), table.shape[1]
    assert out.dtype == torch.float32 and out.shape[0] == tokens and out.shape[1] % width == 0
    _check(_fn("li_embedding_streams")(_code(table), ids.data_ptr(), table.data_ptr(), out.data_ptr(), tokens, width,
                                       table.shape[0], float(scale), out.shape[1] // width, _ptr(error_flag),
                                       _stream()), "embedding_streams")
    return out


def stream_rmsnorm(x: torch.Tensor, weight: torch.Tensor | None, eps: float, out: torch.Tensor | None,
                   read: torch.Tensor | None = None, update: StreamUpdate | None = None,
                   rows: torch.Tensor | None = None, out_scale: float = 1.0) -> torch.Tensor | None:
    """The pending rewrite of the streams (`update`, stored back into x unless `rows` is given), then
    out[r] = u / sqrt(mean(u^2) + eps) * weight * out_scale with u = sum_s read[s] * stream s of row rows[r] (or r);
    read None sums the streams.  x float32 [tokens, S * width]; weight float32 [width]; out [n, width] in the
    engine's dtype, None: only the rewrite is done.  Everything in between is 32-bit."""
    _on_gpu(x, weight, out, read, rows, update.value if update else None, update.gain if update else None,
            update.write if update else None, update.mix if update else None)
    _int32(rows, "rows")
    assert x.dtype == torch.float32 and (weight is None) == (out is None)
    if out is not None:
        width, n = out.shape[1], out.shape[0]
        assert weight.dtype == torch.float32 and weight.numel() == width
        dtype = out.dtype
    else:
        width, n, dtype = update.value.shape[1], x.shape[0], update.value.dtype
    S = x.shape[1] // width
    assert x.shape[1] == S * width and (rows is None or rows.numel() == n) and (rows is not None or n == x.shape[0])
    assert read is None or (read.dtype == torch.float32 and read.numel() == S)
    if update is not None:
        assert update.value.shape == (x.shape[0], width) and update.value.dtype == dtype
        assert update.write.dtype == update.mix.dtype == torch.float32
        assert update.write.numel() == S and update.mix.shape == (S, S)
        assert update.gain is None or (update.gain.dtype == torch.float32 and update.gain.numel() == width)
    _check(_fn("li_stream_rmsnorm")(
        _DTYPE_CODE[dtype], x.data_ptr(), _ptr(update.value if update else None), _ptr(update.gain if update else None),
        _ptr(update.write if update else None), _ptr(update.mix if update else None), _ptr(read), _ptr(weight),
        _ptr(out), _ptr(rows), n, width, S, float(eps), float(out_scale), int(update is not None and rows is None),
        _stream()), "stream_rmsnorm")
    return out


def activation(x: torch.Tensor, out: torch.Tensor, name: str) -> torch.Tensor:
    """out = act(x) element by element (out may be x); `name` from UNARY_ACTIVATIONS."""
    _on_gpu(x, out)
    assert x.shape == out.shape and x.dtype == out.dtype
    if name not in UNARY_ACTIVATIONS:
        raise KernelLibraryError(f"activation {name!r} has no kernel; known: {sorted(UNARY_ACTIVATIONS)}")
    _check(_fn("li_activation")(_code(x), x.data_ptr(), out.data_ptr(), x.numel(), UNARY_ACTIVATIONS[name], _stream()),
           "activation")
    return out


_unary = activation      # for callers whose own `activation` argument hides the function's name


def batched_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[b] = x[b] @ weight[b]^T for every b: x [B, M, K] (any batch and row strides, contiguous k: a head's
    columns of a projection), weight [B, N, K] contiguous, out [B, M, N] contiguous.  float32 runs the FFMA kernel,
    bfloat16 the library's batched product (32-bit accumulation)."""
    _on_gpu(weight, out)
    B, M, K = x.shape
    N = weight.shape[1]
    assert weight.shape == (B, N, K) and out.shape == (B, M, N) and x.dtype == weight.dtype == out.dtype
    if not x.is_cuda:
        raise KernelLibraryError(f"liteinfer_b200 kernels run on a CUDA device only; there is no CPU path (got {x.device})")
    if K > 1 and x.stride(2) != 1:
        raise KernelLibraryError("batched_linear takes x with contiguous rows")
    if M == 0:
        return out
    if x.dtype == torch.float32:
        _check(_fn("li_gemm_simt_batched")(0, x.data_ptr(), weight.data_ptr(), out.data_ptr(), M, N, K, B, x.stride(1),
                                           N, x.stride(0), N * K, M * N, _stream()), "gemm_simt_batched")
        return out
    torch.bmm(x, weight.transpose(1, 2), out=out)
    return out


def latent_prep(proj: torch.Tensor, q_off: int, q_rank: int, kv_off: int | None, kv_rank: int, rot_dim: int,
                rot_dims: int, q_weight: torch.Tensor, kv_weight: torch.Tensor | None, eps: float,
                inv_freq: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                block_table: torch.Tensor, pool: torch.Tensor, q_out: torch.Tensor | None, store: bool = True,
                cos_sin_scale: float = 1.0) -> None:
    """Per token of `proj` [tokens, columns]: q_out = rmsnorm(proj[:, q_off:q_off + q_rank]) * q_weight, and, with
    `kv_off` and `store`, the token's cache entry pool[page, slot] = [rmsnorm(latent) * kv_weight | rotated key
    part], latent = proj[:, kv_off:kv_off + kv_rank], the key part the rot_dim columns behind it, of which the
    first `rot_dims` turn by position * inv_freq (pairs i, i + rot_dims / 2).  pool [pages, 1, page_size, kv_rank +
    rot_dim]; norm weights float32; tokens whose sequence is -1 store nothing.  `q_out` None (with `q_weight`
    None): the layer has no query latent.  `cos_sin_scale` multiplies every cosine and sine."""
    _on_gpu(proj, q_weight, kv_weight, inv_freq, positions, seq_of_token, block_table, pool, q_out)
    _int32(positions, "positions"); _int32(seq_of_token, "seq_of_token"); _int32(block_table, "block_table")
    tokens = proj.shape[0]
    pages, one, page_size, entry = pool.shape
    assert one == 1 and entry == kv_rank + rot_dim and pool.dtype == proj.dtype
    assert (q_out is None) == (q_weight is None)
    assert q_out is None or (q_out.dtype == proj.dtype and q_out.shape == (tokens, q_rank)
                             and q_weight.dtype == torch.float32 and q_weight.numel() == q_rank)
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rot_dims
    writes = kv_off is not None and store
    assert not writes or (kv_weight.dtype == torch.float32 and kv_weight.numel() == kv_rank)
    _check(_fn("li_latent_prep")(_code(proj), proj.data_ptr(), proj.stride(0), q_off, q_rank, kv_off if writes else -1,
                                 kv_rank, rot_dim, rot_dims, _ptr(q_weight), _ptr(kv_weight if writes else None),
                                 float(eps), inv_freq.data_ptr(), positions.data_ptr(), seq_of_token.data_ptr(),
                                 block_table.data_ptr(), block_table.stride(0), pool.data_ptr(), page_size,
                                 pages if writes else 0, _ptr(q_out), tokens, float(cos_sin_scale), _stream()),
           "latent_prep")


def latent_attention(q_lat: torch.Tensor, q_raw: torch.Tensor, q_head_stride: int, q_rot_off: int, out: torch.Tensor,
                     pool: torch.Tensor, block_table: torch.Tensor, query_start_loc: torch.Tensor,
                     context_lens: torch.Tensor, inv_freq: torch.Tensor, sink: torch.Tensor | None, num_seqs: int,
                     max_q_len: int, heads: int, kv_rank: int, rot_dim: int, rot_dims: int, scale: float,
                     plan=None, window: int = 0, cos_sin_scale: float = 1.0) -> torch.Tensor:
    """Causal multi-query attention of every head over the shared cache entries [latent | rotated key part]:
    score = (q_lat . latent + rotate(q_rot) . key part) * scale, out = sum_j p_j latent_j, with exp(sink[h]) as one
    more term of the softmax's denominator (sink float32 [heads] or None).  q_lat, out: [heads, tokens, kv_rank];
    q_raw [tokens, columns]: the part of head h that turns lies at columns h * q_head_stride + q_rot_off (rot_dim
    numbers, rotated here by the query's position).  pool [pages, 1, page_size, kv_rank + rot_dim].  `window` > 0:
    a query at position p reads the keys at p - window + 1 ... p.  `cos_sin_scale` multiplies every cosine and
    sine of the query's rotation."""
    _on_gpu(q_lat, out, pool, block_table, query_start_loc, context_lens, inv_freq, sink)
    _rows2d(q_raw, "q_raw")         # a column slice of a wider projection is fine
    _int32(block_table, "block_table"); _int32(query_start_loc, "query_start_loc"); _int32(context_lens, "context_lens")
    pages, one, page_size, entry = pool.shape
    tokens = q_raw.shape[0]
    assert one == 1 and entry == kv_rank + rot_dim and q_lat.shape == out.shape == (heads, tokens, kv_rank)
    assert q_lat.dtype == q_raw.dtype == out.dtype == pool.dtype
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == heads)
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rot_dims
    if latent_mma_supports(q_raw.dtype, kv_rank, rot_dim, rot_dims):
        # Tensor cores: sequences that bring one token in a launch that splits their keys over blocks, the others
        # four queries a block; without a plan every sequence goes the second way.
        def run(seq_index, count, q_len, splits=1, two_blocks=False):
            partial_out = partial_lse = None
            if splits > 1:
                partial_out = torch.empty((splits, heads, tokens, kv_rank), dtype=torch.float32, device=out.device)
                partial_lse = torch.empty((splits, heads, tokens), dtype=torch.float32, device=out.device)
            _check(_fn("li_latent_attention_mma")(
                q_lat.data_ptr(), q_lat.stride(0), q_lat.stride(1), q_raw.data_ptr(), q_raw.stride(0), q_head_stride,
                q_rot_off, out.data_ptr(), out.stride(0), out.stride(1), pool.data_ptr(), block_table.data_ptr(),
                block_table.stride(0), query_start_loc.data_ptr(), context_lens.data_ptr(), _ptr(seq_index),
                inv_freq.data_ptr(), _ptr(sink), count, q_len, heads, kv_rank, rot_dim, rot_dims, page_size, pages,
                float(scale), splits, _ptr(partial_out), _ptr(partial_lse), tokens, int(two_blocks),
                scratch_for(out.device).gemm_error.data_ptr(), int(window), float(cos_sin_scale), _stream()),
                "latent_attention_mma")

        if plan is None:
            run(None, num_seqs, max(max_q_len, 2))
            return out
        if plan.num_prefill:
            run(plan.prefill_seqs, plan.num_prefill, max(plan.max_prefill_query_len, 2))
        if plan.num_decode:
            chunks = -(-heads // 16)
            reach = plan.max_decode_context_len if window <= 0 else min(plan.max_decode_context_len, window + 64)
            tiles = max(1, -(-reach // 64))                                   # two tiles of 32 keys a split at least
            # Two blocks of eight warps per SM where the batch is wide (measured at 16 heads over 2,048 keys: 67
            # against 86 us at 64 sequences), one of sixteen where it is narrow (18.7 against 19.8 us at 8); as many
            # splits as still make one wave of either.
            two_blocks = plan.num_decode * chunks > 16
            splits = max(1, min(tiles, (2 if two_blocks else 1) * NUM_SMS // max(1, plan.num_decode * chunks), 32))
            run(plan.decode_seqs, plan.num_decode, 1, splits, two_blocks)
        return out
    _check(_fn("li_latent_attention")(
        _code(q_raw), q_lat.data_ptr(), q_lat.stride(0), q_lat.stride(1), q_raw.data_ptr(), q_raw.stride(0),
        q_head_stride, q_rot_off, out.data_ptr(), out.stride(0), out.stride(1), pool.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), query_start_loc.data_ptr(), context_lens.data_ptr(), inv_freq.data_ptr(), _ptr(sink),
        num_seqs, max_q_len, heads, kv_rank, rot_dim, rot_dims, page_size, pages, float(scale), int(window),
        float(cos_sin_scale), _stream()),
        "latent_attention")
    return out


# (latent, rotated part) that attention_latent_mma.cu is instantiated for (its own `..._supports` says the same; the
# table stands here too so that a model of other sizes never builds that library).
_LATENT_MMA_SIZES = {(64, 32), (128, 32), (128, 64), (256, 64), (512, 64)}


def latent_mma_supports(dtype: torch.dtype, kv_rank: int, rot_dim: int, rot_dims: int) -> bool:
    """Whether the tensor-core latent attention takes these sizes (bfloat16; LITEINFER_LATENT_MMA=0 keeps every
    size on the SIMT kernel)."""
    return (dtype == torch.bfloat16 and os.environ.get("LITEINFER_LATENT_MMA", "1") != "0"
            and (kv_rank, rot_dim) in _LATENT_MMA_SIZES and 0 <= rot_dims <= rot_dim and rot_dims % 2 == 0)


def gate_heads(v: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor) -> torch.Tensor:
    """out[t, h * e:(h + 1) * e] = v[h, t] * sigmoid(gate[t, h * e:(h + 1) * e]): v [heads, tokens, e] head-major,
    gate [tokens, heads * e] (a column slice is fine; None: no gate, only the transposition), out [tokens, heads *
    e]; the sigmoid is 32-bit."""
    _on_gpu(v, out)
    heads, tokens, e = v.shape
    assert out.shape == (tokens, heads * e) and v.dtype == out.dtype
    if gate is not None:
        _rows2d(gate, "gate")
        assert gate.shape == out.shape and gate.dtype == v.dtype
    _check(_fn("li_gate_heads")(_code(v), v.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                out.data_ptr(), tokens, heads, e, _stream()), "gate_heads")
    return out


# ------------------------------------------------------------- mixture of experts
EXPERT_ACTIVATIONS = {"swiglu": 0, "capped_swiglu": 1}


@dataclass
class ExpertPlan:
    """A step's (token, slot) pairs ordered by expert and cut into tiles of `tile_rows` rows of one expert each."""
    order: torch.Tensor         # [pairs] int32: the pairs (token * top + slot), expert by expert
    offsets: torch.Tensor       # [experts + 1] int32: where each expert's run starts in `order`
    tile_expert: torch.Tensor   # [max_tiles] int32: the expert of each tile (-1: no such tile)
    tile_row0: torch.Tensor     # [max_tiles] int32: its first row in `order`
    tile_rows: int
    max_tiles: int
    place: torch.Tensor | None = None   # [pairs] int32: where in `order` each pair stands


def moe_route(logits: torch.Tensor, top: int, groups: int, keep: int, renormalise: bool, ids: torch.Tensor,
              weights: torch.Tensor) -> None:
    """Per token of `logits` [tokens, experts] (float32): scores = softmax over all experts; with `groups` > 1 the
    experts form that many equal groups of neighbours, a group's score is its largest, and only experts of the best
    `keep` groups can be chosen; ids [tokens, top] int32 = the experts with the largest scores (ties: the lower
    index), weights [tokens, top] float32 = their scores (`renormalise`: divided by their sum)."""
    _on_gpu(logits, ids, weights)
    _int32(ids, "ids")
    tokens, experts = logits.shape
    assert logits.dtype == torch.float32 == weights.dtype and logits.is_contiguous()
    assert ids.shape == weights.shape == (tokens, top) and ids.is_contiguous() and weights.is_contiguous()
    _check(_fn("li_moe_route")(logits.data_ptr(), tokens, experts, top, groups, keep, int(renormalise), ids.data_ptr(),
                               weights.data_ptr(), _stream()), "moe_route")


def moe_router(x: torch.Tensor, weight: torch.Tensor, top: int, groups: int, keep: int, renormalise: bool,
               ids: torch.Tensor, weights: torch.Tensor) -> None:
    """`moe_route` of the logits x @ weight^T, product and routing in one launch: x [tokens, hidden] in the engine's
    dtype (a column slice is fine), weight [experts, hidden] float32; the product is 32-bit, its sums in an order that
    depends on nothing but the sizes."""
    _on_gpu(weight, ids, weights)
    _rows2d(x, "x")
    _int32(ids, "ids")
    tokens, hidden = x.shape
    experts = weight.shape[0]
    assert weight.dtype == torch.float32 == weights.dtype and weight.shape == (experts, hidden)
    assert ids.shape == weights.shape == (tokens, top) and ids.is_contiguous() and weights.is_contiguous()
    _check(_fn("li_moe_router")(_code(x), x.data_ptr(), x.stride(0), weight.data_ptr(), tokens, hidden, experts, top,
                                groups, keep, int(renormalise), ids.data_ptr(), weights.data_ptr(), _stream()),
           "moe_router")


# LITEINFER_MOE_TCGEN05: 1 (default) = bfloat16 experts of steps with at least LITEINFER_MOE_TCGEN05_MIN_PAIRS (1) pairs of
# (token, expert) run their products on the tcgen05 kernel; 0 = every step on the mma.sync tiles (measured on B200 at
# width 2,048 with 32 experts 2,048 wide, four a token: 2,048 tokens 350 against 958 us, 64 tokens 158 against 222, 8
# tokens 124 against 164).
MOE_TCGEN05 = os.environ.get("LITEINFER_MOE_TCGEN05", "1") != "0"
MOE_TCGEN05_MIN_PAIRS = int(os.environ.get("LITEINFER_MOE_TCGEN05_MIN_PAIRS", "1"))


def moe_tile_rows(dtype: torch.dtype, hidden: int, ff: int, pairs: int | None = None) -> int:
    """Rows of a tile of an expert's products: 128 where the tcgen05 kernel takes them (bfloat16, sizes in eights, a
    step of many pairs), 64 where both run on mma.sync tiles, else 32 (FFMA tiles)."""
    if not torch.cuda.is_available():
        return 32
    code = _DTYPE_CODE[dtype]
    both = _fn("li_moe_tile_rows")(code, ff, hidden) == 64 and _fn("li_moe_tile_rows")(code, hidden, ff) == 64
    if both and pairs is not None and MOE_TCGEN05 and pairs >= MOE_TCGEN05_MIN_PAIRS and hidden % 8 == 0 and ff % 8 == 0:
        return 128
    return 64 if both else 32


def moe_sort(ids: torch.Tensor, experts: int, tile_rows: int, with_place: bool = False) -> ExpertPlan:
    """The plan of a step whose pair p = token * top + slot goes to expert ids.flatten()[p]."""
    _on_gpu(ids)
    _int32(ids, "ids")
    pairs = ids.numel()
    max_tiles = -(-pairs // tile_rows) + experts
    scratch = torch.empty(pairs * (2 if with_place else 1) + experts + 1 + 2 * max_tiles, dtype=torch.int32,
                          device=ids.device)
    order, offsets = scratch[:pairs], scratch[pairs:pairs + experts + 1]
    tile_expert = scratch[pairs + experts + 1:pairs + experts + 1 + max_tiles]
    tile_row0 = scratch[pairs + experts + 1 + max_tiles:pairs + experts + 1 + 2 * max_tiles]
    place = scratch[pairs + experts + 1 + 2 * max_tiles:] if with_place else None
    _check(_fn("li_moe_sort")(ids.data_ptr(), pairs, experts, tile_rows, offsets.data_ptr(), order.data_ptr(),
                              tile_expert.data_ptr(), tile_row0.data_ptr(), max_tiles, _ptr(place), _stream()),
           "moe_sort")
    return ExpertPlan(order, offsets, tile_expert, tile_row0, tile_rows, max_tiles, place)


def moe_gather(x: torch.Tensor, plan: ExpertPlan, top: int, out: torch.Tensor) -> torch.Tensor:
    """out[m] = x[plan.order[m] // top]: every pair's token row, in the order of the experts' runs."""
    _on_gpu(out)
    _rows2d(x, "x")
    pairs = plan.order.numel()
    assert out.shape == (pairs, x.shape[1]) and out.dtype == x.dtype and out.is_contiguous()
    _check(_fn("li_moe_gather")(_code(x), x.data_ptr(), x.stride(0), plan.order.data_ptr(), top, out.data_ptr(), pairs,
                                x.shape[1], _stream()), "moe_gather")
    return out


def moe_grouped_tcgen05(mode: str, a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, plan: ExpertPlan,
                        activation: str = "swiglu", limit: float = 0.0, alpha: float = 1.0,
                        pair_weights: torch.Tensor | None = None) -> torch.Tensor:
    """`moe_grouped` on the tcgen05 kernel (bfloat16): `a` [pairs, K] and `out` hold their rows in the order of the
    experts' runs (`plan.order`), the plan's tiles are 128 rows, and in mode "gate_up" an expert's gate and up rows lie
    interleaved in eights.  mode "down" multiplies row m by pair_weights[plan.order[m]]."""
    _on_gpu(a, weight, out, pair_weights)
    experts, rows, K = weight.shape
    pairs = plan.order.numel()
    assert plan.tile_rows == 128 and mode in ("gate_up", "down") and a.dtype == weight.dtype == out.dtype == torch.bfloat16
    assert a.shape == (pairs, K) and out.shape == (pairs, rows // 2 if mode == "gate_up" else rows)
    act = -1 if mode == "down" else {"swiglu": 0, "capped_swiglu": 4}[activation]
    scale = pair_weights if mode == "down" else None
    _check(_fn("li_gemm_tcgen05_grouped")(
        a.data_ptr(), weight.data_ptr(), out.data_ptr(), pairs, rows, K, experts, act, float(limit), float(alpha),
        plan.tile_expert.data_ptr(), plan.tile_row0.data_ptr(), plan.offsets.data_ptr(), plan.max_tiles,
        plan.order.data_ptr() if scale is not None else None, _ptr(scale),
        scratch_for(a.device).gemm_error.data_ptr(), _stream()), "gemm_tcgen05_grouped")
    return out


def moe_grouped(mode: str, a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, plan: ExpertPlan, top: int,
                activation: str = "swiglu", limit: float = 0.0, alpha: float = 1.0,
                pair_weights: torch.Tensor | None = None, eights: bool = False) -> torch.Tensor:
    """The experts' products, grouped by expert.  mode "gate_up": out[p] = act(W_gate,e a[p // top], W_up,e a[p // top])
    for pair p of expert e; a [tokens, hidden], weight [experts, 2 * ff, hidden] (an expert's gate rows, then its up
    rows), out [pairs, ff]; `activation` of `EXPERT_ACTIVATIONS` ("capped_swiglu": g' = min(g, limit), u' = clamp(u,
    -limit, limit), g' * sigmoid(alpha * g') * (u' + 1)).  mode "down": out[p] = (W_down,e a[p]) * pair_weights[p];
    a [pairs, ff], weight [experts, hidden, ff], out [pairs, hidden].  `eights` (mode "gate_up"): an expert's gate and
    up rows lie interleaved in eights (eight gate rows, then their eight up rows) instead of one half after the other."""
    _on_gpu(a, weight, out, pair_weights)
    _rows2d(a, "a")
    assert mode in ("gate_up", "down") and a.dtype == weight.dtype == out.dtype and out.is_contiguous()
    experts, rows, K = weight.shape
    N = rows // 2 if mode == "gate_up" else rows
    assert weight.is_contiguous() and a.shape[1] == K and out.shape == (plan.order.numel(), N)
    assert pair_weights is None or (pair_weights.dtype == torch.float32 and pair_weights.numel() == plan.order.numel())
    _check(_fn("li_moe_grouped")(_code(a), 0 if mode == "gate_up" else 1, a.data_ptr(), a.stride(0), weight.data_ptr(),
                                 out.data_ptr(), out.stride(0), plan.order.data_ptr(), plan.offsets.data_ptr(),
                                 plan.tile_expert.data_ptr(), plan.tile_row0.data_ptr(), _ptr(pair_weights), top, N, K,
                                 EXPERT_ACTIVATIONS[activation], float(limit), float(alpha), plan.max_tiles,
                                 plan.tile_rows, int(eights), _stream()), "moe_grouped")
    return out


def moe_combine(y: torch.Tensor, out: torch.Tensor, top: int, place: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = sum over s < top of y[t * top + s], in slot order, summed in 32-bit; with `place` the row of pair p is
    y[place[p]] (rows in the order of the experts' runs)."""
    _on_gpu(y, out, place)
    tokens, width = out.shape
    assert y.shape == (tokens * top, width) and y.dtype == out.dtype and y.is_contiguous() and out.is_contiguous()
    _check(_fn("li_moe_combine")(_code(y), y.data_ptr(), out.data_ptr(), tokens, top, width, _ptr(place), _stream()),
           "moe_combine")
    return out


def moe_experts(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                activation: str, limit: float, alpha: float, eights: bool, out: torch.Tensor) -> torch.Tensor:
    """out[t] = sum_s weights[t, s] * down_e(act(gate_e x[t], up_e x[t])), e = ids[t, s]: the chosen experts of every
    token, their products grouped by expert.  gate_up [experts, 2 * ff, hidden] (`eights`: gate and up rows interleaved
    in eights), down [experts, hidden, ff].  Steps of many pairs in bfloat16 run the tcgen05 kernel over the pairs'
    rows gathered expert by expert; the others the mma.sync or FFMA tiles, which gather as they load."""
    tokens, top = ids.shape
    experts, hidden, ff = down.shape
    pairs = tokens * top
    tile = moe_tile_rows(x.dtype, hidden, ff, pairs if eights else None)
    plan = moe_sort(ids, experts, tile, with_place=tile == 128)
    act = torch.empty((pairs, ff), dtype=x.dtype, device=x.device)
    each = torch.empty((pairs, hidden), dtype=x.dtype, device=x.device)
    scale = weights.view(-1)
    if tile == 128:
        rows = moe_gather(x, plan, top, torch.empty((pairs, hidden), dtype=x.dtype, device=x.device))
        moe_grouped_tcgen05("gate_up", rows, gate_up, act, plan, activation, limit, alpha)
        moe_grouped_tcgen05("down", act, down, each, plan, pair_weights=scale)
        return moe_combine(each, out, top, place=plan.place)
    moe_grouped("gate_up", x, gate_up, act, plan, top, activation, limit, alpha, eights=eights)
    moe_grouped("down", act, down, each, plan, top, pair_weights=scale)
    return moe_combine(each, out, top)


# ------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _on_gpu(logits, out)
    _int32(out, "out")
    rows, vocab = logits.shape
    ws = scratch_for(logits.device)
    _check(_fn("li_argmax")(_code(logits), logits.data_ptr(), rows, vocab, out.data_ptr(), ws.argmax_value.data_ptr(),
                            ws.argmax_index.data_ptr(), ws.argmax_counters.data_ptr(), ws.ARGMAX_ROWS, _stream()),
           "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """One token per row: temperature, top-k, top-p, then the draw `uniform[r]` in [0, 1)."""
    _on_gpu(logits, temperature, top_k, top_p, uniform, out)
    _int32(out, "out"); _int32(top_k, "top_k")
    rows, vocab = logits.shape
    for t in (temperature, top_p, uniform):
        assert t.dtype == torch.float32 and t.numel() == rows
    _check(_fn("li_sample")(_code(logits), logits.data_ptr(), rows, vocab, temperature.data_ptr(), top_k.data_ptr(),
                            top_p.data_ptr(), uniform.data_ptr(), out.data_ptr(), _stream()), "sample")
    return out
