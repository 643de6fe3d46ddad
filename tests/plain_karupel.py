"""A plain, slow implementation of the Karupel decoder in float64: the oracle of the Karupel tests.

One function per mechanism, written from the formulas, token by token where the model is a recurrence.  It reads
a model folder with its own safetensors reader and shares no code with `liteinfer_b200`.  A whole sequence goes in,
logits of every position come out; there is no cache, no batch and no cut.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F = torch.float64


def read_model(model_dir):
    """(config.json as a dict, {tensor name: float64 tensor})."""
    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    blob = (model_dir / "model.safetensors").read_bytes()
    (header_len,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + header_len])
    data = blob[8 + header_len:]
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = np.frombuffer(data[lo:hi], dtype=np.uint8)
        if meta["dtype"] == "BF16":
            bits = raw.view(np.uint16).astype(np.uint32) << 16
            value = torch.from_numpy(bits.view(np.float32).copy())
        elif meta["dtype"] == "F32":
            value = torch.from_numpy(raw.view(np.float32).copy())
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        tensors[name] = value.to(F).reshape(meta["shape"])
    return config, tensors


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def offset_norm(x, stored, eps):
    """The model's norm: the stored weight lies around zero, 1 + weight multiplies."""
    return unit_rms(x, eps) * (1.0 + stored)


def silu(x):
    return x / (1.0 + torch.exp(-x))


def causal_conv(x, taps):
    """y[t, c] = sum_j taps[c, j] * x[t - (K - 1 - j), c], zeros before the start; x [T, C], taps [C, K]."""
    T, K = x.shape[0], taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(K):
            src = t - (K - 1 - j)
            if src >= 0:
                y[t] += taps[:, j] * x[src]
    return y


def delta_rule(q, k, v, beta, decay):
    """q, k [T, G, D]; v [T, H, V]; beta, decay [T, H].  Returns the read-outs [T, H, V]."""
    T, G, D = q.shape
    H, V = v.shape[1], v.shape[2]
    out = torch.zeros(T, H, V, dtype=F)
    for h in range(H):
        g = h // (H // G)
        S = torch.zeros(D, V, dtype=F)
        for t in range(T):
            S = decay[t, h] * S
            u = beta[t, h] * (v[t, h] - S.t() @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, h] = S.t() @ q[t, g]
    return out


def delta_mixer(w, p, m, x, eps):
    T = x.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(x @ w[p + "q"].t(), w[p + "q.conv"])).view(T, G, D)
    k = silu(causal_conv(x @ w[p + "k"].t(), w[p + "k.conv"])).view(T, G, D)
    v = silu(causal_conv(x @ w[p + "v"].t(), w[p + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(x @ w[p + "b"].t())
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(x @ w[p + "a"].t() + w[p + "dt_bias"]))
    o = delta_rule(q, k, v, beta, decay)
    o = unit_rms(o, eps) * w[p + "norm"] * silu(x @ w[p + "g"].t()).view(T, H, V)
    return o.reshape(T, H * V) @ w[p + "o"].t()


def matrix_memory(q, k, v, log_in, log_forget):
    """The mLSTM recurrence of one head: q, k [T, D] (q already scaled), v [T, V], the gates' logarithms [T]."""
    T, D = q.shape
    S, n, m = torch.zeros(D, v.shape[1], dtype=F), torch.zeros(D, dtype=F), 0.0
    out = torch.zeros(T, v.shape[1], dtype=F)
    for t in range(T):
        m_new = max(float(log_forget[t]) + m, float(log_in[t]))
        keep, write = math.exp(float(log_forget[t]) + m - m_new), math.exp(float(log_in[t]) - m_new)
        S = keep * S + write * torch.outer(k[t], v[t])
        n = keep * n + write * k[t]
        m = m_new
        out[t] = S.t() @ q[t] / (max(abs(float(n @ q[t])), math.exp(-m)) + 1e-6)
    return out


def mlstm_mixer(w, p, m, x, eps):
    T = x.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (x @ w[p + "q"].t()).view(T, H, D) * D ** -0.5
    k = (x @ w[p + "k"].t()).view(T, H, D)
    v = (x @ w[p + "v"].t()).view(T, H, V)
    log_in = cap * torch.tanh((x @ w[p + "i"].t() + w[p + "i.b"]) / cap)
    log_forget = torch.nn.functional.logsigmoid(cap * torch.tanh((x @ w[p + "f"].t() + w[p + "f.b"]) / cap))
    o = torch.stack([matrix_memory(q[:, h], k[:, h], v[:, h], log_in[:, h], log_forget[:, h]) for h in range(H)], 1)
    o = unit_rms(o, eps).reshape(T, H * V) * w[p + "norm"] * torch.sigmoid(x @ w[p + "g"].t())
    return o @ w[p + "o"].t()


def turn(x, rot):
    """Rotates the first rot.dims dimensions of every head of x [T, heads, dim]: i pairs with i + dims / 2."""
    if not rot:
        return x
    dims = rot["dims"]
    half = dims // 2
    freq = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    if rot.get("scaling"):
        freq = freq / rot["scaling"]["factor"]
    angle = torch.arange(x.shape[0], dtype=F)[:, None] * freq[None, :]
    c, s = angle.cos()[:, None, :], angle.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def attention_mixer(w, p, m, x, eps, first_values, mixes):
    """`first_values`: None, or the values [T, G, V] of the first value-mixing layer; `mixes`: this layer blends
    them in.  Returns (output, this layer's own values before any blend)."""
    T = x.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (x @ w[p + "q"].t() + w[p + "q.b"]).view(T, H, D)
    k = (x @ w[p + "k"].t() + w[p + "k.b"]).view(T, G, D)
    v = (x @ w[p + "v"].t() + w[p + "v.b"]).view(T, G, V)
    own = v
    q = turn(unit_rms(q, eps) * w[p + "q.norm"], m.get("rot"))
    k = turn(unit_rms(k, eps) * w[p + "k.norm"], m.get("rot"))
    if mixes:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * first_values
    out = torch.zeros(T, H, V, dtype=F)
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            score = (k[:t + 1, g] @ q[t, h]) * m["scale"]
            weight = torch.softmax(score, 0)
            out[t, h] = weight @ v[:t + 1, g]
    out = out * torch.sigmoid(x @ w[p + "g"].t())[:, :, None]
    return out.reshape(T, H * V) @ w[p + "o"].t(), own


def gated_feed_forward(w, p, x):
    return (silu(x @ w[p + "gate"].t()) * (x @ w[p + "up"].t())) @ w[p + "down"].t()


def forward(config, w, tokens, trace=None):
    """Logits [len(tokens), vocab] in float64; `trace` (a list) receives the residual stream after every layer."""
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    first_values = None
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "mlstm":
            y = mlstm_mixer(w, p, m, x, eps)
        elif layer["type"] == "delta":
            y = delta_mixer(w, p, m, x, eps)
        else:
            mixing = bool(m.get("v_mix"))
            y, own = attention_mixer(w, p, m, x, eps, first_values, mixing and first_values is not None)
            if mixing and first_values is None:
                first_values = own
        x = x + offset_norm(y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp"):
            x = x + offset_norm(gated_feed_forward(w, f"l{i}.mlp.", x), w[f"l{i}.norm2"], eps)
        if trace is not None:
            trace.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["embed"].t()
