"""A plain, slow implementation of the Kutolix decoder in float64: the oracle of the Kutolix tests.

One function per mechanism, written from the formulas.  It reads a model folder with its own safetensors reader
and shares no code with `liteinfer_b200`.  A whole sequence goes in, logits of every position come out; there is
no cache, no batch and no cut.
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
        elif meta["dtype"] == "I32":
            value = torch.from_numpy(raw.view(np.int32).copy())
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        tensors[name] = value.to(F).reshape(meta["shape"])
    return config, tensors


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def frequencies(rot):
    """(f_i for i < dims / 2, what multiplies every cosine and sine)."""
    dims, base = rot["dims"], float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    s = rot.get("scaling")
    if not s:
        return f, 1.0

    def index_of(turns):
        return dims * math.log(s["original"] / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(index_of(s["fast"])), 0)
    hi = min(math.ceil(index_of(s["slow"])), dims - 1)
    out = torch.empty_like(f)
    for i in range(dims // 2):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f[i] / s["factor"] * ramp + f[i] * (1.0 - ramp)
    return out, 0.1 * math.log(s["factor"]) + 1.0


def rotate(x, rot, layout):
    """x [T, heads, n]: the first rot.dims numbers of every head turn by position * frequency; `layout` "half"
    pairs dimension i with i + dims / 2, "interleaved" pairs 2i with 2i + 1."""
    dims = rot["dims"]
    f, stretch = frequencies(rot)
    out = x.clone()
    for t in range(x.shape[0]):
        for i in range(dims // 2):
            a, b = (i, i + dims // 2) if layout == "half" else (2 * i, 2 * i + 1)
            c, s = math.cos(t * float(f[i])) * stretch, math.sin(t * float(f[i])) * stretch
            u, v = x[t, :, a], x[t, :, b]
            out[t, :, a] = u * c - v * s
            out[t, :, b] = v * c + u * s
    return out


def windowed_softmax_attention(q, k, v, scale, window, sink=None):
    """q [T, H, D], k [T, H, D], v [T, H, V] (keys and values already per query head) -> [T, H, V].  Position i
    reads the keys at i - window + 1 ... i (None: every key up to i).  `sink` [H]: exp(sink) joins the denominator."""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, h] @ q[i, h]) * scale
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + (0.0 if sink is None else torch.exp(sink[h] - m))
            out[i, h] = (e / den) @ v[lo:i + 1, h]
    return out


def gated_attention(h, w, p, mixer, eps):
    """The 'attention' mixer: grouped queries, half-split partial rotation, unit-RMS q and k, window, sink, gate."""
    T = h.shape[0]
    H, G, D, V = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, V)
    if mixer.get("rot"):
        q, k = rotate(q, mixer["rot"], "half"), rotate(k, mixer["rot"], "half")
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    window = mixer["mask"]["size"] if mixer.get("mask") else None
    a = windowed_softmax_attention(q, k, v, mixer["scale"], window, sink=w[p + "sink"])
    a = a.reshape(T, H * V) * sigmoid(h @ w[p + "g"].T)
    return a @ w[p + "o"].T


def latent_attention(h, w, p, mixer, eps):
    """The 'latent_attention' mixer: keys and values expanded from one normalised latent per token plus one rotated
    key part for all heads; interleaved rotation of the rotated parts; window; ordinary softmax."""
    T = h.shape[0]
    H, D, R, V, C = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    q = (h @ w[p + "q"].T).view(T, H, D + R)
    down = h @ w[p + "dkv"].T
    c = unit_rms(down[:, :C], eps) * w[p + "dkv.norm"]
    shared = down[:, C:].view(T, 1, R)
    q_rot = rotate(q[:, :, D:], mixer["rot"], "interleaved")
    k_rot = rotate(shared, mixer["rot"], "interleaved").expand(T, H, R)
    k_plain = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, V)
    window = mixer["mask"]["size"] if mixer.get("mask") else None
    a = windowed_softmax_attention(torch.cat([q[:, :, :D], q_rot], -1), torch.cat([k_plain, k_rot], -1), v,
                                   mixer["scale"], window)
    return a.reshape(T, H * V) @ w[p + "o"].T


def dense_ff(h, w, p):
    g = h @ w[p + "gate"].T
    return (g * sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, router):
    """(chosen experts [T, top], their weights [T, top]): softmax over all experts; the best `keep` groups of
    neighbours by their largest score; the `top` largest scores within those; weights are the scores themselves."""
    scores = torch.softmax(h @ w[p + "router"].T, dim=-1)
    T, E = scores.shape
    groups = router.get("groups")
    allowed = torch.ones(T, E, dtype=torch.bool)
    if groups:
        per = E // groups["count"]
        best = scores.view(T, groups["count"], per).max(-1).values
        keep = best.topk(groups["keep"], dim=-1).indices
        allowed = torch.zeros(T, groups["count"], dtype=torch.bool).scatter_(1, keep, True).repeat_interleave(per, 1)
    masked = torch.where(allowed, scores, torch.full_like(scores, -1.0))
    chosen = masked.topk(router["top"], dim=-1).indices
    return chosen, scores.gather(1, chosen)


def expert_ff(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def moe_ff(h, w, p, mlp):
    chosen, weights = route(h, w, p, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t].tolist(), weights[t]):
            out[t] += s * expert_ff(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    return out


def forward(config, w, tokens, trace=None):
    """Logits [T, vocab] of a whole sequence.  `trace`: a list that receives the stream after every layer."""
    eps = config["norm"]["eps"]
    m = config.get("residual_mult", 1.0)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    for i, layer in enumerate(config["layers"]):
        mix = {"attention": gated_attention, "latent_attention": latent_attention}[layer["type"]]
        x = x + m * unit_rms(mix(x, w, f"l{i}.mix.", layer["mixer"], eps), eps) * w[f"l{i}.norm1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, w, f"l{i}.mlp.") if mlp["kind"] == "dense" else moe_ff(x, w, f"l{i}.mlp.", mlp)
            x = x + m * unit_rms(y, eps) * w[f"l{i}.norm2"]
        if trace is not None:
            trace.append(x.clone())
    logits = (unit_rms(x, eps) * w["final.norm"]) @ w["embed"].T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
