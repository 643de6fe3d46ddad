"""Plain torch stand-ins for the CUDA kernels, with the kernels' own signatures.

Two uses, both in tests only.  (1) `-m gpu` kernel tests compare each CUDA
kernel with the function of the same name here, on inputs of other sizes than
the engine's.  (2) `-m "not gpu"` tests patch these functions over
`liteinfer_b200.ops` (the `cpu_kernels` fixture) so that the step function, the
cache and the scheduler can be driven on a CPU; the product itself has no such
path.  Everything computes in float32 and rounds where the kernels round.
"""

from __future__ import annotations

import math

import torch

from liteinfer_b200.cache import addressing


def _r(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return x.to(dtype).float()


def embedding(ids, table, out, error_flag=None):
    bad = (ids < 0) | (ids >= table.shape[0])
    out.copy_(table[ids.long().clamp(0, table.shape[0] - 1)])
    out[bad] = 0
    if error_flag is not None and bool(bad.any()):
        error_flag.fill_(1)
    return out


def scatter_tokens(tokens, dst, src, source):
    live = dst >= 0
    tokens[dst[live].long()] = source[src[live].long()]
    return tokens


def rmsnorm(x, weight, eps, out, delta=None, rows=None, write_residual=False):
    dtype = x.dtype
    src = x if rows is None else x[rows.long()]
    v = src.float()
    if delta is not None:
        d = delta if rows is None else delta[rows.long()]
        v = _r(v + d.float(), dtype)
        if write_residual:
            x.copy_(v.to(dtype))
    inv = 1.0 / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    out.copy_((weight.float() * _r(v * inv, dtype)).to(dtype))
    return out


def add_(x, delta):
    x.copy_((x.float() + delta.float()).to(x.dtype))
    return x


def add_bias_(out, bias):
    out.copy_((out.float() + bias.float()).to(out.dtype))
    return out


def _activate(x, activation):
    if activation == "silu":
        return x / (1.0 + torch.exp(-x))
    if activation == "gelu":
        return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))
    if activation in ("gelu_pytorch_tanh", "gelu_tanh"):
        return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))
    if activation == "relu":
        return torch.relu(x)
    raise ValueError(activation)


def act_mul(gate_up, out, activation):
    w = out.shape[1]
    g, u = gate_up[:, :w].float(), gate_up[:, w:].float()
    out.copy_((_r(_activate(g, activation), out.dtype) * u).to(out.dtype))
    return out


def act_mul_interleaved(gate_up, out, activation):
    rows, w = out.shape
    pairs = gate_up.float().view(rows, w // 8, 2, 8)
    g, u = pairs[:, :, 0].reshape(rows, w), pairs[:, :, 1].reshape(rows, w)
    out.copy_((_r(_activate(g, activation), out.dtype) * u).to(out.dtype))
    return out


def gated_linear_supported(x, weight):
    return False


def gated_linear(x, weight, out, activation, bias=None):
    gate_up = torch.empty(x.shape[0], weight.shape[0], dtype=x.dtype, device=x.device)
    linear(x, weight, gate_up, bias)
    return act_mul_interleaved(gate_up, out, activation)


def linear(x, weight, out, bias=None, residual=None, activation=None):
    """The product alone: a norm that is still pending runs first, and the result is never added into `residual`
    here (the caller gets it back as the delta still to be added)."""
    if hasattr(x, "materialise"):
        x = x.materialise()
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias.float()
    if out is None:
        out = torch.empty(y.shape, dtype=x.dtype, device=x.device)
    out.copy_(y.to(out.dtype))
    if activation is not None:
        _unary(out, out, activation)
    return out


gemm_simt = linear


def rope_kv_write(qkv, positions, seq_of_token, block_table, k_pool, v_pool, inv_freq, heads, kv_heads,
                  head_dim, rotary_dim, store=True, v_head_dim=None, cos_sin_scale=1.0):
    T = qkv.shape[0]
    dtype = qkv.dtype
    page_size = k_pool.shape[2]
    v_head_dim = head_dim if v_head_dim is None else v_head_dim
    q = qkv[:, :heads * head_dim].float().view(T, heads, head_dim)
    k = qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].float().view(T, kv_heads, head_dim)
    v = qkv[:, (heads + kv_heads) * head_dim:].view(T, kv_heads, v_head_dim)
    if inv_freq is not None and rotary_dim > 0:
        half = rotary_dim // 2
        angle = positions.float()[:, None] * inv_freq.float()[None, :]
        cos, sin = angle.cos()[:, None, :] * cos_sin_scale, angle.sin()[:, None, :] * cos_sin_scale

        def rot(x):
            a, b = x[..., :half], x[..., half:rotary_dim]
            return torch.cat((a * cos - b * sin, b * cos + a * sin, x[..., rotary_dim:]), dim=-1)

        q, k = rot(q), rot(k)
        qkv[:, :heads * head_dim] = q.reshape(T, -1).to(dtype)
    if not store:
        return
    # Where each token is written: its slot, from the block tables (tokens of padding belong to no sequence).
    real = seq_of_token >= 0
    tables = block_table.tolist()
    seqs, pos = seq_of_token[real].tolist(), positions[real].tolist()
    if all(n == 1 for n in _run_lengths(seqs)):
        slots = addressing.newest_slots([tables[s] for s in seqs], pos, page_size, qkv.device)[0]
    else:
        runs = _runs(seqs, pos)
        slots = addressing.packed_addresses([tables[s] for s, _, _ in runs], [a for _, a, _ in runs],
                                            [n for _, _, n in runs], page_size, qkv.device).slots[0]
    ok = (slots >= 0) & (slots < k_pool.shape[0] * page_size)
    rows = torch.nonzero(real)[:, 0][ok]
    k_pool[slots[ok] // page_size, :, slots[ok] % page_size, :] = k.to(dtype)[rows]
    v_pool[slots[ok] // page_size, :, slots[ok] % page_size, :] = v[rows]


def _run_lengths(seqs):
    lengths, last = [], object()
    for s in seqs:
        if s == last:
            lengths[-1] += 1
        else:
            lengths.append(1)
            last = s
    return lengths


def _runs(seqs, positions):
    """(sequence, first position, count) of each run of consecutive tokens of one sequence."""
    runs = []
    for s, p in zip(seqs, positions):
        if runs and runs[-1][0] == s and runs[-1][1] + runs[-1][2] == p:
            runs[-1][2] += 1
        else:
            runs.append([s, p, 1])
    return runs


def paged_attention(q, q_row_stride, out, k_pool, v_pool, block_table, query_start_loc, context_lens, num_seqs,
                    max_q_len, heads, kv_heads, head_dim, scale, window=0, plan=None, decode_splits=None,
                    keep_first=0, softcap=0.0, sink=None):
    dtype = out.dtype
    v_dim = v_pool.shape[3]
    page_size = k_pool.shape[2]
    groups = heads // kv_heads
    qsl = query_start_loc.tolist()
    ctx = context_lens.tolist()
    qmat = q[:, :heads * head_dim].float().view(-1, heads, head_dim)
    # What each sequence reads: the slots of its whole context, from the block tables.
    slots_of = addressing.slot_table(block_table.tolist()[:num_seqs], [max(c, 0) for c in ctx[:num_seqs]], page_size,
                                     q.device)
    k_flat = k_pool.permute(0, 2, 1, 3).reshape(-1, kv_heads, head_dim)      # [slot, kv_heads, head_dim]
    v_flat = v_pool.permute(0, 2, 1, 3).reshape(-1, kv_heads, v_dim)
    for s in range(num_seqs):
        q0, q1 = qsl[s], qsl[s + 1]
        n, c = q1 - q0, ctx[s]
        if n == 0:
            continue
        first = 0 if window <= 0 or keep_first > 0 else max(0, (c - n) - window + 1)
        kpos = torch.arange(first, c, device=q.device)
        slots = slots_of[s, first:c]
        pages = torch.where(slots >= 0, slots // page_size, slots)
        keys = k_flat[slots.clamp(min=0)].float()
        vals = v_flat[slots.clamp(min=0)].float()
        keys = torch.where((slots >= 0)[:, None, None], keys, torch.zeros_like(keys))      # a page given back holds nothing
        vals = torch.where((slots >= 0)[:, None, None], vals, torch.zeros_like(vals))
        keys = keys.repeat_interleave(groups, dim=1)
        vals = vals.repeat_interleave(groups, dim=1)
        scores = torch.einsum("qhd,khd->hqk", qmat[q0:q1], keys) * scale
        if softcap > 0:
            scores = softcap * torch.tanh(scores / softcap)
        qpos = torch.arange(c - n, c, device=q.device)
        hidden = kpos[None, :] > qpos[:, None]
        if window > 0:
            hidden = hidden | ((kpos[None, :] <= qpos[:, None] - window) & (kpos[None, :] >= keep_first))
        hidden = hidden | (pages < 0)[None, :]
        scores = scores.masked_fill(hidden[None], float("-inf"))
        m = scores.amax(-1, keepdim=True)
        if sink is not None:
            m = torch.maximum(m, sink.float()[:, None, None])
        p = torch.exp(scores - m)
        denom = p.sum(-1, keepdim=True)
        if sink is not None:
            denom = denom + torch.exp(sink.float()[:, None, None] - m)
        o = torch.einsum("hqk,khd->qhd", _r(p, dtype), vals) / denom.permute(1, 0, 2)
        out[q0:q1] = o.reshape(n, heads * v_dim).to(dtype)
    return out


def convert(src, dst):
    dst.copy_(src.to(dst.dtype))
    return dst


def _norm(v, eps, centre=True):
    if centre:
        v = v - v.mean(-1, keepdim=True)
    return v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)


def layernorm(x, weight, eps, out, delta=None, rows=None, write_stream=False, centre=True):
    v = (x if rows is None else x[rows.long()]).float()
    if delta is not None:
        d = (delta.value if rows is None else delta.value[rows.long()]).float()
        v = v + delta.weight.float() * _norm(d, delta.eps, getattr(delta, "centred", True))
        if write_stream:
            x.copy_(v.to(x.dtype))
            v = x.float()
    out.copy_((weight.float() * _norm(v, eps, centre)).to(out.dtype))
    return out


def layernorm_add(stream, value, weight, eps, centred=True, out=None):
    stream.copy_((stream.float() + weight.float() * _norm(value.float(), eps, centred)).to(stream.dtype))
    if out is not None:
        out.copy_(stream.to(out.dtype))
    return stream


def projection_rmsnorm_(x, weight, eps):
    x.copy_((weight.float() * _norm(x.float(), eps, centre=False)).to(x.dtype))
    return x


def qk_projection_rmsnorm_(q, q_weight, k, k_weight, eps):
    projection_rmsnorm_(q, q_weight, eps)
    projection_rmsnorm_(k, k_weight, eps)


def gated_rmsnorm(x, gate, weight, eps, out, heads, gate_activation="silu", den=None):
    tokens, width = out.shape
    size = width // heads
    g = gate.float()
    v = x.view(tokens, heads, size)
    if den is not None:
        v = v / den.view(tokens, heads, 1)
    y = _norm(v, eps, centre=False) * weight.float().view(-1, size)
    act = torch.sigmoid(g) if gate_activation == "sigmoid" else g / (1.0 + torch.exp(-g))
    out.copy_((y.reshape(tokens, width) * act).to(out.dtype))
    return out


def head_norm_rope_kv_write(qkv, positions, seq_of_token, block_table, k_pool, v_pool, inv_freq, heads, kv_heads,
                            head_dim, rotary_dim, q_norm, k_norm, norm_eps, store=True, v_other=None, blend=None,
                            unit_norm=False, norm_after_rotation=False, cos_sin_scale=1.0):
    """Per-head norms of q and k, the blend of v, then what `rope_kv_write` does, on a compact copy of the row.
    With the norm behind the rotation, q and k are rotated here and stored unrotated-as-they-are."""
    T, dtype = qkv.shape[0], qkv.dtype
    vd = v_pool.shape[-1]
    qw, kw, vw = heads * head_dim, kv_heads * head_dim, kv_heads * vd
    q = qkv[:, :qw].float().view(T, heads, head_dim)
    k = qkv[:, qw:qw + kw].float().view(T, kv_heads, head_dim)
    v = qkv[:, qw + kw:qw + kw + vw].float()
    if norm_after_rotation and inv_freq is not None and rotary_dim > 0:
        q, k = _turn(q, positions, inv_freq, rotary_dim, cos_sin_scale), _turn(k, positions, inv_freq, rotary_dim, cos_sin_scale)
        inv_freq, rotary_dim, cos_sin_scale = None, 0, 1.0
    if q_norm is not None or unit_norm:
        q = _norm(q, norm_eps, centre=False) * (q_norm.float() if q_norm is not None else 1.0)
    if k_norm is not None or unit_norm:
        k = _norm(k, norm_eps, centre=False) * (k_norm.float() if k_norm is not None else 1.0)
    if v_other is not None:
        v = (1.0 - blend.float()) * v + blend.float() * v_other.float()
    # The norm's result is not rounded before the rotation (the kernel rounds once); float32 rows carry it over.
    compact = torch.cat([q.reshape(T, qw), k.reshape(T, kw), v], dim=1)
    wide_k = torch.empty(k_pool.shape, dtype=torch.float32, device=k_pool.device) if dtype != torch.float32 else k_pool
    wide_v = torch.empty(v_pool.shape, dtype=torch.float32, device=v_pool.device) if dtype != torch.float32 else v_pool
    if dtype != torch.float32:
        wide_k.copy_(k_pool); wide_v.copy_(v_pool)
    rope_kv_write(compact, positions, seq_of_token, block_table, wide_k, wide_v, inv_freq, heads, kv_heads, head_dim,
                  rotary_dim, store=store, v_head_dim=vd, cos_sin_scale=cos_sin_scale)
    if dtype != torch.float32:
        k_pool.copy_(wide_k); v_pool.copy_(wide_v)
    qkv[:, :qw] = compact[:, :qw].to(dtype)


def sigmoid_gate_(x, gate):
    x.copy_((x.float() * torch.sigmoid(gate.float())).to(x.dtype))
    return x


def softcap_(x, cap):
    x.copy_((cap * torch.tanh(x.float() / cap)).to(x.dtype))
    return x


def sigmoid_gate_heads_(x, gate, heads):
    tokens, width = x.shape
    y = x.float().view(tokens, heads, width // heads) * torch.sigmoid(gate.float())[:, :, None]
    x.copy_(y.reshape(tokens, width).to(x.dtype))
    return x


def mlstm(proj, offsets, i_bias, f_bias, cap, state, maxima, query_start_loc, state_slots, num_seqs, heads, dim,
          vdim, out, den, max_query_len=0):
    """state: [slots, heads, vdim + 1, dim]: the transpose of S [dim, vdim] per head, then n; maxima: a copy of m
    per column."""
    qsl, slots = query_start_loc.tolist(), state_slots.tolist()
    T = proj.shape[0]
    q_off, k_off, v_off, i_off, f_off = offsets
    q = proj[:, q_off:q_off + heads * dim].float().view(T, heads, dim) * dim ** -0.5
    k = proj[:, k_off:k_off + heads * dim].float().view(T, heads, dim)
    v = proj[:, v_off:v_off + heads * vdim].float().view(T, heads, vdim)
    gi = cap * torch.tanh((proj[:, i_off:i_off + heads].float() + i_bias) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((proj[:, f_off:f_off + heads].float() + f_bias) / cap))
    for s in range(num_seqs):
        for t in range(qsl[s], qsl[s + 1]):
            for h in range(heads):
                cols = state[slots[s], h]                       # [vdim + 1, dim]
                m = maxima[slots[s], h, 0]
                m_new = torch.maximum(gf[t, h] + m, gi[t, h])
                a, b = torch.exp(gf[t, h] + m - m_new), torch.exp(gi[t, h] - m_new)
                values = torch.cat([v[t, h], torch.ones(1)])
                cols.copy_(a * cols + b * values[:, None] * k[t, h][None, :])
                maxima[slots[s], h] = m_new
                read = cols @ q[t, h]
                out[t, h * vdim:(h + 1) * vdim] = read[:vdim]
                den[t, h] = torch.maximum(read[vdim].abs(), torch.exp(-m_new)) + 1e-6
    return out


def short_conv_step(x, taps, tail, seq_of_token, query_start_loc, state_slots, num_seqs, out, activation="silu",
                    single_tokens=False):
    short_conv(x, taps, tail, seq_of_token, query_start_loc, state_slots, out, activation)
    short_conv_update(x, tail, query_start_loc, state_slots, num_seqs)
    return out


def short_conv(x, taps, tail, seq_of_token, query_start_loc, state_slots, out, activation="silu", move_tail=False):
    K = taps.shape[0]                  # taps: [K, channels]
    qsl, slots = query_start_loc.tolist(), state_slots.tolist()
    out.zero_()
    for s in range(len(qsl) - 1):
        a, b = qsl[s], qsl[s + 1]
        if b <= a:
            continue
        padded = torch.cat([tail[slots[s]].float(), x[a:b].float()])
        acc = torch.zeros(b - a, x.shape[1], device=x.device)
        for j in range(K):
            acc = acc + padded[j:j + b - a] * taps[j].float()
        out[a:b] = (acc / (1.0 + torch.exp(-acc)) if activation == "silu" else acc).to(out.dtype)
    return out


def short_conv_update(x, tail, query_start_loc, state_slots, num_seqs):
    keep = tail.shape[1]
    qsl, slots = query_start_loc.tolist(), state_slots.tolist()
    for s in range(num_seqs):
        a, b = qsl[s], qsl[s + 1]
        if b <= a or keep == 0:
            continue
        tail[slots[s]] = torch.cat([tail[slots[s]], x[a:b].to(tail.dtype)])[-keep:]


def gated_delta_rule(qkv, ab, a_log, dt_bias, state, query_start_loc, state_slots, num_seqs, heads, kv_heads, dim,
                     vdim, out, max_query_len=0):
    """state: [slots, heads, vdim, dim], the transpose of S [dim, vdim] per head."""
    qsl, slots = query_start_loc.tolist(), state_slots.tolist()
    T = qkv.shape[0]
    qk = kv_heads * dim
    q = qkv[:, :qk].float().view(T, kv_heads, dim)
    k = qkv[:, qk:2 * qk].float().view(T, kv_heads, dim)
    v = qkv[:, 2 * qk:].float().view(T, heads, vdim)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(ab[:, :heads].float())
    decay = torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(ab[:, heads:].float() + dt_bias))
    for s in range(num_seqs):
        for t in range(qsl[s], qsl[s + 1]):
            S = state[slots[s]].transpose(1, 2)       # a view: [heads, dim, vdim]
            for h in range(heads):
                g = h // (heads // kv_heads)
                S[h] *= decay[t, h]
                u = beta[t, h] * (v[t, h] - S[h].t() @ k[t, g])
                S[h] += torch.outer(k[t, g], u)
                out[t, h * vdim:(h + 1) * vdim] = S[h].t() @ q[t, g]
    return out


def gemm_error_flag(device):
    return 0


def error_flags(device):
    return (0, 0)


def token_error_flag(device):
    return None


def argmax(logits, out):
    out.copy_(torch.argmax(logits.float(), dim=-1).to(torch.int32))
    return out


def sample_row(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, uniform: float) -> int:
    """The sampling kernel's rule for one row (liteinfer/sampling/sampler.py:50-97), in float64 where it sums."""
    logits = logits.float()
    if not temperature > 0 or top_k == 1:
        return int(torch.argmax(logits))
    x = logits / temperature
    n = x.numel()
    order = sorted(range(n), key=lambda i: (-float(x[i]), i))   # descending, equal values by index
    keep = order[:top_k] if 0 < top_k < n else order
    w = torch.exp(x - x.max()).double()
    if 0.0 < top_p < 1.0:
        total = float(sum(w[i] for i in keep))
        kept, before = [], 0.0
        for i in keep:
            if before > top_p * total:
                break
            kept.append(i)
            before += float(w[i])
        keep = kept
    keep = sorted(keep)
    total = float(sum(w[i] for i in keep))
    target, run = uniform * total, 0.0
    for i in keep:
        run += float(w[i])
        if run > target:
            return i
    return keep[-1]


def sample(logits, temperature, top_k, top_p, uniform, out):
    for r in range(logits.shape[0]):
        out[r] = sample_row(logits[r], float(temperature[r]), int(top_k[r]), float(top_p[r]), float(uniform[r]))
    return out


# ------------------------------------------------- residual streams, latent attention
def embedding_streams(ids, table, out, scale=1.0, error_flag=None):
    bad = (ids < 0) | (ids >= table.shape[0])
    rows = table[ids.long().clamp(0, table.shape[0] - 1)].float() * scale
    rows[bad] = 0
    if error_flag is not None and bool(bad.any()):
        error_flag.fill_(1)
    out.copy_(rows.repeat(1, out.shape[1] // table.shape[1]))
    return out


def stream_rmsnorm(x, weight, eps, out, read=None, update=None, rows=None, out_scale=1.0):
    width = out.shape[1] if out is not None else update.value.shape[1]
    T, S = x.shape[0], x.shape[1] // width
    streams = x.view(T, S, width)
    if update is not None:
        add = update.value.float() * (update.gain if update.gain is not None else 1.0)
        streams = torch.einsum("st,nsd->ntd", update.mix, streams) + update.write[None, :, None] * add[:, None, :]
        if rows is None:
            x.copy_(streams.reshape(T, S * width))
    if out is None:
        return None
    if rows is not None:
        streams = streams[rows.long()]
    u = streams.sum(1) if read is None else torch.einsum("s,nsd->nd", read, streams)
    out.copy_((u / torch.sqrt(u.pow(2).mean(-1, keepdim=True) + eps) * weight * out_scale).to(out.dtype))
    return out


def activation(x, out, name):
    v = x.float()
    out.copy_((torch.relu(v) ** 2 if name == "relu_squared" else _activate(v, name)).to(out.dtype))
    return out


_unary = activation


def batched_linear(x, weight, out):
    out.copy_(torch.einsum("bmk,bnk->bmn", x.float(), weight.float()).to(out.dtype))
    return out


def _turn(x, positions, inv_freq, dims, stretch=1.0):
    """Half-split rotation of the first `dims` numbers of the last axis of x [T, ..., n]; `stretch` multiplies
    every cosine and sine."""
    half = dims // 2
    angle = positions.float()[:, None] * inv_freq.float()[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = angle.cos().reshape(shape) * stretch, angle.sin().reshape(shape) * stretch
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat((a * cos - b * sin, b * cos + a * sin, x[..., dims:]), dim=-1)


def latent_prep(proj, q_off, q_rank, kv_off, kv_rank, rot_dim, rot_dims, q_weight, kv_weight, eps, inv_freq, positions,
                seq_of_token, block_table, pool, q_out, store=True, cos_sin_scale=1.0):
    dtype = proj.dtype
    page_size = pool.shape[2]
    if q_out is not None:
        q = proj[:, q_off:q_off + q_rank].float()
        q_out.copy_((q / torch.sqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_weight).to(dtype))
    if kv_off is None or not store:
        return
    latent = proj[:, kv_off:kv_off + kv_rank].float()
    latent = latent / torch.sqrt(latent.pow(2).mean(-1, keepdim=True) + eps) * kv_weight
    shared = _turn(proj[:, kv_off + kv_rank:kv_off + kv_rank + rot_dim].float(), positions, inv_freq, rot_dims,
                   cos_sin_scale)
    entries = torch.cat([latent, shared], dim=-1).to(dtype)
    tables = block_table.tolist()
    for t, (seq, pos) in enumerate(zip(seq_of_token.tolist(), positions.tolist())):
        if seq < 0:
            continue
        page = tables[seq][pos // page_size]
        if 0 <= page < pool.shape[0]:
            pool[page, 0, pos % page_size] = entries[t]


def latent_attention(q_lat, q_raw, q_head_stride, q_rot_off, out, pool, block_table, query_start_loc, context_lens,
                     inv_freq, sink, num_seqs, max_q_len, heads, kv_rank, rot_dim, rot_dims, scale, plan=None, window=0,
                     cos_sin_scale=1.0):
    dtype = out.dtype
    page_size = pool.shape[2]
    qsl, ctx = query_start_loc.tolist(), context_lens.tolist()
    slots_of = addressing.slot_table(block_table.tolist()[:num_seqs], [max(c, 0) for c in ctx[:num_seqs]], page_size,
                                     q_raw.device)
    flat = pool[:, 0].reshape(-1, kv_rank + rot_dim).float()
    tokens = q_raw.shape[0]
    q_rot_all = q_raw[:, :heads * q_head_stride].float().unflatten(1, (heads, q_head_stride))[:, :, q_rot_off:q_rot_off + rot_dim]
    for s in range(num_seqs):
        q0, q1 = qsl[s], qsl[s + 1]
        n, c = q1 - q0, ctx[s]
        if n == 0:
            continue
        qpos = torch.arange(c - n, c, device=q_raw.device)
        q_rot = _r(_turn(q_rot_all[q0:q1], qpos, inv_freq, rot_dims, cos_sin_scale), dtype)          # [n, H, r]
        q = torch.cat([q_lat[:, q0:q1].float(), q_rot.transpose(0, 1)], dim=-1)           # [H, n, c + r]
        slots = slots_of[s, :c]
        entries = flat[slots.clamp(min=0)]
        entries = torch.where((slots >= 0)[:, None], entries, torch.zeros_like(entries))    # a page given back holds nothing
        scores = torch.einsum("hqd,kd->hqk", q, entries) * scale
        kpos = torch.arange(c, device=q_raw.device)
        hidden = (kpos[None, :] > qpos[:, None]) | (slots < 0)[None, :]
        if window > 0:
            hidden = hidden | (kpos[None, :] <= qpos[:, None] - window)
        scores = scores.masked_fill(hidden[None], float("-inf"))
        m = scores.amax(-1, keepdim=True)
        if sink is not None:
            m = torch.maximum(m, sink[:, None, None])
        p = torch.exp(scores - m)
        denom = p.sum(-1, keepdim=True)
        if sink is not None:
            denom = denom + torch.exp(sink[:, None, None] - m)
        out[:, q0:q1] = (torch.einsum("hqk,kd->hqd", _r(p, dtype), entries[:, :kv_rank]) / denom).to(dtype)
    return out


def gate_heads(v, gate, out):
    heads, tokens, e = v.shape
    joined = v.float().transpose(0, 1).reshape(tokens, heads * e)
    if gate is not None:
        joined = joined * torch.sigmoid(gate.float())
    out.copy_(joined.to(out.dtype))
    return out


def moe_route(logits, top, groups, keep, renormalise, ids, weights):
    scores = torch.softmax(logits.float(), dim=-1)
    tokens, experts = scores.shape
    allowed = torch.ones_like(scores, dtype=torch.bool)
    if groups > 1:
        per = experts // groups
        best = scores.view(tokens, groups, per).amax(-1)
        kept = torch.zeros(tokens, groups, dtype=torch.bool, device=scores.device)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        allowed = kept.repeat_interleave(per, dim=1)
    chosen = torch.where(allowed, scores, torch.full_like(scores, -1.0)).topk(top, dim=-1).indices
    picked = scores.gather(1, chosen)
    if renormalise:
        picked = picked / picked.sum(-1, keepdim=True)
    ids.copy_(chosen.to(torch.int32))
    weights.copy_(picked)


def moe_router(x, weight, top, groups, keep, renormalise, ids, weights):
    moe_route(x.float() @ weight.float().t(), top, groups, keep, renormalise, ids, weights)


def moe_tile_rows(dtype, hidden, ff, pairs=None):
    return 32


class _Plan:
    def __init__(self, ids, experts):
        self.ids, self.experts = ids.reshape(-1).long(), experts
        self.order = torch.argsort(self.ids, stable=True)
        self.place = torch.argsort(self.order)


def moe_sort(ids, experts, tile_rows, with_place=False):
    return _Plan(ids, experts)


def _halves(w, eights):
    """(gate rows, up rows) of one expert's [2 * ff, hidden] matrix."""
    if not eights:
        return w[:w.shape[0] // 2], w[w.shape[0] // 2:]
    blocks = w.unflatten(0, (-1, 2, 8))
    return blocks[:, 0].flatten(0, 1), blocks[:, 1].flatten(0, 1)


def moe_experts(x, gate_up, down, ids, weights, activation, limit, alpha, eights, out):
    tokens, top = ids.shape
    plan = moe_sort(ids, gate_up.shape[0], 32)
    act = torch.empty(tokens * top, down.shape[2], dtype=x.dtype, device=x.device)
    each = torch.empty(tokens * top, down.shape[1], dtype=x.dtype, device=x.device)
    moe_grouped("gate_up", x, gate_up, act, plan, top, activation, limit, alpha, eights=eights)
    moe_grouped("down", act, down, each, plan, top, pair_weights=weights.view(-1))
    return moe_combine(each, out, top)


def moe_grouped(mode, a, weight, out, plan, top, activation="swiglu", limit=0.0, alpha=1.0, pair_weights=None,
                eights=False):
    for pair, e in enumerate(plan.ids.tolist()):
        w = weight[e].float()
        if mode == "gate_up":
            x = a[pair // top].float()
            gate, up = _halves(w, eights)
            g, u = gate @ x, up @ x
            if activation == "capped_swiglu":
                g, u = g.clamp(max=limit), u.clamp(min=-limit, max=limit)
                y = g * torch.sigmoid(alpha * g) * (u + 1.0)
            else:
                y = g * torch.sigmoid(g) * u
        else:
            y = (w @ a[pair].float()) * (1.0 if pair_weights is None else pair_weights[pair])
        out[pair] = y.to(out.dtype)
    return out


def moe_combine(y, out, top, place=None):
    rows = y if place is None else y[place.long()]
    out.copy_(rows.float().view(out.shape[0], top, -1).sum(1).to(out.dtype))
    return out


def fused_decode_supports(*args) -> bool:
    return False      # the stand-ins rotate and store in `rope_kv_write`, never inside the attention


ALL = ("moe_router", "moe_experts", "moe_route", "moe_tile_rows", "moe_sort", "moe_grouped", "moe_combine", "sigmoid_gate_", "softcap_",
       "head_norm_rope_kv_write", "sigmoid_gate_heads_", "mlstm", "embedding_streams", "stream_rmsnorm", "activation", "batched_linear", "latent_prep", "latent_attention",
       "gate_heads", "convert", "layernorm", "layernorm_add", "projection_rmsnorm_", "qk_projection_rmsnorm_", "gated_rmsnorm",
       "short_conv", "short_conv_step", "short_conv_update", "gated_delta_rule", "fused_decode_supports", "scatter_tokens", "embedding", "rmsnorm", "add_", "add_bias_", "act_mul", "act_mul_interleaved", "gated_linear_supported",
       "gated_linear", "gemm_error_flag", "error_flags", "token_error_flag", "linear", "gemm_simt", "rope_kv_write", "paged_attention", "argmax", "sample")
