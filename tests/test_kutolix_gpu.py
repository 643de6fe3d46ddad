"""Kutolix's kernels each against the plain torch function of the same name (`torch_kernels.py`), the plain
mechanisms of `plain_kutolix.py` or a closed form, and the whole model through `bin/trace_run` in float32 and
bfloat16 against `plain_kutolix.py`."""

from __future__ import annotations

import pytest
import torch

import kutolix_configs as kc
import plain_kutolix
import replay_harness as rh
import torch_kernels as ref
from test_gifudra_gpu import _attention_inputs, _batch, _plan
from test_kernels_gpu import _paged_case, _plan_for

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2 ** -6, atol=2 ** -6)


def _randn(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(dtype)


def _ints(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ small kernels
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,lead", [(48, 3), (512, 8), (20, 0)])
def test_elementwise_gate_and_soft_cap(dtype, width, lead):
    from liteinfer_b200 import ops

    x = _randn(9, width, seed=1, dtype=dtype)
    wide = _randn(9, lead + width + 5, seed=2, scale=3.0, dtype=dtype)
    gate = wide[:, lead:lead + width]
    want = (x.float() * torch.sigmoid(gate.float())).to(dtype)
    torch.testing.assert_close(ops.sigmoid_gate_(x.clone(), gate).float(), want.float(), **_tol(dtype))
    logits = _randn(5, 333, seed=3, scale=20.0, dtype=dtype)
    want = (7.5 * torch.tanh(logits.float() / 7.5)).to(dtype)
    got = ops.softcap_(logits.clone(), 7.5)
    torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))
    assert float(got.float().abs().max()) <= 7.5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,v_dim,rot,weights,after,lead", [
    (4, 2, 16, 12, 4, False, True, 0), (3, 3, 6, 10, 2, False, True, 3), (8, 2, 128, 128, 64, False, True, 0),
    (2, 1, 64, 64, 64, True, True, 8), (2, 2, 24, 8, 24, True, False, 0), (4, 4, 128, 64, 0, False, False, 0)])
def test_unit_norm_behind_the_rotation(dtype, heads, kv_heads, head_dim, v_dim, rot, weights, after, lead):
    """q and k divided by their root mean square per head, without a weight or with one, in front of the rotation
    or behind it; against the plain twin and, for the unit norm behind the rotation, against the plain mechanism."""
    from liteinfer_b200 import ops

    page = 8
    table, positions, seq_of, _, _ = _batch([5, 1, 3], [9, 14, 3], page, 12)
    width = (heads + kv_heads) * head_dim + kv_heads * v_dim
    rows = [_randn(9, lead + width + 5, seed=1, dtype=dtype)[:, lead:] for _ in range(2)]
    inv_freq = (100.0 ** (-torch.arange(rot // 2, dtype=torch.float64) * 2 / max(rot, 1))).float().to(DEV) if rot else None
    qn = (1 + 0.2 * _randn(head_dim, seed=2)).to(dtype) if weights else None
    kn = (1 + 0.2 * _randn(head_dim, seed=3)).to(dtype) if weights else None
    pools = [[torch.zeros(12, kv_heads, page, n, dtype=dtype, device=DEV) for n in (head_dim, v_dim)] for _ in range(2)]
    options = dict(unit_norm=not weights, norm_after_rotation=after)
    if weights and rot:
        options["cos_sin_scale"] = 1.3          # stretched cosines and sines: the rotation then changes a head's norm
    for impl, qkv, (kp, vp) in ((ops, rows[0], pools[0]), (ref, rows[1], pools[1])):
        impl.head_norm_rope_kv_write(qkv, positions, seq_of, table, kp, vp, inv_freq, heads, kv_heads, head_dim, rot,
                                     qn, kn, 1e-5, **options)
    torch.testing.assert_close(rows[0][:, :heads * head_dim].float(), rows[1][:, :heads * head_dim].float(), **_tol(dtype))
    torch.testing.assert_close(pools[0][0].float(), pools[1][0].float(), **_tol(dtype))
    torch.testing.assert_close(pools[0][1].float(), pools[1][1].float(), **_tol(dtype))
    if not weights and rot:
        fresh = _randn(9, lead + width + 5, seed=1, dtype=dtype)[:, lead:]
        q = fresh[:, :heads * head_dim].double().cpu().view(9, heads, head_dim)
        for t in (0, 5, 8):
            turned = plain_kutolix.rotate(q[t:t + 1].repeat(int(positions[t]) + 1, 1, 1), {"dims": rot, "base": 100.0}, "half")[-1]
            want = plain_kutolix.unit_rms(turned, 1e-5)
            got = rows[0][t, :heads * head_dim].double().cpu().view(heads, head_dim)
            torch.testing.assert_close(got, want, rtol=_tol(dtype)["rtol"] * 2, atol=_tol(dtype)["atol"] * 2)


# ------------------------------------------------------------------ the sink, on every attention kernel
def _sink_case(dtype, heads, kv_heads, d, page, q_lens, ctx_lens):
    from liteinfer_b200 import ops

    case = _paged_case(dtype, heads, kv_heads, d, page, q_lens, ctx_lens)
    ops.rope_kv_write(case["qkv"], case["positions"], case["seq_of"], case["table"], case["k_pool"], case["v_pool"], None,
                      heads, kv_heads, d, 0)
    return case, (case["k_pool"], case["v_pool"], case["table"], case["qsl"], case["ctx"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,d,page,window", [(4, 2, 16, 16, 0), (6, 3, 48, 8, 7), (3, 1, 32, 4, 37), (2, 2, 80, 16, 1)])
def test_sink_on_the_plain_kernel(dtype, heads, kv_heads, d, page, window):
    from liteinfer_b200 import ops

    q_lens, ctx_lens = [1, 33, 1, 7, 2], [90, 50, 1, 7, 45]
    case, rest = _sink_case(dtype, heads, kv_heads, d, page, q_lens, ctx_lens)
    sink = _randn(heads, seed=9, scale=2.0)
    tail = (case["B"], max(q_lens), heads, kv_heads, d, 0.3, window)
    out = lambda: torch.empty(case["T"], heads * d, dtype=dtype, device=DEV)
    want = ref.paged_attention(case["qkv"], case["qkv"].shape[1], out(), *rest, *tail, sink=sink)
    got = ops.paged_attention(case["qkv"], case["qkv"].shape[1], out(), *rest, *tail, sink=sink)
    torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))
    without = ops.paged_attention(case["qkv"], case["qkv"].shape[1], out(), *rest, *tail)
    assert float((got.float() - without.float()).abs().max()) > 1e-2        # the sink is felt


@pytest.mark.parametrize("heads,kv_heads,d,page", [(4, 2, 64, 16), (8, 2, 128, 16), (5, 1, 64, 32), (16, 16, 128, 64)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("splits", [None, 1, 3, 13])
def test_sink_on_the_tensor_core_kernels(heads, kv_heads, d, page, window, splits):
    """tcgen05 over prompts and portions, the streaming kernel over single tokens (keys unsplit and split over
    blocks that merge), and the mma.sync kernel in both roles: the sink joins every row's denominator once."""
    from liteinfer_b200 import ops

    dtype = torch.bfloat16
    q_lens, ctx_lens = [1, 130, 1, 7, 64, 1, 257], [700, 190, 1, 7, 64, 129, 300]
    case, rest = _sink_case(dtype, heads, kv_heads, d, page, q_lens, ctx_lens)
    sink = _randn(heads, seed=9, scale=2.0)
    tail = (case["B"], max(q_lens), heads, kv_heads, d, d ** -0.5, window)
    out = lambda: torch.full((case["T"], heads * d), float("nan"), dtype=dtype, device=DEV)
    want = ref.paged_attention(case["qkv"], case["qkv"].shape[1], out(), *rest, *tail, sink=sink)
    plan = _plan_for(q_lens, ctx_lens)
    got = ops.paged_attention(case["qkv"], case["qkv"].shape[1], out(), *rest, *tail, plan=plan, decode_splits=splits, sink=sink)
    torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))
    # The mma.sync kernel alone, prompts and single tokens in one unsplit launch, and split single tokens.
    alone = ops.paged_attention_mma(case["qkv"], case["qkv"].shape[1], out(), *rest, None, *tail, sink=sink)
    torch.testing.assert_close(alone.float(), want.float(), **_tol(dtype))
    if splits and splits > 1:
        part = out()
        ops.paged_attention_mma(case["qkv"], case["qkv"].shape[1], part, *rest, plan.decode_seqs, plan.num_decode, 1,
                                heads, kv_heads, d, d ** -0.5, window, splits, sink=sink)
        rows = plan.decode_tokens.long()
        torch.testing.assert_close(part[rows].float(), want[rows].float(), **_tol(dtype))
    assert ops.gemm_error_flag(DEV) == 0


@pytest.mark.parametrize("d,page", [(64, 16), (128, 16), (48, 8)])
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_stands_out_against_a_sink_at_the_windows_edge(d, page, decode):
    """One key's score is lifted far above all others.  Just inside the window the query reads that key's value, and
    a sink as large as the lifted score halves the result; just outside the window the key is not seen."""
    from liteinfer_b200 import ops

    dtype, heads, kv_heads, ctx, window = torch.bfloat16, 4, 2, 520, 200
    n = 1 if decode else 9
    qpos = ctx - 1
    for target in (qpos - window + 1, qpos - window, qpos, qpos - 64, qpos - 128):
        case, rest = _sink_case(dtype, heads, kv_heads, d, page, [n], [ctx])
        k_pool, v_pool, table = case["k_pool"], case["v_pool"], case["table"]
        k_pool.mul_(0.05)
        lifted = _randn(d, seed=3)
        k_pool[int(table[0, target // page]), :, target % page] = lifted.to(dtype)
        case["qkv"][-1, :heads * d] = (lifted * 3.0).to(dtype).repeat(heads)
        found = v_pool[int(table[0, target // page]), :, target % page].float().repeat_interleave(heads // kv_heads, 0)
        tail = (1, n, heads, kv_heads, d, 1.0, window)
        plan = _plan_for([n], [ctx])
        out = lambda: torch.empty(n, heads * d, dtype=dtype, device=DEV)
        got = ops.paged_attention(case["qkv"], case["qkv"].shape[1], out(), *rest, *tail, plan=plan,
                                  sink=torch.full((heads,), -50.0, device=DEV))[-1].float().view(heads, d)
        if target > qpos - window:
            torch.testing.assert_close(got, found, rtol=3e-2, atol=3e-2)
            score = float((case["qkv"][-1, :d].float() * k_pool[int(table[0, target // page]), 0, target % page].float()).sum())
            halved = ops.paged_attention(case["qkv"], case["qkv"].shape[1], out(), *rest, *tail, plan=plan,
                                         sink=torch.full((heads,), score, device=DEV))[-1].float().view(heads, d)
            torch.testing.assert_close(halved, 0.5 * found, rtol=4e-2, atol=4e-2)
        else:
            assert float((got - found).abs().max()) > 0.3


# ------------------------------------------------------------------ latent attention: window and stretch
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,c,r,dims,d,page,window", [(3, 40, 10, 6, 12, 4, 13), (1, 24, 2, 2, 5, 8, 1), (6, 96, 32, 32, 16, 16, 50),
                                                          (16, 64, 32, 32, 32, 16, 45), (9, 128, 64, 64, 8, 64, 100)])
def test_latent_attention_with_a_window_and_stretched_rotation(dtype, heads, c, r, dims, d, page, window):
    from liteinfer_b200 import ops

    query_lens, context_lens = [17, 1, 2, 1, 40], [17, 70, 2 * page + 2, 1, 40 + 3 * page]
    pages = sum(-(-n // page) for n in context_lens) + 3
    table, qsl, ctxl, pool, q_lat, q_raw = _attention_inputs(dtype, heads, c, r, d, query_lens, context_lens, page, pages, 5)
    inv_freq = (1000.0 ** (-torch.arange(dims // 2, dtype=torch.float64) * 2 / dims)).float().to(DEV)
    args = (q_lat, q_raw, d + r, d)
    rest = (pool, table, qsl, ctxl, inv_freq, None, 5, 40, heads, c, r, dims, 0.11)
    for plan in (None, _plan(query_lens, context_lens)):
        got = ops.latent_attention(*args, torch.zeros_like(q_lat), *rest, plan=plan, window=window, cos_sin_scale=1.14)
        want = ref.latent_attention(*args, torch.empty_like(q_lat), *rest, window=window, cos_sin_scale=1.14)
        torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))
    unwindowed = ref.latent_attention(*args, torch.empty_like(q_lat), *rest, cos_sin_scale=1.14)
    assert float((want.float() - unwindowed.float()).abs().max()) > 1e-2


@pytest.mark.parametrize("heads,c,r,page", [(16, 64, 32, 16), (20, 128, 64, 16), (5, 512, 64, 32)])
@pytest.mark.parametrize("window", [33, 64, 500])
def test_latent_window_on_tensor_cores(heads, c, r, page, window):
    """Portions beside single tokens whose keys several blocks share, windows shorter and longer than a round of
    keys, contexts far longer than the window (the pages behind it are gone: their table entries are -1)."""
    from liteinfer_b200 import ops

    dtype, d = torch.bfloat16, 8
    assert ops.latent_mma_supports(dtype, c, r, r)
    query_lens, context_lens = [1, 37, 1, 6, 1, 130, 1], [900, 37, 1, 70, 65, 130 + 2 * page + 3, 1500]
    pages = sum(-(-n // page) for n in context_lens) + 3
    table, qsl, ctxl, pool, q_lat, q_raw = _attention_inputs(dtype, heads, c, r, d, query_lens, context_lens, page, pages, 7)
    for s, (n, total) in enumerate(zip(query_lens, context_lens)):      # what a window has passed is given back
        gone = max(0, total - n - window + 1) // page
        if gone:
            pool[table[s, :gone].long()] = float("nan")
            table[s, :gone] = -1
    inv_freq = (1000.0 ** (-torch.arange(r // 2, dtype=torch.float64) * 2 / r)).float().to(DEV)
    common = (q_lat, q_raw, d + r, d)
    rest = (pool, table, qsl, ctxl, inv_freq, None, 7, 130, heads, c, r, r, 0.09)
    want = ref.latent_attention(*common, torch.empty_like(q_lat), *rest, window=window, cos_sin_scale=0.9)
    planned = ops.latent_attention(*common, torch.zeros_like(q_lat), *rest, plan=_plan(query_lens, context_lens),
                                   window=window, cos_sin_scale=0.9)
    unplanned = ops.latent_attention(*common, torch.zeros_like(q_lat), *rest, window=window, cos_sin_scale=0.9)
    torch.testing.assert_close(planned.float(), want.float(), **_tol(dtype))
    torch.testing.assert_close(unplanned.float(), want.float(), **_tol(dtype))
    assert ops.gemm_error_flag(DEV) == 0


@pytest.mark.parametrize("dtype,c,r", [(torch.float32, 48, 8), (torch.bfloat16, 48, 8), (torch.bfloat16, 64, 32)])
@pytest.mark.parametrize("decode", [False, True])
def test_latent_key_just_inside_and_just_outside_the_window(dtype, c, r, decode):
    from liteinfer_b200 import ops

    heads, d, page, ctx, window = 3, 6, 16, 700, 150
    n = 1 if decode else 9
    plan = _plan([n], [ctx]) if c == 64 else None
    pages = -(-ctx // page) + 2
    inv_freq = (1000.0 ** (-torch.arange(r // 2, dtype=torch.float64) * 2 / r)).float().to(DEV)
    qpos = ctx - 1
    for target in (qpos - window + 1, qpos - window, qpos - window - 1, qpos, qpos - 31, qpos - 32):
        table, qsl, ctxl, pool, q_lat, q_raw = _attention_inputs(dtype, heads, c, r, d, [n], [ctx], page, pages, 11)
        pool.mul_(0.05)
        entry_page, slot = int(table[0, target // page]), target % page
        lifted = torch.zeros(c + r, device=DEV)
        lifted[:c] = _randn(c, seed=3)
        pool[entry_page, 0, slot] = lifted.to(dtype)
        q_lat[:, -1] = (lifted[:c] * 3.0).to(dtype)
        out = ops.latent_attention(q_lat, q_raw, d + r, d, torch.empty_like(q_lat), pool, table, qsl, ctxl, inv_freq,
                                   None, 1, n, heads, c, r, r, 1.0, plan=plan, window=window)
        found = pool[entry_page, 0, slot, :c].float()
        if target > qpos - window:
            torch.testing.assert_close(out[:, -1].float(), found.expand(heads, c), rtol=2e-2, atol=2e-2)
        else:
            assert float(out[:, -1].float().abs().max()) < 0.2


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_prep_without_a_query_latent_and_with_stretch(dtype):
    from liteinfer_b200 import ops

    c, r, dims, page = 40, 10, 6, 4
    table, positions, seq_of, _, _ = _batch([5, 1, 3], [9, 14, 3], page, 12)
    proj = _randn(9, 100, seed=1, dtype=dtype)
    wkv = 1 + 0.2 * _randn(c, seed=3)
    inv_freq = (100.0 ** (-torch.arange(dims // 2, dtype=torch.float64) * 2 / dims)).float().to(DEV)
    pools = [torch.full((12, 1, page, c + r), 7.0, dtype=dtype, device=DEV) for _ in range(2)]
    args = (0, 0, 27, c, r, dims, None, wkv, 1e-5, inv_freq, positions, seq_of, table)
    ops.latent_prep(proj, *args, pools[0], None, cos_sin_scale=1.2)
    ref.latent_prep(proj, *args, pools[1], None, cos_sin_scale=1.2)
    torch.testing.assert_close(pools[0].float(), pools[1].float(), **_tol(dtype))
    # The rotated part of one entry against the plain mechanism with the neighbours' pairs brought into halves.
    t, pos = 5, 13
    shared = proj[t, 27 + c:27 + c + r].double().cpu()
    order = list(range(0, dims, 2)) + list(range(1, dims, 2)) + list(range(dims, r))
    inverse = [order.index(i) for i in range(r)]
    near = shared[inverse].view(1, 1, r).repeat(pos + 1, 1, 1)        # what a checkpoint with neighbour pairs would hold
    turned = plain_kutolix.rotate(near, {"dims": dims, "base": 100.0}, "interleaved")[-1, 0][order] * 1.2
    turned[dims:] = shared[dims:]
    entry = pools[0][int(table[1, pos // page]), 0, pos % page, c:].double().cpu()
    torch.testing.assert_close(entry, turned, rtol=_tol(dtype)["rtol"] * 2, atol=_tol(dtype)["atol"] * 2)


# ------------------------------------------------------------------ the mixture of experts
@pytest.mark.parametrize("experts,top,groups,keep", [(6, 2, 3, 2), (12, 4, 4, 2), (8, 2, 4, 1), (64, 6, 8, 3), (5, 2, 1, 1),
                                                      (3, 1, 1, 1), (256, 8, 8, 4), (4, 4, 2, 2)])
@pytest.mark.parametrize("renormalise", [False, True])
def test_router_against_the_plain_mechanism(experts, top, groups, keep, renormalise):
    from liteinfer_b200 import ops

    tokens = 77
    logits = _randn(tokens, experts, seed=experts, scale=2.0)
    ids = torch.empty(tokens, top, dtype=torch.int32, device=DEV)
    weights = torch.empty(tokens, top, device=DEV)
    ops.moe_route(logits, top, groups, keep, renormalise, ids, weights)
    router = {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}
    chosen, scores = plain_kutolix.route(logits.double().cpu(), {"p.router": torch.eye(experts, dtype=torch.float64)}, "p.", router)
    if renormalise:
        scores = scores / scores.sum(-1, keepdim=True)
    assert torch.equal(ids.cpu().long().sort(-1).values, chosen.sort(-1).values)
    torch.testing.assert_close(weights.cpu().double().sort(-1).values, scores.sort(-1).values, rtol=1e-5, atol=1e-6)
    assert torch.equal(ids.cpu().long(), chosen)            # the largest first, as the plain top-k orders them
    # The router's product and the routing in one launch, in both dtypes and both widths of block, rows of a slice.
    for dtype in DTYPES:
        for count in (tokens, 300):
            wide = _randn(count, 3 + 40 + 2, seed=5, dtype=dtype)
            x, w = wide[:, 3:43], _randn(experts, 40, seed=6, scale=0.7)
            ops.moe_route(x.float() @ w.t(), top, groups, keep, renormalise,
                          want_ids := torch.empty(count, top, dtype=torch.int32, device=DEV), want_w := torch.empty(count, top, device=DEV))
            got_ids, got_w = torch.empty_like(want_ids), torch.empty_like(want_w)
            ops.moe_router(x, w, top, groups, keep, renormalise, got_ids, got_w)
            same = (got_ids == want_ids).all(-1)
            assert float(same.float().mean()) > 0.97            # (a close call may fall the other way: the sums' order differs)
            torch.testing.assert_close(got_w[same], want_w[same], rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,hidden,ff,experts,top", [(1, 64, 20, 6, 2), (9, 36, 10, 8, 2), (70, 128, 64, 8, 2), (300, 128, 64, 4, 4),
                                                           (33, 48, 16, 3, 1), (200, 512, 256, 8, 2), (5, 40, 7, 5, 2)])
def test_grouped_expert_products(dtype, tokens, hidden, ff, experts, top):
    """Sort, both grouped products and the combination against the experts run pair by pair: experts with no token,
    with one, with more than a tile; sizes that take the mma.sync tiles and sizes that do not."""
    from liteinfer_b200 import ops

    x = _randn(tokens, hidden, seed=1, dtype=dtype)
    gate_up = _randn(experts, 2 * ff, hidden, seed=2, scale=hidden ** -0.5, dtype=dtype)
    down = _randn(experts, hidden, ff, seed=3, scale=ff ** -0.5, dtype=dtype)
    g = torch.Generator().manual_seed(4)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(tokens)]).to(torch.int32)
    if top == 1 and experts > 2:
        ids[ids == 1] = 0                                           # expert 1 gets no token at all
    ids = ids.to(DEV)
    weights = torch.rand(tokens, top, generator=g).to(DEV)
    pairs = tokens * top
    tile = ops.moe_tile_rows(dtype, hidden, ff)
    assert tile == (64 if dtype == torch.bfloat16 and hidden % 8 == 0 and ff % 8 == 0 else 32)
    assert ops.moe_tile_rows(dtype, hidden, ff, 10) == (128 if tile == 64 else tile)      # a step's pairs: the tcgen05 kernel where it fits
    results = []
    for impl, plan in ((ops, ops.moe_sort(ids, experts, tile)), (ref, ref.moe_sort(ids, experts, tile))):
        act = torch.zeros(pairs, ff, dtype=dtype, device=DEV)
        impl.moe_grouped("gate_up", x, gate_up, act, plan, top, "capped_swiglu", 1.2, 1.702)
        each = torch.zeros(pairs, hidden, dtype=dtype, device=DEV)
        impl.moe_grouped("down", act, down, each, plan, top, pair_weights=weights.view(-1))
        results.append((act, each, impl.moe_combine(each, torch.empty(tokens, hidden, dtype=dtype, device=DEV), top)))
    for got, want in zip(*results):
        torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))
    plan = ops.moe_sort(ids, experts, tile)
    counts = torch.bincount(ids.view(-1).long(), minlength=experts)
    assert torch.equal(plan.offsets.long().diff(), counts)
    assert torch.equal(ids.view(-1)[plan.order.long()].long(), torch.repeat_interleave(torch.arange(experts, device=DEV), counts))
    assert int((plan.tile_expert >= 0).sum()) == int(((counts + tile - 1) // tile).sum())
    plain = ops.moe_grouped("gate_up", x, gate_up, torch.zeros(pairs, ff, dtype=dtype, device=DEV), plan, top, "swiglu")
    want = ref.moe_grouped("gate_up", x, gate_up, torch.zeros(pairs, ff, dtype=dtype, device=DEV), ref.moe_sort(ids, experts, tile), top, "swiglu")
    torch.testing.assert_close(plain.float(), want.float(), **_tol(dtype))


@pytest.mark.parametrize("tokens,hidden,ff,experts,top", [(300, 128, 64, 4, 4), (200, 512, 256, 8, 2), (2048, 256, 384, 16, 4),
                                                           (700, 136, 40, 5, 3), (130, 64, 128, 3, 1)])
def test_expert_products_on_the_tcgen05_kernel(tokens, hidden, ff, experts, top, monkeypatch):
    """The whole of `moe_experts` with the pairs' rows gathered expert by expert and both products on the tcgen05
    kernel (tiles of 128 rows, experts with no row, one row, more than a tile; widths that are no multiple of the
    kernel's tiles), against the mma.sync tiles and the plain twin."""
    from liteinfer_b200 import ops
    from liteinfer_b200.ops import kernels

    dtype = torch.bfloat16
    x = _randn(tokens, hidden, seed=1, dtype=dtype)
    gate = _randn(experts, ff, hidden, seed=2, scale=hidden ** -0.5, dtype=dtype)
    up = _randn(experts, ff, hidden, seed=5, scale=hidden ** -0.5, dtype=dtype)
    eights = torch.stack([gate.unflatten(1, (-1, 8)), up.unflatten(1, (-1, 8))], dim=2).flatten(1, 3).contiguous()
    down = _randn(experts, hidden, ff, seed=3, scale=ff ** -0.5, dtype=dtype)
    g = torch.Generator().manual_seed(4)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(tokens)]).to(torch.int32)
    if top == 1:
        ids[ids == 1] = 0
    ids = ids.to(DEV)
    weights = torch.rand(tokens, top, generator=g).to(DEV)
    out = lambda: torch.empty(tokens, hidden, dtype=dtype, device=DEV)
    want = ref.moe_experts(x, eights, down, ids, weights, "capped_swiglu", 1.2, 1.702, True, out())
    monkeypatch.setattr(kernels, "MOE_TCGEN05_MIN_PAIRS", 1)
    assert ops.moe_tile_rows(dtype, hidden, ff, tokens * top) == 128
    got = ops.moe_experts(x, eights, down, ids, weights, "capped_swiglu", 1.2, 1.702, True, out())
    torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))
    monkeypatch.setattr(kernels, "MOE_TCGEN05", False)
    tiles = ops.moe_experts(x, eights, down, ids, weights, "capped_swiglu", 1.2, 1.702, True, out())
    torch.testing.assert_close(tiles.float(), want.float(), **_tol(dtype))
    halves = ops.moe_experts(x, torch.cat([gate, up], dim=1).contiguous(), down, ids, weights, "swiglu", 0.0, 1.0, False, out())
    plain = ref.moe_experts(x, torch.cat([gate, up], dim=1), down, ids, weights, "swiglu", 0.0, 1.0, False, out())
    torch.testing.assert_close(halves.float(), plain.float(), **_tol(dtype))
    assert ops.gemm_error_flag(DEV) == 0


def test_router_gives_every_row_an_expert_whatever_it_holds():
    """A row of padding may hold anything (what an attention that found no work left in its output): NaN and
    infinities still choose experts inside the table, so that nothing behind the router reads out of bounds."""
    from liteinfer_b200 import ops

    experts, top = 12, 3
    x = _randn(9, 64, seed=1, dtype=torch.bfloat16)
    x[2], x[5, 7], x[6] = float("nan"), float("inf"), float("-inf")
    ids = torch.full((9, top), -7, dtype=torch.int32, device=DEV)
    weights = torch.empty(9, top, device=DEV)
    ops.moe_router(x, _randn(experts, 64, seed=2), top, 3, 2, False, ids, weights)
    assert int(ids.min()) >= 0 and int(ids.max()) < experts
    logits = _randn(9, experts, seed=3)
    logits[1], logits[4, 2] = float("nan"), float("inf")
    ops.moe_route(logits, top, 3, 2, False, ids, weights)
    assert int(ids.min()) >= 0 and int(ids.max()) < experts


def test_expert_rows_do_not_depend_on_the_batch():
    """A token's expert outputs are the same bits whatever else is in the step (32-bit)."""
    from liteinfer_b200 import ops

    hidden, ff, experts, top = 48, 16, 4, 2
    x = _randn(40, hidden, seed=1)
    gate_up, down = _randn(experts, 2 * ff, hidden, seed=2, scale=0.2), _randn(experts, hidden, ff, seed=3, scale=0.2)
    ids = torch.stack([torch.randperm(experts)[:top] for _ in range(40)]).to(torch.int32).to(DEV)

    def run(rows):
        plan = ops.moe_sort(ids[rows].contiguous(), experts, 32)
        act = ops.moe_grouped("gate_up", x[rows].contiguous(), gate_up, torch.zeros(len(rows) * top, ff, device=DEV), plan, top)
        return ops.moe_grouped("down", act, down, torch.zeros(len(rows) * top, hidden, device=DEV), plan, top)

    whole = run(list(range(40)))
    assert torch.equal(run([7])[0], whole[7 * top]) and torch.equal(run([3, 7, 39])[2 * top + 1], whole[39 * top + 1])


# ------------------------------------------------------------------ the whole model
@pytest.fixture(scope="module")
def kutolix_dirs(tmp_path_factory):
    from liteinfer_b200.weights.random_init import write_random_model

    base = tmp_path_factory.mktemp("kutolix")
    return {name: write_random_model(cfg, base / name, seed) for name, (cfg, seed, _) in kc.ALL.items()}


def _expected(model_dir, requests):
    config, tensors = plain_kutolix.read_model(model_dir)
    return {name: plain_kutolix.forward(config, tensors, tokens).float() for name, tokens in requests.items()}


@pytest.mark.parametrize("name,lengths", [("kut_a", (1, 7, 61, 90)), ("kut_b", (2, 30, 45)), ("kut_c", (5, 52, 150, 18, 210)),
                                           ("kut_d", (4, 33, 58, 21)), ("kut_e", (300, 17, 420))])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_all_cuts(kutolix_dirs, tmp_path, name, lengths, dtype):
    """Whole, the tail decoded, portions down to two tokens, four live requests whose pages are used again, and every
    token a step of its own from the first one on: the same logits as the plain implementation."""
    config, _, page = kc.ALL[name]
    requests = {f"r{i}": kc.prompt(config["vocab"], n, 100 + i) for i, n in enumerate(lengths)}
    expected = _expected(kutolix_dirs[name], requests)
    trace = rh.Trace()
    rh.whole(trace, requests)
    rh.tail_decoded(trace, requests, tail=40)
    rh.portions(trace, requests)
    rh.mixed(trace, requests)
    longest = max(requests, key=lambda r: len(requests[r]))
    for i, token in enumerate(requests[longest]):
        trace.add([(f"o-{longest}", [token], [0])], end=[f"o-{longest}"] if i == len(requests[longest]) - 1 else [])
    results = rh.run_program(trace, kutolix_dirs[name], dtype, tmp_path / "out", config["vocab"], page_size=page)
    wanted = rh.gather_expected(trace, expected)
    if dtype == "float32":
        worst, where = rh.worst_error(results, wanted)
        assert worst < 2 * kc.FLOAT32_TOLERANCE[name], f"worst difference {worst} at step {where}"
        return
    # bfloat16: a router's close call may choose another expert than the 64-bit run does, at a position here and
    # there; every other position is held to the rounding's size, and so is the typical one.
    rows = torch.cat([(got.double() - want.double()).abs().amax(dim=1) for got, want in zip(results, wanted) if want is not None])
    assert float(rows.median()) < kc.BFLOAT16_TOLERANCE[name] / 4, f"typical difference {float(rows.median())}"
    assert float((rows > kc.BFLOAT16_TOLERANCE[name]).double().mean()) < 0.02, f"worst difference {float(rows.max())}"


@pytest.mark.parametrize("seed", [3, 11, 12, 16])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    """Layer orders, sizes and options drawn at random, every way of cutting, against the plain implementation.  In
    32-bit no router's choice is close enough to fall the other way, so every position is held to rounding; in
    bfloat16 (where the sizes drawn bring in the tensor-core kernels) the typical position is."""
    from liteinfer_b200.weights.random_init import write_random_model

    config = kc.random_config(seed)
    model_dir = write_random_model(config, tmp_path / "model", seed)
    requests = {f"r{i}": kc.prompt(config["vocab"], n, 7 + i) for i, n in enumerate((1, 23, 150, 240))}
    expected = _expected(model_dir, requests)
    trace = rh.Trace()
    rh.whole(trace, requests)
    rh.tail_decoded(trace, requests, tail=40)
    rh.portions(trace, requests)
    rh.mixed(trace, requests)
    results = rh.run_program(trace, model_dir, dtype, tmp_path / "out", config["vocab"], page_size=16)
    wanted = rh.gather_expected(trace, expected)
    if dtype == "float32":
        worst, where = rh.worst_error(results, wanted)
        assert worst < 2e-4, f"worst difference {worst} at step {where}"
        return
    rows = []
    for got, want in zip(results, wanted):
        if want is not None:
            diff = got.double() - want.double()
            diff -= diff.mean(dim=1, keepdim=True)
            rows.append(diff.pow(2).mean(dim=1).sqrt() / want.double().std())
    typical = float(torch.cat(rows).median())
    assert typical < 0.03, f"typical relative difference {typical}"


def test_layers_one_by_one_against_plain(kutolix_dirs):
    """The residual stream after every layer (32-bit engine) equals the plain implementation's."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    for name in ("kut_a", "kut_b", "kut_c", "kut_d"):
        config, tensors = plain_kutolix.read_model(kutolix_dirs[name])
        tokens = kc.prompt(config["vocab"], 45, 3)
        want: list = []
        plain_kutolix.forward(config, tensors, tokens, want)
        runner = build_runner(kutolix_dirs[name], torch.float32, DEV, 16, 8, 2)
        runner.cache.reserve(["a"], [45])
        context = runner.build_context([StepEntry("a", tokens, [44])])
        context.layer_trace = []
        runner.model.forward(context, runner.layer_caches)
        assert len(context.layer_trace) == len(want) == len(config["layers"])
        for stop, (got, plain) in enumerate(zip(context.layer_trace, want)):
            assert float((got.cpu().double() - plain).abs().max()) < 2e-4, f"{name}: layer {stop}"


def test_bfloat16_engine_keeps_the_stream_and_the_router_32_bit(kutolix_dirs):
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    runner = build_runner(kutolix_dirs["kut_a"], torch.bfloat16, DEV, 16, 8, 2)
    tokens = kc.prompt(kc.KUT_A["vocab"], 20, 3)
    runner.cache.reserve(["a"], [20])
    context = runner.build_context([StepEntry("a", tokens, [19])])
    context.layer_trace = []
    runner.model.forward(context, runner.layer_caches)
    assert all(t.dtype == torch.float32 for t in context.layer_trace)
    experts = runner.model.layers[0].parts["feed_forward"]
    assert experts.router.dtype == torch.float32 and experts.gate_up.dtype == torch.bfloat16
    assert runner.model.layers[1].parts["mixer"].sink.dtype == torch.float32


def test_greedy_generation_through_the_engine_on_gpu(kutolix_dirs):
    """`LLM.generate` (scheduler with portions of 16 tokens, three seats for five requests, CUDA graphs, sampler)
    picks the plain implementation's tokens over 24 decoded tokens, the windows passing over decoded tokens."""
    from liteinfer_b200.engine.llm import LLM
    from liteinfer_b200.sampling.params import SamplingParams

    config, tensors = plain_kutolix.read_model(kutolix_dirs["kut_d"])
    prompts = [kc.prompt(config["vocab"], n, 40 + n) for n in (3, 26, 9, 14, 2)]
    with LLM(str(kutolix_dirs["kut_d"]), dtype="float32", block_size=4, num_gpu_blocks=96, max_num_seqs=3,
             max_model_len=80, max_num_batched_tokens=16) as llm:
        outputs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24))
    for prompt, output in zip(prompts, outputs):
        tokens = list(prompt)
        for _ in range(24):
            tokens.append(int(plain_kutolix.forward(config, tensors, tokens)[-1].argmax()))
        assert list(output.token_ids) == tokens[len(prompt):]
