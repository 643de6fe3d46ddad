"""Karupel's kernels each against the plain torch function of the same name (`torch_kernels.py`) or a closed form,
and the whole model through `bin/trace_run` in float32 and bfloat16 against `plain_karupel.py`."""

from __future__ import annotations

import math

import pytest
import torch

import karupel_configs as kc
import plain_karupel
import replay_harness as rh
import torch_kernels as ref

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


def _cut(lengths, cuts):
    """Per step, the (begin, end) of every sequence's tokens: sequence i brings its next cuts[k][i] tokens."""
    steps, at = [], [0] * len(lengths)
    for counts in cuts:
        steps.append([(a, min(a + c, n)) for a, c, n in zip(at, counts, lengths)])
        at = [b for _, b in steps[-1]]
    assert at == list(lengths)
    return steps


# ------------------------------------------------------------------ the matrix memory
def _run_mlstm(impl, proj, lengths, cuts, slots, heads, dim, vdim, cap, i_bias, f_bias, offsets, num_slots=5):
    dev = proj[0].device
    state = torch.zeros(num_slots, heads, vdim + 1, dim, device=dev)
    maxima = torch.zeros(num_slots, heads, vdim + 1, device=dev)
    outs, dens = [[] for _ in lengths], [[] for _ in lengths]
    for step in _cut(lengths, cuts):
        rows = torch.cat([proj[i][a:b] for i, (a, b) in enumerate(step)])
        counts = [b - a for a, b in step]
        qsl = [0]
        for c in counts:
            qsl.append(qsl[-1] + c)
        out = torch.zeros(rows.shape[0], heads * vdim, device=dev)
        den = torch.zeros(rows.shape[0], heads, device=dev)
        # The longest sequence of the step is told as the engine tells it, but not for a step that is the whole run,
        # so that both ways of sizing the kernel's buffers are compared with each other.
        impl.mlstm(rows, offsets, i_bias, f_bias, cap, state, maxima, torch.tensor(qsl, dtype=torch.int32, device=dev),
                   slots.to(dev), len(lengths), heads, dim, vdim, out, den, max(counts) if len(cuts) > 1 else 0)
        for i in range(len(lengths)):
            outs[i].append(out[qsl[i]:qsl[i + 1]]); dens[i].append(den[qsl[i]:qsl[i + 1]])
    return [torch.cat(o) for o in outs], [torch.cat(d) for d in dens], state, maxima


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim", [(3, 18, 20), (1, 40, 56), (5, 4, 7), (2, 64, 32), (2, 128, 128), (1, 256, 15),
                                             (4, 32, 48), (1, 1, 1), (2, 7, 16), (1, 200, 31), (2, 256, 40),
                                             (3, 8, 24), (2, 16, 8)])
@pytest.mark.parametrize("lead", [3, 8])
def test_mlstm_in_portions_equals_whole(dtype, heads, dim, vdim, lead):
    """Whole sequences, portions (of 1, 2 and more tokens, longer than the kernel's chunk too) and steps in which a
    sequence brings nothing give the same read-outs and leave the same state, through slots out of order.  `lead`:
    the column at which q begins (8: rows and columns on 16-byte borders, which the kernel's wide loads need)."""
    from liteinfer_b200 import ops

    lengths, slots = (45, 6), _ints([3, 0])
    width = lead + 2 * heads * dim + heads * vdim + 2 * heads
    width += -width % lead
    offsets = (lead, lead + heads * dim, lead + 2 * heads * dim, width - 2 * heads, width - heads)
    proj = [_randn(n, width, seed=20 + i, dtype=dtype) for i, n in enumerate(lengths)]
    for p in proj:
        p[:, offsets[3]:] *= 4.0                                  # gates that move: the maximum changes hands
    i_bias, f_bias = _randn(heads, seed=5), _randn(heads, seed=6) + 2.0
    args = (slots, heads, dim, vdim, 7.5, i_bias, f_bias, offsets)
    whole = _run_mlstm(ops, proj, lengths, [lengths], *args)
    cuts = [(2, 1), (1, 1), (1, 0), (1, 1), (17, 0), (2, 2), (21, 1)]
    parts = _run_mlstm(ops, proj, lengths, cuts, *args)
    proj_cpu = [p.cpu() for p in proj]
    want = _run_mlstm(ref, proj_cpu, lengths, cuts, slots.cpu(), heads, dim, vdim, 7.5, i_bias.cpu(), f_bias.cpu(), offsets)
    for k in (0, 1):                                              # read-outs, denominators
        for a, b, c in zip(whole[k], parts[k], want[k]):
            torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
            torch.testing.assert_close(a.cpu(), c, rtol=2e-4, atol=2e-5)
    torch.testing.assert_close(whole[2], parts[2], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(parts[2].cpu(), want[2], rtol=2e-4, atol=2e-5)
    torch.testing.assert_close(parts[3].cpu(), want[3], rtol=1e-5, atol=1e-5)
    assert not parts[2][[1, 2, 4]].any() and not parts[3][[1, 2, 4]].any()


def _gates(raw_i, raw_f, cap):
    """The gates' logarithms of raw inputs, in float64."""
    i = cap * math.tanh(raw_i / cap)
    z = cap * math.tanh(raw_f / cap)
    return i, -math.log1p(math.exp(-z))


@pytest.mark.parametrize("decode", [False, True])
def test_mlstm_recalls_a_far_key_among_hundreds(decode):
    """Token 0 writes values along an axis that no later key touches; 400 tokens on, a query along that axis reads
    them back: exactly the values while the write's weight is above exp(-m), faded by the forget gates' product
    otherwise.  Both as a prompt and with the last 100 tokens one step each."""
    from liteinfer_b200 import ops

    dim, vdim, n, cap = 32, 16, 401, 9.0
    width = 2 * dim + vdim + 2
    offsets = (0, dim, 2 * dim, 2 * dim + vdim, 2 * dim + vdim + 1)
    values = torch.arange(1, vdim + 1, dtype=torch.float32)
    for raw_first, raw_rest, raw_forget in ((6.0, -3.0, 30.0), (1.0, 2.0, 6.0), (-4.0, -6.0, 8.0)):
        proj = torch.zeros(n, width)
        for t in range(1, n):
            proj[t, dim + 1 + (t % (dim - 1))] = 1.0           # keys along the axes 1 .. dim-1
            proj[t, 2 * dim:2 * dim + vdim] = -7.0
        proj[0, dim] = 1.0
        proj[0, 2 * dim:2 * dim + vdim] = values
        proj[:, offsets[3]] = raw_rest
        proj[0, offsets[3]] = raw_first
        proj[:, offsets[4]] = raw_forget
        proj[-1, 0] = 1.0                                      # the last query asks for axis 0
        # closed form in float64
        m, log_w = 0.0, None
        for t in range(n):
            i, f = _gates(raw_first if t == 0 else raw_rest, raw_forget, cap)
            m_new = max(f + m, i)
            log_w = i - m_new if t == 0 else log_w + f + m - m_new
            m = m_new
        weight = math.exp(log_w) * dim ** -0.5
        want = values.double() * weight / (max(weight, math.exp(-m)) + 1e-6)
        proj = proj.to(DEV)
        cuts = [(n - 100,)] + [(1,)] * 100 if decode else [(n,)]
        zero = torch.zeros(1, device=DEV)
        outs, dens, _, _ = _run_mlstm(ops, [proj], (n,), cuts, _ints([1]), 1, dim, vdim, cap, zero, zero, offsets, 2)
        got = outs[0][-1].double().cpu() / dens[0][-1].double().cpu()
        torch.testing.assert_close(got, want, rtol=3e-4, atol=1e-9)
        assert float(want.abs().max()) > 1e-6                  # the case means something


def test_mlstm_first_token_meets_a_maximum_of_zero():
    """The running maximum starts at 0: a first token whose input gate lies far below 0 is weighted exp(i - f), not
    1, and the denominator's floor is exp(-f), not exp(-i)."""
    from liteinfer_b200 import ops

    dim, vdim, cap = 8, 4, 20.0
    offsets = (0, dim, 2 * dim, 2 * dim + vdim, 2 * dim + vdim + 1)
    proj = torch.zeros(1, 2 * dim + vdim + 2, device=DEV)
    proj[0, 0] = proj[0, dim] = 2.0
    proj[0, 2 * dim:2 * dim + vdim] = torch.tensor([1.0, -2.0, 3.0, 0.5])
    proj[0, offsets[3]], proj[0, offsets[4]] = -9.0, 3.0
    i, f = _gates(-9.0, 3.0, cap)
    assert f > i
    zero = torch.zeros(1, device=DEV)
    outs, dens, state, maxima = _run_mlstm(ops, [proj], (1,), [(1,)], _ints([0]), 1, dim, vdim, cap, zero, zero, offsets, 1)
    write = math.exp(i - f)
    dot = write * 4.0 * dim ** -0.5
    torch.testing.assert_close(outs[0][0].cpu().double(), proj[0, 2 * dim:2 * dim + vdim].cpu().double() * dot, rtol=1e-5, atol=1e-9)
    assert abs(float(dens[0][0, 0]) - (max(dot, math.exp(-f)) + 1e-6)) < 1e-5
    assert abs(float(maxima[0, 0, 0]) - f) < 1e-6 and abs(float(state[0, 0, vdim, 0]) - 2.0 * write) < 1e-8


# ------------------------------------------------------------------ norms and gates
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,size,per_head,activation", [(3, 20, True, "sigmoid"), (2, 128, False, "sigmoid"),
                                                             (5, 1, True, "silu"), (1, 48, True, "sigmoid"), (7, 44, True, "sigmoid"),
                                                             (2, 256, False, "silu"), (1, 512, True, "sigmoid"),
                                                             (3, 260, True, "silu"), (2, 516, False, "sigmoid")])
def test_gated_rmsnorm_with_divisor_and_weights_per_head(dtype, heads, size, per_head, activation):
    """The gate is a column slice of a wider tensor: with rows of 9 more elements than the heads it lies on no
    16-byte border (the element-by-element kernel), with 12 more it does (the kernel that keeps a head's row in
    registers, for heads of up to 512)."""
    from liteinfer_b200 import ops

    x = _randn(13, heads * size, seed=1, scale=2.0)
    weight = 1 + 0.2 * _randn(heads * size if per_head else size, seed=3)
    den = _randn(13, heads, seed=4).abs() + 0.05
    for spare in (9, 12):
        wide = _randn(13, heads * size + spare, seed=2, dtype=dtype)
        for d in (None, den):
            out, want = (torch.empty(13, heads * size, dtype=dtype, device=DEV) for _ in range(2))
            ops.gated_rmsnorm(x, wide[:, 4:4 + heads * size], weight, 1e-5, out, heads, gate_activation=activation, den=d)
            ref.gated_rmsnorm(x, wide[:, 4:4 + heads * size], weight, 1e-5, want, heads, gate_activation=activation, den=d)
            torch.testing.assert_close(out.float(), want.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 80, 257, 2048, 12288])
def test_output_norm_adds_into_a_32_bit_stream_and_hands_it_back_rounded(dtype, width):
    """stream += w * value / rms(value) with w in 32-bit (1 + the stored weight, which bfloat16 would round), the
    sum in 32-bit, and the rounded sum for the next sublayer's products."""
    from liteinfer_b200 import ops

    stream = _randn(9, width, seed=3, scale=3.0) + 1.5
    value = _randn(9, width, seed=4, scale=0.3, dtype=dtype) - 0.4
    weight = 1.0 + 0.001 * _randn(width, seed=5)                    # 32-bit: bfloat16 cannot tell these from 1
    got, want = stream.clone(), stream.clone()
    out, out_want = (torch.empty(9, width, dtype=dtype, device=DEV) for _ in range(2))
    ops.layernorm_add(got, value, weight, 1e-5, centred=False, out=None if dtype == torch.float32 else out)
    ref.layernorm_add(want, value, weight, 1e-5, centred=False, out=out_want)
    torch.testing.assert_close(got, want, rtol=2e-6, atol=2e-6)
    if dtype != torch.float32:
        assert torch.equal(out, got.to(dtype))
    rounded = stream.clone()
    ref.layernorm_add(rounded, value, weight.to(torch.bfloat16).float(), 1e-5, centred=False)
    assert float((rounded - want).abs().max()) > 50 * float((got - want).abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_sigmoid_gate_heads(dtype):
    from liteinfer_b200 import ops

    for heads, size in ((4, 24), (1, 64), (7, 3), (8, 48), (3, 128), (5, 4)):
        x = _randn(11, heads * size, seed=1, dtype=dtype)
        wide = _randn(11, heads + 5, seed=2, scale=3.0, dtype=dtype)
        want = x.clone()
        ref.sigmoid_gate_heads_(want, wide[:, 2:2 + heads], heads)
        ops.sigmoid_gate_heads_(x, wide[:, 2:2 + heads], heads)
        torch.testing.assert_close(x.float(), want.float(), **_tol(dtype))


# ------------------------------------------------------------------ attention's preparation
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,v_dim,rot,norms,mix", [
    (4, 2, 24, 16, 12, True, True), (2, 2, 16, 16, 16, True, False), (6, 2, 8, 16, 4, True, True),
    (3, 1, 20, 28, 0, True, False), (4, 2, 64, 64, 64, True, True), (2, 1, 64, 48, 32, False, True),
    (8, 8, 128, 128, 64, True, True), (1, 1, 40, 7, 2, True, True), (5, 1, 32, 32, 16, "q", True),
    (3, 3, 256, 64, 128, "k", True), (2, 1, 128, 8, 0, True, False)])
@pytest.mark.parametrize("lead", [3, 8])
def test_head_norm_rotation_value_blend_and_store(dtype, heads, kv_heads, head_dim, v_dim, rot, norms, mix, lead):
    """Per-head norms of q and k (or of one of them) before the rotation of the first `rot` dimensions, the blend of v
    with another layer's values, and the pages: against the plain function, with a row of padding and pages out of
    order.  `lead`: where the other layer's values begin in their rows (8: on a 16-byte border, so the kernel that
    moves 16 bytes a thread runs where the sizes allow it; 3: the kernel for any layout)."""
    from liteinfer_b200 import ops

    page, tokens = 8, 21
    inv_freq = None
    if rot:
        inv_freq = (500.0 ** (-torch.arange(0, rot, 2, dtype=torch.float32) / rot) / 3.0).to(DEV)
    width = (heads + kv_heads) * head_dim + kv_heads * v_dim
    qkv = _randn(tokens, width + 16, seed=1, scale=1.5, dtype=dtype)
    other_wide = _randn(tokens, kv_heads * v_dim + 16, seed=2, dtype=dtype)
    other = other_wide[:, lead:lead + kv_heads * v_dim] if mix else None
    blend = torch.tensor([0.37], device=DEV) if mix else None
    qw, kw = (1 + 0.3 * _randn(head_dim, seed=3)).to(dtype), (1 + 0.3 * _randn(head_dim, seed=4)).to(dtype)
    positions, seq_of = _ints(list(range(30, 30 + tokens - 1)) + [0]), _ints([0] * (tokens - 1) + [-1])
    table = _ints([[4, 2, 9, 0, 7, 1, 3]])
    pools = [(torch.zeros(10, kv_heads, page, head_dim, dtype=dtype, device=DEV),
              torch.zeros(10, kv_heads, page, v_dim, dtype=dtype, device=DEV)) for _ in range(2)]
    got, want = qkv.clone(), qkv.clone()
    args = (inv_freq, heads, kv_heads, head_dim, rot, qw if norms in (True, "q") else None,
            kw if norms in (True, "k") else None, 1e-5)
    ops.head_norm_rope_kv_write(got, positions, seq_of, table, *pools[0], *args, v_other=other, blend=blend)
    ref.head_norm_rope_kv_write(want, positions, seq_of, table, *pools[1], *args, v_other=other, blend=blend)
    q_width = heads * head_dim
    torch.testing.assert_close(got[:-1, :q_width].float(), want[:-1, :q_width].float(), **_tol(dtype))
    torch.testing.assert_close(pools[0][0].float(), pools[1][0].float(), **_tol(dtype))
    torch.testing.assert_close(pools[0][1].float(), pools[1][1].float(), **_tol(dtype))
    assert torch.equal(got[:, width:], qkv[:, width:])                     # what rides behind v (the gate) is left alone
    assert not pools[0][0][[5, 6, 8]].any()                                # pages of nobody
    if mix:                                                                # the stored values are blended, 37 to 63
        plain = qkv[:-1, q_width + kv_heads * head_dim:width].float()
        blended = 0.63 * plain + 0.37 * other[:-1].float()
        slot, at = int(table[0, 30 // page]), 30 % page
        torch.testing.assert_close(pools[0][1][slot, :, at].float().reshape(-1), blended[0], **_tol(dtype))


# ------------------------------------------------------------------ the whole model
@pytest.fixture(scope="module")
def karupel_dirs(tmp_path_factory):
    from liteinfer_b200.weights.random_init import write_random_model

    base = tmp_path_factory.mktemp("karupel")
    return {name: write_random_model(cfg, base / name, seed) for name, (cfg, seed, _) in kc.ALL.items()}


def _expected(model_dir, requests):
    config, tensors = plain_karupel.read_model(model_dir)
    return {name: plain_karupel.forward(config, tensors, tokens).float() for name, tokens in requests.items()}


@pytest.mark.parametrize("name,lengths", [("kar_a", (1, 7, 61, 90)), ("kar_b", (2, 30, 45)), ("kar_c", (5, 52, 150, 18, 210)),
                                           ("kar_d", (4, 33, 58, 21)), ("kar_e", (300, 17, 420))])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_all_cuts(karupel_dirs, tmp_path, name, lengths, dtype):
    """Whole, the tail decoded, portions down to two tokens, four live requests whose pages and slots are used
    again, and every token a step of its own from the first one on: the same logits as the plain implementation."""
    config, _, page = kc.ALL[name]
    requests = {f"r{i}": kc.prompt(config["vocab"], n, 100 + i) for i, n in enumerate(lengths)}
    expected = _expected(karupel_dirs[name], requests)
    trace = rh.Trace()
    rh.whole(trace, requests)
    rh.tail_decoded(trace, requests, tail=40)
    rh.portions(trace, requests)
    rh.mixed(trace, requests)
    longest = max(requests, key=lambda r: len(requests[r]))
    for i, token in enumerate(requests[longest]):
        trace.add([(f"o-{longest}", [token], [0])], end=[f"o-{longest}"] if i == len(requests[longest]) - 1 else [])
    results = rh.run_program(trace, karupel_dirs[name], dtype, tmp_path / "out", config["vocab"], page_size=page)
    worst, where = rh.worst_error(results, rh.gather_expected(trace, expected))
    limit = 2 * kc.FLOAT32_TOLERANCE[name] if dtype == "float32" else kc.BFLOAT16_TOLERANCE[name]
    assert worst < limit, f"worst difference {worst} at step {where}"
    if dtype == "bfloat16" and name in kc.BFLOAT16_TYPICAL:
        rows = []
        for got, want in zip(results, rh.gather_expected(trace, expected)):
            if want is not None:
                diff = got.double() - want.double()
                diff -= diff.mean(dim=1, keepdim=True)
                rows.append(diff.pow(2).mean(dim=1).sqrt() / want.double().std())
        typical = float(torch.cat(rows).median())
        assert typical < kc.BFLOAT16_TYPICAL[name], f"typical relative difference {typical}"


@pytest.mark.parametrize("kinds", [("mlstm", "delta"), ("attention",)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_models_of_some_mixers_only(tmp_path, kinds, dtype):
    """A model without attention layers keeps no pages, one without recurrent layers no state: both run through the
    trace runner, whole, in portions and token by token, like the plain implementation."""
    from liteinfer_b200.weights.random_init import write_random_model

    model_dir = write_random_model(kc.only(kinds), tmp_path / "model", 31)
    requests = {f"r{i}": kc.prompt(61, n, 7 + i) for i, n in enumerate((3, 26, 41))}
    expected = _expected(model_dir, requests)
    trace = rh.Trace()
    rh.whole(trace, requests)
    rh.tail_decoded(trace, requests, tail=40)
    rh.portions(trace, requests)
    rh.mixed(trace, requests)
    results = rh.run_program(trace, model_dir, dtype, tmp_path / "out", 61, page_size=4)
    worst, where = rh.worst_error(results, rh.gather_expected(trace, expected))
    assert worst < (1e-4 if dtype == "float32" else 0.08), f"worst difference {worst} at step {where}"


def test_layers_one_by_one_against_plain(karupel_dirs):
    """The residual stream after every layer (32-bit engine) equals the plain implementation's."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    for name in ("kar_a", "kar_b", "kar_c"):
        config, tensors = plain_karupel.read_model(karupel_dirs[name])
        tokens = kc.prompt(config["vocab"], 45, 3)
        want: list = []
        plain_karupel.forward(config, tensors, tokens, want)
        runner = build_runner(karupel_dirs[name], torch.float32, DEV, 16, 8, 2)
        runner.cache.reserve(["a"], [45])
        context = runner.build_context([StepEntry("a", tokens, [44])])
        context.layer_trace = []
        runner.model.forward(context, runner.layer_caches)
        assert len(context.layer_trace) == len(want) == len(config["layers"])
        for stop, (got, plain) in enumerate(zip(context.layer_trace, want)):
            assert float((got.cpu().double() - plain).abs().max()) < 2e-4, f"{name}: layer {stop}"


def test_bfloat16_engine_keeps_the_stream_and_states_32_bit(karupel_dirs):
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    runner = build_runner(karupel_dirs["kar_a"], torch.bfloat16, DEV, 16, 8, 2)
    tokens = kc.prompt(kc.KAR_A["vocab"], 20, 3)
    runner.cache.reserve(["a"], [20])
    context = runner.build_context([StepEntry("a", tokens, [19])])
    context.layer_trace = []
    runner.model.forward(context, runner.layer_caches)
    assert all(t.dtype == torch.float32 for t in context.layer_trace)
    kinds = {name: pool.dtype for cache in runner.layer_caches for name, pool in cache.states.items()}
    assert kinds["mlstm"] == kinds["mlstm_max"] == kinds["delta"] == torch.float32 and kinds["conv"] == torch.bfloat16


def test_greedy_generation_through_the_engine_on_gpu(karupel_dirs):
    """`LLM.generate` (scheduler with portions of 16 tokens, three seats for five requests, CUDA graphs, sampler)
    picks the plain implementation's tokens over 24 decoded tokens."""
    from liteinfer_b200.engine.llm import LLM
    from liteinfer_b200.sampling.params import SamplingParams

    config, tensors = plain_karupel.read_model(karupel_dirs["kar_b"])
    prompts = [kc.prompt(config["vocab"], n, 40 + n) for n in (3, 26, 9, 14, 2)]
    with LLM(str(karupel_dirs["kar_b"]), dtype="float32", block_size=4, num_gpu_blocks=96, max_num_seqs=3,
             max_model_len=80, max_num_batched_tokens=16) as llm:
        outputs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24))
    for prompt, output in zip(prompts, outputs):
        tokens = list(prompt)
        for _ in range(24):
            tokens.append(int(plain_karupel.forward(config, tensors, tokens)[-1].argmax()))
        assert list(output.token_ids) == tokens[len(prompt):]
