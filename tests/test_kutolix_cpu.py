"""Kutolix through the framework's step function, cache manager and engine on a CPU (stand-in kernels), against the
plain implementation of `plain_kutolix.py`: every way of cutting the same requests gives the same logits.  And the
plain implementation's mechanisms on inputs made so that a fault would show."""

from __future__ import annotations

import json
import math

import pytest
import torch

import kutolix_configs as kc
import plain_kutolix
import replay_harness as rh
from test_kegizen_cpu import full_trace


@pytest.fixture(scope="module")
def kutolix_dirs(tmp_path_factory):
    from liteinfer_b200.weights.random_init import write_random_model

    base = tmp_path_factory.mktemp("kutolix")
    return {name: write_random_model(cfg, base / name, seed) for name, (cfg, seed, _) in kc.ALL.items() if name != "kut_e"}


def expected_logits(model_dir, requests):
    config, tensors = plain_kutolix.read_model(model_dir)
    return {name: plain_kutolix.forward(config, tensors, tokens).float() for name, tokens in requests.items()}


def test_config_round_trip_and_names(kutolix_dirs):
    from liteinfer_b200.config.kutolix_config import KutolixConfig
    from liteinfer_b200.config.model_config import ConfigError
    from liteinfer_b200.config.registry import resolve

    for name, (raw, _, _) in kc.ALL.items():
        arch, config = resolve(raw)
        assert arch.name == "Kutolix" and KutolixConfig.from_dict(config.to_dict()) == config
        if name in kutolix_dirs:
            written = json.loads((kutolix_dirs[name] / "config.json").read_text())
            assert KutolixConfig.from_dict(written) == config
    arch, config = resolve(kc.KUT_B)
    assert config.embedding_scale == 1.0 and config.residual_mult == 1.0 and config.logit_softcap is None
    assert config.layers[0].mixer.window is None and config.layers[2].mixer.window == 1 and config.layers[2].mixer.rot is None
    assert config.layers[0].mlp.groups == 1 and config.layers[2].mlp is None
    spec = arch.build_spec(config)
    assert [layer.block for layer in spec.layers] == ["output_norm", "output_norm", "output_norm_mixer_only", "output_norm"]
    _, tensors = plain_kutolix.read_model(kutolix_dirs["kut_a"])
    assert tensors["l0.mix.dkv"].shape == (24 + 8, 64) and tensors["l0.mix.dkv.norm"].shape == (24,)
    assert tensors["l1.mix.sink"].shape == (4,) and tensors["l1.mix.g"].shape == (4 * 12, 64)
    assert tensors["l0.mlp.router"].shape == (6, 64) and tensors["l0.mlp.e5.down"].shape == (64, 20)
    assert "l2.norm2" not in tensors and "head" not in tensors and "l3.mlp.e3.gate" in tensors
    for path, value in ((("layers", 0, "mixer", "kv_rank"), None), (("layers", 0, "mlp", "router", "top"), 5),
                        (("layers", 0, "mlp", "router", "groups", "count"), 4), (("layers", 1, "mixer", "kv_heads"), 3),
                        (("layers", 0, "mixer", "rot", "scaling", "original"), None), (("norm", "eps"), None)):
        bad = json.loads(json.dumps(kc.KUT_A))
        at = bad
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            resolve(bad)


@pytest.mark.parametrize("name,lengths", [("kut_a", (1, 7, 61, 75)), ("kut_b", (2, 30, 45)), ("kut_c", (3, 150, 40, 18, 80)),
                                           ("kut_d", (4, 33, 58, 21))])
def test_all_cuts_match_plain_on_cpu(cpu_kernels, kutolix_dirs, name, lengths):
    """Whole, the tail decoded, portions down to two tokens, four live requests with pages used again, every token a
    step of its own: windows pass over prompts and decoded tokens, pages behind a window are given back."""
    from liteinfer_b200.engine.loading import build_runner

    config, _, page = kc.ALL[name]
    requests = {f"r{i}": kc.prompt(config["vocab"], n, 100 + i) for i, n in enumerate(lengths)}
    expected = expected_logits(kutolix_dirs[name], requests)
    trace = full_trace(requests)
    assert trace.max_live <= 4
    runner = build_runner(kutolix_dirs[name], torch.float32, "cpu", page, -(-trace.max_tokens // page), 4)
    results = rh.run_in_process(runner, trace)
    worst, where = rh.worst_error(results, rh.gather_expected(trace, expected))
    assert worst < kc.FLOAT32_TOLERANCE[name], f"worst difference {worst} at step {where}"
    assert not runner.cache.live_requests
    for group in runner.cache.groups:
        assert group.allocator.num_held == 0


def test_layers_one_by_one_against_plain_on_cpu(cpu_kernels, kutolix_dirs):
    """The residual stream after every layer: which layer differs first, if one does."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    for name in ("kut_a", "kut_b", "kut_d"):
        config, tensors = plain_kutolix.read_model(kutolix_dirs[name])
        tokens = kc.prompt(config["vocab"], 29, 3)
        want: list = []
        plain_kutolix.forward(config, tensors, tokens, want)
        runner = build_runner(kutolix_dirs[name], torch.float32, "cpu", 8, 8, 2)
        runner.cache.reserve(["a"], [29])
        context = runner.build_context([StepEntry("a", tokens, [28])])
        context.layer_trace = []
        runner.model.forward(context, runner.layer_caches)
        assert len(context.layer_trace) == len(want) == len(config["layers"])
        for stop, (got, plain) in enumerate(zip(context.layer_trace, want)):
            assert float((got.double() - plain).abs().max()) < 1e-4, f"{name}: layer {stop}"


def test_windowed_layers_give_pages_back_while_a_request_runs(cpu_kernels, kutolix_dirs):
    """A model whose every layer has a window holds, however long the request grows, only the pages its widest
    window reaches; the pool is smaller than the request."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    config, _, _ = kc.ALL["kut_a"]
    tokens = kc.prompt(config["vocab"], 120, 5)
    want = expected_logits(kutolix_dirs["kut_a"], {"a": tokens})["a"]
    runner = build_runner(kutolix_dirs["kut_a"], torch.float32, "cpu", 4, 20, 1)      # 80 slots a group for 120 tokens
    got = []
    for at in range(0, 120, 10):
        got.append(runner.step([StepEntry("a", tokens[at:at + 10], list(range(10)))]))
    assert float((torch.cat(got) - want).abs().max()) < 5e-5
    assert max(group.allocator.num_held for group in runner.cache.groups) <= 12


def test_greedy_generation_through_the_engine(cpu_kernels, kutolix_dirs):
    """`LLM.generate` (scheduler, sampler, engine loop) on a Kutolix folder picks the plain implementation's tokens."""
    from liteinfer_b200.engine.llm import LLM
    from liteinfer_b200.sampling.params import SamplingParams

    config, tensors = plain_kutolix.read_model(kutolix_dirs["kut_a"])
    prompts = [kc.prompt(config["vocab"], n, 40 + n) for n in (3, 26, 9)]
    llm = LLM(str(kutolix_dirs["kut_a"]), dtype="float32", device="cpu", block_size=16, num_gpu_blocks=32, max_num_seqs=2,
              max_model_len=64, max_num_batched_tokens=16, enable_cuda_graphs=False)
    outputs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))
    for prompt, output in zip(prompts, outputs):
        tokens = list(prompt)
        for _ in range(6):
            tokens.append(int(plain_kutolix.forward(config, tensors, tokens)[-1].argmax()))
        assert list(output.token_ids) == tokens[len(prompt):]


# ------------------------------------------------------------- the plain mechanisms, on inputs that show a fault
def test_plain_window_and_sink_on_a_planted_key():
    """One key's score stands out: the query finds it just inside the window, not just outside; a sink as large as
    that score halves the result."""
    T, D, window = 40, 8, 11
    g = torch.Generator().manual_seed(0)
    q = 0.01 * torch.randn(T, 1, D, generator=g, dtype=torch.float64)
    k = 0.01 * torch.randn(T, 1, D, generator=g, dtype=torch.float64)
    v = torch.randn(T, 1, 4, generator=g, dtype=torch.float64)
    planted = 20
    k[planted, 0] = 0.0
    k[planted, 0, 0] = 30.0
    q[:, 0, 0] = 1.0
    out = plain_kutolix.windowed_softmax_attention(q, k, v, 1.0, window)
    assert torch.allclose(out[planted + window - 1, 0], v[planted, 0], atol=1e-9)        # the last query that sees it
    assert not torch.allclose(out[planted + window, 0], v[planted, 0], atol=0.1)         # the first that does not
    assert torch.allclose(out[planted - 1, 0], v[planted - window:planted, 0].mean(0), atol=1e-2)
    halved = plain_kutolix.windowed_softmax_attention(q, k, v, 1.0, window, sink=torch.tensor([30.0], dtype=torch.float64))
    assert torch.allclose(halved[planted + 3, 0], v[planted, 0] / 2, atol=1e-9)


def test_plain_router_keeps_the_best_groups_and_does_not_renormalise():
    w = {"p.router": torch.eye(6, dtype=torch.float64)}
    h = torch.tensor([[3.0, 0.0, 0.1, 0.2, 2.5, 2.4]], dtype=torch.float64)     # groups (0,1) (2,3) (4,5)
    chosen, weights = plain_kutolix.route(h, w, "p.", {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}})
    scores = torch.softmax(h, -1)[0]
    assert chosen[0].tolist() == [0, 4, 5] and torch.allclose(weights[0], scores[[0, 4, 5]])
    assert float(weights.sum()) < 1.0
    chosen, _ = plain_kutolix.route(h, w, "p.", {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 1}})
    assert sorted(chosen[0].tolist()) == [0, 1, 3] or sorted(chosen[0].tolist())[:2] == [0, 1]   # only group (0,1) is open
    chosen, _ = plain_kutolix.route(h, w, "p.", {"experts": 6, "top": 3})
    assert chosen[0].tolist() == [0, 4, 5]


def test_plain_yarn_frequencies_and_pairing():
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}}
    f, stretch = plain_kutolix.frequencies(rot)
    plain = [100.0 ** (-2.0 * i / 8) for i in range(4)]
    assert math.isclose(stretch, 0.1 * math.log(4.0) + 1.0)
    assert math.isclose(float(f[0]), plain[0]) and math.isclose(float(f[3]), plain[3] / 4.0)   # fast pairs keep, slow ones stretch
    x = torch.arange(1.0, 9.0, dtype=torch.float64).view(1, 1, 8).repeat(3, 1, 1)
    near = plain_kutolix.rotate(x, {"dims": 4, "base": 10.0}, "interleaved")[2, 0]
    half = plain_kutolix.rotate(x, {"dims": 4, "base": 10.0}, "half")[2, 0]
    a = 2.0      # position 2, frequency 1
    assert math.isclose(float(near[0]), 1 * math.cos(a) - 2 * math.sin(a)) and math.isclose(float(near[1]), 2 * math.cos(a) + 1 * math.sin(a))
    assert math.isclose(float(half[0]), 1 * math.cos(a) - 3 * math.sin(a)) and math.isclose(float(half[2]), 3 * math.cos(a) + 1 * math.sin(a))
    assert near[4:].tolist() == half[4:].tolist() == [5.0, 6.0, 7.0, 8.0]


def test_plain_expert_caps_its_products():
    w = {"e.gate": torch.tensor([[10.0], [-10.0]], dtype=torch.float64), "e.up": torch.tensor([[10.0], [-10.0]], dtype=torch.float64),
         "e.down": torch.eye(2, dtype=torch.float64)}
    y = plain_kutolix.expert_ff(torch.ones(1, 1, dtype=torch.float64), w, "e.", 2.0)[0]
    assert math.isclose(float(y[0]), 2.0 / (1 + math.exp(-1.702 * 2.0)) * 3.0)          # gate capped at 2, up at 2, + 1
    assert math.isclose(float(y[1]), -10.0 / (1 + math.exp(17.02)) * (-2.0 + 1.0))      # the gate has no lower cap
