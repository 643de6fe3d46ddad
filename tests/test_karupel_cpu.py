"""Karupel through the framework's step function, cache manager and engine on a CPU (stand-in kernels), against the
plain implementation of `plain_karupel.py`: every way of cutting the same requests gives the same logits."""

from __future__ import annotations

import json

import pytest
import torch

import karupel_configs as kc
import plain_karupel
import replay_harness as rh
from test_kegizen_cpu import full_trace


@pytest.fixture(scope="module")
def karupel_dirs(tmp_path_factory):
    from liteinfer_b200.weights.random_init import write_random_model

    base = tmp_path_factory.mktemp("karupel")
    return {name: write_random_model(cfg, base / name, seed) for name, (cfg, seed, _) in kc.ALL.items()}


def expected_logits(model_dir, requests):
    config, tensors = plain_karupel.read_model(model_dir)
    return {name: plain_karupel.forward(config, tensors, tokens).float() for name, tokens in requests.items()}


def test_config_round_trip_and_names(karupel_dirs):
    from liteinfer_b200.config.karupel_config import KarupelConfig
    from liteinfer_b200.config.model_config import ConfigError
    from liteinfer_b200.config.registry import resolve

    for name, (raw, _, _) in kc.ALL.items():
        arch, config = resolve(raw)
        assert arch.name == "Karupel" and KarupelConfig.from_dict(config.to_dict()) == config
        written = json.loads((karupel_dirs[name] / "config.json").read_text())
        assert KarupelConfig.from_dict(written) == config
    arch, config = resolve(kc.KAR_A)
    spec = arch.build_spec(config)
    mixes = [layer.parts["mixer"].params.get("value_mix") for layer in spec.layers]
    assert mixes == ["source", None, "mixed", None, "mixed"]
    _, tensors = plain_karupel.read_model(karupel_dirs["kar_a"])
    assert "l1.norm2" not in tensors and "l0.mix.q.norm" in tensors and "l3.mix.q.conv" in tensors
    assert "l2.mix.vmix" in tensors and tensors["l2.mix.vmix"].shape == () and "l0.mix.vmix" not in tensors
    assert "l1.mix.i.b" in tensors and "head" not in tensors
    # One layer alone that names value mixing mixes nothing.
    lone = resolve(kc.KAR_B)[0].build_spec(resolve(kc.KAR_B)[1])
    assert [layer.parts["mixer"].params.get("value_mix") for layer in lone.layers] == [None] * 4
    bad = json.loads(json.dumps(kc.KAR_A))
    bad["layers"][4]["mixer"]["vdim"] = 8           # values of another shape than the source layer's
    with pytest.raises(ConfigError):
        resolve(bad)
    bad = json.loads(json.dumps(kc.KAR_A))
    del bad["layers"][1]["mixer"]["gate_cap"]
    with pytest.raises(ConfigError):
        resolve(bad)


@pytest.mark.parametrize("name,lengths", [("kar_a", (1, 7, 61, 75)), ("kar_b", (2, 30, 45)), ("kar_c", (3, 70, 40, 18, 52)),
                                           ("kar_d", (4, 33, 58, 21))])
def test_all_cuts_match_plain_on_cpu(cpu_kernels, karupel_dirs, name, lengths):
    from liteinfer_b200.engine.loading import build_runner

    config, _, page = kc.ALL[name]
    requests = {f"r{i}": kc.prompt(config["vocab"], n, 100 + i) for i, n in enumerate(lengths)}
    expected = expected_logits(karupel_dirs[name], requests)
    trace = full_trace(requests)
    assert trace.max_live <= 4
    runner = build_runner(karupel_dirs[name], torch.float32, "cpu", page, -(-trace.max_tokens // page), 4)
    results = rh.run_in_process(runner, trace)
    worst, where = rh.worst_error(results, rh.gather_expected(trace, expected))
    assert worst < kc.FLOAT32_TOLERANCE[name], f"worst difference {worst} at step {where}"
    assert not runner.cache.live_requests
    for group in runner.cache.groups:
        assert group.allocator.num_held == 0


def test_layers_one_by_one_against_plain_on_cpu(cpu_kernels, karupel_dirs):
    """The residual stream after every layer: which layer differs first, if one does."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    for name in ("kar_a", "kar_b"):
        config, tensors = plain_karupel.read_model(karupel_dirs[name])
        tokens = kc.prompt(config["vocab"], 29, 3)
        want: list = []
        plain_karupel.forward(config, tensors, tokens, want)
        runner = build_runner(karupel_dirs[name], torch.float32, "cpu", 8, 8, 2)
        runner.cache.reserve(["a"], [29])
        context = runner.build_context([StepEntry("a", tokens, [28])])
        context.layer_trace = []
        runner.model.forward(context, runner.layer_caches)
        assert len(context.layer_trace) == len(want) == len(config["layers"])
        for stop, (got, plain) in enumerate(zip(context.layer_trace, want)):
            assert float((got.double() - plain).abs().max()) < 1e-4, f"{name}: layer {stop}"


def test_states_start_at_zero_in_a_slot_that_is_used_again(cpu_kernels, karupel_dirs):
    """A request that takes the slot of a finished one sees none of its state (S, n, the running maximum, the
    convolutions' tails)."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    config, _, page = kc.ALL["kar_b"]
    runner = build_runner(karupel_dirs["kar_b"], torch.float32, "cpu", page, 40, 1)
    first, second = kc.prompt(config["vocab"], 50, 1), kc.prompt(config["vocab"], 12, 2)
    runner.step([StepEntry("a", first, [])])
    runner.release("a")
    got = runner.step([StepEntry("b", second, list(range(12)))])
    want = expected_logits(karupel_dirs["kar_b"], {"b": second})["b"]
    assert float((got - want).abs().max()) < 5e-5


def test_greedy_generation_through_the_engine(cpu_kernels, karupel_dirs):
    """`LLM.generate` (scheduler, sampler, engine loop) on a Karupel folder picks the plain implementation's tokens."""
    from liteinfer_b200.engine.llm import LLM
    from liteinfer_b200.sampling.params import SamplingParams

    config, tensors = plain_karupel.read_model(karupel_dirs["kar_a"])
    prompts = [kc.prompt(config["vocab"], n, 40 + n) for n in (3, 26, 9)]
    llm = LLM(str(karupel_dirs["kar_a"]), dtype="float32", device="cpu", block_size=16, num_gpu_blocks=32, max_num_seqs=2,
              max_model_len=64, max_num_batched_tokens=16, enable_cuda_graphs=False)
    outputs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))
    for prompt, output in zip(prompts, outputs):
        tokens = list(prompt)
        for _ in range(6):
            tokens.append(int(plain_karupel.forward(config, tensors, tokens)[-1].argmax()))
        assert list(output.token_ids) == tokens[len(prompt):]


@pytest.mark.parametrize("kinds", [("mlstm", "delta"), ("attention",), ("delta",), ("mlstm",)])
def test_models_of_some_mixers_only(cpu_kernels, tmp_path, kinds):
    """A model without attention layers keeps no pages, one without recurrent layers no state: both run, cut every
    way, like the plain implementation."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.weights.random_init import write_random_model

    config = kc.only(kinds)
    model_dir = write_random_model(config, tmp_path / "model", 31)
    requests = {f"r{i}": kc.prompt(61, n, 7 + i) for i, n in enumerate((3, 26, 41))}
    expected = expected_logits(model_dir, requests)
    trace = full_trace(requests)
    runner = build_runner(model_dir, torch.float32, "cpu", 4, -(-trace.max_tokens // 4), 4)
    results = rh.run_in_process(runner, trace)
    worst, where = rh.worst_error(results, rh.gather_expected(trace, expected))
    assert worst < 5e-5, f"worst difference {worst} at step {where}"
