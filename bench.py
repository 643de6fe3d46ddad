"""Headline benchmark: decode tokens/s of the Llama 3.2 1B shape on one B200, with prefill and roofline figures.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 with every
sequence near the benchmark context (4,096), timed on the device over K decode
steps of the engine's own step function and sampler.  `e2e` is the same measured
through the Python entry point (`LLM.generate`: host token ids in, host token
ids out; every step its inputs travel from pinned host memory to the device, read
in place by the kernel that stages the batch, and the sampled tokens travel back
to the host).  `prefill` times one 2,048-token prompt,
`roofline` relates the decode step to the bytes it must read, `points` holds
decode at batch 1 and 64.  Weights are random (seeded) and token ids synthetic.

`--compare kegizen` prints another line instead (the default run is unchanged): prefill and decode of the Kegizen
decoder beside the Llama decoder at equal layer sizes, and the Kegizen kernels one by one beside their like.
`--compare gifudra` does the same for the Gifudra decoder (latent attention, residual streams).
`--compare karupel` sets the Karupel decoder (mLSTM, delta-rule and gated attention layers) beside a Kegizen decoder of
the same sizes, its closest relative, and its kernels beside their like.
`--compare kutolix` sets the Kutolix decoder (windowed gated attention with a sink, windowed latent attention, dense
and routed feed-forwards) beside a Gifudra decoder of the same sizes, and its kernels beside their like.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 128256, "hidden_size": 2048, "intermediate_size": 8192,
    "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "max_position_embeddings": 131072, "hidden_act": "silu",
}
# The other shapes of the reference's configurations, for `--shape` (the default run and the contract are the 1B shape).
LLAMA_3B = dict(LLAMA_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, head_dim=128)
LLAMA_8B = dict(LLAMA_1B, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, head_dim=128,
                tie_word_embeddings=False,
                rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                              "original_max_position_embeddings": 8192})
SHAPES = {"1b": ("Llama 3.2 1B", LLAMA_1B, 4096), "3b": ("Llama 3.2 3B", LLAMA_3B, 4096),
          "8b": ("Llama 3.1 8B", LLAMA_8B, 8192)}
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = 16
# A40 decode step of the reference at batch 8 (docs/benchmarks.md:749-753: 6.41 ms -> 1,248 tok/s).
BASELINE_DECODE_B8_TOKS = 1248.0


def _find_number(tree, key: str):
    """The first number stored under `key` anywhere in a JSON tree (the file's layout is the driver's)."""
    if isinstance(tree, dict):
        value = tree.get(key)
        if isinstance(value, (int, float)) and not isinstance(value, bool):
            return float(value)
        if isinstance(value, dict):
            for inner in ("value", "median", "mean"):
                if isinstance(value.get(inner), (int, float)):
                    return float(value[inner])
        for child in tree.values():
            found = _find_number(child, key)
            if found is not None:
                return found
    elif isinstance(tree, list):
        for child in tree:
            found = _find_number(child, key)
            if found is not None:
                return found
    return None


def measured_peaks() -> dict:
    """Copy bandwidth (GB/s) and bfloat16 product throughput (TFLOP/s) to measure against: the driver's
    measurements if it left them, else the stated fallback.  `bf16_tflops_burst` is the library product timed
    alone, `bf16_tflops` the same held for seconds under the power cap; a prefill step of a few milliseconds
    timed alone is measured against the burst figure."""
    fallback = {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "bf16_tflops_burst": 1590.0, "source": "fallback"}
    path = ROOT / "MEASURED_PEAKS.json"
    if not path.is_file():
        return fallback
    try:
        raw = json.loads(path.read_text())
    except (OSError, ValueError):
        return fallback
    hbm = _find_number(raw, "hbm_gbs")
    burst = _find_number(raw, "bf16_tflops")
    flops = _find_number(raw, "bf16_tflops_sustained") or burst
    if hbm is not None and hbm < 100:          # given in TB/s
        hbm *= 1000.0
    if flops is not None and flops > 100000:   # given in GFLOP/s
        flops, burst = flops / 1000.0, (burst or flops) / 1000.0
    if not hbm or not flops:
        return fallback
    return {"hbm_gbs": hbm, "bf16_tflops": flops, "bf16_tflops_burst": burst or flops, "source": "measured"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self._proc = None

    def start(self) -> None:
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self._proc = None

    def _read(self) -> None:
        for line in self._proc.stdout:
            self.samples.append([f.strip() for f in line.split(",")])

    def stop(self) -> dict:
        if self._proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self._proc.terminate()
        rows = [s for s in self.samples if len(s) >= 6 and s[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in rows), "sm_max_mhz": int(rows[0][1]),
                "reasons": reasons, "samples": len(rows)}


def _fill_cache(runner, ids: list[str], lengths: list[int]) -> None:
    """Gives every request `length` tokens of cache without computing them: pages are taken through the
    cache manager and hold small random values (a decode step's time does not depend on what they are)."""
    runner.cache.reserve(ids, lengths)
    for request_id, n in zip(ids, lengths):
        runner.cache.commit(request_id, n)


def _decode_rate(runner, sampler, params, batch: int, start_len: int, steps: int, warmup: int, vocab: int):
    """(tokens/s, ms per step, launches of own kernels per step) of `steps` decode steps at `batch`."""
    import torch

    from liteinfer_b200.engine.runner import StepEntry
    from liteinfer_b200.ops import kernels

    ids = [f"b{batch}-{i}" for i in range(batch)]
    _fill_cache(runner, ids, [start_len] * batch)
    g = torch.Generator().manual_seed(batch)
    tokens = torch.randint(0, vocab, (batch,), generator=g).tolist()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = 0
    for i in range(warmup + steps):
        if i == warmup:
            torch.cuda.synchronize()
            launches = kernels.launch_count + getattr(runner, "graph_launches", 0)
            start.record()
        logits = runner.step([StepEntry(r, [t], (0,)) for r, t in zip(ids, tokens)])
        sampled = sampler(logits, [params] * batch, ids)
        tokens = sampled.tolist()
    stop.record()
    torch.cuda.synchronize()
    launches = kernels.launch_count + getattr(runner, "graph_launches", 0) - launches
    ms = start.elapsed_time(stop) / steps
    for r in ids:
        runner.release(r)
    return batch / ms * 1e3, ms, launches // steps


def run_ours(args) -> dict:
    import torch

    from liteinfer_b200 import LLM, SamplingParams
    from liteinfer_b200.engine.runner import StepEntry
    from liteinfer_b200.ops import kernels
    from liteinfer_b200.sampling.sampler import Sampler
    from liteinfer_b200.weights.random_init import write_random_model

    model_name, shape, CONTEXT = SHAPES[args.shape]     # the context length of the chosen shape
    cfg = dict(shape)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    peaks = measured_peaks()
    steps, warmup, batch = args.steps, max(3, args.warmup), 8
    greedy = SamplingParams(temperature=0.0, max_tokens=warmup + steps + 1, ignore_eos=True)

    with tempfile.TemporaryDirectory() as tmp:
        model_dir = write_random_model(cfg, Path(tmp) / "llama-1b", seed=0)
        decode_start = CONTEXT - (warmup + steps) - 1
        llm = LLM(str(model_dir), dtype="bfloat16", device="cuda:0", max_num_seqs=64, max_model_len=CONTEXT + 1,
                  block_size=PAGE, max_num_batched_tokens=8192, gpu_memory_utilization=0.5)
        runner = llm.engine.runner
        model = runner.model
        for group in runner.cache.groups:                      # random cache contents
            group.pool.normal_(0.0, 0.5)
        vocab, hidden = cfg["vocab_size"], cfg["hidden_size"]
        sampler = Sampler(0)

        g = torch.Generator().manual_seed(7)
        if args.section == "decode":
            value, ms, launches = _decode_rate(runner, sampler, greedy, args.batch, decode_start, steps, warmup, vocab)
            llm.close()
            return {"section": "decode", "batch": args.batch, "value": value, "ms_per_step": ms,
                    "gpu_launches": launches * steps}

        # ---- prefill: one prompt of 2,048 tokens, logits at its last token
        prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=g).tolist()
        times = []
        for i in range(3 + 3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            runner.step([StepEntry("prefill", prompt, (PREFILL_TOKENS - 1,))])
            b.record()
            torch.cuda.synchronize()
            runner.release("prefill")
            if i >= 3:
                times.append(a.elapsed_time(b))
        prefill_ms = statistics.median(times)
        layers = cfg["num_hidden_layers"]
        q, kv, inter = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"], cfg["intermediate_size"]
        linear_params = layers * (hidden * (q + 2 * kv) + q * hidden + 3 * hidden * inter)
        attn_flops = layers * 4 * cfg["num_attention_heads"] * cfg["head_dim"] * PREFILL_TOKENS * (PREFILL_TOKENS + 1) / 2
        prefill_flops = 2 * linear_params * PREFILL_TOKENS + attn_flops + 2 * hidden * vocab
        prefill = {"value": PREFILL_TOKENS / prefill_ms * 1e3, "tokens": PREFILL_TOKENS, "ms": prefill_ms,
                   "frac": prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops_burst"] * 1e12),
                   "frac_of_sustained": prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)}
        if args.section == "prefill":
            llm.close()
            return {"section": "prefill", **prefill}

        # ---- decode, device-timed
        clocks = ClockSampler()
        clocks.start()
        value, ms, launches = _decode_rate(runner, sampler, greedy, batch, decode_start, steps, warmup, vocab)
        clock_record = clocks.stop()
        b1, _, _ = _decode_rate(runner, sampler, greedy, 1, decode_start, steps, warmup, vocab)
        b64, _, _ = _decode_rate(runner, sampler, greedy, 64, decode_start, steps, warmup, vocab)

        # ---- roofline of the batch-8 decode step: every weight once, plus the live requests' cache
        element = 2
        weight_bytes = (linear_params + hidden * vocab + (2 * layers + 1) * hidden) * element
        mean_ctx = decode_start + warmup + steps / 2
        kv_bytes = batch * mean_ctx * layers * 2 * kv * element
        achieved = (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "of": peaks["source"]}

        # ---- end to end through LLM.generate: host ids in, host ids out
        prompts = [torch.randint(0, vocab, (decode_start,), generator=g).tolist() for _ in range(batch)]
        llm.generate(prompts, greedy)          # once untimed: every graph the timed run replays is captured here
        llm.stats.steps.clear()
        outs = llm.generate(prompts, greedy)
        assert all(len(o.token_ids) == warmup + steps + 1 for o in outs)
        # A step's time end to end: from the end of the step before it to its own end (scheduling, the step
        # function, sampling, the read of the tokens, the stop rules and the loop around them).
        decode_steps = [s for s in llm.stats.steps if s.phase == "decode" and s.num_seqs == batch][-steps:]
        e2e_ms = sum(s.stages.loop for s in decode_steps) / len(decode_steps) * 1e3
        stage_us = {name: round(sum(getattr(s.stages, name) for s in decode_steps) / len(decode_steps) * 1e6, 1)
                    for name in ("schedule", "launch", "wait", "finish", "forward_device", "sample_device")}
        pages = -(-CONTEXT // PAGE)
        e2e = {"value": batch / e2e_ms * 1e3, "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 4 * (3 * batch + (batch + 1) + 3 * batch + batch * pages),
               "d2h_bytes_per_step": 4 * batch, "stage_us": stage_us}
        llm.close()

    # ---- the reference's two larger configurations (full depth), each reported as a few flat numbers
    points = {"decode_b1": b1, "decode_b64": b64}
    workloads = {}
    if args.shape == "1b" and not args.layers and not args.no_workloads:
        args.workload = "all"
        workloads = run_workloads(args)
        for name, result in workloads.items():
            for key, number in result.items():
                if key in ("output_tok_s", "decode_hbm_frac", "decode_b1_tok_s", "decode_b8_tok_s", "decode_b64_tok_s",
                           "decode_b1_hbm_frac", "decode_b8_hbm_frac", "decode_b64_hbm_frac", "failed"):
                    points[f"w{name}_{key}"] = number

    return {
        "metric": f"decode tok/s at batch 8 ({model_name} shape)", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / BASELINE_DECODE_B8_TOKS if args.shape == "1b" and not args.layers else None, "dtype": "bf16", "data": "synthetic ids, random weights",
        "impl": "ours",
        "config": {"model": model_name.lower().replace(" ", "-") + "-shape", "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "hidden": hidden, "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": inter, "vocab": vocab, "global_batch": batch,
                   "seq_len": CONTEXT, "page_size": PAGE, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (weights and cache are read every step)",
                   "baseline": "reference A40 batch-8 decode, 1248 tok/s"},
        "clocks": clock_record, "e2e": e2e, "gpu_launches": launches * steps,
        "prefill": prefill, "roofline": roofline, "points": points, "workloads": workloads,
    }


# ---- `--compare kegizen`: the Kegizen decoder beside the Llama decoder at equal layer sizes ----------------------
def _kegizen_config(width: int, ff: int, layers: int, heads: int, kv_heads: int, head_dim: int, vocab: int,
                    plain_attention: bool = False) -> dict:
    """Three delta-rule layers, then one attention layer (a window of 1,024 that keeps 4 tokens, capped scores,
    YaRN-scaled rotation of all of the head), over and over; every projection as wide as the Llama layer's.
    `plain_attention`: causal attention over everything, uncapped, unscaled rotation."""
    delta = {"type": "delta", "mlp": {"kind": "dense", "ff": ff},
             "mixer": {"heads": heads * head_dim // 128, "kv_heads": heads * head_dim // 128, "dim": 128, "vdim": 128, "conv": 4}}
    attention = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
                 "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim,
                           "scale": head_dim ** -0.5, "softcap": 30.0, "mask": {"size": 1024, "keep_first": 4},
                           "rot": {"dims": head_dim, "base": 10000.0,
                                   "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    if plain_attention:
        attention["mixer"] = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim,
                              "scale": head_dim ** -0.5, "rot": {"dims": head_dim, "base": 10000.0, "scaling": None}}
    return {"architecture": "Kegizen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [attention if i % 4 == 3 else delta for i in range(layers)], "loop": None}


def _karupel_config(width: int, ff: int, layers: int, heads: int, kv_heads: int, head_dim: int, vocab: int) -> dict:
    """mLSTM, delta rule, mLSTM, attention, over and over: the recurrent layers with heads of 128 x 128 as wide as the
    model, the attention with the Llama layer's heads (half of each head rotated, scaled frequencies, per-head q/k
    norms, the head gate, values mixed with the first attention's); a feed-forward in every layer."""
    wide = heads * head_dim // 128
    mlp = {"kind": "dense", "ff": ff}
    mlstm = {"type": "mlstm", "mlp": mlp, "mixer": {"heads": wide, "dim": 128, "vdim": 128, "gate_cap": 15.0}}
    delta = {"type": "delta", "mlp": mlp, "mixer": {"heads": wide, "kv_heads": wide, "dim": 128, "vdim": 128, "conv": 4}}
    attention = {"type": "attention", "mlp": mlp,
                 "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim,
                           "scale": head_dim ** -0.5, "v_mix": True,
                           "rot": {"dims": head_dim // 2, "base": 10000.0, "scaling": {"factor": 2.0}}}}
    order = (mlstm, delta, mlstm, attention)
    return {"architecture": "Karupel", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [order[i % 4] for i in range(layers)]}


def _kutolix_config(width: int, ff: int, layers: int, heads: int, kv_heads: int, head_dim: int, vocab: int) -> dict:
    """Gated attention and latent attention in turn, both with a window of 1,024: the attention with the sizes of the
    Llama layer at head size 128 (half of each head rotated), the latent attention with those of the Gifudra layer
    (unrotated part 128, rotated part 64 with YaRN frequencies, values 128, a latent of 512); a dense feed-forward
    behind the attention, 32 experts a quarter as wide behind the latent attention, of which each token runs four
    (eight groups, four kept): as many feed-forward weights per token in either."""
    h = heads * head_dim // 128
    attention = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
                 "mixer": {"heads": h, "kv_heads": max(1, h // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                           "mask": {"size": 1024}, "rot": {"dims": 64, "base": 100000.0}}}
    latent = {"type": "latent_attention",
              "mlp": {"kind": "moe", "expert": {"ff": ff // 4, "limit": 7.0},
                      "router": {"experts": 32, "top": 4, "groups": {"count": 8, "keep": 4}}},
              "mixer": {"heads": h, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5,
                        "mask": {"size": 1024},
                        "rot": {"dims": 64, "base": 10000.0,
                                "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    return {"architecture": "Kutolix", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
            "residual_mult": 0.7, "logit_softcap": 30.0, "layers": [(attention, latent)[i % 2] for i in range(layers)]}


def _timed(fn, repeats: int = 20, warmup: int = 5, inner: int = 1) -> float:
    """Median milliseconds of one `fn()` on the current stream, between CUDA events, after `warmup` calls; with
    `inner` > 1 that many calls stand between the events (a kernel shorter than the host's time to launch it)."""
    import torch

    for _ in range(warmup):
        fn()
    times = []
    for _ in range(repeats):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(inner):
            fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) / inner)
    return statistics.median(times)


def _kegizen_kernels(peaks: dict) -> dict:
    """Each kernel of the design alone beside the like kernel of the Llama path, as fractions of the measured copy
    bandwidth (kernels that stream) or product throughput (attention over prompts).  Inputs are larger than L2
    where a kernel streams, so every call reads from memory."""
    import torch

    from liteinfer_b200 import ops
    from liteinfer_b200.parts.context import AttentionPlan

    dev, bf = "cuda:0", torch.bfloat16
    hbm, tflops = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops_burst"] * 1e12
    out: dict = {}

    def ints(v):
        return torch.tensor(v, dtype=torch.int32, device=dev)

    def in_graph(fn, inner: int = 10) -> float:
        """Milliseconds of one `fn()` replayed from a CUDA graph of `inner` calls (kernels of a few microseconds,
        which the host cannot launch as fast as they run)."""
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(inner):
                fn()
        return _timed(graph.replay, repeats=10, warmup=2) / inner

    # -- norms over a stream of 16,384 x 2,048 (the 32-bit stream: 134 MB; bfloat16: 67 MB)
    T, W = 16384, 2048
    x32, x16 = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev).to(bf)
    value, w = torch.randn(T, W, device=dev).to(bf), torch.ones(W, dtype=bf, device=dev)
    normed = torch.empty(T, W, dtype=bf, device=dev)
    ms = _timed(lambda: ops.layernorm(x32, w, 1e-5, normed, delta=ops.NormedDelta(value, w, 1e-5), write_stream=True))
    out["layernorm_fused_hbm_frac"] = T * W * (4 + 2 + 4 + 2) / (ms * 1e-3) / hbm
    ms = _timed(lambda: ops.rmsnorm(x16, w, 1e-5, normed, delta=value, write_residual=True))
    out["llama_rmsnorm_fused_hbm_frac"] = T * W * (2 + 2 + 2 + 2) / (ms * 1e-3) / hbm

    # -- short convolutions over 16,384 tokens x 6,144 channels
    C = 6144
    xin, taps = torch.randn(T, C, device=dev).to(bf), torch.randn(4, C, device=dev).to(bf)
    tail, conved = torch.zeros(4, 3, C, dtype=bf, device=dev), torch.empty(T, C, dtype=bf, device=dev)
    seq_of, qsl, slots = torch.zeros(T, dtype=torch.int32, device=dev), ints([0, T]), ints([0])
    ms = _timed(lambda: ops.short_conv(xin, taps, tail, seq_of, qsl, slots, conved))
    out["short_conv_hbm_frac"] = T * C * 4 / (ms * 1e-3) / hbm

    # -- the recurrence: decode (64 requests x 16 heads x 128 x 128 states: 134 MB read and written) and a prompt
    H, d = 16, 128
    for batch, tokens_each, key in ((64, 1, "delta_rule_decode_b64"), (8, 1, "delta_rule_decode_b8"), (1, 2048, "delta_rule_prompt_2048")):
        n = batch * tokens_each
        qkv = torch.randn(n, 3 * H * d, device=dev).to(bf)
        ab = torch.randn(n, 2 * H, device=dev).to(bf)
        state = torch.zeros(batch, H, d, d, device=dev)
        read = torch.empty(n, H * d, device=dev)
        a_log, dt = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
        q2 = ints([i * tokens_each for i in range(batch + 1)])
        sl = ints(list(range(batch)))
        run = lambda: ops.gated_delta_rule(qkv, ab, a_log, dt, state, q2, sl, batch, H, H, d, d, read, tokens_each)  # noqa: E731
        ms = in_graph(run) if tokens_each == 1 else _timed(run)
        out[key + "_us"] = ms * 1e3
        if tokens_each == 1:
            out[key + "_hbm_frac"] = batch * H * d * d * 4 * 2 / (ms * 1e-3) / hbm
        else:
            out[key + "_us_per_token"] = ms * 1e3 / tokens_each

    # -- attention: a prompt of 2,048 (window 1,024 + 4 kept, capped) on the mma.sync kernel beside the plain
    #    causal one on the tcgen05 kernel; decode at 64 requests over 1,028 visible keys beside the streaming kernel
    for head_dim, heads, kv_heads in ((64, 32, 8), (128, 32, 8)):
        page, n = 16, 2048
        pages = n // page
        k_pool = torch.randn(pages * 64, kv_heads, page, head_dim, device=dev).to(bf)
        v_pool = torch.randn(pages * 64, kv_heads, page, head_dim, device=dev).to(bf)
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        q = torch.randn(n, heads * head_dim, device=dev).to(bf)
        o = torch.empty_like(q)
        plan = AttentionPlan(num_prefill=1, prefill_seqs=ints([0]), max_prefill_query_len=n)
        args = (q, q.shape[1], o, k_pool, v_pool, table, ints([0, n]), ints([n]), 1, n, heads, kv_heads, head_dim, head_dim ** -0.5)
        ms = _timed(lambda: ops.paged_attention(*args, 1024, plan=plan, keep_first=4, softcap=30.0))
        visible = sum(min(i + 1, 1024 + 4) for i in range(n))
        out[f"attention_prompt_d{head_dim}_masked_tflops_frac"] = 4 * heads * head_dim * visible / (ms * 1e-3) / tflops
        out[f"attention_prompt_d{head_dim}_masked_us"] = ms * 1e3
        ms = _timed(lambda: ops.paged_attention(*args, 0, plan=plan))
        out[f"llama_attention_prompt_d{head_dim}_tflops_frac"] = 4 * heads * head_dim * n * (n + 1) / 2 / (ms * 1e-3) / tflops
        out[f"llama_attention_prompt_d{head_dim}_us"] = ms * 1e3
        B = 64
        table = torch.arange(B * pages, dtype=torch.int32, device=dev).view(B, pages)
        q = torch.randn(B, heads * head_dim, device=dev).to(bf)
        o = torch.empty_like(q)
        plan = AttentionPlan(num_decode=B, decode_seqs=ints(list(range(B))), decode_tokens=ints(list(range(B))),
                             max_decode_context_len=n)
        args = (q, q.shape[1], o, k_pool, v_pool, table, ints(list(range(B + 1))), ints([n] * B), B, 1, heads, kv_heads, head_dim, head_dim ** -0.5)
        ms = in_graph(lambda: ops.paged_attention(*args, 1024, plan=plan, keep_first=4, softcap=30.0))
        out[f"attention_decode_d{head_dim}_masked_hbm_frac"] = B * 1028 * kv_heads * head_dim * 2 * 2 / (ms * 1e-3) / hbm
        ms = in_graph(lambda: ops.paged_attention(*args, 1024, plan=plan))
        out[f"llama_attention_decode_d{head_dim}_window_hbm_frac"] = B * 1024 * kv_heads * head_dim * 2 * 2 / (ms * 1e-3) / hbm
    return {k: round(v, 4) for k, v in out.items()}


def _gifudra_config(width: int, ff: int, layers: int, heads: int, kv_heads: int, head_dim: int, vocab: int) -> dict:
    """Latent attention with as many heads as the Llama layer has at head size 128 (unrotated part 128, rotated
    part 64, values 128, a query latent of three quarters of the width, a key/value latent of 512), four residual
    streams, a squared-relu feed-forward as wide as the Llama layer's; every fourth layer reads the cache entries of
    the layer before it."""
    h = heads * head_dim // 128
    mixer = {"heads": h, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": width * 3 // 4, "kv_rank": 512,
             "scale": 192 ** -0.5, "rot": {"dims": 64, "base": 10000.0}}
    return {"architecture": "Gifudra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0},
            "logit_scale": 0.5, "streams": 4,
            "layers": [{"type": "latent_attention", "mlp": {"kind": "dense", "ff": ff},
                        "mixer": dict(mixer, kv_from=i - 1) if i % 4 == 3 else mixer} for i in range(layers)]}


def _gifudra_kernels(peaks: dict) -> dict:
    """Each kernel of the design alone beside the like kernel of the Llama path, as fractions of the measured copy
    bandwidth (kernels that stream) or product throughput (attention over prompts); inputs larger than L2."""
    import torch

    from liteinfer_b200 import ops
    from liteinfer_b200.parts.context import AttentionPlan

    dev, bf = "cuda:0", torch.bfloat16
    hbm, tflops = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops_burst"] * 1e12
    out: dict = {}

    def ints(v):
        return torch.tensor(v, dtype=torch.int32, device=dev)

    def in_graph(fn, inner: int = 10) -> float:
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(inner):
                fn()
        return _timed(graph.replay, repeats=10, warmup=2) / inner

    # -- the norm between two sublayers: four 32-bit streams of 16,384 x 2,048 rewritten, read and normalised
    T, W, S = 16384, 2048, 4
    x = torch.randn(T, S * W, device=dev)
    y, normed = torch.randn(T, W, device=dev).to(bf), torch.empty(T, W, dtype=bf, device=dev)
    weight, gain = torch.ones(W, device=dev), torch.ones(W, device=dev)
    read, write, mix = torch.full((S,), 0.25, device=dev), torch.full((S,), 0.1, device=dev), torch.eye(S, device=dev)
    ms = _timed(lambda: ops.stream_rmsnorm(x, weight, 1e-5, normed, read=read, update=ops.StreamUpdate(y, gain, write, mix)))
    out["stream_rmsnorm_fused_hbm_frac"] = T * W * (8 * S + 2 + 2) / (ms * 1e-3) / hbm
    out["stream_rmsnorm_fused_us"] = ms * 1e3
    x16, w16 = torch.randn(T, W, device=dev).to(bf), torch.ones(W, dtype=bf, device=dev)
    ms = _timed(lambda: ops.rmsnorm(x16, w16, 1e-5, normed, delta=y, write_residual=True))
    out["llama_rmsnorm_fused_hbm_frac"] = T * W * (2 + 2 + 2 + 2) / (ms * 1e-3) / hbm

    # -- the feed-forward's activation (16,384 x 8,192) beside the gated one
    F = 8192
    hidden, gate_up, act = torch.randn(T, F, device=dev).to(bf), torch.randn(T, 2 * F, device=dev).to(bf), torch.empty(T, F, dtype=bf, device=dev)
    ms = _timed(lambda: ops.activation(hidden, act, "relu_squared"))
    out["relu_squared_hbm_frac"] = T * F * 4 / (ms * 1e-3) / hbm
    ms = _timed(lambda: ops.act_mul(gate_up, act, "silu"))
    out["llama_act_mul_hbm_frac"] = T * F * 6 / (ms * 1e-3) / hbm

    # -- latent attention (16 heads, latent 512 + 64 rotated) beside grouped-query attention (16 / 4 heads of 128)
    H, C, R, dm, page, n = 16, 512, 64, 128, 16, 2048
    pages = n // page
    inv_freq = (10000.0 ** (-torch.arange(R // 2, dtype=torch.float64) * 2 / R)).float().to(dev)
    sink = torch.zeros(H, device=dev)
    pool = (torch.randn(pages * 64, 1, page, C + R, device=dev) * 0.3).to(bf)
    kv_heads, hd = 4, 128
    k_pool = torch.randn(pages * 64, kv_heads, page, hd, device=dev).to(bf)
    v_pool = torch.randn(pages * 64, kv_heads, page, hd, device=dev).to(bf)
    # a prompt of 2,048
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
    q_lat, q_raw = (torch.randn(H, n, C, device=dev) * 0.3).to(bf), torch.randn(n, H * (dm + R), device=dev).to(bf)
    o_lat = torch.empty_like(q_lat)
    plan = AttentionPlan(num_prefill=1, prefill_seqs=ints([0]), max_prefill_query_len=n)
    qsl, ctxl = ints([0, n]), ints([n])
    ms = _timed(lambda: ops.latent_attention(q_lat, q_raw, dm + R, dm, o_lat, pool, table, qsl, ctxl, inv_freq,
                                             sink, 1, n, H, C, R, R, 0.07, plan=plan))
    out["latent_attention_prompt_us"] = ms * 1e3
    out["latent_attention_prompt_tflops_frac"] = 2 * H * (2 * C + R) * n * (n + 1) / 2 / (ms * 1e-3) / tflops
    q = torch.randn(n, H * hd, device=dev).to(bf)
    o = torch.empty_like(q)
    args = (q, q.shape[1], o, k_pool, v_pool, table, ints([0, n]), ints([n]), 1, n, H, kv_heads, hd, hd ** -0.5)
    ms = _timed(lambda: ops.paged_attention(*args, 0, plan=plan))
    out["llama_attention_prompt_us"] = ms * 1e3
    out["llama_attention_prompt_tflops_frac"] = 4 * H * hd * n * (n + 1) / 2 / (ms * 1e-3) / tflops
    # single tokens at batch 64 and 8 over 2,048 keys
    for B in (64, 8):
        table = torch.arange(B * pages, dtype=torch.int32, device=dev).view(B, pages)
        q_lat, q_raw = (torch.randn(H, B, C, device=dev) * 0.3).to(bf), torch.randn(B, H * (dm + R), device=dev).to(bf)
        o_lat = torch.empty_like(q_lat)
        plan = AttentionPlan(num_decode=B, decode_seqs=ints(list(range(B))), decode_tokens=ints(list(range(B))),
                             max_decode_context_len=n)
        qsl, ctxl = ints(list(range(B + 1))), ints([n] * B)
        ms = in_graph(lambda: ops.latent_attention(q_lat, q_raw, dm + R, dm, o_lat, pool, table, qsl, ctxl, inv_freq, sink,
                                                   B, 1, H, C, R, R, 0.07, plan=plan))
        out[f"latent_attention_decode_b{B}_us"] = ms * 1e3
        out[f"latent_attention_decode_b{B}_hbm_frac"] = B * n * (C + R) * 2 / (ms * 1e-3) / hbm
        q = torch.randn(B, H * hd, device=dev).to(bf)
        o = torch.empty_like(q)
        args = (q, q.shape[1], o, k_pool, v_pool, table, qsl, ctxl, B, 1, H, kv_heads, hd, hd ** -0.5)
        ms = in_graph(lambda: ops.paged_attention(*args, 0, plan=plan))
        out[f"llama_attention_decode_b{B}_us"] = ms * 1e3
        out[f"llama_attention_decode_b{B}_hbm_frac"] = B * n * kv_heads * hd * 2 * 2 / (ms * 1e-3) / hbm
    return {k: round(v, 4) for k, v in out.items()}


def _karupel_kernels(peaks: dict) -> dict:
    """Each kernel that the Karupel design brought, alone beside the like kernel of the Kegizen path, as fractions of
    the measured copy bandwidth; inputs larger than L2, so every call reads from memory."""
    import torch

    from liteinfer_b200 import ops

    dev, bf = "cuda:0", torch.bfloat16
    hbm = peaks["hbm_gbs"] * 1e9
    out: dict = {}

    def ints(v):
        return torch.tensor(v, dtype=torch.int32, device=dev)

    def in_graph(fn, inner: int = 10) -> float:
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(inner):
                fn()
        return _timed(graph.replay, repeats=10, warmup=2) / inner

    # -- the norm on a sublayer's way out: stream (32-bit) += (1 + w) * value / rms(value), and the sum rounded
    T, W = 16384, 2048
    x32, value = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev).to(bf)
    w32, w16 = torch.ones(W, device=dev), torch.ones(W, dtype=bf, device=dev)
    rounded = torch.empty(T, W, dtype=bf, device=dev)
    ms = _timed(lambda: ops.layernorm_add(x32, value, w32, 1e-5, centred=False, out=rounded))
    out["output_norm_hbm_frac"] = T * W * (4 + 2 + 4 + 2) / (ms * 1e-3) / hbm
    ms = _timed(lambda: ops.layernorm(x32, w16, 1e-5, rounded, delta=ops.NormedDelta(value, w16, 1e-5), write_stream=True))
    out["kegizen_layernorm_fused_hbm_frac"] = T * W * (4 + 2 + 4 + 2) / (ms * 1e-3) / hbm

    # -- the gated norm behind a recurrence: the mLSTM's (divisor, sigmoid gate, weights per head) and the delta rule's
    H, d = 16, 128
    read, gate = torch.randn(T, H * d, device=dev), torch.randn(T, H * d, device=dev).to(bf)
    den, gated = torch.rand(T, H, device=dev) + 0.5, torch.empty(T, H * d, dtype=bf, device=dev)
    wide_w, head_w = torch.ones(H * d, device=dev), torch.ones(d, device=dev)
    ms = _timed(lambda: ops.gated_rmsnorm(read, gate, wide_w, 1e-5, gated, H, gate_activation="sigmoid", den=den))
    out["mlstm_gated_norm_hbm_frac"] = T * H * d * (4 + 2 + 2) / (ms * 1e-3) / hbm
    ms = _timed(lambda: ops.gated_rmsnorm(read, gate, head_w, 1e-5, gated, H))
    out["kegizen_gated_norm_hbm_frac"] = T * H * d * (4 + 2 + 2) / (ms * 1e-3) / hbm

    # -- the recurrences: single tokens of 64 and 8 requests (16 heads of 128 x 128: 134 MB of state read and written
    #    at 64) and a prompt of 2,048
    for batch, tokens_each, key in ((64, 1, "decode_b64"), (8, 1, "decode_b8"), (1, 2048, "prompt_2048")):
        n = batch * tokens_each
        q2, sl = ints([i * tokens_each for i in range(batch + 1)]), ints(list(range(batch)))
        proj = torch.randn(n, 4 * H * d + 2 * H, device=dev).to(bf)
        state, maxima = torch.zeros(batch, H, d + 1, d, device=dev), torch.zeros(batch, H, d + 1, device=dev)
        o, dn = torch.empty(n, H * d, device=dev), torch.empty(n, H, device=dev)
        bias = torch.zeros(H, device=dev)
        offsets = (0, H * d, 2 * H * d, 4 * H * d, 4 * H * d + H)
        run_m = lambda: ops.mlstm(proj, offsets, bias, bias, 15.0, state, maxima, q2, sl, batch, H, d, d, o, dn,  # noqa: E731
                                  tokens_each)
        qkv, ab = torch.randn(n, 3 * H * d, device=dev).to(bf), torch.randn(n, 2 * H, device=dev).to(bf)
        s2 = torch.zeros(batch, H, d, d, device=dev)
        run_d = lambda: ops.gated_delta_rule(qkv, ab, bias, bias, s2, q2, sl, batch, H, H, d, d, o, tokens_each)  # noqa: E731
        for name, run, rows in (("mlstm", run_m, d + 1), ("kegizen_delta_rule", run_d, d)):
            ms = in_graph(run) if tokens_each == 1 else _timed(run)
            out[f"{name}_{key}_us"] = ms * 1e3
            if tokens_each == 1:
                out[f"{name}_{key}_hbm_frac"] = batch * H * rows * d * 4 * 2 / (ms * 1e-3) / hbm
            else:
                out[f"{name}_{key}_us_per_token"] = ms * 1e3 / tokens_each

    # -- what stands in front of the attention: per-head norms, rotation, blend of the values, pages; beside the
    #    plain rotation and store.  16,384 tokens of 32 / 8 heads of 128.
    heads, kv_heads, hd, page = 32, 8, 128, 16
    pages = T // page
    row = (heads + 2 * kv_heads) * hd
    qkv = torch.randn(T, row + 32, device=dev).to(bf)
    other = torch.randn(T, kv_heads * hd, device=dev).to(bf)
    k_pool, v_pool = (torch.empty(pages, kv_heads, page, hd, dtype=bf, device=dev) for _ in range(2))
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
    positions, seq_of = torch.arange(T, dtype=torch.int32, device=dev), torch.zeros(T, dtype=torch.int32, device=dev)
    inv_half = (10000.0 ** (-torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2)) / 2.0).to(dev)
    inv_full = (10000.0 ** (-torch.arange(0, hd, 2, dtype=torch.float32) / hd)).to(dev)
    norm_w, blend = torch.ones(hd, dtype=bf, device=dev), torch.tensor([0.4], device=dev)
    ms = _timed(lambda: ops.head_norm_rope_kv_write(qkv, positions, seq_of, table, k_pool, v_pool, inv_half, heads,
                                                    kv_heads, hd, hd // 2, norm_w, norm_w, 1e-5, v_other=other, blend=blend))
    moved = T * hd * 2 * (2 * heads + 2 * kv_heads + 3 * kv_heads)      # q read and written; k, v read and stored; the other v
    out["head_norm_rope_store_hbm_frac"] = moved / (ms * 1e-3) / hbm
    exact = qkv[:, :row].contiguous()
    ms = _timed(lambda: ops.rope_kv_write(exact, positions, seq_of, table, k_pool, v_pool, inv_full, heads, kv_heads, hd, hd))
    out["kegizen_rope_store_hbm_frac"] = T * hd * 2 * (2 * heads + 4 * kv_heads) / (ms * 1e-3) / hbm

    # -- the gate on the heads' outputs (in place)
    attended, gates = torch.randn(T, heads * hd, device=dev).to(bf), torch.randn(T, heads, device=dev).to(bf)
    ms = _timed(lambda: ops.sigmoid_gate_heads_(attended, gates, heads))
    out["head_gate_hbm_frac"] = T * heads * hd * 2 * 2 / (ms * 1e-3) / hbm
    return {k: round(v, 4) for k, v in out.items()}


def _kutolix_kernels(peaks: dict) -> dict:
    """Each kernel that the Kutolix design brought or changed, alone beside its like, as fractions of the measured
    copy bandwidth (kernels that stream) or product throughput (attention and experts over prompts); inputs larger
    than L2."""
    import torch

    from liteinfer_b200 import ops
    from liteinfer_b200.parts.context import AttentionPlan

    dev, bf = "cuda:0", torch.bfloat16
    hbm, tflops = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops_burst"] * 1e12
    out: dict = {}

    def ints(v):
        return torch.tensor(v, dtype=torch.int32, device=dev)

    def in_graph(fn, inner: int = 10) -> float:
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(inner):
                fn()
        return _timed(graph.replay, repeats=10, warmup=2) / inner

    # -- gated attention (16 / 4 heads of 128, a window of 1,024, a sink) beside the same launch without a sink
    H, kv_heads, hd, page, n, window = 16, 4, 128, 16, 2048, 1024
    pages = n // page
    sink = torch.zeros(H, device=dev)
    k_pool = torch.randn(pages * 64, kv_heads, page, hd, device=dev).to(bf)
    v_pool = torch.randn(pages * 64, kv_heads, page, hd, device=dev).to(bf)
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
    q = torch.randn(n, H * hd, device=dev).to(bf)
    o = torch.empty_like(q)
    plan = AttentionPlan(num_prefill=1, prefill_seqs=ints([0]), max_prefill_query_len=n)
    args = (q, q.shape[1], o, k_pool, v_pool, table, ints([0, n]), ints([n]), 1, n, H, kv_heads, hd, hd ** -0.5, window)
    seen = n * (n + 1) // 2 - (n - window) * (n - window + 1) // 2          # (query, key) pairs inside the window
    for name, extra in (("sink_attention", dict(sink=sink)), ("plain_attention", {})):
        ms = _timed(lambda: ops.paged_attention(*args, plan=plan, **extra))
        out[f"{name}_prompt_us"] = ms * 1e3
        out[f"{name}_prompt_tflops_frac"] = 4 * H * hd * seen / (ms * 1e-3) / tflops
    for B in (64, 8):
        table = torch.arange(B * pages, dtype=torch.int32, device=dev).view(B, pages)
        plan = AttentionPlan(num_decode=B, decode_seqs=ints(list(range(B))), decode_tokens=ints(list(range(B))),
                             max_decode_context_len=n)
        qsl, ctxl = ints(list(range(B + 1))), ints([n] * B)
        q = torch.randn(B, H * hd, device=dev).to(bf)
        o = torch.empty_like(q)
        args = (q, q.shape[1], o, k_pool, v_pool, table, qsl, ctxl, B, 1, H, kv_heads, hd, hd ** -0.5, window)
        for name, extra in (("sink_attention", dict(sink=sink)), ("plain_attention", {})):
            ms = in_graph(lambda: ops.paged_attention(*args, plan=plan, **extra))
            out[f"{name}_decode_b{B}_us"] = ms * 1e3
            out[f"{name}_decode_b{B}_hbm_frac"] = B * window * kv_heads * hd * 2 * 2 / (ms * 1e-3) / hbm

    # -- latent attention with a window of 1,024 (16 heads, latent 512 + 64 rotated) beside the same launch without
    C, R, dm = 512, 64, 128
    inv_freq = (10000.0 ** (-torch.arange(R // 2, dtype=torch.float64) * 2 / R)).float().to(dev)
    pool = (torch.randn(pages * 64, 1, page, C + R, device=dev) * 0.3).to(bf)
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
    q_lat, q_raw = (torch.randn(H, n, C, device=dev) * 0.3).to(bf), torch.randn(n, H * (dm + R), device=dev).to(bf)
    o_lat = torch.empty_like(q_lat)
    plan = AttentionPlan(num_prefill=1, prefill_seqs=ints([0]), max_prefill_query_len=n)
    qsl, ctxl = ints([0, n]), ints([n])
    for name, extra, pairs in (("windowed_latent", dict(window=window, cos_sin_scale=1.14), seen),
                               ("causal_latent", {}, n * (n + 1) // 2)):
        ms = _timed(lambda: ops.latent_attention(q_lat, q_raw, dm + R, dm, o_lat, pool, table, qsl, ctxl, inv_freq, None,
                                                 1, n, H, C, R, R, 0.07, plan=plan, **extra))
        out[f"{name}_prompt_us"] = ms * 1e3
        out[f"{name}_prompt_tflops_frac"] = 2 * H * (2 * C + R) * pairs / (ms * 1e-3) / tflops
    for B in (64, 8):
        table = torch.arange(B * pages, dtype=torch.int32, device=dev).view(B, pages)
        q_lat, q_raw = (torch.randn(H, B, C, device=dev) * 0.3).to(bf), torch.randn(B, H * (dm + R), device=dev).to(bf)
        o_lat = torch.empty_like(q_lat)
        plan = AttentionPlan(num_decode=B, decode_seqs=ints(list(range(B))), decode_tokens=ints(list(range(B))),
                             max_decode_context_len=n)
        qsl, ctxl = ints(list(range(B + 1))), ints([n] * B)
        for name, extra, keys in (("windowed_latent", dict(window=window, cos_sin_scale=1.14), window), ("causal_latent", {}, n)):
            ms = in_graph(lambda: ops.latent_attention(q_lat, q_raw, dm + R, dm, o_lat, pool, table, qsl, ctxl, inv_freq,
                                                       None, B, 1, H, C, R, R, 0.07, plan=plan, **extra))
            out[f"{name}_decode_b{B}_us"] = ms * 1e3
            out[f"{name}_decode_b{B}_hbm_frac"] = B * keys * (C + R) * 2 / (ms * 1e-3) / hbm

    # -- what stands in front of the gated attention (rotation of half a head, unit norm behind it, store) beside the
    #    Karupel form (norm with a weight in front of the rotation); the element-wise gate beside the gate per head
    T = 16384
    heads, kvh = 32, 8
    pages_t = T // page
    row = (heads + 2 * kvh) * hd
    qkv = torch.randn(T, row + heads * hd, device=dev).to(bf)
    kp, vp = (torch.empty(pages_t, kvh, page, hd, dtype=bf, device=dev) for _ in range(2))
    table = torch.arange(pages_t, dtype=torch.int32, device=dev).view(1, pages_t)
    positions, seq_of = torch.arange(T, dtype=torch.int32, device=dev), torch.zeros(T, dtype=torch.int32, device=dev)
    inv_half = (100000.0 ** (-torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2))).to(dev)
    norm_w = torch.ones(hd, dtype=bf, device=dev)
    moved = T * hd * 2 * (2 * heads + 4 * kvh)
    ms = _timed(lambda: ops.head_norm_rope_kv_write(qkv, positions, seq_of, table, kp, vp, inv_half, heads, kvh, hd, hd // 2,
                                                    None, None, 1e-6, unit_norm=True, norm_after_rotation=True))
    out["unit_norm_behind_rotation_store_hbm_frac"] = moved / (ms * 1e-3) / hbm
    ms = _timed(lambda: ops.head_norm_rope_kv_write(qkv, positions, seq_of, table, kp, vp, inv_half, heads, kvh, hd, hd // 2,
                                                    norm_w, norm_w, 1e-6))
    out["karupel_head_norm_rope_store_hbm_frac"] = moved / (ms * 1e-3) / hbm
    attended = torch.randn(T, heads * hd, device=dev).to(bf)
    ms = _timed(lambda: ops.sigmoid_gate_(attended, qkv[:, row:]))
    out["output_gate_hbm_frac"] = T * heads * hd * 2 * 3 / (ms * 1e-3) / hbm
    ms = _timed(lambda: ops.sigmoid_gate_heads_(attended, qkv[:, row:row + heads], heads))
    out["karupel_head_gate_hbm_frac"] = T * heads * hd * 2 * 2 / (ms * 1e-3) / hbm

    # -- the routed feed-forward (width 2,048; 32 experts 2,048 wide; 4 per token) beside the dense one (8,192 wide)
    W, F, E, top = 2048, 2048, 32, 4
    gate_up = (torch.randn(E, 2 * F, W, device=dev) * 0.02).to(bf)
    down = (torch.randn(E, W, F, device=dev) * 0.02).to(bf)
    router = torch.randn(E, W, device=dev) * 0.02
    dense_gate_up = (torch.randn(2 * 4 * F, W, device=dev) * 0.02).to(bf)
    dense_down = (torch.randn(W, 4 * F, device=dev) * 0.02).to(bf)
    from liteinfer_b200.ops import kernels as op_kernels

    for tokens, key in ((2048, "prompt_2048"), (64, "decode_b64"), (8, "decode_b8")):
        x = torch.randn(tokens, W, device=dev).to(bf)
        ids, weights = torch.empty(tokens, top, dtype=torch.int32, device=dev), torch.empty(tokens, top, device=dev)
        y = torch.empty(tokens, W, dtype=bf, device=dev)

        def route():
            ops.moe_router(x, router, top, 8, 4, False, ids, weights)

        def experts():
            ops.moe_experts(x, gate_up, down, ids, weights, "capped_swiglu", 7.0, 1.702, True, y)

        dense_hidden = torch.empty(tokens, 4 * F, dtype=bf, device=dev)
        interleaved = ops.gated_linear_supported(x, dense_gate_up)

        def dense():
            if interleaved:
                ops.gated_linear(x, dense_gate_up, dense_hidden, "silu")
            else:
                ops.act_mul(ops.linear(x, dense_gate_up, None), dense_hidden, "silu")
            ops.linear(dense_hidden, dense_down, None)

        route()
        timer = _timed if tokens > 64 else in_graph
        out[f"moe_router_{key}_us"] = timer(route) * 1e3
        ms_d = timer(dense)
        out[f"dense_ff_{key}_us"] = ms_d * 1e3
        flops = 2 * tokens * top * 3 * F * W
        active = int(torch.unique(ids).numel())
        for form, least in (("tcgen05", 1), ("mma", 1 << 30)):      # both forms of the experts' products at every width
            kept = op_kernels.MOE_TCGEN05_MIN_PAIRS
            op_kernels.MOE_TCGEN05_MIN_PAIRS = least
            ms_e = timer(experts)
            op_kernels.MOE_TCGEN05_MIN_PAIRS = kept
            out[f"moe_experts_{form}_{key}_us"] = ms_e * 1e3
            if tokens > 64:
                out[f"moe_experts_{form}_{key}_tflops_frac"] = flops / (ms_e * 1e-3) / tflops
            else:
                out[f"moe_experts_{form}_{key}_hbm_frac"] = active * 3 * F * W * 2 / (ms_e * 1e-3) / hbm
        if tokens > 64:
            out[f"dense_ff_{key}_tflops_frac"] = flops / (ms_d * 1e-3) / tflops
        else:
            out[f"moe_experts_{key}_active"] = active
            out[f"dense_ff_{key}_hbm_frac"] = 3 * 4 * F * W * 2 / (ms_d * 1e-3) / hbm

    # -- the soft cap on 64 rows of logits
    logits = torch.randn(64, 32000, device=dev).to(bf)
    out["softcap_b64_us"] = in_graph(lambda: ops.softcap_(logits, 30.0)) * 1e3
    return {k: round(v, 4) for k, v in out.items()}


def run_kegizen(args, which: str = "kegizen") -> dict:
    """Prefill (one prompt of 2,048 tokens) and decode (batch 8 and 64 near a context of 2,048) of a Kegizen (or
    Gifudra) model and of a Llama model with the same width, depth, head sizes and feed-forward, random weights,
    bfloat16; and the design's kernels one by one.  Printed as one JSON line; the default run of this file does not
    include it."""
    import torch

    from liteinfer_b200 import LLM, SamplingParams
    from liteinfer_b200.engine.runner import StepEntry
    from liteinfer_b200.sampling.sampler import Sampler
    from liteinfer_b200.weights.random_init import write_random_model

    peaks = measured_peaks()
    steps, warmup, context, vocab = min(args.steps, 32), max(3, min(args.warmup, 8)), 2048, 32000
    greedy = SamplingParams(temperature=0.0, max_tokens=warmup + steps + 1, ignore_eos=True)
    sizes = {"w2048": dict(width=2048, ff=8192, layers=8, heads=32, kv_heads=8, head_dim=64),
             "w4096": dict(width=4096, ff=14336, layers=4, heads=32, kv_heads=8, head_dim=128)}
    if which == "gifudra":      # heads of 128 in both sizes: the latent attention's heads are 128 + 64 wide
        sizes = {"w2048": dict(width=2048, ff=8192, layers=8, heads=16, kv_heads=4, head_dim=128),
                 "w4096": dict(width=4096, ff=14336, layers=4, heads=32, kv_heads=8, head_dim=128)}
    if which == "kutolix":
        sizes = {"w2048": dict(width=2048, ff=8192, layers=8, heads=16, kv_heads=4, head_dim=128),
                 "w4096": dict(width=4096, ff=14336, layers=4, heads=32, kv_heads=8, head_dim=128)}
    design = {"gifudra": _gifudra_config, "karupel": _karupel_config, "kutolix": _kutolix_config}.get(which, _kegizen_config)
    result: dict = {"impl": "ours", "compare": which, "dtype": "bf16", "data": "synthetic ids, random weights",
                    "peaks": peaks, "models": {}}
    for name, size in sizes.items():
        llama = dict(LLAMA_1B, vocab_size=vocab, hidden_size=size["width"], intermediate_size=size["ff"],
                     num_hidden_layers=size["layers"], num_attention_heads=size["heads"],
                     num_key_value_heads=size["kv_heads"], head_dim=size["head_dim"], tie_word_embeddings=False)
        beside = ("llama", llama)
        if which == "karupel":      # its closest relative: delta-rule layers and plain causal attention, the same sizes
            beside = ("kegizen", _kegizen_config(vocab=vocab, plain_attention=True, **size))
        if which == "kutolix":      # its closest relative: latent attention with a sink and a gate, dense feed-forwards
            beside = ("gifudra", _gifudra_config(vocab=vocab, **size))
        for arch, cfg in ((which, design(vocab=vocab, **size)), beside):
            with tempfile.TemporaryDirectory() as tmp:
                model_dir = write_random_model(cfg, Path(tmp) / arch, seed=0)
                llm = LLM(str(model_dir), dtype="bfloat16", device="cuda:0", max_num_seqs=64, max_model_len=context + 1,
                          block_size=PAGE, max_num_batched_tokens=8192, gpu_memory_utilization=0.5)
                runner = llm.engine.runner
                g = torch.Generator().manual_seed(7)
                prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=g).tolist()

                def prefill():
                    runner.step([StepEntry("prefill", prompt, (PREFILL_TOKENS - 1,))])
                    runner.release("prefill")

                numbers = {"prefill_2048_ms": round(_timed(prefill, repeats=5, warmup=3), 3)}
                numbers["prefill_tok_s"] = round(PREFILL_TOKENS / numbers["prefill_2048_ms"] * 1e3)
                start = context - (warmup + steps) - 1
                for batch in (8, 64):
                    rate, ms, launches = _decode_rate(runner, Sampler(0), greedy, batch, start, steps, warmup, vocab)
                    numbers[f"decode_b{batch}_tok_s"] = round(rate)
                    numbers[f"decode_b{batch}_ms"] = round(ms, 4)
                    numbers[f"decode_b{batch}_launches"] = launches
                numbers["weight_gb"] = round(runner.model.weight_bytes() / 1e9, 3)
                numbers["decode_b8_weight_hbm_frac"] = round(
                    runner.model.weight_bytes() / (numbers["decode_b8_ms"] * 1e-3) / (peaks["hbm_gbs"] * 1e9), 3)
                runner.check_kernels()
                llm.close()
                result["models"][f"{name}_{arch}"] = numbers
    kernels = {"gifudra": _gifudra_kernels, "karupel": _karupel_kernels, "kutolix": _kutolix_kernels}.get(which, _kegizen_kernels)
    result["kernels"] = kernels(peaks)
    return result


def _shape_numbers(cfg: dict) -> dict:
    layers, hidden, vocab = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    linear = layers * (hidden * (q + 2 * kv) + q * hidden + 3 * hidden * cfg["intermediate_size"])
    return {"weight_bytes": (linear + hidden * vocab + (2 * layers + 1) * hidden) * 2,     # every weight a step reads, once
            "kv_bytes_per_token": layers * 2 * kv * 2}


def workload_3b(args, peaks: dict) -> dict:
    """The reference's serving workload at the Llama 3.2 3B layer sizes: 64 requests with prompts of 128 to 2,048
    tokens (uniform, seeded) and 256 forced output tokens each, all offered at once to `LLM.generate` (continuous
    batching under a token budget of 8,192).  One untimed run of the same requests comes first, as the reference's
    harness warms up (benchmarks/harness.py:110-122).  Reported: output tokens per second over the whole run, and
    for its decode steps the bytes they had to read (weights once, the live requests' cache) over their time."""
    import random

    import torch

    from liteinfer_b200 import LLM, SamplingParams
    from liteinfer_b200.weights.random_init import write_random_model

    cfg = dict(LLAMA_3B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    numbers = _shape_numbers(cfg)
    rng = random.Random(3)
    lengths = [rng.randint(128, 2048) for _ in range(64)]
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in lengths]
    params = SamplingParams(temperature=0.0, max_tokens=256, min_tokens=256, ignore_eos=True)
    with tempfile.TemporaryDirectory() as tmp:
        model_dir = write_random_model(cfg, Path(tmp) / "llama-3b", seed=0)
        with LLM(str(model_dir), dtype="bfloat16", device="cuda:0", max_num_seqs=64, max_model_len=2048 + 256 + 1,
                 block_size=PAGE, max_num_batched_tokens=8192) as llm:
            llm.generate(prompts, params)                       # warm-up: every graph this run needs is captured
            steps: list[tuple[str, float, int]] = []
            scheduler = llm.engine.scheduler
            llm.stats.on_step(lambda m: steps.append(
                (m.phase, m.stages.loop, sum(len(s) for s in scheduler.running if not s.is_finished))))
            torch.cuda.synchronize()
            start = time.perf_counter()
            outs = llm.generate(prompts, params)
            torch.cuda.synchronize()
            wall = time.perf_counter() - start
    assert all(len(o.token_ids) == 256 for o in outs)
    decode = [(t, held) for phase, t, held in steps if phase == "decode"]
    decode_bytes = sum(numbers["weight_bytes"] + held * numbers["kv_bytes_per_token"] for _, held in decode)
    decode_s = sum(t for t, _ in decode)
    return {"model": "llama-3.2-3b-shape", "layers": cfg["num_hidden_layers"], "layers_full": LLAMA_3B["num_hidden_layers"],
            "requests": 64, "prompt_tokens": sum(lengths), "output_tokens": 64 * 256, "wall_s": wall,
            "output_tok_s": 64 * 256 / wall, "total_tok_s": (sum(lengths) + 64 * 256) / wall, "steps": len(steps),
            "decode_steps": len(decode), "decode_ms_per_step": decode_s / max(1, len(decode)) * 1e3,
            "decode_hbm_frac": decode_bytes / decode_s / 1e9 / peaks["hbm_gbs"] if decode_s else None}


def workload_8b(args, peaks: dict) -> dict:
    """Decode at the Llama 3.1 8B layer sizes with every sequence at a context of 8,192: batch 1, 8 and 64, the cache
    sized for 64 such sequences (68.7 GB beside 16 GB of weights).  Tokens per second of the step function and the
    sampler, device-timed, and the fraction of the copy bandwidth that the bytes of a step come to."""
    from liteinfer_b200 import LLM, SamplingParams
    from liteinfer_b200.sampling.sampler import Sampler
    from liteinfer_b200.weights.random_init import write_random_model

    cfg = dict(LLAMA_8B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    numbers = _shape_numbers(cfg)
    context, steps, warmup = 8192, args.steps, max(3, args.warmup)
    start_len = context - (warmup + steps) - 1
    greedy = SamplingParams(temperature=0.0, max_tokens=warmup + steps + 1, ignore_eos=True)
    out = {"model": "llama-3.1-8b-shape", "layers": cfg["num_hidden_layers"], "layers_full": LLAMA_8B["num_hidden_layers"],
           "context": context}
    with tempfile.TemporaryDirectory() as tmp:
        model_dir = write_random_model(cfg, Path(tmp) / "llama-8b", seed=0)
        pages = 64 * (-(-(context + 1) // PAGE)) + 16
        with LLM(str(model_dir), dtype="bfloat16", device="cuda:0", max_num_seqs=64, max_model_len=context + 1,
                 block_size=PAGE, max_num_batched_tokens=8192, num_gpu_blocks=pages) as llm:
            runner = llm.engine.runner
            for group in runner.cache.groups:
                group.pool.normal_(0.0, 0.5)
            out["cache_gb"] = pages * runner.cache.bytes_per_page() / 1e9
            for batch in (1, 8, 64):
                value, ms, _ = _decode_rate(runner, Sampler(0), greedy, batch, start_len, steps, warmup, cfg["vocab_size"])
                nbytes = numbers["weight_bytes"] + batch * (start_len + warmup + steps / 2) * numbers["kv_bytes_per_token"]
                out[f"decode_b{batch}_tok_s"] = value
                out[f"decode_b{batch}_ms"] = ms
                out[f"decode_b{batch}_hbm_frac"] = nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]
    return out


def run_workloads(args) -> dict:
    """The two larger configurations of the reference's benchmark set; a failure is reported, not raised."""
    peaks = measured_peaks()
    results = {}
    for name, fn in (("3b", workload_3b), ("8b", workload_8b)):
        if args.workload not in ("all", name):
            continue
        try:
            started = time.perf_counter()
            results[name] = {**fn(args, peaks), "took_s": round(time.perf_counter() - started, 1)}
        except Exception as error:  # noqa: BLE001
            results[name] = {"failed": f"{type(error).__name__}: {str(error)[:200]}"}
    return results


def run_reference(args) -> dict:
    """The unmodified reference through its own public API: `baseline/_ref` holds its package (put there by
    `baseline/install_reference.py`), `baseline/reference_arm.py` drives it.  Whatever keeps it from running
    here (the package missing, a dependency missing on this box, its Triton kernels failing to compile for
    this GPU) is printed as the reason for `unavailable`."""
    if not (ROOT / "baseline" / "_ref" / "liteinfer").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref holds no copy of the reference package "
                "(run python baseline/install_reference.py <reference checkout> where one exists)"}
    try:
        sys.path.insert(0, str(ROOT / "baseline"))
        from reference_arm import run  # noqa: PLC0415
        helpers = {"ClockSampler": ClockSampler, "peaks": measured_peaks(), "baseline_toks": BASELINE_DECODE_B8_TOKS}
        return run(args, LLAMA_1B, CONTEXT, PAGE, helpers)
    except Exception as error:  # noqa: BLE001
        import traceback
        traceback.print_exc()
        return {"impl": "reference", "unavailable": f"{type(error).__name__}: {str(error)[:300]}"}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    parser.add_argument("--section", default="all", choices=["all", "decode", "prefill"],
                        help="run one part only (for profiling); the JSON line then lacks the other parts")
    parser.add_argument("--batch", type=int, default=8, help="decode batch of --section decode")
    parser.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="layer sizes: Llama 3.2 1B (the contract's), 3B or 3.1 8B")
    parser.add_argument("--workload", default="none", choices=["none", "3b", "8b", "all"],
                        help="run the reference's larger configurations instead (64 requests under continuous batching "
                             "at the 3B sizes; decode at a context of 8,192 at the 8B sizes) and print their line")
    parser.add_argument("--compare", default="none", choices=["none", "kegizen", "gifudra", "karupel", "kutolix"],
                        help="instead of the default run: the Kegizen (or Gifudra) decoder beside the Llama decoder, "
                             "the Karupel decoder beside the Kegizen decoder, or the Kutolix decoder beside the Gifudra "
                             "decoder, at equal layer sizes (prefill, decode, and the design's kernels one by one)")
    parser.add_argument("--no-workloads", action="store_true",
                        help="leave the 3B and 8B configurations out of the default run (they add about 80 s)")
    args = parser.parse_args()
    if args.gpus != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print("liteinfer_b200 is a single-GPU engine: bench.py runs at --gpus 1 only")
        return 2
    if args.compare != "none" and args.impl == "ours":
        print(json.dumps(run_kegizen(args, args.compare)))
        return 0
    if args.workload != "none" and args.impl == "ours":
        print(json.dumps({"impl": "ours", "workloads": run_workloads(args)}))
        return 0
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
