"""The Kutolix decoder as a `ModelSpec`.

Every layer has one of two mixers and an optional feed-forward.  The mixers: a grouped-query softmax attention
with a sliding window, a half-split rotation of the first `rot.dims` dimensions, q and k divided by their root mean
square per head after the rotation, a learned sink per head in the softmax's denominator and an element-wise
sigmoid output gate; and a latent attention (keys and values expanded from one normalised latent per token plus
one rotated key part shared by all heads, queries straight from the stream, pairs of neighbours rotated with YaRN
frequencies, a sliding window).  The feed-forward is a gated silu one, or a mixture of experts (softmax scores,
experts chosen from the best groups of neighbours, weights not renormalised, experts with capped products).
The sublayers read the residual stream as it is; only what they give back is normalised and scaled:
x <- x + m * norm(sublayer(x)).  The embedding's rows are scaled, the stream is summed in 32-bit, the head is the
embedding's table and the logits pass c * tanh(. / c).  Tensor names: `embed`, `l<i>.norm1|norm2`, `l<i>.mix.*`,
`l<i>.mlp.gate|up|down` or `l<i>.mlp.router`, `l<i>.mlp.e<j>.gate|up|down`, `final.norm`.
"""

from __future__ import annotations

from liteinfer_b200.config.kutolix_config import KutolixConfig, KutolixMixer, KutolixMLP, KutolixRotation
from liteinfer_b200.config.registry import register_architecture
from liteinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_BARE = {"weight": ""}      # a tensor stored under the part's prefix itself
_ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                    "gate_proj.weight": "g", "sink": "sink"}
_LATENT_NAMES = {"q.weight": "q", "dkv.weight": "dkv", "dkv_norm.weight": "dkv.norm", "uk.weight": "uk",
                 "uv.weight": "uv", "o.weight": "o"}
_MLP_NAMES = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}

EXPERT_GATE_SLOPE = 1.702       # an expert's gate passes g * sigmoid(1.702 g)


def _rotation(rot: KutolixRotation | None, size: int, pairs: str) -> PartSpec:
    if rot is None:
        return PartSpec("none", {})
    params = {"head_dim": size, "rotary_dim": rot.dims, "theta": rot.base, "pairs": pairs}
    if rot.scaling is not None:
        s = rot.scaling
        params.update({"rope_type": "yarn", "factor": s.factor, "original_max_position_embeddings": s.original,
                       "fast": s.fast, "slow": s.slow})
    else:
        params["exact"] = True
    return PartSpec("rotary", params)


def _mixer(config: KutolixConfig, mixer: KutolixMixer) -> tuple[PartSpec, dict[str, str]]:
    if mixer.type == "attention":
        return PartSpec("attention", {
            "hidden_size": config.hidden_size, "heads": mixer.heads, "kv_heads": mixer.kv_heads, "head_dim": mixer.dim,
            "v_head_dim": mixer.vdim, "position": _rotation(mixer.rot, mixer.dim, "half"), "scale": mixer.scale,
            "window": mixer.window, "qk_norm": "head", "qk_norm_weight": False, "qk_norm_after_rotation": True,
            "qk_norm_eps": config.norm_eps, "sink": True, "output_gate": True}), _ATTENTION_NAMES
    return PartSpec("latent_attention", {
        "hidden_size": config.hidden_size, "heads": mixer.heads, "dim": mixer.dim, "rot_dim": mixer.rot_dim,
        "vdim": mixer.vdim, "q_rank": None, "kv_rank": mixer.kv_rank, "scale": mixer.scale,
        "norm_eps": config.norm_eps, "position": _rotation(mixer.rot, mixer.rot_dim, "interleaved"),
        "window": mixer.window, "sink": False, "gate": False}), _LATENT_NAMES


def _feed_forward(config: KutolixConfig, mlp: KutolixMLP) -> tuple[PartSpec, dict[str, str]]:
    if mlp.kind == "dense":
        return PartSpec("gated_mlp", {"hidden_size": config.hidden_size, "intermediate_size": mlp.ff,
                                      "activation": "silu"}), _MLP_NAMES
    names = {"router.weight": "router"}
    for e in range(mlp.experts):
        names.update({f"experts.{e}.{ours}": f"e{e}.{theirs}" for ours, theirs in _MLP_NAMES.items()})
    return PartSpec("routed_experts", {
        "hidden_size": config.hidden_size, "intermediate_size": mlp.ff, "experts": mlp.experts, "top": mlp.top,
        "groups": mlp.groups, "groups_keep": mlp.groups_keep, "activation": "capped_swiglu", "limit": mlp.limit,
        "alpha": EXPERT_GATE_SLOPE, "renormalise": False}), names


def kutolix_spec(config: KutolixConfig) -> ModelSpec:
    out_norm = PartSpec("rmsnorm_affine", {"size": config.hidden_size, "eps": config.norm_eps,
                                           "mult": config.residual_mult})
    layers, ignored = [], []
    for i, layer in enumerate(config.layers):
        mixer, mixer_names = _mixer(config, layer.mixer)
        parts = {"mixer": mixer, "mixer_out_norm": out_norm}
        prefixes = {"mixer": f"l{i}.mix.", "mixer_out_norm": f"l{i}.norm1"}
        renames = {"mixer": mixer_names, "mixer_out_norm": _BARE}
        if layer.mlp is not None:
            feed_forward, ff_names = _feed_forward(config, layer.mlp)
            parts.update({"feed_forward_out_norm": out_norm, "feed_forward": feed_forward})
            prefixes.update({"feed_forward": f"l{i}.mlp.", "feed_forward_out_norm": f"l{i}.norm2"})
            renames.update({"feed_forward": ff_names, "feed_forward_out_norm": _BARE})
        else:
            ignored.append(f"l{i}.norm2")
        layers.append(LayerSpec("output_norm" if layer.mlp is not None else "output_norm_mixer_only", parts, prefixes,
                                renames))
    sizes = {"vocab_size": config.vocab_size, "hidden_size": config.hidden_size}
    return ModelSpec(
        vocab_size=config.vocab_size, hidden_size=config.hidden_size,
        embedding=PartSpec("token_embedding", {**sizes, "scale": config.embedding_scale}), embedding_prefix="embed",
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm_affine", {"size": config.hidden_size, "eps": config.norm_eps}),
        final_norm_prefix="final.norm",
        head=PartSpec("linear", {**sizes, "softcap": config.logit_softcap}), head_prefix="head", tied={"head": "embed"},
        stream_dtype="float32",
        renames={"embedding": _BARE, "final_norm": _BARE, "head": _BARE},
        ignored=tuple(ignored),
    )


register_architecture("Kutolix", KutolixConfig, kutolix_spec, replace=True)
