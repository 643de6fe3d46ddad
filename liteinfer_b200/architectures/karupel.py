"""The Karupel decoder as a `ModelSpec`.

Every layer has one of three mixers (an mLSTM matrix memory, a gated delta-rule recurrence, a softmax attention with
per-head query/key norms, a per-head output gate and values mixed with those of the first such layer) and an
optional gated feed-forward.  The sublayers read the residual stream as it is; only what they give back is
normalised: x <- x + norm(sublayer(x)), an RMS norm whose stored weight lies around zero (1 + w multiplies).  The
residual stream is summed in 32-bit; the head is the embedding's table.  Tensor names: `embed`,
`l<i>.norm1|norm2`, `l<i>.mix.*`, `l<i>.mlp.gate|up|down`, `final.norm`.
"""

from __future__ import annotations

from liteinfer_b200.config.karupel_config import KarupelConfig, KarupelMixer
from liteinfer_b200.config.registry import register_architecture
from liteinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_BARE = {"weight": ""}      # a tensor stored under the part's prefix itself
_ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                    "q_proj.bias": "q.b", "k_proj.bias": "k.b", "v_proj.bias": "v.b", "q_norm.weight": "q.norm",
                    "k_norm.weight": "k.norm", "g_proj.weight": "g", "value_mix": "vmix"}
_DELTA_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "g_proj.weight": "g",
                "b_proj.weight": "b", "a_proj.weight": "a", "o_proj.weight": "o", "q_conv.weight": "q.conv",
                "k_conv.weight": "k.conv", "v_conv.weight": "v.conv", "norm.weight": "norm"}
_MLSTM_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "g_proj.weight": "g",
                "o_proj.weight": "o", "norm.weight": "norm", "i_proj.weight": "i", "i_proj.bias": "i.b",
                "f_proj.weight": "f", "f_proj.bias": "f.b"}
_MLP_NAMES = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}

VALUE_MIX_KEY = "karupel.first_values"      # where a step keeps the first mixing layer's values for the later ones


def _mixer(config: KarupelConfig, mixer: KarupelMixer, value_mix: str | None) -> tuple[PartSpec, dict[str, str]]:
    if mixer.type == "mlstm":
        return PartSpec("mlstm", {"hidden_size": config.hidden_size, "heads": mixer.heads, "dim": mixer.dim,
                                  "vdim": mixer.vdim, "gate_cap": mixer.gate_cap,
                                  "norm_eps": config.norm_eps}), _MLSTM_NAMES
    sizes = {"hidden_size": config.hidden_size, "heads": mixer.heads, "kv_heads": mixer.kv_heads}
    if mixer.type == "delta":
        return PartSpec("gated_delta_rule", {**sizes, "dim": mixer.dim, "vdim": mixer.vdim, "conv": mixer.conv,
                                             "norm_eps": config.norm_eps}), _DELTA_NAMES
    if mixer.rot is None:
        position = PartSpec("none", {})
    else:
        scaled = mixer.rot.factor is not None
        position = PartSpec("rotary", {"head_dim": mixer.dim, "rotary_dim": mixer.rot.dims, "theta": mixer.rot.base,
                                       "rope_type": "linear" if scaled else "default",
                                       "factor": mixer.rot.factor if scaled else 1.0})
    return PartSpec("attention", {**sizes, "head_dim": mixer.dim, "v_head_dim": mixer.vdim, "position": position,
                                  "scale": mixer.scale, "bias": True, "out_bias": False, "qk_norm": "head",
                                  "qk_norm_eps": config.norm_eps, "head_gate": True, "value_mix": value_mix,
                                  "value_mix_key": VALUE_MIX_KEY}), _ATTENTION_NAMES


def karupel_spec(config: KarupelConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm_unit_offset", {"size": config.hidden_size, "eps": config.norm_eps})
    layers, ignored = [], []
    mixing = [i for i, layer in enumerate(config.layers) if layer.mixer.v_mix]
    for i, layer in enumerate(config.layers):
        value_mix = None
        if layer.mixer.v_mix and len(mixing) > 1:
            value_mix = "source" if i == mixing[0] else "mixed"
        if layer.mixer.type == "attention" and value_mix != "mixed":
            ignored.append(f"l{i}.mix.vmix")        # stored for every attention layer, read only where values are mixed
        mixer, mixer_names = _mixer(config, layer.mixer, value_mix)
        parts = {"mixer": mixer, "mixer_out_norm": norm}
        prefixes = {"mixer": f"l{i}.mix.", "mixer_out_norm": f"l{i}.norm1"}
        renames = {"mixer": mixer_names, "mixer_out_norm": _BARE}
        if layer.ff is not None:
            parts.update({"feed_forward_out_norm": norm, "feed_forward": PartSpec(
                "gated_mlp", {"hidden_size": config.hidden_size, "intermediate_size": layer.ff, "activation": "silu"})})
            prefixes.update({"feed_forward": f"l{i}.mlp.", "feed_forward_out_norm": f"l{i}.norm2"})
            renames.update({"feed_forward": _MLP_NAMES, "feed_forward_out_norm": _BARE})
        else:
            ignored.append(f"l{i}.norm2")
        layers.append(LayerSpec("output_norm" if layer.ff is not None else "output_norm_mixer_only", parts, prefixes,
                                renames))
    sizes = {"vocab_size": config.vocab_size, "hidden_size": config.hidden_size}
    return ModelSpec(
        vocab_size=config.vocab_size, hidden_size=config.hidden_size,
        embedding=PartSpec("token_embedding", sizes), embedding_prefix="embed",
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear", sizes), head_prefix="head", tied={"head": "embed"},
        stream_dtype="float32",
        renames={"embedding": _BARE, "final_norm": _BARE, "head": _BARE},
        ignored=tuple(ignored),
    )


register_architecture("Karupel", KarupelConfig, karupel_spec, replace=True)
