"""Typed configuration of the Karupel decoder, read from its config.json.

A Karupel config.json names everything per layer:

    {"architecture": "Karupel", "vocab": V, "width": D, "norm": {"eps": e},
     "layers": [{"type": "mlstm" | "delta" | "attention", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F} | null}, ...]}

`mlstm` mixers give `heads, dim, vdim, gate_cap`; `delta` mixers give `heads, kv_heads, dim, vdim, conv`;
`attention` mixers give `heads, kv_heads, dim, vdim, scale` and optionally `v_mix` and
`rot: {dims, base, scaling: {factor} | null}`.  Sizes have no defaults: a missing size is a `ConfigError`.  An
option that is absent, null or false is off (no rotation, no frequency scaling, no value mixing, no feed-forward).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from liteinfer_b200.config.kegizen_config import _need
from liteinfer_b200.config.model_config import ConfigError

MIXER_TYPES = ("mlstm", "delta", "attention")


@dataclass(frozen=True)
class KarupelRotation:
    dims: int
    base: float
    factor: float | None = None      # linear scaling: every frequency is divided by it; None = unscaled


@dataclass(frozen=True)
class KarupelMixer:
    type: str
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0                # delta, attention: heads of q/k (delta) or of k/v (attention)
    conv: int = 0                    # delta: taps of the short convolutions
    gate_cap: float = 0.0            # mlstm: the raw gates pass cap * tanh(x / cap)
    scale: float = 0.0               # attention: what a score is multiplied by
    v_mix: bool = False              # attention: values are mixed with those of the first such layer
    rot: KarupelRotation | None = None

    def __post_init__(self) -> None:
        if self.type not in MIXER_TYPES:
            raise ConfigError(f"mixer type {self.type!r} is not supported; known: {list(MIXER_TYPES)}")
        for name in ("heads", "dim", "vdim"):
            if getattr(self, name) < 1:
                raise ConfigError(f"mixer {name} must be >= 1, got {getattr(self, name)}")
        if self.type != "mlstm":
            if self.kv_heads < 1 or self.heads % self.kv_heads:
                raise ConfigError(f"heads={self.heads} is not a multiple of kv_heads={self.kv_heads}")
        if self.type == "delta" and self.conv < 1:
            raise ConfigError("a delta mixer needs conv >= 1")
        if self.type == "mlstm" and not self.gate_cap > 0:
            raise ConfigError("an mlstm mixer needs gate_cap > 0")
        if self.rot is not None:
            if self.rot.dims < 2 or self.rot.dims % 2 or self.rot.dims > self.dim:
                raise ConfigError(f"rot.dims={self.rot.dims} must be even and within the head's {self.dim} dimensions")
            if self.rot.factor is not None and not self.rot.factor > 0:
                raise ConfigError("rot.scaling.factor must be > 0")

    @classmethod
    def from_dict(cls, kind: str, raw: dict[str, Any], where: str) -> KarupelMixer:
        sizes = {name: _need(raw, name, int, where) for name in ("heads", "dim", "vdim")}
        if kind == "mlstm":
            return cls(kind, gate_cap=_need(raw, "gate_cap", float, where), **sizes)
        sizes["kv_heads"] = _need(raw, "kv_heads", int, where)
        if kind == "delta":
            return cls(kind, conv=_need(raw, "conv", int, where), **sizes)
        rot = None
        if raw.get("rot") and raw["rot"].get("dims") != 0:      # no dimension rotated: as good as no rotation
            r = raw["rot"]
            factor = _need(r["scaling"], "factor", float, where + " rot.scaling") if r.get("scaling") else None
            rot = KarupelRotation(_need(r, "dims", int, where + " rot"), _need(r, "base", float, where + " rot"), factor)
        return cls(kind, scale=_need(raw, "scale", float, where), v_mix=bool(raw.get("v_mix")), rot=rot, **sizes)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.type == "mlstm":
            out["gate_cap"] = self.gate_cap
            return out
        out["kv_heads"] = self.kv_heads
        if self.type == "delta":
            out["conv"] = self.conv
            return out
        out["scale"] = self.scale
        if self.v_mix:
            out["v_mix"] = True
        if self.rot is not None:
            out["rot"] = {"dims": self.rot.dims, "base": self.rot.base,
                          "scaling": None if self.rot.factor is None else {"factor": self.rot.factor}}
        return out


@dataclass(frozen=True)
class KarupelLayer:
    mixer: KarupelMixer
    ff: int | None                   # width of the gated feed-forward; None = the layer has none


@dataclass(frozen=True)
class KarupelConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple[KarupelLayer, ...]
    eos_token_id: tuple[int, ...] = ()
    architecture: str = "Karupel"

    def __post_init__(self) -> None:
        if self.vocab_size < 1 or self.hidden_size < 1:
            raise ConfigError("vocab and width must be >= 1")
        if not self.layers:
            raise ConfigError("config.json names no layer")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be > 0")
        mixing = [layer.mixer for layer in self.layers if layer.mixer.v_mix]
        for mixer in mixing[1:]:
            if (mixer.kv_heads, mixer.vdim) != (mixing[0].kv_heads, mixing[0].vdim):
                raise ConfigError("layers that mix values need values of one shape: "
                                  f"{mixer.kv_heads} x {mixer.vdim} against {mixing[0].kv_heads} x {mixing[0].vdim}")

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> KarupelConfig:
        if not isinstance(raw.get("layers"), list):
            raise ConfigError("config.json has no 'layers' list")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            kind = entry.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json {where} has type {kind!r}; known: {list(MIXER_TYPES)}")
            mixer = KarupelMixer.from_dict(kind, entry.get("mixer"), where + ".mixer")
            mlp = entry.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"config.json {where}.mlp has kind {mlp.get('kind')!r}; known: ['dense']")
            layers.append(KarupelLayer(mixer, None if mlp is None else _need(mlp, "ff", int, where + ".mlp")))
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab_size=_need(raw, "vocab", int, ""), hidden_size=_need(raw, "width", int, ""),
                   norm_eps=_need(raw.get("norm"), "eps", float, "norm"), layers=tuple(layers), eos_token_id=eos_ids,
                   architecture=str(raw.get("architecture", "Karupel")))

    def to_dict(self) -> dict[str, Any]:
        """config.json contents that `from_dict` reads back to an equal config."""
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": layer.mixer.type, "mixer": layer.mixer.to_dict(),
                        "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}} for layer in self.layers],
        }
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
