"""Typed configuration of the Kutolix decoder, read from its config.json.

A Kutolix config.json names everything per layer:

    {"architecture": "Kutolix", "vocab": V, "width": D, "norm": {"eps": e}, "embedding": {"scale": s},
     "residual_mult": m, "logit_softcap": c,
     "layers": [{"type": "attention" | "latent_attention", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F}
                      | {"kind": "moe", "expert": {"ff": F, "limit": L},
                         "router": {"experts": E, "top": k, "groups": {"count": n, "keep": g}}}
                      | null}, ...]}

`attention` mixers give `heads, kv_heads, dim, vdim, scale`; `latent_attention` mixers give `heads, dim, rot_dim,
vdim, kv_rank, scale`; both optionally `mask: {size}` (a sliding window) and
`rot: {dims, base, scaling: {factor, original, fast, slow} | null}`.  Sizes have no defaults: a missing size is a
`ConfigError`.  An option that is absent or null is off (no window, no rotation, no frequency scaling, no expert
groups, no soft-cap, no feed-forward); `embedding.scale` and `residual_mult` absent are 1.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from liteinfer_b200.config.kegizen_config import YarnScaling, _need
from liteinfer_b200.config.model_config import ConfigError

MIXER_TYPES = ("attention", "latent_attention")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class KutolixRotation:
    dims: int
    base: float
    scaling: YarnScaling | None = None

    @classmethod
    def from_dict(cls, raw: dict[str, Any] | None, where: str) -> "KutolixRotation | None":
        if not raw or raw.get("dims") == 0:         # no dimension rotated: as good as no rotation
            return None
        scaling = None
        if raw.get("scaling"):
            s, at = raw["scaling"], where + ".scaling"
            scaling = YarnScaling(_need(s, "factor", float, at), _need(s, "original", float, at),
                                  _need(s, "fast", float, at), _need(s, "slow", float, at))
            if not scaling.factor > 0 or not scaling.original > 0:
                raise ConfigError(f"config.json {at}: factor and original must be > 0")
        rot = cls(_need(raw, "dims", int, where), _need(raw, "base", float, where), scaling)
        if rot.dims < 2 or rot.dims % 2 or not rot.base > 0:
            raise ConfigError(f"config.json {where}: dims={rot.dims} must be even and >= 2, base > 0")
        return rot

    def to_dict(self) -> dict[str, Any]:
        s = self.scaling
        return {"dims": self.dims, "base": self.base,
                "scaling": None if s is None else {"factor": s.factor, "original": s.original, "fast": s.fast,
                                                   "slow": s.slow}}


@dataclass(frozen=True)
class KutolixMixer:
    type: str
    heads: int
    dim: int                         # attention: size of a query/key head; latent_attention: its unrotated part
    vdim: int
    scale: float
    kv_heads: int = 0                # attention
    rot_dim: int = 0                 # latent_attention: the rotated part of a query/key head
    kv_rank: int = 0                 # latent_attention: size of the latent
    window: int | None = None        # a query at position p reads the keys at p - window + 1 ... p
    rot: KutolixRotation | None = None

    def __post_init__(self) -> None:
        if self.type not in MIXER_TYPES:
            raise ConfigError(f"mixer type {self.type!r} is not supported; known: {list(MIXER_TYPES)}")
        for name in ("heads", "dim", "vdim"):
            if getattr(self, name) < 1:
                raise ConfigError(f"mixer {name} must be >= 1, got {getattr(self, name)}")
        if self.window is not None and self.window < 1:
            raise ConfigError(f"mask.size must be >= 1, got {self.window}")
        if self.type == "attention":
            if self.kv_heads < 1 or self.heads % self.kv_heads:
                raise ConfigError(f"heads={self.heads} is not a multiple of kv_heads={self.kv_heads}")
            if self.rot is not None and self.rot.dims > self.dim:
                raise ConfigError(f"rot.dims={self.rot.dims} exceeds the head's {self.dim} dimensions")
        else:
            if self.kv_rank < 1 or self.rot_dim < 0:
                raise ConfigError("a latent_attention mixer needs kv_rank >= 1 and rot_dim >= 0")
            if self.rot is not None and self.rot.dims > self.rot_dim:
                raise ConfigError(f"rot.dims={self.rot.dims} exceeds the rotated part's {self.rot_dim} dimensions")

    @classmethod
    def from_dict(cls, kind: str, raw: dict[str, Any], where: str) -> "KutolixMixer":
        sizes = {name: _need(raw, name, int, where) for name in ("heads", "dim", "vdim")}
        mask = raw.get("mask")
        common = dict(scale=_need(raw, "scale", float, where), rot=KutolixRotation.from_dict(raw.get("rot"), where + ".rot"),
                      window=_need(mask, "size", int, where + ".mask") if mask else None)
        if kind == "attention":
            return cls(kind, kv_heads=_need(raw, "kv_heads", int, where), **sizes, **common)
        return cls(kind, rot_dim=_need(raw, "rot_dim", int, where), kv_rank=_need(raw, "kv_rank", int, where), **sizes,
                   **common)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.type == "attention":
            out["kv_heads"] = self.kv_heads
        else:
            out.update({"rot_dim": self.rot_dim, "kv_rank": self.kv_rank})
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class KutolixMLP:
    kind: str
    ff: int                          # dense: its width; moe: the width of one expert
    experts: int = 0
    top: int = 0
    limit: float = 0.0               # moe: the expert's gate is capped from above, its up product from both sides
    groups: int = 1                  # moe: experts form this many equal groups of neighbours ...
    groups_keep: int = 1             # ... of which only the best this many can be chosen from

    def __post_init__(self) -> None:
        if self.kind not in MLP_KINDS:
            raise ConfigError(f"mlp kind {self.kind!r} is not supported; known: {list(MLP_KINDS)}")
        if self.ff < 1:
            raise ConfigError(f"mlp ff must be >= 1, got {self.ff}")
        if self.kind == "moe":
            if self.experts < 1 or not 1 <= self.top <= self.experts or not self.limit > 0:
                raise ConfigError(f"a moe needs 1 <= top <= experts and limit > 0, got top={self.top}, "
                                  f"experts={self.experts}, limit={self.limit}")
            if self.groups < 1 or self.experts % self.groups or not 1 <= self.groups_keep <= self.groups:
                raise ConfigError(f"groups.count={self.groups} must divide experts={self.experts}, and 1 <= groups.keep "
                                  f"<= count")
            if self.groups_keep * (self.experts // self.groups) < self.top:
                raise ConfigError("the kept groups hold fewer experts than `top`")

    @classmethod
    def from_dict(cls, raw: dict[str, Any] | None, where: str) -> "KutolixMLP | None":
        if raw is None:
            return None
        kind = raw.get("kind", "dense")
        if kind == "dense":
            return cls("dense", _need(raw, "ff", int, where))
        if kind != "moe":
            raise ConfigError(f"config.json {where} has kind {kind!r}; known: {list(MLP_KINDS)}")
        expert, router = raw.get("expert"), raw.get("router")
        groups = (router or {}).get("groups")
        return cls("moe", _need(expert, "ff", int, where + ".expert"),
                   experts=_need(router, "experts", int, where + ".router"), top=_need(router, "top", int, where + ".router"),
                   limit=_need(expert, "limit", float, where + ".expert"),
                   groups=_need(groups, "count", int, where + ".router.groups") if groups else 1,
                   groups_keep=_need(groups, "keep", int, where + ".router.groups") if groups else 1)

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        router: dict[str, Any] = {"experts": self.experts, "top": self.top}
        if self.groups > 1:
            router["groups"] = {"count": self.groups, "keep": self.groups_keep}
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit}, "router": router}


@dataclass(frozen=True)
class KutolixLayer:
    mixer: KutolixMixer
    mlp: KutolixMLP | None


@dataclass(frozen=True)
class KutolixConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple[KutolixLayer, ...]
    embedding_scale: float = 1.0
    residual_mult: float = 1.0
    logit_softcap: float | None = None
    eos_token_id: tuple[int, ...] = ()
    architecture: str = "Kutolix"

    def __post_init__(self) -> None:
        if self.vocab_size < 1 or self.hidden_size < 1:
            raise ConfigError("vocab and width must be >= 1")
        if not self.layers:
            raise ConfigError("config.json names no layer")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be > 0")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError("logit_softcap must be > 0 (or absent)")

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "KutolixConfig":
        if not isinstance(raw.get("layers"), list):
            raise ConfigError("config.json has no 'layers' list")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            kind = entry.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json {where} has type {kind!r}; known: {list(MIXER_TYPES)}")
            layers.append(KutolixLayer(KutolixMixer.from_dict(kind, entry.get("mixer"), where + ".mixer"),
                                       KutolixMLP.from_dict(entry.get("mlp"), where + ".mlp")))
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        embedding = raw.get("embedding") or {}
        cap = raw.get("logit_softcap")
        return cls(vocab_size=_need(raw, "vocab", int, ""), hidden_size=_need(raw, "width", int, ""),
                   norm_eps=_need(raw.get("norm"), "eps", float, "norm"), layers=tuple(layers),
                   embedding_scale=float(embedding.get("scale", 1.0) if embedding.get("scale") is not None else 1.0),
                   residual_mult=float(raw["residual_mult"]) if raw.get("residual_mult") is not None else 1.0,
                   logit_softcap=float(cap) if cap else None, eos_token_id=eos_ids,
                   architecture=str(raw.get("architecture", "Kutolix")))

    def to_dict(self) -> dict[str, Any]:
        """config.json contents that `from_dict` reads back to an equal config."""
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
            "residual_mult": self.residual_mult,
            "layers": [{"type": layer.mixer.type, "mixer": layer.mixer.to_dict(),
                        "mlp": None if layer.mlp is None else layer.mlp.to_dict()} for layer in self.layers],
        }
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
