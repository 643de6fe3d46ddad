"""Tiny Kutolix configurations for the tests: they differ in every size, option and layer order.

KUT_A: starts with a latent attention (three heads, a window of 13, YaRN frequencies) and a mixture of six experts
in three groups of which two are kept; a gated attention with two key/value heads for four query heads, a quarter of
each head rotated, a window of 9; a latent layer without feed-forward; an attention layer with experts.
KUT_B: what a configuration may leave out: no windows in two layers, no embedding scale, no residual multiplier, no
soft-cap, experts without groups with the best one of three chosen; a window of one token (a position sees itself
only); one head; every dimension rotated; a latent layer whose frequencies are not scaled.
KUT_C: sizes of the tensor-core kernels (keys and values of 64 with windows longer than a tile of keys, a latent of
64 with a rotated part of 32, experts whose products run on tensor-core tiles).
KUT_D: small sizes that are multiples of little (width 36, heads of 6 with 2 dimensions rotated, values of 10, a
latent of 20 with a rotated part of 4, eight experts in four groups of which one is kept, experts 10 wide; an
attention layer whose frequencies are scaled too).
KUT_E: a width of 512 with heads of 128 x 128 and windows of some hundred tokens, a latent of 128 with a rotated
part of 64: prompts of a few hundred tokens take the tensor-core products and attention kernels.
"""

import random

KUT_A = {
    "architecture": "Kutolix", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.7},
    "residual_mult": 0.6, "logit_softcap": 9.0,
    "layers": [
        {"type": "latent_attention",
         "mixer": {"heads": 3, "dim": 12, "rot_dim": 8, "vdim": 10, "kv_rank": 24, "scale": 0.21, "mask": {"size": 13},
                   "rot": {"dims": 8, "base": 1000.0,
                           "scaling": {"factor": 3.0, "original": 16, "fast": 8.0, "slow": 1.0}}},
         "mlp": {"kind": "moe", "expert": {"ff": 20, "limit": 1.5},
                 "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}}},
        {"type": "attention",
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 12, "scale": 0.3, "mask": {"size": 9},
                   "rot": {"dims": 4, "base": 500.0}},
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "latent_attention",
         "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 16, "kv_rank": 12, "scale": 0.4, "mask": {"size": 30},
                   "rot": {"dims": 4, "base": 100.0,
                           "scaling": {"factor": 8.0, "original": 8, "fast": 4.0, "slow": 0.5}}},
         "mlp": None},
        {"type": "attention",
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 8, "scale": 0.25, "mask": {"size": 17},
                   "rot": {"dims": 24, "base": 10000.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 12, "limit": 0.8},
                 "router": {"experts": 4, "top": 3, "groups": {"count": 2, "keep": 2}}}},
    ],
}

KUT_B = {
    "architecture": "Kutolix", "vocab": 129, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention",
         "mixer": {"heads": 1, "kv_heads": 1, "dim": 20, "vdim": 28, "scale": 0.5, "rot": {"dims": 20, "base": 50.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 16, "limit": 3.0}, "router": {"experts": 3, "top": 1}}},
        {"type": "latent_attention",
         "mixer": {"heads": 2, "dim": 10, "rot_dim": 6, "vdim": 7, "kv_rank": 18, "scale": 0.3,
                   "rot": {"dims": 6, "base": 300.0}},
         "mlp": {"kind": "dense", "ff": 24}},
        {"type": "attention",
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 8, "vdim": 8, "scale": 0.35, "mask": {"size": 1}},
         "mlp": None},
        {"type": "latent_attention",
         "mixer": {"heads": 1, "dim": 16, "rot_dim": 2, "vdim": 24, "kv_rank": 9, "scale": 0.2, "mask": {"size": 5},
                   "rot": {"dims": 2, "base": 20.0, "scaling": {"factor": 2.0, "original": 4, "fast": 2.0, "slow": 1.0}}},
         "mlp": {"kind": "dense", "ff": 20}},
    ],
}

KUT_C = {
    "architecture": "Kutolix", "vocab": 200, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
    "residual_mult": 0.8, "logit_softcap": 20.0,
    "layers": [
        {"type": "attention",
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.15, "mask": {"size": 70},
                   "rot": {"dims": 32, "base": 5000.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 64, "limit": 2.5},
                 "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 3}}}},
        {"type": "latent_attention",
         "mixer": {"heads": 4, "dim": 32, "rot_dim": 32, "vdim": 32, "kv_rank": 64, "scale": 0.12, "mask": {"size": 45},
                   "rot": {"dims": 32, "base": 10000.0,
                           "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}}},
         "mlp": {"kind": "dense", "ff": 96}},
        {"type": "attention",
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 64, "scale": 0.11, "mask": {"size": 128},
                   "rot": {"dims": 64, "base": 5000.0}},
         "mlp": None},
        {"type": "latent_attention",
         "mixer": {"heads": 2, "dim": 64, "rot_dim": 32, "vdim": 48, "kv_rank": 64, "scale": 0.1, "mask": {"size": 100},
                   "rot": {"dims": 32, "base": 2000.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 32, "limit": 1.0}, "router": {"experts": 4, "top": 4}}},
    ],
}

KUT_D = {
    "architecture": "Kutolix", "vocab": 97, "width": 36, "norm": {"eps": 1e-4}, "embedding": {"scale": 2.0},
    "residual_mult": 0.3, "logit_softcap": 5.0,
    "layers": [
        {"type": "attention",
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 6, "vdim": 10, "scale": 0.5, "mask": {"size": 4},
                   "rot": {"dims": 2, "base": 37.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 10, "limit": 0.5},
                 "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 1}}}},
        {"type": "attention",
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 4, "scale": 0.2, "mask": {"size": 21},
                   "rot": {"dims": 8, "base": 900.0,
                           "scaling": {"factor": 2.5, "original": 16, "fast": 8.0, "slow": 1.0}}},
         "mlp": {"kind": "dense", "ff": 28}},
        {"type": "latent_attention",
         "mixer": {"heads": 5, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 20, "scale": 0.33, "mask": {"size": 8},
                   "rot": {"dims": 4, "base": 60.0,
                           "scaling": {"factor": 16.0, "original": 32, "fast": 4.0, "slow": 2.0}}},
         "mlp": {"kind": "moe", "expert": {"ff": 7, "limit": 4.0},
                 "router": {"experts": 5, "top": 2, "groups": {"count": 1, "keep": 1}}}},
    ],
}

KUT_E = {
    "architecture": "Kutolix", "vocab": 1500, "width": 512, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
    "residual_mult": 0.7, "logit_softcap": 30.0,
    "layers": [
        {"type": "attention",
         "mixer": {"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.088, "mask": {"size": 200},
                   "rot": {"dims": 64, "base": 10000.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 256, "limit": 7.0},
                 "router": {"experts": 8, "top": 2, "groups": {"count": 2, "keep": 1}}}},
        {"type": "latent_attention",
         "mixer": {"heads": 4, "dim": 64, "rot_dim": 64, "vdim": 64, "kv_rank": 128, "scale": 0.09, "mask": {"size": 180},
                   "rot": {"dims": 64, "base": 10000.0,
                           "scaling": {"factor": 6.0, "original": 128, "fast": 24.0, "slow": 1.0}}},
         "mlp": {"kind": "dense", "ff": 768}},
        {"type": "attention",
         "mixer": {"heads": 4, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 0.1, "mask": {"size": 333},
                   "rot": {"dims": 128, "base": 20000.0}},
         "mlp": {"kind": "dense", "ff": 1024}},
    ],
}

# name -> (config, seed, page size)
ALL = {"kut_a": (KUT_A, 41, 16), "kut_b": (KUT_B, 42, 4), "kut_c": (KUT_C, 43, 16), "kut_d": (KUT_D, 44, 8),
       "kut_e": (KUT_E, 45, 16)}


def random_config(seed: int) -> dict:
    """A configuration drawn at random: three to six layers of either mixer with sizes of the SIMT kernels and of the
    tensor-core ones, windows or none, rotations or none, every kind of feed-forward or none."""
    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(3, 6)):
        window = rng.choice([None, 17, 24, 50, 64, 100, 130])
        if rng.random() < 0.5:
            dim = rng.choice([32, 48, 64, 128])
            heads = rng.choice([2, 4, 6, 8])
            mixer = {"heads": heads, "kv_heads": rng.choice([k for k in (1, 2, 3, 4, 8) if heads % k == 0]), "dim": dim,
                     "vdim": rng.choice([dim, dim, 32, 64, 128]), "scale": dim ** -0.5}
            if rng.random() < 0.8:
                mixer["rot"] = {"dims": rng.choice([d for d in (8, 16, 32, 64, 128) if d <= dim]),
                                "base": rng.choice([10000.0, 100000.0, 500.0])}
            kind = "attention"
        else:
            kv_rank, rot_dim = rng.choice([(64, 32), (128, 32), (128, 64), (128, 8), (96, 16), (256, 64), (48, 8)])
            scaling = rng.choice([None, {"factor": rng.choice([2.0, 3.0, 8.0]), "original": rng.choice([64, 256, 2048]),
                                         "fast": rng.choice([16.0, 32.0]), "slow": 1.0}])
            mixer = {"heads": rng.choice([2, 4, 8]), "dim": rng.choice([16, 32, 64]), "rot_dim": rot_dim,
                     "vdim": rng.choice([24, 32, 48, 64]), "kv_rank": kv_rank, "scale": 0.12,
                     "rot": {"dims": rot_dim, "base": 10000.0, "scaling": scaling}}
            kind = "latent_attention"
        if window:
            mixer["mask"] = {"size": window}
        draw = rng.random()
        if draw < 0.15:
            mlp = None
        elif draw < 0.55:
            mlp = {"kind": "dense", "ff": rng.choice([64, 200, 320, 512])}
        else:
            groups, per = rng.choice([1, 2, 4]), rng.choice([2, 3, 4])
            keep = rng.randint(1, groups)
            router = {"experts": groups * per, "top": rng.randint(1, min(keep * per, 4))}
            if groups > 1 or rng.random() < 0.5:
                router["groups"] = {"count": groups, "keep": keep}
            mlp = {"kind": "moe", "expert": {"ff": rng.choice([24, 64, 96, 128]), "limit": rng.choice([1.0, 3.0, 7.0])},
                   "router": router}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    config = {"architecture": "Kutolix", "vocab": rng.choice([300, 777, 1000]), "width": rng.choice([96, 128, 160, 256, 320]),
              "norm": {"eps": 1e-5}, "layers": layers}
    if rng.random() < 0.8:
        config["embedding"] = {"scale": rng.choice([0.25, 2.0, 1.3])}
    if rng.random() < 0.8:
        config["residual_mult"] = rng.choice([0.4, 0.7, 1.5])
    if rng.random() < 0.8:
        config["logit_softcap"] = rng.choice([12.0, 30.0, 8.0])
    return config


def prompt(vocab: int, length: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(length)]


# Largest absolute difference of float32 logits from the float64 plain implementation that rounding alone explains.
FLOAT32_TOLERANCE = {"kut_a": 5e-5, "kut_b": 5e-5, "kut_c": 1e-4, "kut_d": 5e-5, "kut_e": 2e-4}
# The same for bfloat16 (products' operands, pages and the sublayers' outputs are rounded; logits are of size 1).
BFLOAT16_TOLERANCE = {"kut_a": 0.08, "kut_b": 0.08, "kut_c": 0.12, "kut_d": 0.08, "kut_e": 0.3}
