"""Tiny Logivik configurations for the tests.  They differ in every size and option: widths (also one
that is no multiple of 8), vocabularies, head counts and groups of the delta rule (1, 2, all heads on
one key head), key and value sizes (equal, larger, smaller, wider than one block of the recurrence),
convolutions of 1 to 5 taps, latent sizes, rotated parts (all of it turned, or only its first
elements), stretched and unstretched rotations, windows (1, a few tokens, longer than a page), layer
orders (each mixer comes first somewhere, layers without a feed-forward), embedding scales, and the
cache's page size."""

from __future__ import annotations


def _delta(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _latent(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, dims=None, scaling=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": rot}


def _window(heads, dim, vdim, rank, q_rank, scale, window):
    return {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank, "scale": scale,
            "mask": {"size": window}}


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


LV_A = {
    "architecture": "Logivik", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "layers": [
        _layer("delta", _delta(4, 2, 16, 24, 3), 96),
        _layer("latent_attention", _latent(3, 16, 8, 20, 24, 0.3, scaling=(4.0, 32, 8.0, 1.0)), None),
        _layer("latent_attention_2", _window(2, 24, 16, 40, 12, 0.2, 9), 80),
        _layer("delta", _delta(2, 2, 20, 8, 2), None),
        _layer("latent_attention_2", _window(5, 8, 12, 16, 20, 0.35, 33), 72),
    ],
}
LV_B = {
    "architecture": "Logivik", "vocab": 157, "width": 52, "norm": {"eps": 1e-6},
    "layers": [
        _layer("latent_attention", _latent(4, 8, 12, 40, 16, 0.4, base=500.0, dims=8), 64),
        _layer("delta", _delta(6, 1, 12, 10, 5), 56),
        _layer("latent_attention_2", _window(1, 32, 32, 8, 8, 0.18, 3), None),
        _layer("delta", _delta(3, 3, 6, 40, 1), 40),
        _layer("latent_attention_2", _window(3, 12, 20, 24, 16, 0.3, 1), None),
    ],
}
# sizes that the products' own kernels take (blocks of 64 in the feed-forward), a state wider than one
# block of value channels, a key size that is no multiple of the rows a thread holds
LV_C = {
    "architecture": "Logivik", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
    "layers": [
        _layer("latent_attention_2", _window(4, 64, 32, 64, 48, 0.125, 40), 192),
        _layer("delta", _delta(2, 1, 130, 80, 4), None),
        _layer("latent_attention", _latent(4, 32, 64, 48, 96, 0.1, base=1e6, scaling=(2.0, 64, 16.0, 2.0)), 128),
        _layer("delta", _delta(4, 2, 64, 64, 4), 64),
    ],
}
# latents in steps of 16 (the tensor-core attention kernels) with head counts that fill no tile evenly, values
# narrower than one warp's share of columns, a rotated part turned only in its first half
LV_D = {
    "architecture": "Logivik", "vocab": 333, "width": 192, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
    "layers": [
        _layer("delta", _delta(6, 3, 96, 48, 2), 160),
        _layer("latent_attention", _latent(5, 24, 16, 40, 48, 0.16, base=2000.0, dims=8, scaling=(3.0, 48, 6.0, 1.5)), None),
        _layer("latent_attention_2", _window(7, 16, 24, 32, 40, 0.25, 20), 96),
        _layer("latent_attention", _latent(18, 8, 32, 16, 80, 0.2), 64),
    ],
}
# a latent attention layer with sink and gate but no rotated part (and so no positions at all in the model)
LV_E = {
    "architecture": "Logivik", "vocab": 120, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        _layer("latent_attention", {"heads": 4, "dim": 16, "rot_dim": 0, "vdim": 16, "kv_rank": 32, "scale": 0.25}, 64),
        _layer("delta", _delta(2, 2, 32, 32, 4), None),
    ],
}
# (configuration, how the random weights are drawn, page size)
ALL = {
    "LA": (LV_A, {"seed": 21, "std": 0.08, "norm_std": 0.1}, 16),
    "LB": (LV_B, {"seed": 22, "std": 0.1, "norm_std": 0.1}, 8),
    "LC": (LV_C, {"seed": 23, "std": 0.06, "norm_std": 0.1}, 32),
    "LD": (LV_D, {"seed": 24, "std": 0.07, "norm_std": 0.1}, 16),
    "LE": (LV_E, {"seed": 25, "std": 0.1, "norm_std": 0.1}, 16),
}
