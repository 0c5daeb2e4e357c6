"""Tiny Ketalix configurations for the tests.  They differ in every size and option: widths,
vocabularies, head counts and groups, key and value sizes (equal, larger, smaller), rotated
part of a head, windows (none, a few tokens, longer than a page), caps, layer orders (which
mixer comes first, layers without a feed-forward, attention layers that blend values or do
not), decay temperatures and ranks, embedding scales, and the cache's page size."""

from __future__ import annotations


def _attn(heads, kv, dim, vdim, scale, window=None, softcap=None, rot=None, base=10000.0, v_mix=False):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if window is not None:
        m["mask"] = {"size": window}
    if softcap is not None:
        m["softcap"] = softcap
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    return m


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


KX_A = {
    "architecture": "Ketalix", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "layers": [
        _layer("attention", _attn(4, 2, 16, 24, 0.6, window=9, softcap=15.0, rot=8, v_mix=True), 96),
        _layer("gla", {"heads": 2, "dim": 12, "vdim": 20, "tau": 8.0, "rank": 5}, 80),
        _layer("attention", _attn(4, 2, 16, 24, 0.6, window=20, softcap=15.0, rot=8, v_mix=True), None),
        _layer("gla", {"heads": 3, "dim": 20, "vdim": 8, "tau": 4.0, "rank": 3}, None),
        _layer("attention", _attn(6, 2, 8, 24, 0.9, window=33, softcap=6.0, rot=8, base=500.0, v_mix=True), 72),
    ],
}
KX_B = {
    "architecture": "Ketalix", "vocab": 157, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        _layer("gla", {"heads": 1, "dim": 40, "vdim": 40, "tau": 2.0, "rank": 8}, 64),
        _layer("attention", _attn(3, 3, 32, 32, 0.4, rot=32, base=1e6), 56),
        _layer("attention", _attn(4, 1, 8, 40, 1.2, window=3, softcap=30.0, rot=4, v_mix=True), None),
        _layer("gla", {"heads": 4, "dim": 6, "vdim": 10, "tau": 32.0, "rank": 2}, 40),
    ],
}
# head sizes that tensor-core attention kernels take, a state wider than one block of value channels
KX_C = {
    "architecture": "Ketalix", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
    "layers": [
        _layer("attention", _attn(4, 2, 64, 64, 0.25, window=40, softcap=12.0, rot=32, v_mix=True), 192),   # blocks of 64: the products apply the gate
        _layer("gla", {"heads": 2, "dim": 64, "vdim": 80, "tau": 16.0, "rank": 4}, None),
        _layer("attention", _attn(4, 2, 64, 64, 0.25, softcap=12.0, rot=64, v_mix=True), 96),
    ],
}
# (configuration, how the random weights are drawn, page size)
ALL = {
    "KA": (KX_A, {"seed": 11, "std": 0.08, "norm_std": 0.1}, 16),
    "KB": (KX_B, {"seed": 12, "std": 0.1, "norm_std": 0.1}, 8),
    "KC": (KX_C, {"seed": 13, "std": 0.06, "norm_std": 0.1}, 32),
}
