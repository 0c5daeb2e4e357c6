"""The Logivik design without a GPU: the reader of config.json and its refusals, the tensors it
expects, the cache needs of its mixers, the stretched rotation's frequencies, and the plain
implementation's own consistency."""

from __future__ import annotations

import copy
import math

import pytest
import torch

import logivik_configs as lc
from plain import logivik_plain as plain
from tokamak_b200.cache.manager import KVPagesNeed, StateNeed
from tokamak_b200.config.model_config import ConfigError
from tokamak_b200.config.registry import architecture_of, supported_architectures
from tokamak_b200.models.decoder import DecoderModel


def spec_of(raw):
    arch = architecture_of(raw)
    return arch.build_spec(arch.parse(raw))


def test_registered_and_parsed():
    assert "Logivik" in supported_architectures()
    arch = architecture_of(lc.LV_A)
    cfg = arch.parse(lc.LV_A)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps, cfg.embedding_scale) == (211, 64, 1e-5, 3.0)
    assert [l.type for l in cfg.layers] == [l["type"] for l in lc.LV_A["layers"]]
    assert cfg.layers[0].mixer.conv == 3 and cfg.layers[3].ff is None
    rot = cfg.layers[1].mixer
    assert rot.rot_dims == 8 and rot.yarn.factor == 4.0 and rot.sinks and rot.gate and rot.window is None
    win = cfg.layers[2].mixer
    assert win.window == 9 and win.q_rank == 12 and not win.sinks and not win.gate and win.rot_dim == 0
    assert arch.parse(lc.LV_B).embedding_scale == 1.0
    assert arch.parse(lc.LV_B).layers[0].mixer.yarn is None
    with pytest.raises(ConfigError):
        arch.build_spec(cfg, window=8)           # the design has windows of its own per layer


def test_expected_tensors_and_cache_needs():
    spec = spec_of(lc.LV_A)
    names = DecoderModel.expected_tensors(spec)
    assert names["embed"].shape == (211, 64) and names["head"].shape == (211, 64) and names["final.norm"].shape == (64,)
    assert names["l0.mix.q.conv"].shape == (32, 3) and names["l0.mix.v.conv"].shape == (96, 3)
    assert names["l0.mix.b"].shape == (4, 64) and names["l0.mix.A_log"].shape == (4,) and names["l0.mix.norm"].shape == (24,)
    assert names["l1.mix.q"].shape == (3 * 24, 64) and names["l1.mix.dkv"].shape == (32, 64)
    assert names["l1.mix.dkv.norm"].shape == (24,) and names["l1.mix.uk"].shape == (48, 24) and names["l1.mix.uv"].shape == (60, 24)
    assert names["l1.mix.sink"].shape == (3,) and names["l1.mix.g"].shape == (60, 64) and names["l1.mix.o"].shape == (64, 60)
    assert names["l2.mix.dq"].shape == (12, 64) and names["l2.mix.uq"].shape == (48, 12) and names["l2.mix.dkv"].shape == (40, 64)
    assert "l2.mix.sink" not in names and "l2.mix.g" not in names and "l1.norm2" not in names and "l1.mlp.gate" not in names
    assert names["l0.norm1"].role == "bias" and names["l2.mlp.down"].shape == (64, 80)
    # a latent cache keeps one row per token, values inside the keys; the delta rule one record per request
    from tokamak_b200.parts.base import MIXERS
    needs = {}
    for block in spec.blocks:
        cls = MIXERS.get(block.mixer.kind)
        part = cls.__new__(cls)
        part.spec = block.mixer
        if block.mixer.kind == "gated_delta":
            from tokamak_b200.csrc.ops import delta_record_floats
            part.record_floats, _ = delta_record_floats(block.mixer.num_heads, block.mixer.num_kv_heads, block.mixer.key_dim,
                                                        block.mixer.value_dim, block.mixer.conv_taps)
        needs[block.name] = part.cache_need()
    assert needs["l1"] == KVPagesNeed(1, 32, None, 24, values_in_keys=True) and needs["l1"].stored_dim == 32
    assert needs["l2"] == KVPagesNeed(1, 40, 9, 40, values_in_keys=True)
    assert needs["l0"] == StateNeed((4 * 16 * 24 + 2 * (2 * 32 + 96),), "float32")
    assert needs["l3"] == StateNeed((2 * 20 * 8 + 1 * (2 * 40 + 16),), "float32")
    assert KVPagesNeed(2, 16, None, 24).stored_dim == 40


@pytest.mark.parametrize("change,message", [
    (lambda r: r["layers"][0].update(type="conv"), "not a mixer"),
    (lambda r: r["layers"][0]["mixer"].pop("conv"), "conv"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda r: r["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"]["rot"].pop("base"), "base"),
    (lambda r: r["layers"][1]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda r: r["layers"][2]["mixer"].pop("mask"), "mask"),
    (lambda r: r["layers"][2]["mixer"].update(q_rank=0), "q_rank"),
    (lambda r: r["layers"][2]["mlp"].update(kind="experts"), "feed-forward"),
    (lambda r: r.pop("width"), "width"),
    (lambda r: r["norm"].update(eps=0.0), "eps"),
    (lambda r: r.update(layers=[]), "layers"),
])
def test_refusals(change, message):
    raw = copy.deepcopy(lc.LV_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        architecture_of(raw).parse(raw)


@pytest.mark.parametrize("dims,base,scaling", [(8, 10000.0, (4.0, 32, 8.0, 1.0)), (32, 1e6, (2.0, 512, 32.0, 1.0)),
                                               (64, 500.0, (8.0, 64, 4.0, 0.5)), (6, 100.0, (3.0, 16, 2.0, 1.0))])
def test_stretched_frequencies(dims, base, scaling):
    from tokamak_b200.parts.position import YarnScaling, yarn_frequencies
    factor, original, fast, slow = scaling
    freq, mag = yarn_frequencies(dims, base, YarnScaling(*scaling))
    want, want_mag = plain.yarn_frequencies(dims, base, dict(factor=factor, original=original, fast=fast, slow=slow))
    assert torch.allclose(freq, want, rtol=1e-13, atol=0) and mag == pytest.approx(0.1 * math.log(factor) + 1.0)
    assert want_mag == pytest.approx(mag)
    plainf = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    assert (freq <= plainf * (1 + 1e-12)).all() and (freq >= plainf / factor * (1 - 1e-12)).all()
    # a pair that turns more than `fast` times over the original length keeps its frequency, one that
    # turns less than `slow` times is slowed by the whole factor
    turns = original * plainf / (2 * math.pi)
    where = lambda t: dims * math.log(original / (2 * math.pi * t)) / (2 * math.log(base))
    lo, hi = max(math.floor(where(fast)), 0), min(math.ceil(where(slow)), dims - 1)
    for i in range(dims // 2):
        if i <= lo:
            assert freq[i] == pytest.approx(plainf[i].item(), rel=1e-12)
        if i >= hi and hi > lo:
            assert freq[i] == pytest.approx(plainf[i].item() / factor, rel=1e-12)
    assert turns[0] > turns[-1]
    unstretched, one = yarn_frequencies(dims, base, None)
    assert one == 1.0 and torch.allclose(unstretched, plainf, rtol=1e-13, atol=0)


def test_plain_mechanisms_agree_with_themselves():
    """The plain delta rule over a sequence equals the same rule continued from a carried state; the plain
    convolution equals a direct sum; a window of the sequence's length equals no window."""
    g = torch.Generator().manual_seed(0)
    T, dk, dv = 12, 5, 4
    q, k = torch.randn(T, dk, generator=g, dtype=torch.float64), torch.randn(T, dk, generator=g, dtype=torch.float64)
    v = torch.randn(T, dv, generator=g, dtype=torch.float64)
    beta, gate = torch.rand(T, generator=g, dtype=torch.float64), torch.rand(T, generator=g, dtype=torch.float64)
    S = torch.zeros(dk, dv, dtype=torch.float64)
    outs = []
    for t in range(T):
        S = gate[t] * S
        S = S + torch.outer(k[t], beta[t] * (v[t] - S.T @ k[t]))
        outs.append(S.T @ q[t])
    assert torch.allclose(plain.delta_rule(q, k, v, beta, gate), torch.stack(outs))
    x, taps = torch.randn(9, 3, generator=g, dtype=torch.float64), torch.randn(3, 4, generator=g, dtype=torch.float64)
    y = plain.short_conv(x, taps)
    assert torch.allclose(y[0], taps[:, 3] * x[0]) and torch.allclose(y[5], sum(taps[:, j] * x[2 + j] for j in range(4)))
    qq, kk, vv = (torch.randn(7, 2, 3, generator=g, dtype=torch.float64) for _ in range(3))
    assert torch.allclose(plain.softmax_attention(qq, kk, vv, 0.5, 7), plain.softmax_attention(qq, kk, vv, 0.5, None))
    one = plain.softmax_attention(qq, kk, vv, 0.5, 1)
    assert torch.allclose(one, vv)
    sunk = plain.softmax_attention(qq, kk, vv, 0.5, 1, torch.zeros(2, dtype=torch.float64))
    s = (qq * kk).sum(-1) * 0.5
    assert torch.allclose(sunk, vv * (torch.exp(s) / (torch.exp(s) + 1.0))[..., None])


def test_random_folder_round_trip(tmp_path):
    from tokamak_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "m", lc.LV_B, seed=3, dtype="bfloat16")
    cfg, w = plain.load_folder(folder)
    assert cfg["width"] == 52 and set(w) == set(DecoderModel.expected_tensors(spec_of(lc.LV_B)))
    logits = plain.forward(cfg, w, [1, 5, 9, 2])
    assert logits.shape == (4, 157) and torch.isfinite(logits).all()
    rounded = plain.forward(cfg, w, [1, 5, 9, 2], round_to=torch.bfloat16)
    assert 0 < (rounded - logits).abs().max() < 0.5 * logits.std()
