"""The Ketalix design in the registry: configuration, model description, expected tensors, and
the plain implementation's two ways of computing the same thing."""

from __future__ import annotations

import copy

import pytest
import torch

import ketalix_configs as kc
from plain import ketalix_plain as plain
from tokamak_b200.cache.device import plan_groups
from tokamak_b200.cache.manager import KVPagesNeed, StateNeed
from tokamak_b200.config import ConfigError, architecture_of
from tokamak_b200.models.decoder import DecoderModel
from tokamak_b200.weights import write_random_model
from tokamak_b200.weights.loader import checkpoint_shapes


def spec_of(raw, shapes=None):
    arch = architecture_of(raw)
    return arch.build_spec(arch.parse(raw, None, tensor_shapes=shapes))


def test_design_is_chosen_by_the_architecture_key():
    arch = architecture_of(kc.KX_A)
    assert arch.name == "Ketalix" and arch.reads_tensor_shapes
    cfg = arch.parse(kc.KX_A)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps, cfg.embedding_scale) == (211, 64, 1e-5, 3.0)
    assert [l.type for l in cfg.layers] == ["attention", "gla", "attention", "gla", "attention"]
    assert [l.ff for l in cfg.layers] == [96, 80, None, None, 72]
    assert arch.parse(kc.KX_B).embedding_scale == 1.0


def test_layers_become_blocks_with_their_own_caches():
    spec = spec_of(kc.KX_A)
    mixers = [b.mixer for b in spec.blocks]
    assert [m.kind for m in mixers] == ["attention_capped", "gla", "attention_capped", "gla", "attention_capped"]
    # the first blending layer keeps its values, the later ones blend
    assert [getattr(m, "value_mix", None) for m in mixers] == ["source", None, "blend", None, "blend"]
    assert [m.window for m in mixers if m.kind == "attention_capped"] == [9, 20, 33]
    assert mixers[0].position.rotary_dim == 8 and mixers[4].position.theta == 500.0
    assert spec.blocks[2].feed_forward is None and spec.blocks[0].feed_forward.activation == "gelu_tanh"
    assert [c.cache for c in spec.schedule] == [f"l{i}" for i in range(5)]
    b = spec_of(kc.KX_B)
    assert [getattr(m.mixer, "value_mix", None) for m in b.blocks] == [None, None, "source", None]
    assert b.blocks[1].mixer.window is None and b.blocks[1].mixer.softcap is None


def test_expected_tensors_and_the_rank_that_only_the_checkpoint_gives(tmp_path):
    exp = DecoderModel.expected_tensors(spec_of(kc.KX_A))
    assert exp["l0.mix.q"].shape == (64, 64) and exp["l0.mix.v"].shape == (48, 64) and exp["l0.mix.o"].shape == (64, 96)
    assert exp["l0.mix.sink"].shape == (4,) and exp["l0.mix.vmix"].shape == ()
    assert exp["l1.mix.a1"].shape == (5, 64) and exp["l1.mix.a2"].shape == (24, 5) and exp["l1.mix.a2.b"].shape == (24,)
    assert exp["l1.mix.norm"].shape == (20,) and exp["l3.mix.g"].shape == (24, 64)
    assert "l2.mlp.gate" not in exp and "l2.norm2" not in exp and "l2.ls2" not in exp and "l2.ls1" in exp
    assert {"embed", "head", "final.norm"} <= set(exp)
    # a folder whose configuration does not name the rank: the header of the checkpoint does
    folder = write_random_model(tmp_path / "m", kc.KX_A, seed=1)
    raw = copy.deepcopy(kc.KX_A)
    for lay in raw["layers"]:
        lay["mixer"].pop("rank", None)
    shapes = checkpoint_shapes(folder)
    assert shapes["l3.mix.a1"] == (3, 64)
    spec = spec_of(raw, shapes)
    assert [b.mixer.decay_rank for b in spec.blocks if b.mixer.kind == "gla"] == [5, 3]
    assert [b.mixer.decay_rank for b in spec_of(raw).blocks if b.mixer.kind == "gla"] == [16, 16]


@pytest.mark.parametrize("change,match", [
    (lambda r: r["layers"][0].update(type="conv"), "not a mixer"),
    (lambda r: r["layers"][0]["mixer"].update(heads=5), "multiple of kv_heads"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"].update(tau=0.0), "tau"),
    (lambda r: r["layers"][0]["mlp"].update(kind="moe"), "not a feed-forward"),
    (lambda r: r.pop("width"), "width"),
    (lambda r: r["layers"][2]["mixer"].update(vdim=16), "blends its values"),
])
def test_faulty_configurations_are_refused(change, match):
    raw = copy.deepcopy(kc.KX_A)
    change(raw)
    with pytest.raises(ConfigError, match=match):
        spec_of(raw)


def test_cache_needs_group_by_sizes():
    needs = {"a": KVPagesNeed(2, 16, 9, 24), "b": KVPagesNeed(2, 16, 9, 24), "c": KVPagesNeed(2, 16, 9),
             "s": StateNeed((2, 12, 20)), "t": StateNeed((2, 12, 20)), "u": StateNeed((3, 20, 8))}
    kv, st = plan_groups(needs, 64, 16)
    assert sorted(len(g.cache_keys) for g in kv) == [1, 2] and sorted(len(g.cache_keys) for g in st) == [1, 2]
    assert KVPagesNeed(2, 16).value_dim == 16 and KVPagesNeed(2, 16, None, 24).value_dim == 24


def test_plain_prefix_property_and_state_carry():
    """The oracle agrees with itself: logits of a prefix are the first rows of the logits of the
    whole, and the recurrence continued from a carried state equals the recurrence in one go."""
    torch.manual_seed(0)
    folder_cfg = kc.KX_B
    from tokamak_b200.weights.random_init import random_tensors
    arch = architecture_of(folder_cfg)
    tensors = random_tensors(DecoderModel.expected_tensors(arch.build_spec(arch.parse(folder_cfg))), 3, std=0.1)
    toks = torch.randint(0, folder_cfg["vocab"], (40,)).tolist()
    whole = plain.forward_logits(folder_cfg, tensors, toks)
    part = plain.forward_logits(folder_cfg, tensors, toks[:17])
    assert torch.allclose(whole[:17], part, atol=1e-10)
    q, k, a = torch.randn(30, 2, 6).double(), torch.randn(30, 2, 6).double(), torch.rand(30, 2, 6).double()
    v = torch.randn(30, 2, 5).double()
    o, s = plain.gla_recurrence(q, k, v, a)
    o1, s1 = plain.gla_recurrence(q[:11], k[:11], v[:11], a[:11])
    o2, s2 = plain.gla_recurrence(q[11:], k[11:], v[11:], a[11:], s1)
    assert torch.allclose(torch.cat([o1, o2]), o, atol=1e-12) and torch.allclose(s2, s, atol=1e-12)
    # the closed form of the same state: S_T = sum_t (prod_{u>t} alpha_u) * k_t v_t^T
    S = torch.zeros(2, 6, 5, dtype=torch.float64)
    for t in range(30):
        decay = a[t + 1:].prod(dim=0)
        S += decay[:, :, None] * k[t][:, :, None] * v[t][:, None, :]
    assert torch.allclose(S, s, atol=1e-10)


def test_random_folder_from_the_command_line(tmp_path, capsys):
    """The writer of seeded random folders takes the design's config.json like any other."""
    import json

    from tokamak_b200.cli import main
    from tokamak_b200.weights.loader import checkpoint_shapes

    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(kc.KX_B))
    out = tmp_path / "model"
    assert main(["--write-random", str(out), "--config", str(cfg), "--seed", "4", "--weights-dtype", "float32"]) == 0
    assert "wrote" in capsys.readouterr().out
    shapes = checkpoint_shapes(out)
    assert shapes["embed"] == (kc.KX_B["vocab"], kc.KX_B["width"]) and shapes["l0.mix.a1"][1] == kc.KX_B["width"]
    assert "l2.mlp.gate" not in shapes and "l1.mlp.gate" in shapes          # the third layer has no feed-forward
