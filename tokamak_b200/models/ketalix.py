"""The Ketalix decoder as a :class:`ModelSpec`.

A stack of sandwich-normed blocks (a norm in front of and behind every sublayer, a learned
per-channel scale on what joins the residual stream) whose mixers alternate freely between
windowed grouped-query attention with sinks, capped scores and blended values, and gated linear
attention with a recurrent state; gated feed-forwards with the tanh form of gelu, which a layer
may also lack; a scaled embedding and an untied head.

``config.json`` names the design in ``architecture`` and lists the layers one by one:

    {"architecture": "Ketalix", "vocab": V, "width": W, "norm": {"eps": e},
     "embedding": {"scale": s},
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale",
                 "softcap", "mask": {"size"}, "rot": {"base", "dims"}, "v_mix"}, "mlp": {"kind": "dense", "ff"} | null},
                {"type": "gla", "mixer": {"heads", "dim", "vdim", "tau"}, "mlp": ...}, ...]}

Tensors are ``embed``, ``head``, ``final.norm`` and, for layer ``i``, ``l<i>.norm1``, ``l<i>.norm1b``,
``l<i>.ls1``, ``l<i>.mix.*`` and, with a feed-forward, ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.ls2``,
``l<i>.mlp.{gate,up,down}``.  The inner size of a gla layer's decay projection is not in the
configuration; ``decay_rank`` of the typed configuration is filled from the checkpoint's header
(``l<i>.mix.a1`` is ``[rank, width]``) or, for a folder of random weights, from the optional key
``mixer.rank`` (default 16).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..config.model_config import ConfigError
from ..parts.attention import CappedAttentionSpec
from ..parts.block import SandwichBlockSpec
from ..parts.embedding import EmbeddingSpec, HeadSpec
from ..parts.feedforward import SwiGLUSpec
from ..parts.gla import GatedLinearAttentionSpec
from ..parts.norm import RMSNormSpec
from ..parts.position import RopePairsSpec
from .decoder import LayerCall, ModelSpec

ARCHITECTURE = "Ketalix"
DEFAULT_MAX_POSITIONS = 1 << 17     # the design has no limit of its own; positions are exact in float32 far beyond
DEFAULT_DECAY_RANK = 16


@dataclass(frozen=True)
class AttentionLayer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float | None
    window: int | None
    rot_base: float
    rot_dims: int
    v_mix: bool


@dataclass(frozen=True)
class GlaLayer:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int


@dataclass(frozen=True)
class KetalixLayer:
    type: str                      # "attention" or "gla"
    mixer: Any                     # AttentionLayer or GlaLayer
    ff: int | None                 # inner size of the feed-forward, None for a layer without one


@dataclass(frozen=True)
class KetalixConfig:
    """Typed configuration; the first four fields are what the engine reads."""

    architecture: str
    vocab_size: int
    max_position_embeddings: int
    eos_token_ids: tuple
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    layers: tuple


def _need(raw: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(raw, Mapping) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json is missing {where}{key!r}")
    return raw[key]


def _positive(value: Any, what: str) -> int:
    if isinstance(value, bool) or int(value) != value or int(value) < 1:
        raise ConfigError(f"{what} must be a positive integer, got {value!r}")
    return int(value)


def _parse_layer(i: int, raw: Mapping[str, Any], ranks: Mapping[int, int]) -> KetalixLayer:
    where = f"layers[{i}]."
    kind = _need(raw, "type", where)
    m = _need(raw, "mixer", where)
    w = where + "mixer."
    if kind == "attention":
        heads, kv = _positive(_need(m, "heads", w), w + "heads"), _positive(_need(m, "kv_heads", w), w + "kv_heads")
        if heads % kv:
            raise ConfigError(f"{w}heads ({heads}) must be a multiple of kv_heads ({kv})")
        dim = _positive(_need(m, "dim", w), w + "dim")
        rot = m.get("rot") or {}
        rot_dims = int(rot.get("dims", 0) or 0)
        if rot_dims % 2 or rot_dims > dim or rot_dims < 0:
            raise ConfigError(f"{w}rot.dims must be even and at most dim ({dim}), got {rot_dims}")
        if rot_dims and "base" not in rot:
            raise ConfigError(f"config.json is missing {w}rot.base")
        mask = m.get("mask") or {}
        window = mask.get("size")
        softcap = m.get("softcap")
        mixer = AttentionLayer(heads=heads, kv_heads=kv, dim=dim, vdim=_positive(m.get("vdim", dim), w + "vdim"),
                               scale=float(_need(m, "scale", w)),
                               softcap=float(softcap) if softcap else None,
                               window=_positive(window, w + "mask.size") if window is not None else None,
                               rot_base=float(rot.get("base", 1.0)), rot_dims=rot_dims, v_mix=bool(m.get("v_mix", False)))
    elif kind == "gla":
        dim = _positive(_need(m, "dim", w), w + "dim")
        tau = float(_need(m, "tau", w))
        if not tau > 0.0:
            raise ConfigError(f"{w}tau must be > 0, got {tau}")
        mixer = GlaLayer(heads=_positive(_need(m, "heads", w), w + "heads"), dim=dim,
                         vdim=_positive(m.get("vdim", dim), w + "vdim"), tau=tau,
                         rank=_positive(ranks.get(i, m.get("rank", DEFAULT_DECAY_RANK)), w + "rank"))
    else:
        raise ConfigError(f"{where}type {kind!r} is not a mixer of this design (attention, gla)")
    mlp = raw.get("mlp")
    ff = None
    if mlp is not None:
        if mlp.get("kind", "dense") != "dense":
            raise ConfigError(f"{where}mlp.kind {mlp.get('kind')!r} is not a feed-forward of this design (dense)")
        ff = _positive(_need(mlp, "ff", where + "mlp."), where + "mlp.ff")
    return KetalixLayer(type=kind, mixer=mixer, ff=ff)


def parse_config(raw: Mapping[str, Any], eos_token_ids=None, tensor_shapes: Mapping[str, tuple] | None = None
                 ) -> KetalixConfig:
    """The typed configuration of a ``config.json`` dictionary.  ``tensor_shapes`` (name -> shape,
    from the checkpoint's header) supplies the sizes that only the tensors give."""
    layers_raw = _need(raw, "layers", "")
    if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
        raise ConfigError("config.json: layers must be a non-empty list")
    ranks = {}
    for i in range(len(layers_raw)):
        shape = (tensor_shapes or {}).get(f"l{i}.mix.a1")
        if shape is not None and len(shape) == 2:
            ranks[i] = int(shape[0])
    eps = float(_need(_need(raw, "norm", ""), "eps", "norm."))
    if not eps > 0.0:
        raise ConfigError(f"norm.eps must be > 0, got {eps}")
    emb = raw.get("embedding") or {}
    return KetalixConfig(
        architecture=ARCHITECTURE,
        vocab_size=_positive(_need(raw, "vocab", ""), "vocab"),
        max_position_embeddings=_positive(raw.get("max_position_embeddings", DEFAULT_MAX_POSITIONS),
                                          "max_position_embeddings"),
        eos_token_ids=tuple(int(e) for e in (eos_token_ids or ())),
        hidden_size=_positive(_need(raw, "width", ""), "width"),
        norm_eps=eps,
        embedding_scale=float(emb.get("scale", 1.0)),
        layers=tuple(_parse_layer(i, lay, ranks) for i, lay in enumerate(layers_raw)),
    )


def model_spec(cfg: KetalixConfig) -> ModelSpec:
    """Blocks and schedule: every layer once, with a cache of its own (pages for an attention
    layer, a state record for a gla layer).  Among the attention layers that blend values, the
    first keeps its raw values for the step and the later ones blend with them."""
    norm = RMSNormSpec(cfg.hidden_size, cfg.norm_eps)
    blocks, schedule = [], []
    source = None       # (kv heads, value size) of the first blending layer
    for i, lay in enumerate(cfg.layers):
        prefix = f"l{i}."
        m = lay.mixer
        if lay.type == "attention":
            mix = None
            if m.v_mix:
                if source is None:
                    source, mix = (m.kv_heads, m.vdim), "source"
                elif source != (m.kv_heads, m.vdim):
                    raise ConfigError(f"layer {i} blends its values with the first blending layer's, but has "
                                      f"{m.kv_heads} x {m.vdim} values per token against {source[0]} x {source[1]}")
                else:
                    mix = "blend"
            mixer = CappedAttentionSpec(
                hidden_size=cfg.hidden_size, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                v_head_dim=m.vdim, position=RopePairsSpec(m.rot_dims, m.rot_base), softmax_scale=m.scale,
                unit_norm_eps=cfg.norm_eps, window=m.window, softcap=m.softcap, sinks=True, value_mix=mix)
        else:
            mixer = GatedLinearAttentionSpec(
                hidden_size=cfg.hidden_size, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim,
                decay_rank=m.rank, decay_tau=m.tau, norm_eps=cfg.norm_eps)
        ffn = {}
        if lay.ff is not None:
            ffn = dict(norm_in2=norm, norm_out2=norm,
                       feed_forward=SwiGLUSpec(cfg.hidden_size, lay.ff, activation="gelu_tanh",
                                               gate_name="gate", up_name="up", down_name="down"),
                       norm_in2_name=prefix + "norm2", ffn_prefix=prefix + "mlp.",
                       norm_out2_name=prefix + "norm2b", scale2_name=prefix + "ls2")
        blocks.append(SandwichBlockSpec(
            name=f"l{i}", norm_in1=norm, mixer=mixer, norm_out1=norm, norm_in1_name=prefix + "norm1",
            mixer_prefix=prefix + "mix.", norm_out1_name=prefix + "norm1b", scale1_name=prefix + "ls1", **ffn))
        schedule.append(LayerCall(block=f"l{i}", cache=f"l{i}"))
    return ModelSpec(
        embedding=EmbeddingSpec(cfg.vocab_size, cfg.hidden_size, name="embed", scale=cfg.embedding_scale),
        blocks=tuple(blocks),
        schedule=tuple(schedule),
        final_norm=norm,
        final_norm_name="final.norm",
        head=HeadSpec(cfg.vocab_size, cfg.hidden_size, tied=False, name="head"),
    )
