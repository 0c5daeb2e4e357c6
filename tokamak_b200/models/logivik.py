"""The Logivik decoder as a :class:`ModelSpec`.

A stack of blocks whose sublayers read the residual stream itself and are normalised only on the
way out, ``x <- x + norm(sublayer(x))``, with norm weights stored around zero.  The mixers, listed
layer by layer in ``config.json``, are the gated delta rule (a recurrent state per head, short
convolutions on q, k and v), latent attention with a rotated key part (YaRN-stretched rotation of
neighbouring pairs, a sink per head, a sigmoid output gate) and latent attention without positions
(queries through a latent of their own, a sliding window).  Feed-forwards are silu-gated units, which
a layer may lack; the embedding is scaled; the head is untied.

    {"architecture": "Logivik", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "delta", "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": {"kind": "dense", "ff"} | null},
                {"type": "latent_attention", "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale",
                 "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}}, "mlp": ...},
                {"type": "latent_attention_2", "mixer": {"heads", "dim", "vdim", "kv_rank", "q_rank", "scale",
                 "mask": {"size"}}, "mlp": ...}, ...]}

Tensors are ``embed``, ``head``, ``final.norm`` and, for layer ``i``, ``l<i>.norm1``, ``l<i>.mix.*`` and, with a
feed-forward, ``l<i>.norm2`` and ``l<i>.mlp.{gate,up,down}``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..config.model_config import ConfigError
from ..parts.block import SandwichBlockSpec
from ..parts.delta import GatedDeltaSpec
from ..parts.embedding import EmbeddingSpec, HeadSpec
from ..parts.feedforward import SwiGLUSpec
from ..parts.latent import LatentAttentionSpec
from ..parts.norm import CastNormSpec, OffsetRMSNormSpec
from ..parts.position import NoPositionSpec, RopePairsSpec, YarnScaling
from .decoder import LayerCall, ModelSpec

ARCHITECTURE = "Logivik"
DEFAULT_MAX_POSITIONS = 1 << 17     # the design has no limit of its own
UNIT_EPS = 1e-6                     # under the root when q and k of the delta rule are scaled to unit length


@dataclass(frozen=True)
class DeltaLayer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class LatentLayer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int | None
    scale: float
    window: int | None
    rot_dims: int
    rot_base: float
    yarn: YarnScaling | None
    sinks: bool
    gate: bool


@dataclass(frozen=True)
class LogivikLayer:
    type: str                      # "delta", "latent_attention" or "latent_attention_2"
    mixer: Any                     # DeltaLayer or LatentLayer
    ff: int | None                 # inner size of the feed-forward, None for a layer without one


@dataclass(frozen=True)
class LogivikConfig:
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
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value or int(value) < 1:
        raise ConfigError(f"{what} must be a positive integer, got {value!r}")
    return int(value)


def _parse_rot(m: Mapping[str, Any], w: str, rot_dim: int) -> tuple[int, float, YarnScaling | None]:
    rot = _need(m, "rot", w)
    dims = int(rot.get("dims", rot_dim))
    if dims % 2 or dims < 0 or dims > rot_dim:
        raise ConfigError(f"{w}rot.dims must be even and at most rot_dim ({rot_dim}), got {dims}")
    base = float(_need(rot, "base", w + "rot."))
    if not base > 1.0:
        raise ConfigError(f"{w}rot.base must be > 1, got {base}")
    sc = rot.get("scaling")
    yarn = None
    if sc is not None:
        ws = w + "rot.scaling."
        yarn = YarnScaling(factor=float(_need(sc, "factor", ws)), original=float(_need(sc, "original", ws)),
                           fast=float(_need(sc, "fast", ws)), slow=float(_need(sc, "slow", ws)))
        if not (yarn.factor > 0 and yarn.original > 0 and yarn.fast > 0 and yarn.slow > 0):
            raise ConfigError(f"{ws}factor, original, fast and slow must be > 0")
    return dims, base, yarn


def _parse_layer(i: int, raw: Mapping[str, Any]) -> LogivikLayer:
    where = f"layers[{i}]."
    kind = _need(raw, "type", where)
    m = _need(raw, "mixer", where)
    w = where + "mixer."
    num = lambda key: _positive(_need(m, key, w), w + key)
    if kind == "delta":
        heads, kv = num("heads"), _positive(m.get("kv_heads", m.get("heads")), w + "kv_heads")
        if heads % kv:
            raise ConfigError(f"{w}heads ({heads}) must be a multiple of kv_heads ({kv})")
        dim = num("dim")
        mixer = DeltaLayer(heads=heads, kv_heads=kv, dim=dim, vdim=_positive(m.get("vdim", dim), w + "vdim"),
                           conv=num("conv"))
    elif kind == "latent_attention":
        rot_dim = m.get("rot_dim", 0) or 0
        if isinstance(rot_dim, bool) or int(rot_dim) != rot_dim or rot_dim < 0:
            raise ConfigError(f"{w}rot_dim must be a non-negative integer, got {rot_dim!r}")
        rot_dim = int(rot_dim)
        dims, base, yarn = _parse_rot(m, w, rot_dim) if rot_dim else (0, 1.0, None)     # no rotated part: no positions
        dim = num("dim")
        mixer = LatentLayer(heads=num("heads"), dim=dim, rot_dim=rot_dim, vdim=_positive(m.get("vdim", dim), w + "vdim"),
                            kv_rank=num("kv_rank"), q_rank=None, scale=float(_need(m, "scale", w)), window=None,
                            rot_dims=dims, rot_base=base, yarn=yarn, sinks=True, gate=True)
    elif kind == "latent_attention_2":
        dim = num("dim")
        mixer = LatentLayer(heads=num("heads"), dim=dim, rot_dim=0, vdim=_positive(m.get("vdim", dim), w + "vdim"),
                            kv_rank=num("kv_rank"), q_rank=num("q_rank"), scale=float(_need(m, "scale", w)),
                            window=_positive(_need(_need(m, "mask", w), "size", w + "mask."), w + "mask.size"),
                            rot_dims=0, rot_base=1.0, yarn=None, sinks=False, gate=False)
    else:
        raise ConfigError(f"{where}type {kind!r} is not a mixer of this design "
                          f"(delta, latent_attention, latent_attention_2)")
    mlp = raw.get("mlp")
    ff = None
    if mlp is not None:
        if mlp.get("kind", "dense") != "dense":
            raise ConfigError(f"{where}mlp.kind {mlp.get('kind')!r} is not a feed-forward of this design (dense)")
        ff = _positive(_need(mlp, "ff", where + "mlp."), where + "mlp.ff")
    return LogivikLayer(type=kind, mixer=mixer, ff=ff)


def parse_config(raw: Mapping[str, Any], eos_token_ids=None) -> LogivikConfig:
    """The typed configuration of a ``config.json`` dictionary."""
    layers_raw = _need(raw, "layers", "")
    if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
        raise ConfigError("config.json: layers must be a non-empty list")
    eps = float(_need(_need(raw, "norm", ""), "eps", "norm."))
    if not eps > 0.0:
        raise ConfigError(f"norm.eps must be > 0, got {eps}")
    emb = raw.get("embedding") or {}
    return LogivikConfig(
        architecture=ARCHITECTURE,
        vocab_size=_positive(_need(raw, "vocab", ""), "vocab"),
        max_position_embeddings=_positive(raw.get("max_position_embeddings", DEFAULT_MAX_POSITIONS),
                                          "max_position_embeddings"),
        eos_token_ids=tuple(int(e) for e in (eos_token_ids or ())),
        hidden_size=_positive(_need(raw, "width", ""), "width"),
        norm_eps=eps,
        embedding_scale=float(emb.get("scale", 1.0)),
        layers=tuple(_parse_layer(i, lay) for i, lay in enumerate(layers_raw)),
    )


def model_spec(cfg: LogivikConfig) -> ModelSpec:
    """Blocks and schedule: every layer once, with a cache of its own (pages of latents for an
    attention layer, a state record for a delta layer).  A block is the sandwich arrangement without
    a norm in front of its sublayers and without layer scales."""
    width = cfg.hidden_size
    norm, front = OffsetRMSNormSpec(width, cfg.norm_eps), CastNormSpec(width)
    blocks, schedule = [], []
    for i, lay in enumerate(cfg.layers):
        prefix = f"l{i}."
        m = lay.mixer
        if lay.type == "delta":
            mixer = GatedDeltaSpec(hidden_size=width, num_heads=m.heads, num_kv_heads=m.kv_heads, key_dim=m.dim,
                                   value_dim=m.vdim, conv_taps=m.conv, norm_eps=cfg.norm_eps, unit_eps=UNIT_EPS)
        else:
            position = RopePairsSpec(m.rot_dims, m.rot_base, m.yarn) if m.rot_dims else NoPositionSpec()
            mixer = LatentAttentionSpec(hidden_size=width, num_heads=m.heads, head_dim=m.dim, v_head_dim=m.vdim,
                                        kv_rank=m.kv_rank, softmax_scale=m.scale, norm_eps=cfg.norm_eps,
                                        rot_dim=m.rot_dim, q_rank=m.q_rank, position=position, window=m.window,
                                        sinks=m.sinks, gate=m.gate)
        ffn = {}
        if lay.ff is not None:
            ffn = dict(norm_in2=front, norm_out2=norm,
                       feed_forward=SwiGLUSpec(width, lay.ff, activation="silu", gate_name="gate", up_name="up",
                                               down_name="down"),
                       norm_in2_name="", ffn_prefix=prefix + "mlp.", norm_out2_name=prefix + "norm2")
        blocks.append(SandwichBlockSpec(name=f"l{i}", norm_in1=front, mixer=mixer, norm_out1=norm, norm_in1_name="",
                                        mixer_prefix=prefix + "mix.", norm_out1_name=prefix + "norm1", **ffn))
        schedule.append(LayerCall(block=f"l{i}", cache=f"l{i}"))
    return ModelSpec(
        embedding=EmbeddingSpec(cfg.vocab_size, width, name="embed", scale=cfg.embedding_scale),
        blocks=tuple(blocks),
        schedule=tuple(schedule),
        final_norm=norm,
        final_norm_name="final.norm",
        head=HeadSpec(cfg.vocab_size, width, tied=False, name="head"),
    )
