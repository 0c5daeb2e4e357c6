"""Gated linear attention: a mixer whose memory is a matrix-valued state per request and head."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache.manager import StateNeed
from ..csrc import ops
from .base import MIXERS, Runtime, TensorReq, linear, tensor_bytes


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """Sizes and constants of one gated-linear-attention mixer.

    ``key_dim`` / ``value_dim`` are per head; ``decay_rank`` is the inner size of the low-rank
    decay projection; ``decay_tau`` the temperature of the decay (``alpha = sigmoid(z) ** (1 / tau)``);
    ``norm_eps`` the eps of the output norm.  The ``*_name`` fields are the tensors' names after
    the part's prefix.
    """

    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    decay_rank: int
    decay_tau: float
    norm_eps: float
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    gate_name: str = "g"
    o_name: str = "o"
    norm_name: str = "norm"
    decay_in_name: str = "a1"
    decay_out_name: str = "a2"
    decay_bias_name: str = "a2.b"
    kind: str = "gla"


@MIXERS.register("gla")
class GatedLinearAttention:
    """``S_t = diag(alpha_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` per head, with
    ``q = W_q h / sqrt(key_dim)``, a decay per key channel ``alpha = sigmoid(W_2 (W_1 h) + b) ** (1 / tau)``,
    an RMS norm of every head's ``o`` over ``value_dim`` (one weight vector for all heads), a
    ``silu`` gate and an output projection.

    The state ``[heads, key_dim, value_dim]`` is a float32 record in the request's slot of the
    cache (:class:`~tokamak_b200.cache.manager.StateNeed`): cleared when the slot is handed out,
    read at the start of a step's portion and stored at its end.  The five input projections are
    one stacked operand, so a step is one product, the kernel that lays out the
    recurrence's float32 inputs (scaled q, k, decays, v), the recurrence, the output stage and the output product.  Decays, state, recurrence and norm are float32 in every dtype.
    """

    GRAPH_SAFE = True

    def __init__(self, spec: GatedLinearAttentionSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        hk, hv = spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim
        self.w_in = torch.cat([tensors[prefix + spec.q_name], tensors[prefix + spec.k_name],
                               tensors[prefix + spec.v_name], tensors[prefix + spec.gate_name],
                               tensors[prefix + spec.decay_in_name]], dim=0).contiguous()
        self.q_off, self.k_off, self.v_off, self.g_off, self.a_off = 0, hk, 2 * hk, 2 * hk + hv, 2 * hk + 2 * hv
        self.w_decay = tensors[prefix + spec.decay_out_name].contiguous()
        self.decay_bias = tensors[prefix + spec.decay_bias_name]
        self.norm_w = tensors[prefix + spec.norm_name]
        self.w_o = tensors[prefix + spec.o_name]

    @staticmethod
    def expected_tensors(spec: GatedLinearAttentionSpec, prefix: str) -> dict[str, TensorReq]:
        h = spec.hidden_size
        hk, hv = spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim
        return {
            prefix + spec.q_name: TensorReq((hk, h)),
            prefix + spec.k_name: TensorReq((hk, h)),
            prefix + spec.v_name: TensorReq((hv, h)),
            prefix + spec.gate_name: TensorReq((hv, h)),
            prefix + spec.o_name: TensorReq((h, hv)),
            prefix + spec.norm_name: TensorReq((spec.value_dim,), role="vector"),
            prefix + spec.decay_in_name: TensorReq((spec.decay_rank, h)),
            prefix + spec.decay_out_name: TensorReq((hk, spec.decay_rank)),
            prefix + spec.decay_bias_name: TensorReq((hk,), role="bias"),
        }

    def cache_need(self) -> StateNeed:
        return StateNeed((self.spec.num_heads, self.spec.key_dim, self.spec.value_dim), "float32")

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_in, self.w_decay, self.decay_bias, self.norm_w, self.w_o)

    def forward(self, h, step, cache_view):
        spec = self.spec
        proj = linear(h, self.w_in, err=step.err)
        prep = ops.gla_prepare(proj, self.q_off, self.k_off, self.v_off, self.a_off, self.w_decay, self.decay_bias,
                               heads=spec.num_heads, key_dim=spec.key_dim, value_dim=spec.value_dim,
                               tau=spec.decay_tau, q_scale=spec.key_dim ** -0.5)
        o = ops.gla_scan(prep, cache_view.records, step.req_q_start, step.req_q_len, step.req_slot, step.err)
        y = ops.gla_out(o, proj, self.g_off, self.norm_w, spec.norm_eps, h.dtype)
        return linear(y, self.w_o, err=step.err)
