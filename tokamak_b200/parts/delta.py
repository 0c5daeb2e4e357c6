"""The gated delta rule: a mixer whose memory is a matrix-valued state per request and head that
every token decays and then corrects towards its own value."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache.manager import StateNeed
from ..csrc import ops
from .base import MIXERS, Runtime, TensorReq, linear, tensor_bytes


@dataclass(frozen=True)
class GatedDeltaSpec:
    """Sizes, constants and tensor names of one gated-delta-rule mixer.

    ``num_heads`` value heads of ``value_dim`` read ``num_kv_heads`` query/key heads of ``key_dim``
    (value head ``i`` reads q/k head ``i // (num_heads / num_kv_heads)``).  ``conv_taps`` is the
    length of the causal convolution that q, k and v pass; ``unit_eps`` the eps under the root when q
    and k heads are scaled to unit length; ``norm_eps`` the eps of the output norm.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float
    unit_eps: float = 1e-6
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    conv_suffix: str = ".conv"
    beta_name: str = "b"
    decay_name: str = "a"
    decay_log_name: str = "A_log"
    decay_bias_name: str = "dt_bias"
    gate_name: str = "g"
    norm_name: str = "norm"
    o_name: str = "o"
    kind: str = "gated_delta"


@MIXERS.register("gated_delta")
class GatedDeltaRule:
    """Per head, with ``S`` the ``[key_dim, value_dim]`` state: ``S <- g S``, ``u = beta (v - S^T k)``,
    ``S <- S + k u^T``, ``o = S^T q`` (the read-out sees the token's own write).  q, k and v pass a
    short causal convolution and silu; q and k heads are scaled to unit length (q also by
    ``key_dim ** -0.5``); ``beta = sigmoid(W_b h)`` and ``g = exp(-exp(A_log) softplus(W_a h + dt_bias))``
    are one number per head.  Every head's ``o`` is RMS-normed over ``value_dim`` (one weight vector for
    all heads), multiplied by ``silu(W_g h)``, and projected out.

    The request's record in the cache (:class:`~tokamak_b200.cache.manager.StateNeed`, float32, cleared
    when the slot is handed out) holds the state of every head and the last ``conv_taps - 1`` inputs of
    the convolution.  The six input projections are one stacked operand; convolution, unit norm, beta,
    the decay, the recurrence and the output norm are float32 in every dtype (``csrc/delta.cu``; the
    output stage is the kernel that gated linear attention uses).
    """

    GRAPH_SAFE = True

    def __init__(self, spec: GatedDeltaSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} value heads are not a multiple of {spec.num_kv_heads} key heads")
        if spec.key_dim > 256:
            raise ValueError(f"key_dim {spec.key_dim} is beyond the recurrence kernel's limit of 256")
        if not 1 <= spec.conv_taps <= 8:
            raise ValueError(f"a convolution of {spec.conv_taps} taps is not taken (1 to 8)")
        self.spec = spec
        self.rt = rt
        hk, hv, hh = spec.num_kv_heads * spec.key_dim, spec.num_heads * spec.value_dim, spec.num_heads
        t = lambda name: tensors[prefix + name]
        self.w_in = torch.cat([t(spec.q_name), t(spec.k_name), t(spec.v_name), t(spec.gate_name), t(spec.beta_name),
                               t(spec.decay_name)], dim=0).contiguous()
        self.q_off, self.k_off, self.v_off = 0, hk, 2 * hk
        self.g_off, self.b_off, self.a_off = 2 * hk + hv, 2 * hk + 2 * hv, 2 * hk + 2 * hv + hh
        self.taps = torch.cat([t(name + spec.conv_suffix).float() for name in (spec.q_name, spec.k_name, spec.v_name)],
                              dim=0).contiguous()
        self.a_log = t(spec.decay_log_name).float().contiguous()
        self.dt_bias = t(spec.decay_bias_name).float().contiguous()
        self.norm_w = t(spec.norm_name)
        self.w_o = t(spec.o_name)
        self.record_floats, _ = ops.delta_record_floats(spec.num_heads, spec.num_kv_heads, spec.key_dim,
                                                        spec.value_dim, spec.conv_taps)

    @staticmethod
    def expected_tensors(spec: GatedDeltaSpec, prefix: str) -> dict[str, TensorReq]:
        w = spec.hidden_size
        hk, hv, hh = spec.num_kv_heads * spec.key_dim, spec.num_heads * spec.value_dim, spec.num_heads
        conv = lambda name: prefix + name + spec.conv_suffix
        return {
            prefix + spec.q_name: TensorReq((hk, w)),
            conv(spec.q_name): TensorReq((hk, spec.conv_taps), role="bias"),
            prefix + spec.k_name: TensorReq((hk, w)),
            conv(spec.k_name): TensorReq((hk, spec.conv_taps), role="bias"),
            prefix + spec.v_name: TensorReq((hv, w)),
            conv(spec.v_name): TensorReq((hv, spec.conv_taps), role="bias"),
            prefix + spec.beta_name: TensorReq((hh, w)),
            prefix + spec.decay_log_name: TensorReq((hh,), role="bias"),
            prefix + spec.norm_name: TensorReq((spec.value_dim,), role="vector"),
            prefix + spec.decay_name: TensorReq((hh, w)),
            prefix + spec.decay_bias_name: TensorReq((hh,), role="bias"),
            prefix + spec.gate_name: TensorReq((hv, w)),
            prefix + spec.o_name: TensorReq((w, hv)),
        }

    def cache_need(self) -> StateNeed:
        return StateNeed((self.record_floats,), "float32")

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_in, self.taps, self.a_log, self.dt_bias, self.norm_w, self.w_o)

    def forward(self, h, step, cache_view):
        spec = self.spec
        proj = linear(h, self.w_in, err=step.err)
        q, k, v, beta, g = ops.delta_prepare(
            proj, self.taps, self.a_log, self.dt_bias, cache_view.records, step.tok_req, step.req_q_start,
            step.req_q_len, step.req_slot, step.err, dtype=h.dtype, q_off=self.q_off, k_off=self.k_off,
            v_off=self.v_off, b_off=self.b_off, a_off=self.a_off, heads=spec.num_heads, kv_heads=spec.num_kv_heads,
            key_dim=spec.key_dim, value_dim=spec.value_dim, unit_eps=spec.unit_eps, q_scale=spec.key_dim ** -0.5)
        o = ops.delta_scan(q, k, v, beta, g, cache_view.records, step.req_q_start, step.req_q_len, step.req_slot,
                           step.err)
        y = ops.gla_out(o, proj, self.g_off, self.norm_w, spec.norm_eps, h.dtype)
        return linear(y, self.w_o, err=step.err)
