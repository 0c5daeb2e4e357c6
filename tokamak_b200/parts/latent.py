"""Latent attention: every head's keys and values are products of one small latent vector per token,
and only the latent (and one rotated key part that all heads share) is cached."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache.manager import KVPagesNeed
from ..csrc import ops
from .attention import paged_attention
from .base import MIXERS, POSITIONS, Runtime, TensorReq, graph_safe, linear, tensor_bytes
from .position import NoPositionSpec


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Sizes, constants and tensor names of one latent-attention mixer.

    A head has ``head_dim`` unrotated and ``rot_dim`` rotated query/key elements and ``v_head_dim``
    value elements; ``kv_rank`` is the size of the cached latent.  ``q_rank`` (``None``: the queries
    are a direct projection) is the size of a latent that the queries pass through, with a norm of
    its own.  ``position`` rotates the ``rot_dim`` part (a spec whose part rotates neighbouring pairs,
    or none).  ``window``: positions a query sees, itself included (``None``: all).  ``sinks``: a learned
    number per head joins the softmax denominator.  ``gate``: the concatenated heads are multiplied by
    the sigmoid of a projection of the mixer's input.  ``norm_eps`` is the eps of the latents' norms.
    """

    hidden_size: int
    num_heads: int
    head_dim: int
    v_head_dim: int
    kv_rank: int
    softmax_scale: float
    norm_eps: float
    rot_dim: int = 0
    q_rank: int | None = None
    position: object = NoPositionSpec()
    window: int | None = None
    sinks: bool = False
    gate: bool = False
    q_name: str = "q"
    q_down_name: str = "dq"
    q_norm_name: str = "dq.norm"
    q_up_name: str = "uq"
    kv_down_name: str = "dkv"
    kv_norm_name: str = "dkv.norm"
    k_up_name: str = "uk"
    v_up_name: str = "uv"
    sink_name: str = "sink"
    gate_name: str = "g"
    o_name: str = "o"
    kind: str = "latent_attention"


@MIXERS.register("latent_attention")
class LatentAttention:
    """``c = rmsnorm(W_dkv h)`` is the latent; head ``i`` has ``k_i = [W_uk,i c | rot(k_r)]`` and ``v_i = W_uv,i c``
    with ``k_r`` further rows of ``W_dkv h`` shared by the heads, and scores ``q_i . k_i * scale``.

    The cache holds one row ``[c | rot(k_r)]`` per token (one "head", values being the leading part of
    the keys: :class:`~tokamak_b200.cache.manager.KVPagesNeed` with ``values_in_keys``), and attention
    runs in the latent space: since ``q_i . W_uk,i c = (W_uk,i^T q_i) . c``, the query of head ``i``
    becomes ``[W_uk,i^T q_i | rot(q_r,i)]`` (float32), the heads all read the same rows, the weighted
    sum of latents comes out, and ``W_uv,i`` is applied to that sum.  Nothing per head is ever formed
    for a cached token.  Norms, angles, scores and softmax are float32 in every dtype.
    """

    def __init__(self, spec: LatentAttentionSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.kv_rank + spec.rot_dim > 1024:
            raise ValueError(f"a cache row of {spec.kv_rank} + {spec.rot_dim} elements is beyond the attention "
                             f"kernel's limit of 1024")
        if spec.q_rank and spec.rot_dim:
            raise ValueError("queries through a latent of their own together with a rotated part are not built")
        self.spec = spec
        self.rt = rt
        h, d, dr, dv, r = spec.num_heads, spec.head_dim, spec.rot_dim, spec.v_head_dim, spec.kv_rank
        t = lambda name: tensors[prefix + name]
        mats = [t(spec.q_down_name) if spec.q_rank else t(spec.q_name), t(spec.kv_down_name)]
        self.q_off = 0
        self.kv_off = mats[0].shape[0]
        self.g_off = self.kv_off + r + dr
        if spec.gate:
            mats.append(t(spec.gate_name))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_q_up = t(spec.q_up_name) if spec.q_rank else None
        self.q_norm_w = t(spec.q_norm_name) if spec.q_rank else None
        self.kv_norm_w = t(spec.kv_norm_name)
        # [heads, rank, head_dim]: the product with a head's unrotated query gives its query in the latent space
        self.w_uk_t = t(spec.k_up_name).view(h, d, r).transpose(1, 2).contiguous()
        self.w_uv = t(spec.v_up_name).view(h, dv, r).contiguous()
        self.sinks = t(spec.sink_name).contiguous() if spec.sinks else None
        self.w_o = t(spec.o_name)
        self.position = POSITIONS.get(spec.position.kind)(spec.position, tensors, rt)
        if dr and spec.position.kind != "none" and getattr(self.position, "PAIRING", None) != "neighbours":
            raise ValueError(f"position encoding {spec.position.kind!r} does not rotate neighbouring pairs")

    @staticmethod
    def expected_tensors(spec: LatentAttentionSpec, prefix: str) -> dict[str, TensorReq]:
        w, h, d, dr, dv, r = (spec.hidden_size, spec.num_heads, spec.head_dim, spec.rot_dim, spec.v_head_dim,
                              spec.kv_rank)
        out = {
            prefix + spec.kv_down_name: TensorReq((r + dr, w)),
            prefix + spec.kv_norm_name: TensorReq((r,), role="vector"),
            prefix + spec.k_up_name: TensorReq((h * d, r)),
            prefix + spec.v_up_name: TensorReq((h * dv, r)),
            prefix + spec.o_name: TensorReq((w, h * dv)),
        }
        if spec.q_rank:
            out[prefix + spec.q_down_name] = TensorReq((spec.q_rank, w))
            out[prefix + spec.q_norm_name] = TensorReq((spec.q_rank,), role="vector")
            out[prefix + spec.q_up_name] = TensorReq((h * (d + dr), spec.q_rank))
        else:
            out[prefix + spec.q_name] = TensorReq((h * (d + dr), w))
        if spec.sinks:
            out[prefix + spec.sink_name] = TensorReq((h,), role="bias")
        if spec.gate:
            out[prefix + spec.gate_name] = TensorReq((h * dv, w))
        out.update(POSITIONS.get(spec.position.kind).expected_tensors(spec.position))
        return out

    def cache_need(self) -> KVPagesNeed:
        s = self.spec
        return KVPagesNeed(1, s.kv_rank + s.rot_dim, s.window, s.kv_rank, values_in_keys=True)

    def GRAPH_SAFE(self) -> bool:
        return graph_safe(self.position)

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_in, self.w_q_up, self.q_norm_w, self.kv_norm_w, self.w_uk_t, self.w_uv, self.sinks,
                            self.w_o)

    def _per_head(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """``out[i, t] = w[i] @ x[t, i]`` for ``x`` ``[tokens, heads, K]`` (a view) and ``w`` ``[heads, M, K]``:
        the engine's float32 product, or the library's batched product in bfloat16."""
        if x.dtype == torch.float32:
            return ops.gemm_f32_heads(x, w)
        ops.flush_chains()
        return torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out_dtype=out_dtype)

    def forward(self, h, step, cache_view):
        spec = self.spec
        n, heads, d, dr, r = h.shape[0], spec.num_heads, spec.head_dim, spec.rot_dim, spec.kv_rank
        proj = linear(h, self.w_in, err=step.err)
        table, _ = self.position.rotary_table(step)
        prepare = dict(kv_off=self.kv_off, rank=r, rot=dr, kv_norm_w=self.kv_norm_w, eps=spec.norm_eps, table=table,
                       req_q_len=step.req_q_len, req_kv_len=step.req_kv_len)
        where = (cache_view.k, step.positions, step.tok_req, step.req_slot, cache_view.table, step.err)
        if spec.q_rank:
            # the kernel that writes the cache rows also norms the query latent; its up-projection follows
            _, cq = ops.latent_prepare(proj, *where, cq_off=self.q_off, cq_norm_w=self.q_norm_w, **prepare)
            q = _dense(linear(cq, self.w_q_up, err=step.err), h.dtype).view(n, heads, d)
            q_lat = self._per_head(q, self.w_uk_t, torch.float32).transpose(0, 1)      # a view [n, heads, r]
        else:
            proj = _dense(proj, h.dtype)
            q = proj[:, self.q_off:self.q_off + heads * (d + dr)].view(n, heads, d + dr)
            q_abs = self._per_head(q[:, :, :d], self.w_uk_t, torch.float32)            # [heads, n, r] float32
            q_lat, _ = ops.latent_prepare(proj, *where, q_abs=q_abs, q_off=self.q_off, q_head_cols=d + dr,
                                          q_rot_off=d, **prepare)
        o_lat = torch.empty((n, heads, r), dtype=h.dtype, device=h.device)
        paged_attention(q_lat, o_lat, cache_view, step, scale=spec.softmax_scale, window=spec.window, sinks=self.sinks)
        o = self._per_head(o_lat, self.w_uv, h.dtype)                                  # [heads, n, dv]
        y = ops.heads_gate(o, proj if spec.gate else None, self.g_off)
        return linear(y, self.w_o, err=step.err)


def _dense(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A product's result as one tensor in the activation type (partial sums are added up)."""
    from .base import sum_parts
    ops.flush_chains()
    return sum_parts(x, dtype)
