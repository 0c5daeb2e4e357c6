"""Plain, slow implementation of the Ketalix decoder: whole sequences, no cache, no batching,
one function per mechanism, sharing no code with the engine.  Everything runs on the CPU in
float64 by default, so that the result can serve as the truth for the float32 and the bfloat16
engine alike.

``round_to`` (e.g. ``torch.bfloat16``) makes the same functions round their intermediate
results (norm outputs, products, rotated heads, cached keys and values, mixer outputs) to that
type and widen them again, while sums, norms' statistics, softmax, decays, state and the
residual stream stay wide: what a 16-bit engine loses to rounding alone at a position.

Notation: ``x`` is the residual stream [T, W]; a linear weight is stored [out, in] and applied
as ``x @ W.T``; positions count from 0.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def load_folder(model_dir):
    """config.json as a dict and every tensor of the folder's safetensors files, by name."""
    from safetensors import safe_open

    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    tensors = {}
    for file in sorted(model_dir.glob("*.safetensors")):
        with safe_open(str(file), framework="pt", device="cpu") as f:
            for name in f.keys():
                tensors[name] = f.get_tensor(name)
    return cfg, tensors


# ----------------------------------------------------------------------------- mechanisms

def _rounder(round_to):
    if round_to is None:
        return lambda x: x
    return lambda x: x.to(round_to).to(x.dtype)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight.to(x.dtype)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_unit(h, w_gate, w_up, w_down, round_to=None):
    """down(gelu_tanh(gate h) * (up h))."""
    r = _rounder(round_to)
    return r(r(gelu_tanh(r(h @ w_gate.T)) * r(h @ w_up.T)) @ w_down.T)


def rotate_pairs(x, positions, rot_dims, base):
    """Pair i = (x[2i], x[2i+1]) of every head turns by position * base^(-2i / rot_dims);
    elements from rot_dims on pass unchanged.  x: [T, heads, dim]."""
    out = x.clone()
    for i in range(rot_dims // 2):
        angle = positions.to(x.dtype) * (base ** (-2.0 * i / rot_dims))
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        u, w = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - w * s
        out[..., 2 * i + 1] = w * c + u * s
    return out


def blend_values(v, v_first, lam):
    return (1.0 - lam) * v + lam * v_first


def attend(q, k, v, scale, softcap, window, sinks):
    """One row at a time.  q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key/value
    head h // (H / G); position i sees j with 0 <= i - j < window (window None: every j <= i);
    the softmax denominator also holds exp(sink_h)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            if softcap is not None:
                s = softcap * torch.tanh(s / softcap)
            terms = s if sinks is None else torch.cat([s, sinks[h].to(q.dtype).reshape(1)])
            p = torch.softmax(terms, dim=0)[: i + 1 - lo]
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def attention_mixer(h, w, m, eps, ctx, positions=None, round_to=None):
    """w: the mixer's tensors by short name; m: its configuration; ctx carries the first
    blending layer's values."""
    r = _rounder(round_to)
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
    positions = torch.arange(T) if positions is None else positions
    q = r(h @ w["q"].T).view(T, H, d)
    k = r(h @ w["k"].T).view(T, G, d)
    v = r(h @ w["v"].T).view(T, G, dv)
    rot = m.get("rot") or {}
    if rot.get("dims"):
        q = rotate_pairs(q, positions, rot["dims"], rot["base"])
        k = rotate_pairs(k, positions, rot["dims"], rot["base"])
    q, k = r(unit_rms(q, eps)), r(unit_rms(k, eps))
    if m.get("v_mix"):
        if "v_first" in ctx:
            v = blend_values(v, ctx["v_first"], w["vmix"].to(h.dtype))
        else:
            ctx["v_first"] = v
    window = (m.get("mask") or {}).get("size")
    o = r(attend(q, k, r(v), m["scale"], m.get("softcap") or None, window, w["sink"]))
    return r(o.reshape(T, H * dv) @ w["o"].T)


def gla_decays(h, w_a1, w_a2, bias, tau):
    """alpha = sigmoid(W_a2 (W_a1 h) + b) ** (1 / tau)."""
    return torch.sigmoid((h @ w_a1.T) @ w_a2.T + bias.to(h.dtype)).pow(1.0 / tau)


def gla_recurrence(q, k, v, alpha, state=None):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T; o_t = S_t^T q_t, head by head, token by token.
    q, k, alpha: [T, H, d]; v: [T, H, dv].  Returns (o [T, H, dv], the last state [H, d, dv])."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=q.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        for hd in range(H):
            S[hd] = alpha[t, hd][:, None] * S[hd] + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ q[t, hd]
    return o, S


def gla_mixer(h, w, m, eps, round_to=None):
    r = _rounder(round_to)
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m.get("vdim", m["dim"])
    q = r(h @ w["q"].T).view(T, H, d) * d ** -0.5
    k = r(h @ w["k"].T).view(T, H, d)
    v = r(h @ w["v"].T).view(T, H, dv)
    alpha = torch.sigmoid(r(h @ w["a1"].T) @ w["a2"].T + w["a2.b"].to(h.dtype)).pow(1.0 / m["tau"]).view(T, H, d)
    o, _ = gla_recurrence(q, k, v, alpha)
    o = rms_norm(o, w["norm"], eps).reshape(T, H * dv)
    g = r(h @ w["g"].T)
    return r(r(o * g * torch.sigmoid(g)) @ w["o"].T)


# ----------------------------------------------------------------------------- the model

def _sub(tensors, prefix, dtype):
    return {k[len(prefix):]: v.to(dtype) for k, v in tensors.items() if k.startswith(prefix)}


def forward_hidden(cfg, tensors, tokens, dtype=torch.float64, round_to=None):
    """The residual stream after every layer, [layers, T, W], and after the last one."""
    r = _rounder(round_to)
    eps = cfg["norm"]["eps"]
    t = {k: v.to(dtype) for k, v in tensors.items()}
    x = t["embed"][torch.tensor(tokens, dtype=torch.long)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    ctx, after = {}, []
    for i, lay in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = r(rms_norm(x, t[p + "norm1"], eps))
        w = _sub(tensors, p + "mix.", dtype)
        if lay["type"] == "attention":
            y = attention_mixer(h, w, lay["mixer"], eps, ctx, round_to=round_to)
        else:
            y = gla_mixer(h, w, lay["mixer"], eps, round_to=round_to)
        x = x + rms_norm(y, t[p + "norm1b"], eps) * t[p + "ls1"]
        if lay.get("mlp") is not None:
            h = r(rms_norm(x, t[p + "norm2"], eps))
            y = gated_unit(h, t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"], round_to=round_to)
            x = x + rms_norm(y, t[p + "norm2b"], eps) * t[p + "ls2"]
        after.append(x)
    return torch.stack(after), x


def forward_logits(cfg, tensors, tokens, dtype=torch.float64, round_to=None):
    """Logits [T, V] of a whole sequence."""
    _, x = forward_hidden(cfg, tensors, tokens, dtype, round_to)
    h = _rounder(round_to)(rms_norm(x, tensors["final.norm"].to(dtype), cfg["norm"]["eps"]))
    return h @ tensors["head"].to(dtype).T


def greedy_generate(cfg, tensors, prompt, n_new, dtype=torch.float64):
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward_logits(cfg, tensors, seq, dtype)[-1].argmax()))
    return seq[len(prompt):]
