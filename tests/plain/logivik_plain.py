"""A slow float64 implementation of every mechanism of the Logivik design, one function each,
written from the equations.  It shares nothing with the package: tests compare the engine with it.

All functions take and return ``torch.float64`` tensors on the CPU; a sequence is processed whole
(``[T, ...]``), position ``t`` of the sequence being row ``t``.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64

# ``ROUND`` is applied wherever an engine that keeps activations in 16 bits rounds them: after every
# matrix product and after the norms and gates whose result feeds one.  The identity by default;
# :func:`forward` with ``round_to`` swaps it for the duration of a call.
ROUND = lambda x: x


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The block norm: the weight is stored around zero, the factor is ``1 + w``."""
    return rms(x, eps) * (1.0 + w)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def short_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """Causal convolution per channel: ``y[t, c] = sum_j taps[c, j] x[t - (K - 1) + j, c]`` with
    zeros before the start (the last column weighs the current token)."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(K):
            s = t - (K - 1) + j
            if s >= 0:
                y[t] += taps[:, j] * x[s]
    return y


def delta_rule(q, k, v, beta, g):
    """Gated delta rule of one head.  ``q, k`` ``[T, dk]``, ``v`` ``[T, dv]``, ``beta, g`` ``[T]``.
    Per token: decay the state, write the error-corrected value under the key, read with the query."""
    T, dk = k.shape
    dv = v.shape[1]
    S = torch.zeros(dk, dv, dtype=F64)
    out = torch.zeros(T, dv, dtype=F64)
    for t in range(T):
        S = g[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(h, w, m, eps):
    """``w``: name -> tensor of one mixer (``q``, ``q.conv``, ...); ``m``: its sizes."""
    T = h.shape[0]
    H, HK, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(ROUND(h @ w["q"].T), w["q.conv"])).view(T, HK, dk)
    k = silu(short_conv(ROUND(h @ w["k"].T), w["k.conv"])).view(T, HK, dk)
    v = silu(short_conv(ROUND(h @ w["v"].T), w["v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(ROUND(h @ w["b"].T))
    g = torch.exp(-torch.exp(w["A_log"]) * torch.nn.functional.softplus(ROUND(h @ w["a"].T) + w["dt_bias"]))
    gate = silu(ROUND(h @ w["g"].T)).view(T, H, dv)
    rep = H // HK
    o = torch.stack([delta_rule(q[:, i // rep], k[:, i // rep], v[:, i], beta[:, i], g[:, i]) for i in range(H)], 1)
    y = ROUND(rms(o, eps) * w["norm"] * gate)
    return ROUND(y.reshape(T, H * dv) @ w["o"].T)


def yarn_frequencies(dims: int, base: float, scaling: dict | None):
    """``(frequencies [dims / 2], factor on cos and sin)``."""
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = scaling["factor"], scaling["original"]
    where = lambda t: dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(where(scaling["fast"])), 0)
    hi = min(math.ceil(where(scaling["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, freqs, mag):
    """Turns the neighbouring pairs ``(x[2i], x[2i + 1])`` of the last axis by ``position * freqs[i]``;
    ``x`` is ``[T, ..., 2 n]`` with ``n = len(freqs)``."""
    a = positions.to(F64)[:, None] * freqs[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [freqs.numel()]
    c, s = (torch.cos(a) * mag).view(shape), (torch.sin(a) * mag).view(shape)
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


def softmax_attention(q, k, v, scale, window=None, sinks=None):
    """``q`` ``[T, H, d]``, ``k`` ``[T, H, d]``, ``v`` ``[T, H, dv]``.  Query ``i`` sees ``j <= i`` and, with a
    window, ``i - j < window``.  ``sinks`` ``[H]`` adds ``exp(sink)`` to each denominator."""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        s = torch.einsum("jhd,hd->hj", k[lo:i + 1], q[i]) * scale                 # [H, keys]
        m = s.max(dim=1).values if sinks is None else torch.maximum(s.max(dim=1).values, sinks)
        e = torch.exp(s - m[:, None])
        den = e.sum(dim=1) + (torch.exp(sinks - m) if sinks is not None else 0.0)
        out[i] = torch.einsum("hj,jhd->hd", e / den[:, None], v[lo:i + 1])
    return out


def latent_attention(h, w, m, eps, positions):
    """Latent attention with a rotated part: the keys and values of all heads come from one latent
    per token, one rotated key part is shared by the heads; sink in the softmax; sigmoid output gate."""
    T = h.shape[0]
    H, d, dr, dv, r = m["heads"], m["dim"], m.get("rot_dim", 0), m["vdim"], m["kv_rank"]
    q = ROUND(h @ w["q"].T).view(T, H, d + dr)
    dkv = ROUND(h @ w["dkv"].T)
    c = ROUND(rms(dkv[:, :r], eps) * w["dkv.norm"])
    k_rot = dkv[:, r:].clone()
    q_rot = q[..., d:].clone()
    if dr:
        rot = m["rot"]
        n_rot = rot.get("dims", dr)
        freqs, mag = yarn_frequencies(n_rot, rot["base"], rot.get("scaling"))
        k_rot[:, :n_rot] = rotate_pairs(k_rot[:, :n_rot], positions, freqs, mag)
        q_rot[..., :n_rot] = rotate_pairs(q_rot[..., :n_rot], positions, freqs, mag)
    k_rot = ROUND(k_rot)
    k = torch.cat([ROUND(c @ w["uk"].T).view(T, H, d), k_rot[:, None, :].expand(T, H, dr)], -1)
    v = ROUND(c @ w["uv"].T).view(T, H, dv)
    o = softmax_attention(torch.cat([q[..., :d], q_rot], -1), k, v, m["scale"], None, w["sink"])
    o = ROUND(ROUND(o.reshape(T, H * dv)) * torch.sigmoid(ROUND(h @ w["g"].T)))
    return ROUND(o @ w["o"].T)


def latent_window_attention(h, w, m, eps):
    """Latent attention without positions: queries through a latent of their own, a sliding window,
    an ordinary softmax."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    cq = ROUND(rms(ROUND(h @ w["dq"].T), eps) * w["dq.norm"])
    q = ROUND(cq @ w["uq"].T).view(T, H, d)
    c = ROUND(rms(ROUND(h @ w["dkv"].T), eps) * w["dkv.norm"])
    k = ROUND(c @ w["uk"].T).view(T, H, d)
    v = ROUND(c @ w["uv"].T).view(T, H, dv)
    o = softmax_attention(q, k, v, m["scale"], m["mask"]["size"], None)
    return ROUND(ROUND(o.reshape(T, H * dv)) @ w["o"].T)


def dense_ff(h, w):
    return ROUND(ROUND(silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T)


def forward(config: dict, tensors: dict, tokens, return_layers: bool = False, round_to=None):
    """Logits ``[T, vocab]`` of one sequence from position 0; ``tensors``: name -> float64 tensor.
    ``round_to`` (a 16-bit dtype) rounds activations where a 16-bit engine does; the residual stream,
    norms' statistics, scores and the recurrence stay exact."""
    global ROUND
    keep = ROUND
    if round_to is not None:
        ROUND = lambda x: x.to(round_to).to(F64)
    try:
        return _forward(config, tensors, tokens, return_layers)
    finally:
        ROUND = keep


def _forward(config, tensors, tokens, return_layers):
    eps = config["norm"]["eps"]
    x = tensors["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config.get("embedding", {}).get("scale", 1.0)
    positions = torch.arange(x.shape[0])
    after = []
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        w = {k[len(pre) + 4:]: v for k, v in tensors.items() if k.startswith(pre + "mix.")}
        m = layer["mixer"]
        h = ROUND(x)
        if layer["type"] == "delta":
            y = delta_mixer(h, w, m, eps)
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, w, m, eps, positions)
        elif layer["type"] == "latent_attention_2":
            y = latent_window_attention(h, w, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + offset_norm(y, tensors[pre + "norm1"], eps)
        if layer.get("mlp") is not None:
            wf = {k[len(pre) + 4:]: v for k, v in tensors.items() if k.startswith(pre + "mlp.")}
            x = x + offset_norm(dense_ff(ROUND(x), wf), tensors[pre + "norm2"], eps)
        after.append(x.clone())
    logits = ROUND(offset_norm(x, tensors["final.norm"], eps)) @ tensors["head"].T
    return (logits, torch.stack(after)) if return_layers else logits


def load_folder(folder) -> tuple[dict, dict]:
    """``(config, name -> float64 tensor)`` of a model folder; the safetensors file is read by its header
    (an 8-byte length, that many bytes of JSON, then the data)."""
    import json
    import struct
    from pathlib import Path
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + a:8 + n + b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        tensors[name] = t.to(F64)
    return config, tensors


def greedy_generate(config: dict, tensors: dict, prompt, new_tokens: int) -> list[int]:
    seq = list(prompt)
    for _ in range(new_tokens):
        seq.append(int(forward(config, tensors, seq)[-1].argmax()))
    return seq[len(prompt):]
