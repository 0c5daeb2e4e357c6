"""The Logivik design on the GPU: every mechanism's kernel against the plain implementation, then
whole models under every way of cutting and batching their requests, and generation through the
engine's entry point."""

from __future__ import annotations

import functools
import json
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch

import logivik_configs as lc
import traces
from helpers import assert_logits_close, random_tokens
from plain import logivik_plain as plain

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_TMP = []


@functools.lru_cache(maxsize=None)
def folder_of(tag: str, dtype: str) -> Path:
    from tokamak_b200.weights import write_random_model
    raw, init, _ = lc.ALL[tag]
    tmp = tempfile.TemporaryDirectory(prefix=f"tk_{tag}_{dtype}_")
    _TMP.append(tmp)
    write_random_model(tmp.name, raw, dtype=dtype, **init)
    return Path(tmp.name)


@functools.lru_cache(maxsize=None)
def _truth(folder: str, tokens: tuple) -> torch.Tensor:
    cfg, w = plain.load_folder(folder)
    return plain.forward(cfg, w, list(tokens))


def truth(folder, tokens) -> torch.Tensor:
    return _truth(str(folder), tuple(int(t) for t in tokens))


@functools.lru_cache(maxsize=None)
def _rounded(folder: str, tokens: tuple) -> torch.Tensor:
    cfg, w = plain.load_folder(folder)
    return plain.forward(cfg, w, list(tokens), round_to=torch.bfloat16)


# bfloat16: a row is judged against what rounding alone costs in its request: the plain implementation
# rounding where a 16-bit engine rounds gives, row by row, an error of its own; rows differ by the luck of
# the draw (measured over these models: the engine's mean error equals that baseline's, the ratio of the two
# on single rows scatters from 0.1 to 20), so the level is the worst row of the request, the limit four times
# that, and never below the level of a well-conditioned row.  A wrong key, page, state or mask moves a row
# by about its spread.
BF16_FLOOR_RMS, BF16_FLOOR_MAX, BF16_TIMES = 0.05, 0.2, 4.0


@functools.lru_cache(maxsize=None)
def _rounding_level(folder: str, tokens: tuple) -> tuple[float, float]:
    want = _truth(folder, tokens)
    rel = (_rounded(folder, tokens) - want).abs() / want.std(dim=-1, keepdim=True).clamp_min(1e-6)
    return rel.pow(2).mean(-1).sqrt().max().item(), rel.max().item()


def check_rows(results, rows, reqs, folder, dtype, what) -> int:
    n = 0
    for step in sorted(rows):
        got = torch.from_numpy(np.asarray(results[step])).double()
        for i, (rid, p) in enumerate(rows[step]):
            where = f"{what}: step {step}, request {rid!r}, position {p}"
            want = truth(folder, reqs[rid])[p]
            if dtype == "float32":
                assert_logits_close(got[i:i + 1], want[None], dtype, where)
            else:
                mine = (got[i] - want).abs() / want.std().clamp_min(1e-6)
                base_rms, base_max = _rounding_level(str(folder), tuple(int(t) for t in reqs[rid]))
                assert torch.isfinite(got[i]).all(), where
                rms = mine.pow(2).mean().sqrt().item()
                assert rms <= max(BF16_FLOOR_RMS, BF16_TIMES * base_rms), (
                    f"{where}: off by {rms:.3e} (rms) of the row's spread; rounding alone costs up to {base_rms:.3e}")
                assert mine.max().item() <= max(BF16_FLOOR_MAX, BF16_TIMES * base_max), (
                    f"{where}: off by {mine.max().item():.3e} (max) of the row's spread; rounding alone costs up to "
                    f"{base_max:.3e}")
            n += 1
    return n


def dev(x, dtype=None):
    return x.to("cuda", dtype) if dtype is not None else x.to("cuda")


def i32(*v):
    return torch.tensor(v, dtype=torch.int32, device="cuda")


def close(got, want, dtype, scale=1.0):
    got, want = got.detach().cpu().double(), want.double()
    tol = (2e-5 if dtype == "float32" else 2e-2) * scale
    err = (got - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), f"off by {err:.3e}"


def new_err():
    return torch.zeros(4, dtype=torch.int32, device="cuda")


# ======================================================================= mechanisms alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [40, 1030, 2048])        # the general kernel (1030) and the one on 16-byte pieces
def test_branch_joins_the_stream_and_the_rows_go_on_unnormalised(dtype, width):
    """x += (1 + w) * rms(branch); the next sublayer reads x itself, rounded to the engine's type."""
    from tokamak_b200.parts.base import NormedBranch, Runtime
    from tokamak_b200.parts.norm import CastNorm, CastNormSpec, OffsetRMSNorm, OffsetRMSNormSpec
    g = torch.Generator().manual_seed(width)
    n = 6
    rt = Runtime(torch.device("cuda"), TORCH[dtype])
    resid = torch.randn(n, width, generator=g)
    branch = (3 * torch.randn(n, width, generator=g)).to(TORCH[dtype]).float()
    w = 0.4 * torch.randn(width, generator=g)
    norm = OffsetRMSNorm(OffsetRMSNormSpec(width, 1e-5), "n", {"n": dev(w)}, rt)
    assert torch.equal(norm.weight.cpu(), 1.0 + w)
    cast = CastNorm(CastNormSpec(width), "", {}, rt)
    want = resid.double() + plain.offset_norm(branch.double(), w.double(), 1e-5)
    weight, eps = norm.owed_norm_params()
    r = dev(resid.clone())
    h = cast.add_norm(r, NormedBranch(dev(branch, TORCH[dtype]), weight, eps))
    close(r, want, "float32")
    assert h.dtype == TORCH[dtype] and torch.equal(h.float(), r.to(TORCH[dtype]).float())
    # split sums of a product, and only chosen rows: the stream is left alone
    r2 = dev(resid.clone())
    parts = dev(torch.stack([branch * 0.25, branch * 0.75]))
    rows = i32(4, 1)
    h2 = cast.add_norm(r2, NormedBranch(parts, weight, eps), rows=rows)
    assert torch.equal(r2.cpu(), resid)
    close(h2, want[[4, 1]], dtype)
    # nothing pending (the first sublayer of a model): the rows as they are
    assert torch.equal(cast.add_norm(r, None).float(), r.to(TORCH[dtype]).float())
    # the model's last norm joins the branch and norms with 1 + w
    last = OffsetRMSNorm(OffsetRMSNormSpec(width, 1e-6), "f", {"f": dev(w)}, rt)
    r3 = dev(resid.clone())
    out = last.add_norm(r3, NormedBranch(dev(branch, TORCH[dtype]), weight, eps))
    close(out, plain.offset_norm(want, w.double(), 1e-6), dtype, scale=2.0)


@pytest.mark.parametrize("dims,base,scaling", [(8, 10000.0, (4.0, 32, 8.0, 1.0)), (32, 1e6, (2.0, 512, 32.0, 1.0)),
                                               (64, 500.0, (8.0, 64, 4.0, 0.5)), (16, 10000.0, None)])
def test_stretched_pair_rotation_table(dims, base, scaling):
    from tokamak_b200.csrc import ops
    from tokamak_b200.parts.position import YarnScaling, yarn_frequencies
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    want_f, want_mag = plain.yarn_frequencies(dims, base, sc)
    freq, mag = yarn_frequencies(dims, base, YarnScaling(*scaling) if scaling else None)
    assert mag == pytest.approx(want_mag, rel=1e-12) and torch.allclose(freq, want_f, rtol=1e-12, atol=0)
    if scaling:
        assert (freq <= want_f.new_tensor(base) ** (-torch.arange(0, dims, 2, dtype=torch.float64) / dims) + 1e-15).all()
    pos = torch.tensor([0, 1, 2, 63, 64, 1000, 5000], dtype=torch.int32)
    table = ops.rope_table(dev(pos), dev(freq.float()), mag).cpu().double()
    ang = pos.double()[:, None] * freq.float().double()[None, :]
    assert (table[..., 0] - torch.cos(ang) * mag).abs().max() < 5e-4      # float32 angles at position 5000
    assert (table[:5, :, 0] - torch.cos(ang[:5]) * mag).abs().max() < 2e-6
    assert (table[:5, :, 1] - torch.sin(ang[:5]) * mag).abs().max() < 2e-6


def _latent_case(dtype, n, heads, d, dr, rank, n_rot, q_rank, seed):
    g = torch.Generator().manual_seed(seed)
    cols_q = q_rank if q_rank else heads * (d + dr)
    row = cols_q + rank + dr + 5
    proj = torch.randn(n, row, generator=g).to(TORCH[dtype])
    wc = 1 + 0.3 * torch.randn(rank, generator=g)
    return g, proj, row, cols_q, wc


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,d,dr,rank,n_rot", [(3, 16, 8, 24, 8), (4, 8, 12, 16, 8), (2, 32, 64, 96, 64), (5, 4, 6, 300, 2)])
def test_latent_rows_rotated_part_and_query_rows(dtype, heads, d, dr, rank, n_rot):
    """The cache row [c | rot(k_r)] lands in the token's page and slot, the query rows are the absorbed part
    beside the turned part; positions come from a table that already holds the stretch."""
    from tokamak_b200.csrc import ops
    n, page, n_pages = 11, 4, 9
    g, proj, row, cols_q, wc = _latent_case(dtype, n, heads, d, dr, rank, n_rot, None, seed=d * dr)
    positions = [5, 6, 7, 8, 9, 0, 1, 2, 13, 14, 15]          # three requests: 5 tokens from 5, 3 from 0, 3 from 13
    tok_req = [0] * 5 + [1] * 3 + [2] * 3
    slots = [2, 0, 1]
    table_pages = torch.full((3, 6), -1, dtype=torch.int32)
    table_pages[2, :3] = torch.tensor([7, 3, 8]); table_pages[0, :1] = 5; table_pages[1, :4] = torch.tensor([1, 0, 2, 6])
    freqs, mag = plain.yarn_frequencies(n_rot, 10000.0, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0})
    pos_t = torch.tensor(positions)
    rope = ops.rope_table(dev(pos_t.int()), dev(freqs.float()), mag)
    cache = torch.zeros(n_pages, 1, page, rank + dr, dtype=TORCH[dtype], device="cuda")
    q_abs = torch.randn(heads, n, rank, generator=g)
    err = new_err()
    args = (dev(pos_t.int()), dev(torch.tensor(tok_req, dtype=torch.int32)), i32(*slots), dev(table_pages), err)
    kw = dict(kv_off=cols_q, rank=rank, rot=dr, kv_norm_w=dev(wc), eps=1e-5, table=rope, q_abs=dev(q_abs), q_off=0,
              q_head_cols=d + dr, q_rot_off=d)
    q_lat, cq = ops.latent_prepare(dev(proj), cache, *args, **kw)
    assert err.cpu().tolist()[0] == 0 and cq is None
    x = proj.double()
    f32 = freqs.float().double()
    c = plain.rms(x[:, cols_q:cols_q + rank], 1e-5) * wc.double()
    kr = x[:, cols_q + rank:cols_q + rank + dr].clone()
    kr[:, :n_rot] = plain.rotate_pairs(kr[:, :n_rot], pos_t, f32, mag)
    want_rows = torch.cat([c, kr], 1)
    for t in range(n):
        pg = table_pages[slots[tok_req[t]], positions[t] // page].item()
        close(cache[pg, 0, positions[t] % page], want_rows[t], dtype, scale=2.0)
    qr = x[:, :cols_q].reshape(n, heads, d + dr)[..., d:].clone()
    qr[..., :n_rot] = plain.rotate_pairs(qr[..., :n_rot], pos_t, f32, mag)
    close(q_lat[..., :rank], q_abs.transpose(0, 1), "float32")
    close(q_lat[..., rank:], qr, "float32", scale=2.0)
    # the same from the partial sums of a split product
    cache2 = torch.zeros_like(cache)
    halves = dev(torch.stack([proj.float() * 0.5, proj.float() * 0.5]))
    q_lat2, _ = ops.latent_prepare(halves, cache2, *args, **kw)
    assert torch.equal(q_lat2, q_lat) and torch.equal(cache2, cache)
    # untouched pages stay untouched
    assert not cache[4].any()


@pytest.mark.parametrize("dtype", DTYPES)
def test_query_latent_is_normed_beside_the_cache_write(dtype):
    from tokamak_b200.csrc import ops
    n, rank, q_rank, page = 7, 40, 12, 8
    g, proj, row, cols_q, wc = _latent_case(dtype, n, 2, 24, 0, rank, 0, q_rank, seed=3)
    wq = 1 + 0.3 * torch.randn(q_rank, generator=g)
    cache = torch.zeros(3, 1, page, rank, dtype=TORCH[dtype], device="cuda")
    err = new_err()
    table_pages = torch.tensor([[2, 0, -1]], dtype=torch.int32)
    q_lat, cq = ops.latent_prepare(dev(proj), cache, dev(torch.arange(4, 4 + n, dtype=torch.int32)),
                                   dev(torch.zeros(n, dtype=torch.int32)), i32(0), dev(table_pages), err, kv_off=cols_q,
                                   rank=rank, rot=0, kv_norm_w=dev(wc), eps=1e-6, cq_off=0, cq_norm_w=dev(wq))
    assert q_lat is None and err.cpu().tolist()[0] == 0
    x = proj.double()
    close(cq, plain.rms(x[:, :q_rank], 1e-6) * wq.double(), dtype, scale=2.0)
    c = plain.rms(x[:, cols_q:cols_q + rank], 1e-6) * wc.double()
    got = torch.cat([cache[2, 0, 4:], cache[0, 0, :3]])
    close(got, c, dtype, scale=2.0)


def _attend(q, rows_by_pos, n_ctx, scale, window, sinks, rank):
    """Plain attention of one query over latent rows 0 .. n_ctx - 1 (values: the leading ``rank`` elements)."""
    H = q.shape[0]
    k = rows_by_pos[:n_ctx, None, :].expand(n_ctx, H, rows_by_pos.shape[1])
    out = plain.softmax_attention(torch.cat([torch.zeros(n_ctx - 1, H, q.shape[1], dtype=torch.float64), q[None]]),
                                  k, k[..., :rank], scale, window, sinks)
    return out[-1]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rank,dr,window", [(24, 8, None), (40, 0, 9), (96, 64, None), (300, 4, 33), (16, 0, 1)])
def test_attention_over_latent_rows_with_stand_out_keys(dtype, rank, dr, window):
    """Float32 queries over pages whose values are the leading part of the key rows.  One key far back, at a
    page border or just inside / just outside the window is made to stand out (its score beats all others),
    so a key that is lost, or seen when it should not be, changes the result by about its own value; a sink
    that is left out changes every weight."""
    from tokamak_b200.csrc import ops
    H, page, ctx = 3, 8, 150
    g = torch.Generator().manual_seed(rank + dr)
    width = rank + dr
    rows = (0.3 * torch.randn(ctx, width, generator=g)).to(TORCH[dtype])
    n_pages = -(-ctx // page)
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    cache = torch.zeros(n_pages + 3, 1, page, width, dtype=TORCH[dtype], device="cuda")
    for p in range(ctx):
        cache[perm[p // page], 0, p % page] = dev(rows[p])
    table = torch.full((2, n_pages + 2), -1, dtype=torch.int32)
    table[1, :n_pages] = perm.int()
    sinks = torch.tensor([0.5, -1.0, 2.0]) if window is None else None
    scale = 0.4
    v_view = cache[..., :rank]
    # queries: decoded single tokens and a prompt portion's tokens at chosen positions
    w = window or ctx
    special = sorted({ctx - 1, page * 5, page * 5 - 1, w - 1, min(ctx - 1, w), 0, 1})
    for qpos in special:
        targets = [0, qpos, max(0, qpos - w + 1), max(0, qpos - w), (qpos // page) * page, max(0, (qpos // page) * page - 1)]
        for far in sorted({t for t in targets if t <= qpos}):
            q = 0.2 * torch.randn(H, width, generator=g)
            key = rows[far].double()
            q[1] = (key / key.norm() * 25.0 / scale / key.norm()).float()        # head 1 scores 25 on key `far`
            q_dev = dev(q[None].contiguous())
            out = torch.empty(1, H, rank, dtype=TORCH[dtype], device="cuda")
            err = new_err()
            ops.attention_plain(q_dev, out, cache, v_view, i32(qpos), i32(0), i32(1), dev(table), err, scale=scale,
                                window=window, sinks=dev(sinks) if sinks is not None else None)
            assert err.cpu().tolist()[0] == 0
            want = _attend(q.double(), rows.double(), qpos + 1, scale, window, sinks.double() if sinks is not None else None, rank)
            close(out[0], want, dtype, scale=2.0)
            seen = qpos - far < w
            near = (out[0, 1].cpu().double() - rows[far, :rank].double()).abs().max().item()
            assert (near < 0.05) == seen, (qpos, far, near)
    # a portion of a prompt beside a single token of another request, chosen rows only
    pos = torch.tensor([40, 41, 42, 43, 149], dtype=torch.int32)
    q = 0.2 * torch.randn(5, H, width, generator=g)
    out = torch.zeros(5, H, rank, dtype=TORCH[dtype], device="cuda")
    err = new_err()
    table2 = torch.cat([table, table[1:2]])
    ops.attention_plain(dev(q), out, cache, v_view, dev(pos), i32(0, 0, 0, 0, 1), i32(1, 2), dev(table2), err,
                        scale=scale, window=window, sinks=dev(sinks) if sinks is not None else None, items=i32(4, 1, 3))
    assert err.cpu().tolist()[0] == 0 and not out[0].any() and not out[2].any()
    for t in (1, 3, 4):
        want = _attend(q[t].double(), rows.double(), int(pos[t]) + 1, scale, window, sinks.double() if sinks is not None else None, rank)
        close(out[t], want, dtype, scale=2.0)
    # queries given head-major (the layout a per-head product leaves) are read through their strides
    q_hm = dev(q.transpose(0, 1).contiguous())
    out2 = torch.zeros_like(out)
    ops.attention_plain(q_hm.transpose(0, 1), out2, cache, v_view, dev(pos), i32(0, 0, 0, 0, 1), i32(1, 2), dev(table2), err,
                        scale=scale, window=window, sinks=dev(sinks) if sinks is not None else None, items=i32(4, 1, 3))
    assert torch.equal(out2, out)


@pytest.mark.parametrize("H,rank,dr,window", [(3, 64, 32, None), (16, 128, 64, 70), (4, 512, 64, None), (5, 16, 0, 1),
                                              (70, 32, 16, 9)])
def test_tensor_core_attention_over_latent_rows(H, rank, dr, window):
    """The kernel that stacks a token's heads as rows of a tile: a portion of a prompt (two 64-token tiles,
    the second one ragged) beside single tokens of two other requests whose keys are cut into 1, 2 and 5
    shares; every query token makes one key stand out for head 1: far back, at a page border, the first or
    the last key inside its window, the first one outside."""
    from types import SimpleNamespace
    from tokamak_b200.csrc import ops
    page, ctx, scale = 8, 150, 0.4
    width = rank + dr
    assert ops.latent_kernel_takes(width, rank)
    g = torch.Generator().manual_seed(H + rank)
    w = window or ctx
    seqs = [(0.3 * torch.randn(n, width, generator=g)).bfloat16() for n in (ctx, 131, 64)]
    n_pages = sum(-(-len(x) // page) for x in seqs)
    perm = torch.randperm(n_pages + 2, generator=g)
    cache = torch.zeros(n_pages + 2, 1, page, width, dtype=torch.bfloat16, device="cuda")
    table = torch.full((4, 32), -1, dtype=torch.int32)
    slots, at = [2, 0, 3], 0
    for x, slot in zip(seqs, slots):
        for p in range(len(x)):
            if p % page == 0:
                table[slot, p // page] = perm[at]; at += 1
            cache[table[slot, p // page], 0, p % page] = dev(x[p])
    q_len = [70, 1, 1]
    kv_len = [len(x) for x in seqs]
    starts = [0, 70, 71]
    positions = list(range(ctx - 70, ctx)) + [130, 63]
    tok_req = [0] * 70 + [1, 2]
    q = 0.2 * torch.randn(72, H, width, generator=g)
    targets = []
    for t, (pos, r) in enumerate(zip(positions, tok_req)):
        choices = [pos, max(0, pos - w + 1), max(0, pos - w), (pos // page) * page, max(0, (pos // page) * page - 1), 0, pos // 2]
        far = choices[t % len(choices)]
        key = seqs[r][far].double()
        q[t, 1 % H] = (key * 25.0 / scale / key.norm() ** 2).float()
        targets.append(far)
    sinks = torch.linspace(-1.0, 2.0, H) if window is None else None
    step = SimpleNamespace(positions=dev(torch.tensor(positions, dtype=torch.int32)), tok_req=dev(torch.tensor(tok_req, dtype=torch.int32)),
                           req_q_start=i32(*starts), req_q_len=i32(*q_len), req_kv_len=i32(*kv_len), req_slot=i32(*slots),
                           err=new_err())
    want = torch.zeros(72, H, rank, dtype=torch.float64)
    for t, (pos, r) in enumerate(zip(positions, tok_req)):
        want[t] = _attend(q[t].bfloat16().double(), seqs[r].double(), pos + 1, scale, window,
                          sinks.double() if sinks is not None else None, rank)
    kw = dict(scale=scale, window=window, sinks=dev(sinks) if sinks is not None else None)
    tiles = i32(0, 1, 0, 0)                    # (request row, tile) pairs, the ragged tile first
    for q_dev in (dev(q), dev(q.bfloat16()), dev(q.transpose(0, 1).contiguous()).transpose(0, 1)):
        for n_splits in (1, 2, 5):
            out = torch.zeros(72, H, rank, dtype=torch.bfloat16, device="cuda")
            ops.attention_latent(q_dev, out, cache, rank, step, dev(table), tiles=tiles, **kw)
            ops.attention_latent(q_dev, out, cache, rank, step, dev(table), items=i32(71, 70), n_splits=n_splits, **kw)
            assert step.err.cpu().tolist()[0] == 0
            close(out, want, "bfloat16", scale=2.0)
            for t, far in enumerate(targets):
                seen = positions[t] - far < w
                near = (out[t, 1 % H].cpu().double() - seqs[tok_req[t]][far, :rank].double()).abs().max().item()
                assert (near < 0.05) == seen, (t, positions[t], far, near)


@pytest.mark.parametrize("dtype", DTYPES)
def test_per_head_products_and_the_gated_way_back(dtype):
    from tokamak_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    n, H, K, M = 37, 3, 20, 70
    x = torch.randn(n, H, K + 6, generator=g)
    w = torch.randn(H, M, K, generator=g)
    out = ops.gemm_f32_heads(dev(x)[:, :, 2:2 + K], dev(w))
    want = torch.einsum("nhk,hmk->hnm", x[:, :, 2:2 + K].double(), w.double())
    close(out, want, "float32", scale=4.0)
    o = torch.randn(H, n, 12, generator=g).to(TORCH[dtype])
    proj = torch.randn(n, 9 + H * 12, generator=g).to(TORCH[dtype])
    y = ops.heads_gate(dev(o), dev(proj), 9)
    want = o.double().permute(1, 0, 2).reshape(n, H * 12) * torch.sigmoid(proj.double()[:, 9:])
    close(y, want, dtype)
    y2 = ops.heads_gate(dev(o), dev(torch.stack([proj.float() * 0.5, proj.float() * 0.5])), 9)
    close(y2, want, dtype)
    close(ops.heads_gate(dev(o)), o.double().permute(1, 0, 2).reshape(n, H * 12), dtype)


def _delta_inputs(dtype, H, HK, dk, dv, taps, lens, seed):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    hk, hv = HK * dk, H * dv
    row = 2 * hk + 2 * hv + 2 * H + 3
    proj = torch.randn(T, row, generator=g).to(TORCH[dtype])
    conv = 0.5 * torch.randn(2 * hk + hv, taps, generator=g)
    a_log = 0.5 * torch.randn(H, generator=g)
    dt_bias = 0.5 * torch.randn(H, generator=g)
    offs = dict(q_off=0, k_off=hk, v_off=2 * hk, b_off=2 * hk + 2 * hv + 3, a_off=2 * hk + 2 * hv + 3 + H)
    return g, proj, conv, a_log, dt_bias, offs


def _delta_plain(x, conv, a_log, dt_bias, offs, H, HK, dk, dv):
    """q, k, v, beta, g of one request's whole sequence ``x`` [T, row] by the plain functions."""
    T = x.shape[0]
    hk, hv = HK * dk, H * dv
    cut = lambda off, n: x[:, off:off + n]
    q = plain.silu(plain.short_conv(cut(offs["q_off"], hk), conv[:hk].double())).view(T, HK, dk)
    k = plain.silu(plain.short_conv(cut(offs["k_off"], hk), conv[hk:2 * hk].double())).view(T, HK, dk)
    v = plain.silu(plain.short_conv(cut(offs["v_off"], hv), conv[2 * hk:].double())).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(cut(offs["b_off"], H))
    g = torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(cut(offs["a_off"], H) + dt_bias.double()))
    return q, k, v, beta, g


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,HK,dk,dv,taps", [(4, 2, 16, 24, 3), (6, 1, 12, 10, 5), (3, 3, 6, 40, 1), (2, 1, 130, 80, 4),
                                             (2, 2, 64, 64, 2), (1, 1, 256, 33, 4)])
def test_delta_rule_inputs_recurrence_and_state_over_steps(dtype, H, HK, dk, dv, taps):
    """Three requests in slots 2, 0, 3 of 4, fed in two steps of unequal portions (the second step's first
    tokens read the convolution's tail of the first) and a step of one token each (the kernel of the inputs
    moves the tails on itself): inputs, outputs, state and tail against the plain functions run over each
    request's whole sequence."""
    from tokamak_b200.csrc import ops
    first, second, third = [9, 1, 30], [2, 5, 1], [1, 1, 1]
    slots = [2, 0, 3]
    totals = [a + b + c for a, b, c in zip(first, second, third)]
    g, proj, conv, a_log, dt_bias, offs = _delta_inputs(dtype, H, HK, dk, dv, taps, totals, seed=dk + dv)
    floats, tail_off = ops.delta_record_floats(H, HK, dk, dv, taps)
    records = torch.zeros(4, floats, device="cuda")
    records[1] = 7.0                                     # a slot of no request: left alone
    starts_all = [0, totals[0], totals[0] + totals[1]]
    seqs = [proj[s:s + n] for s, n in zip(starts_all, totals)]
    err = new_err()
    got_o = [[] for _ in seqs]
    got_in = [[] for _ in seqs]
    for lens, at in ((first, [0, 0, 0]), (second, first), (third, [a + b for a, b in zip(first, second)])):
        step_proj = torch.cat([seq[a:a + n] for seq, a, n in zip(seqs, at, lens)])
        starts = [0, lens[0], lens[0] + lens[1]]
        tok_req = sum(([r] * n for r, n in enumerate(lens)), [])
        meta = (dev(torch.tensor(tok_req, dtype=torch.int32)), i32(*starts), i32(*lens), i32(*slots), err)
        kw = dict(dtype=TORCH[dtype], heads=H, kv_heads=HK, key_dim=dk, value_dim=dv, unit_eps=1e-6, q_scale=dk ** -0.5, **offs)
        # both launch shapes and the split sums of a product give the same bits (on copies: the tail moves on)
        halves = dev(torch.stack([step_proj.float() * 0.5, step_proj.float() * 0.5]))
        others = [ops.delta_prepare(x, dev(conv), dev(a_log), dev(dt_bias), records.clone(), *meta, shape=shape, **kw)
                  for x, shape in ((dev(step_proj), 1), (dev(step_proj), 2), (halves, 0))]
        q, k, v, beta, gg = ops.delta_prepare(dev(step_proj), dev(conv), dev(a_log), dev(dt_bias), records, *meta, **kw)
        for other in others:
            assert all(torch.equal(a, b) for a, b in zip(other, (q, k, v, beta, gg)))
        o = ops.delta_scan(q, k, v, beta, gg, records, *meta[1:])
        for r, (s, n) in enumerate(zip(starts, lens)):
            got_o[r].append(o[s:s + n].cpu())
            got_in[r].append([t[s:s + n].cpu() for t in (q, k, v, beta, gg)])
    assert err.cpu().tolist()[0] == 0
    assert (records[1] == 7.0).all()
    for r, seq in enumerate(seqs):
        q, k, v, beta, gg = _delta_plain(seq.double(), conv, a_log, dt_bias, offs, H, HK, dk, dv)
        for i, want in enumerate((q, k, v, beta, gg)):
            close(torch.cat([part[i] for part in got_in[r]]), want, "float32", scale=5.0)
        rep = H // HK
        want_o = torch.stack([plain.delta_rule(q[:, h // rep], k[:, h // rep], v[:, h], beta[:, h], gg[:, h]) for h in range(H)], 1)
        close(torch.cat(got_o[r]), want_o, "float32", scale=20.0)
        # the state after all tokens, and the tail: the last taps - 1 inputs
        S = torch.zeros(H, dk, dv, dtype=torch.float64)
        for h in range(H):
            for t in range(seq.shape[0]):
                S[h] = gg[t, h] * S[h]
                u = beta[t, h] * (v[t, h] - S[h].T @ k[t, h // rep])
                S[h] += torch.outer(k[t, h // rep], u)
        close(records[slots[r], :tail_off].view(H, dk, dv), S, "float32", scale=20.0)
        if taps > 1:
            hk, hv = HK * dk, H * dv
            chans = torch.cat([seq[:, :2 * hk + hv]], 1).float()
            want_tail = torch.zeros(taps - 1, 2 * hk + hv)
            have = min(taps - 1, seq.shape[0])
            want_tail[taps - 1 - have:] = chans[seq.shape[0] - have:]
            assert torch.equal(records[slots[r], tail_off:].view(taps - 1, -1).cpu(), want_tail)


def test_delta_rule_is_bit_equal_however_the_tokens_are_cut_and_split():
    from tokamak_b200.csrc import ops
    H, HK, dk, dv, T = 4, 2, 48, 40, 67
    g = torch.Generator().manual_seed(5)
    q = torch.randn(T, HK, dk, generator=g) / dk
    k = torch.nn.functional.normalize(torch.randn(T, HK, dk, generator=g), dim=-1)
    v = torch.randn(T, H, dv, generator=g)
    beta, gg = torch.rand(T, H, generator=g), torch.exp(-0.3 * torch.rand(T, H, generator=g))
    err = new_err()

    def run(cuts, cols=0):
        records = torch.zeros(2, H * dk * dv + 5, device="cuda")
        outs, at = [], 0
        for n in cuts:
            part = [dev(t[at:at + n].contiguous()) for t in (q, k, v, beta, gg)]
            outs.append(ops.delta_scan(*part, records, i32(0), i32(n), i32(1), err, cols=cols))
            at += n
        return torch.cat(outs), records
    o1, s1 = run([T])
    o2, s2 = run([2, 7, 1, 1, 16, 8, 9, 23])
    assert torch.equal(o1, o2) and torch.equal(s1, s2)
    assert not s1[0].any() and not s1[1, H * dk * dv:].any()
    for cols in (16, 32, 64):            # other splits of the columns add in another order: equal to rounding
        o3, s3 = run([T], cols)
        o4, s4 = run([5, 62], cols)
        assert torch.equal(o3, o4) and torch.equal(s3, s4)
        assert (o3 - o1).abs().max() <= 1e-5 * o1.abs().max()
    assert err.cpu().tolist()[0] == 0


def test_delta_rule_remembers_a_far_write_and_forgets_by_its_decay():
    """A value written under a key 300 tokens back is read out exactly while the decay is 1 and other keys
    are orthogonal, and is gone when the decay is small: a state that is lost or not decayed shows."""
    from tokamak_b200.csrc import ops
    H, dk, dv, T = 1, 32, 16, 301
    k = torch.zeros(T, 1, dk); v = torch.zeros(T, 1, dv)
    k[0, 0, 3] = 1.0; v[0, 0] = torch.arange(1, dv + 1).float()
    for t in range(1, T - 1):
        k[t, 0, 4 + t % 20] = 1.0
        v[t, 0] = 0.01 * t
    k[T - 1, 0, 31] = 1.0
    q = torch.zeros(T, 1, dk); q[T - 1, 0, 3] = 1.0
    beta = torch.ones(T, 1)
    err = new_err()
    for decay, want in ((1.0, v[0, 0]), (0.99, v[0, 0] * 0.99 ** 300)):
        gg = torch.full((T, 1), decay)
        for cuts in ([T], [100, 1, 199, 1]):
            records = torch.zeros(1, dk * dv, device="cuda")
            at, outs = 0, []
            for n in cuts:
                part = [dev(t[at:at + n].contiguous()) for t in (q, k, v, beta, gg)]
                outs.append(ops.delta_scan(*part, records, i32(0), i32(n), i32(0), err))
                at += n
            assert torch.allclose(torch.cat(outs)[-1, 0].cpu(), want, rtol=1e-4, atol=1e-12)
    assert err.cpu().tolist()[0] == 0


# ======================================================================= whole models

LENGTHS = {"LA": [5, 17, 33, 70, 130, 96, 41, 128], "LB": [1, 7, 31, 64, 100, 143, 52, 90],
           "LC": [3, 40, 77, 150, 64, 110, 25, 95], "LD": [2, 66, 129, 20, 90, 151, 47, 80],
           "LE": [4, 70, 33, 100]}


def requests_for(tag):
    vocab = lc.ALL[tag][0]["vocab"]
    return {f"r{i}": random_tokens(vocab, n, seed=100 * i + n) for i, n in enumerate(LENGTHS[tag])}


def make_core(tag, dtype, max_tokens, max_live=4):
    from tokamak_b200.engine.replay import build_core
    return build_core(folder_of(tag, dtype), dtype, max_tokens, page_size=lc.ALL[tag][2], max_live=max_live)


def replay(tag, dtype, builder, max_tokens, poison=False, max_live=4, **kw):
    from tokamak_b200.engine.replay import run_step
    reqs = requests_for(tag)
    if builder is traces.mixed:
        kw.update(max_tokens=max_tokens, max_live=max_live)
    records, rows = builder(reqs, **kw)
    core = make_core(tag, dtype, max_tokens, max_live)
    results = {}
    for rec in records:
        if poison:
            core.cache.poison_free_pages()
            core.cache.poison_free_state()
        out = run_step(core, rec)
        if out is not None:
            results[rec["step"]] = out
        core.manager.check_invariants()
    assert not core.manager.live_requests()
    assert all(g.num_free == g.num_pages for g in core.manager.kv_groups)
    n = check_rows(results, rows, reqs, folder_of(tag, dtype), dtype, f"{tag}/{dtype}")
    assert n == sum(len(v) for v in rows.values())
    return core


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", ["LA", "LB", "LC", "LD"])
def test_whole_prompts(tag, dtype):
    replay(tag, dtype, traces.whole, max_tokens=192)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", ["LA", "LB", "LC", "LD"])
def test_tail_decoded_one_by_one_across_every_window(tag, dtype):
    replay(tag, dtype, traces.tail_one_by_one, max_tokens=192, tail=60)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", ["LA", "LB", "LC", "LD"])
def test_portions_of_changing_size(tag, dtype):
    replay(tag, dtype, traces.portions, max_tokens=192)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", ["LA", "LB", "LC", "LD"])
def test_mixed_batches_with_pages_and_slots_used_again(tag, dtype):
    replay(tag, dtype, traces.mixed, max_tokens=384, poison=True, seed=7)
    assert sum(LENGTHS[tag]) > 384


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_without_a_rotated_part(dtype):
    replay("LE", dtype, traces.portions, max_tokens=128)
    replay("LE", dtype, traces.mixed, max_tokens=192, poison=True, seed=4)


@pytest.mark.parametrize("seed", [1, 2])
@pytest.mark.parametrize("tag,dtype", [("LA", "float32"), ("LB", "bfloat16"), ("LC", "bfloat16")])
def test_mixed_batches_in_other_orders_with_two_slots(tag, dtype, seed):
    replay(tag, dtype, traces.mixed, max_tokens=320, poison=True, seed=seed, max_live=2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_long_decode(dtype):
    """Positions 0, 1, 2 one by one, then 220 more decoded one by one: over many pages, past every
    window, with a state and a convolution tail carried through every one of them."""
    from tokamak_b200.engine.replay import run_trace
    tag = "LA"
    reqs = {"long": random_tokens(lc.ALL[tag][0]["vocab"], 224, seed=5)}
    records, rows = traces.tail_one_by_one(reqs, tail=223)
    results = run_trace(make_core(tag, dtype, 256), records)
    check_rows(results, rows, reqs, folder_of(tag, dtype), dtype, f"long/{dtype}")


def test_same_logits_however_cut_float32():
    from tokamak_b200.engine.replay import run_trace
    tag = "LB"
    reqs = requests_for(tag)
    got = {}
    for name, builder in (("whole", traces.whole), ("portions", traces.portions)):
        records, rows = builder(reqs)
        res = run_trace(make_core(tag, "float32", 192), records)
        got[name] = {rp: res[s][i] for s in rows for i, rp in enumerate(rows[s])}
    for rp, a in got["whole"].items():
        b = got["portions"][rp]
        assert np.abs(a - b).max() <= 2e-5 * max(1.0, np.abs(a).max()), rp


@pytest.mark.parametrize("tag", ["LA", "LC"])
def test_residual_stream_after_every_layer_float32(tag):
    """Layer by layer: what each block leaves, joined to the stream, against the plain implementation."""
    from tokamak_b200.engine.step import StepEntry
    core = make_core(tag, "float32", 64)
    caught = []
    for block in core.model.blocks.values():
        def wrapped(resid, pending, step, view, fwd=block.forward):
            r, p = fwd(resid, pending, step, view)
            x = p.x.float() if p.x.dim() == 2 else p.x.sum(0)
            assert p.layer_scale is None
            caught.append(r.double().cpu() + plain.rms(x.double().cpu(), p.eps) * p.weight.double().cpu())
            return r, p
        block.forward = wrapped
    toks = random_tokens(lc.ALL[tag][0]["vocab"], 40, seed=9)
    core.step.run([StepEntry("a", toks, [39])])
    cfg, w = plain.load_folder(folder_of(tag, "float32"))
    _, want = plain.forward(cfg, w, toks, return_layers=True)
    assert len(caught) == want.shape[0]
    for i, got in enumerate(caught):
        err = (got - want[i]).abs().max().item()
        assert err <= 2e-4 * max(1.0, want[i].abs().max().item()), f"layer {i} is off by {err:.3e}"


@pytest.mark.parametrize("tag", ["LA", "LB"])
def test_greedy_generation_through_the_entry_point_float32(tag):
    """LLM.generate with its scheduler: prompts in portions beside decoding requests, fewer slots
    than requests, a pool that is used again; the tokens are the plain implementation's."""
    from tokamak_b200 import LLM, SamplingParams
    folder = folder_of(tag, "float32")
    llm = LLM(folder, dtype="float32", block_size=lc.ALL[tag][2], max_seq_len=128, kv_pool_tokens=256,
              prefill_chunk=24, max_num_batched_tokens=40, max_batch_size=3)
    vocab = lc.ALL[tag][0]["vocab"]
    prompts = [random_tokens(vocab, n, seed=7 * n + 1) for n in (5, 33, 1, 61, 18)]
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0.0, max_new_tokens=10))
    assert llm.last_stats["mixed_steps"] > 0
    cfg, w = plain.load_folder(folder)
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == plain.greedy_generate(cfg, w, p, 10), len(p)


def test_greedy_generation_bfloat16_picks_a_top_token():
    from tokamak_b200 import LLM, SamplingParams
    tag = "LC"
    folder = folder_of(tag, "bfloat16")
    llm = LLM(folder, dtype="bfloat16", block_size=lc.ALL[tag][2], max_seq_len=128, max_batch_size=4)
    prompts = [random_tokens(lc.ALL[tag][0]["vocab"], n, seed=n) for n in (9, 40, 70)]
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0.0, max_new_tokens=12))
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.output_token_ids:
            logits = truth(folder, seq)[-1]
            assert logits[tok] >= logits.max() - 0.05 * logits.std(), (len(p), len(seq))
            seq.append(tok)


def test_trace_run_program_on_this_design(tmp_path):
    tag, dtype = "LB", "float32"
    reqs = {k: v for k, v in list(requests_for(tag).items())[:4]}
    records, rows = traces.mixed(reqs, max_tokens=256, seed=3)
    folder = folder_of(tag, dtype)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
         "--out", str(out), "--max-tokens", "256", "--page-size", "8"],
        input="".join(json.dumps(r) + "\n" for r in records), text=True, capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for r in records for w in ("done", str(r["step"]))]
    vocab = lc.ALL[tag][0]["vocab"]
    results = {s: np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, vocab) for s in rows}
    check_rows(results, rows, reqs, folder, dtype, "trace_run")


def test_generation_from_the_command_line(capsys):
    from tokamak_b200.cli import main
    folder = folder_of("LA", "float32")
    argv = ["--model", str(folder), "--dtype", "float32", "--prompt-len", "21", "--temperature", "0",
            "--max-new-tokens", "9", "--ignore-eos", "--block-size", "16", "--max-seq-len", "64", "--kv-pool-tokens", "256"]
    assert main(argv) == 0
    first = capsys.readouterr().out
    assert main(argv) == 0
    assert capsys.readouterr().out == first and first.strip()
