"""The Ketalix design on the GPU: every mechanism's kernel against the plain implementation, then
whole models under every way of cutting and batching their requests, and generation through the
engine's entry point."""

from __future__ import annotations

import functools
import json
import math
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch

import ketalix_configs as kc
import traces
from helpers import assert_logits_close, random_tokens
from plain import ketalix_plain as plain

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_TMP = []


@functools.lru_cache(maxsize=None)
def folder_of(tag: str, dtype: str) -> Path:
    from tokamak_b200.weights import write_random_model
    raw, init, _ = kc.ALL[tag]
    tmp = tempfile.TemporaryDirectory(prefix=f"tk_{tag}_{dtype}_")
    _TMP.append(tmp)
    write_random_model(tmp.name, raw, dtype=dtype, **init)
    return Path(tmp.name)


@functools.lru_cache(maxsize=None)
def _truth(folder: str, tokens: tuple) -> torch.Tensor:
    cfg, w = plain.load_folder(folder)
    return plain.forward_logits(cfg, w, list(tokens))


def truth(folder, tokens) -> torch.Tensor:
    return _truth(str(folder), tuple(int(t) for t in tokens))


@functools.lru_cache(maxsize=None)
def _rounded(folder: str, tokens: tuple) -> torch.Tensor:
    cfg, w = plain.load_folder(folder)
    return plain.forward_logits(cfg, w, list(tokens), round_to=torch.bfloat16)


# bfloat16: a row is judged against what rounding alone costs at that row.  With heads of a few
# elements and the norm behind every mixer, a row can be ill-conditioned (a dot product near zero
# that the norm scales back up), so one limit for all rows would be either blind or wrong.  The
# plain implementation, rounding where a 16-bit engine rounds, gives the row's own level; the limit
# is four times that, and never below the level of a well-conditioned row.  A wrong key, page,
# state or mask moves a row by about its spread, twenty times the floor.
BF16_FLOOR_RMS, BF16_FLOOR_MAX, BF16_TIMES = 0.05, 0.2, 4.0


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
                spread = want.std().clamp_min(1e-6)
                mine = (got[i] - want).abs() / spread
                base = (_rounded(str(folder), tuple(int(t) for t in reqs[rid]))[p] - want).abs() / spread
                assert torch.isfinite(got[i]).all(), where
                rms, base_rms = mine.pow(2).mean().sqrt().item(), base.pow(2).mean().sqrt().item()
                assert rms <= max(BF16_FLOOR_RMS, BF16_TIMES * base_rms), (
                    f"{where}: off by {rms:.3e} (rms) of the row's spread; rounding alone costs {base_rms:.3e}")
                assert mine.max().item() <= max(BF16_FLOOR_MAX, BF16_TIMES * base.max().item()), (
                    f"{where}: off by {mine.max().item():.3e} (max) of the row's spread; rounding alone costs "
                    f"{base.max().item():.3e}")
            n += 1
    return n


def dev(x, dtype=None):
    return x.to("cuda", dtype) if dtype is not None else x.to("cuda")


def close(got, want, dtype, scale=1.0):
    got, want = got.detach().cpu().double(), want.double()
    tol = (2e-5 if dtype == "float32" else 2e-2) * scale
    err = (got - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), f"off by {err:.3e}"


# ======================================================================= mechanisms alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [40, 1030, 2048, 4104, 10240])     # the general kernel (1030) and 1, 1, 3, 5 pieces a thread
def test_branch_norm_layer_scale_residual_and_next_norm(dtype, width):
    from tokamak_b200.csrc import ops
    g = torch.Generator().manual_seed(width)
    n = 7
    resid = torch.randn(n, width, generator=g)
    branch = (3 * torch.randn(n, width, generator=g)).to(TORCH[dtype]).float()
    wb, ls, wn = (1 + 0.3 * torch.randn(width, generator=g) for _ in range(3))
    want_x = resid.double() + plain.rms_norm(branch.double(), wb.double(), 1e-5) * ls.double()
    want_h = plain.rms_norm(want_x, wn.double(), 1e-6)
    # every row, written back, with the norm that follows
    r = dev(resid.clone()); out = torch.empty(n, width, dtype=TORCH[dtype], device="cuda")
    ops.branch_norm_add(r, dev(branch, TORCH[dtype]), dev(wb), dev(ls), 1e-5, dev(wn), out, 1e-6)
    close(r, want_x, "float32"); close(out, want_h, dtype)
    # partial sums of a split product, no layer scale, nothing follows
    parts = torch.stack([branch * 0.25, branch * 0.75])
    r = dev(resid.clone())
    ops.branch_norm_add(r, dev(parts), dev(wb), None, 1e-5, None, None)
    close(r, resid.double() + plain.rms_norm(branch.double(), wb.double(), 1e-5), "float32")
    # chosen rows: the stream stays as it is
    rows = torch.tensor([5, 0, 2], dtype=torch.int32)
    r = dev(resid.clone()); out = torch.empty(3, width, dtype=TORCH[dtype], device="cuda")
    ops.branch_norm_add(r, dev(branch, TORCH[dtype]), dev(wb), dev(ls), 1e-5, dev(wn), out, 1e-6, dev(rows))
    assert torch.equal(r.cpu(), resid)
    close(out, want_h[rows.long()], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gelu_gated_unit_and_scaled_embedding(dtype):
    from tokamak_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    gate_up = (2 * torch.randn(5, 2 * 24, generator=g)).to(TORCH[dtype])
    out = torch.empty(5, 24, dtype=TORCH[dtype], device="cuda")
    ops.swiglu(dev(gate_up), out, activation="gelu_tanh")
    gu = gate_up.double()
    close(out, plain.gelu_tanh(gu[:, :24]) * gu[:, 24:], dtype)
    table = torch.randn(11, 20, generator=g).to(TORCH[dtype])
    ids = torch.tensor([3, 10, 0], dtype=torch.int32)
    resid = torch.empty(3, 20, dtype=torch.float32, device="cuda")
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    ops.embed_gather(dev(table), dev(ids), resid, err, scale=7.5)
    close(resid, table.double()[ids.long()] * 7.5, "float32")


def _paged(k, v, page, seed, dtype, extra_pages=3):
    """Keys [T, G, d] and values [T, G, dv] of one request in pages handed out in a shuffled order."""
    T, G, d = k.shape
    n_pages = -(-T // page)
    order = torch.randperm(n_pages + extra_pages, generator=torch.Generator().manual_seed(seed))[:n_pages]
    kc_ = torch.full((n_pages + extra_pages, G, page, d), float("nan"))
    vc_ = torch.full((n_pages + extra_pages, G, page, v.shape[-1]), float("nan"))
    for t in range(T):
        kc_[order[t // page], :, t % page] = k[t]
        vc_[order[t // page], :, t % page] = v[t]
    return dev(kc_, dtype), dev(vc_, dtype), dev(order.to(torch.int32).reshape(1, -1))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,dv,rot", [(16, 24, 8), (32, 32, 32), (8, 40, 0), (70, 6, 34), (128, 128, 64), (64, 256, 64), (256, 8, 256)])
def test_pair_rotation_unit_norm_value_blend_and_page_write(dtype, d, dv, rot):
    from tokamak_b200.csrc import ops
    H, G, T, page = 4, 2, 37, 8
    g = torch.Generator().manual_seed(d)
    row = (H + G) * d + G * dv
    qkv = torch.randn(T, row, generator=g).to(TORCH[dtype])
    v_first = torch.randn(T, G * dv, generator=g)
    lam = torch.tensor([0.3])
    x = qkv.double()
    q, k, v = x[:, :H * d].view(T, H, d), x[:, H * d:(H + G) * d].view(T, G, d), x[:, (H + G) * d:].view(T, G, dv)
    pos = torch.arange(100, 100 + T)
    want_q = plain.unit_rms(plain.rotate_pairs(q, pos, rot, 5000.0), 1e-5)
    want_k = plain.unit_rms(plain.rotate_pairs(k, pos, rot, 5000.0), 1e-5)
    want_v = plain.blend_values(v, v_first.double().view(T, G, dv), 0.3)
    n_pages = -(-(100 + T) // page)
    kcache = torch.zeros(n_pages, G, page, d, dtype=TORCH[dtype], device="cuda")
    vcache = torch.zeros(n_pages, G, page, dv, dtype=TORCH[dtype], device="cuda")
    order = torch.randperm(n_pages, generator=g).to(torch.int32)
    inv_freq = torch.tensor([5000.0 ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)], dtype=torch.float32)
    table = ops.rope_table(dev(pos.to(torch.int32)), dev(inv_freq)) if rot else None
    q_out = torch.empty(T, H, d, dtype=TORCH[dtype], device="cuda")
    v_out = torch.empty(T, G * dv, dtype=torch.float32, device="cuda")
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    ops.qkv_pairs(dev(qkv), q_out, kcache, vcache, dev(pos.to(torch.int32)), dev(torch.zeros(T, dtype=torch.int32)),
                  dev(torch.zeros(1, dtype=torch.int32)), dev(order.reshape(1, -1)), table, err, n_q_heads=H,
                  n_kv_heads=G, rotary_dim=rot, unit_norm_eps=1e-5, v_first_in=dev(v_first), v_lambda=dev(lam),
                  v_first_out=v_out)
    assert err.cpu().tolist()[0] == 0
    close(q_out, want_q, dtype)
    close(v_out, v.reshape(T, G * dv), "float32")           # the raw values, for later layers
    for t in (0, 5, T - 1):
        p = 100 + t
        close(kcache[order[p // page], :, p % page], want_k[t], dtype)
        close(vcache[order[p // page], :, p % page], want_v[t], dtype)
    # without norm and blend: rotation alone, values as they are
    ops.qkv_pairs(dev(qkv), q_out, kcache, vcache, dev(pos.to(torch.int32)), dev(torch.zeros(T, dtype=torch.int32)),
                  dev(torch.zeros(1, dtype=torch.int32)), dev(order.reshape(1, -1)), table, err, n_q_heads=H,
                  n_kv_heads=G, rotary_dim=rot, unit_norm_eps=None)
    close(q_out, plain.rotate_pairs(q, pos, rot, 5000.0), dtype, scale=4.0)
    p = 100 + T - 1
    close(vcache[order[p // page], :, p % page], v[T - 1], dtype, scale=4.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,dv,H,G,page,window,cap,sink", [
    (16, 24, 4, 2, 8, 19, 10.0, True), (64, 64, 4, 2, 16, 19, 10.0, True), (128, 128, 8, 1, 16, 33, None, True),
    (64, 64, 2, 2, 32, None, 25.0, False), (8, 40, 3, 1, 8, 5, None, False), (64, 64, 8, 2, 16, 64, 12.0, True)])
def test_attention_cap_sink_window_edges_and_page_borders(dtype, d, dv, H, G, page, window, cap, sink):
    """Keys just inside and just outside the window of chosen queries (one of them at a page's
    border) are made to stand out, a far key too, and the sinks are large: leaving one of them out,
    or letting one in, moves the result by far more than the tolerance."""
    from tokamak_b200.csrc import ops
    T = 150
    g = torch.Generator().manual_seed(d + H)
    q = torch.randn(T, H, d, generator=g)
    k = torch.randn(T, G, d, generator=g)
    v = torch.randn(T, G, dv, generator=g)
    w = window or T
    for iq in (w + 3, 2 * page + w - 1, 2 * page + w, T - 1):
        if iq >= T:
            continue
        for j in (iq - w + 1, iq - w):              # the last key inside, the first key outside
            if j >= 0:
                k[j] = 3.0 * q[iq, ::H // G] / q[iq, ::H // G].norm(dim=-1, keepdim=True) * math.sqrt(d)
    k[1] = 3.0 * q[T - 2, ::H // G] / q[T - 2, ::H // G].norm(dim=-1, keepdim=True) * math.sqrt(d)   # far back
    q, k, v = (t.to(TORCH[dtype]) for t in (q, k, v))
    sinks = 2.0 + torch.randn(H, generator=g) if sink else None
    scale = 1.7 / math.sqrt(d)
    want = plain.attend(q.double(), k.double(), v.double(), scale, cap, window, sinks)
    kcache, vcache, table = _paged(k, v, page, seed=page, dtype=TORCH[dtype])
    pos = dev(torch.arange(T, dtype=torch.int32))
    zeros = dev(torch.zeros(T, dtype=torch.int32))
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.empty(T, H, dv, dtype=TORCH[dtype], device="cuda")
    ops.attention_plain(dev(q), out, kcache, vcache, pos, zeros, dev(torch.zeros(1, dtype=torch.int32)), table, err,
                        scale=scale, window=window, softcap=cap, sinks=dev(sinks) if sink else None)
    assert err.cpu().tolist()[0] == 0
    close(out, want, dtype)
    if sink:     # the sink matters: without it the result is another
        ops.attention_plain(dev(q), out, kcache, vcache, pos, zeros, dev(torch.zeros(1, dtype=torch.int32)), table,
                            err, scale=scale, window=window, softcap=cap)
        assert (out.cpu().double() - want).abs().max() > 0.05


@pytest.mark.parametrize("d,H,G,page,window,cap", [(64, 4, 2, 16, 40, 12.0), (128, 8, 2, 16, 33, 20.0),
                                                    (128, 4, 4, 32, None, None), (64, 8, 1, 64, 70, 9.0)])
def test_tiled_attention_kernels_in_prompts_and_in_decoding(d, H, G, page, window, cap):
    """The dispatcher's bfloat16 path (tensor-core kernels for portions and for single tokens) on a
    batch laid out by the step function: a prompt in two portions, then tokens one by one, with
    stand-out keys just inside and just outside the window of the queries that are checked, one of
    them at a page's border, and large sinks."""
    from tokamak_b200.cache.device import DeviceCache, plan_groups
    from tokamak_b200.cache.manager import CacheManager, KVPagesNeed
    from tokamak_b200.engine.step import StepEntry, StepFunction
    from tokamak_b200.parts.attention import paged_attention
    T, n_dec = 300, 40
    g = torch.Generator().manual_seed(d + page)
    q = torch.randn(T, H, d, generator=g)
    k = torch.randn(T, G, d, generator=g)
    v = torch.randn(T, G, d, generator=g)
    w = window or T
    for iq in list(range(T - n_dec - 2, T, 7)) + [4 * page + w - 1, 4 * page + w, 133]:
        for j in (iq - w + 1, iq - w):
            if 0 <= j < T and iq < T:
                k[j] = 3.0 * q[iq, ::H // G] / q[iq, ::H // G].norm(dim=-1, keepdim=True) * math.sqrt(d)
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    sinks = 2.0 + torch.randn(H, generator=g)
    scale = 1.5 / math.sqrt(d)
    want = plain.attend(q.double(), k.double(), v.double(), scale, cap, window, sinks)

    kv, st = plan_groups({"a": KVPagesNeed(G, d, window)}, 512, page)
    manager = CacheManager(kv, st, 2)
    cache = DeviceCache(manager, torch.bfloat16, torch.device("cuda"), 512)
    step = StepFunction(None, cache, 512, 512)
    view = cache.view("a")
    manager.admit("other"); manager.grow("other", 3 * page)       # so that the request's pages are not the first ones

    def run(lo, hi):
        entries = [StepEntry("r", list(range(lo, hi)), [])]
        batch = step.build(entries)
        table = manager.kv_groups[0].table("r")
        for t in range(lo, hi):
            view.k[table[t // page], :, t % page] = k[t].cuda()
            view.v[table[t // page], :, t % page] = v[t].cuda()
        out = torch.empty(hi - lo, H, d, dtype=torch.bfloat16, device="cuda")
        paged_attention(q[lo:hi].cuda().contiguous(), out, view, batch, scale=scale, window=window, softcap=cap,
                        sinks=sinks.cuda())
        step.finish(entries)
        step.check_errors()
        close(out, want[lo:hi], "bfloat16")

    run(0, 133)                  # a portion that ends inside a page
    run(133, T - n_dec)          # the next one, starting there
    for t in range(T - n_dec, T):
        run(t, t + 1)            # single tokens: the decode kernel


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dk,dv,rank", [(2, 12, 20, 5), (1, 40, 40, 8), (3, 64, 80, 4), (2, 130, 33, 1), (2, 32, 24, 16)])
def test_gla_decay_recurrence_state_and_output_stage(dtype, H, dk, dv, rank):
    from tokamak_b200.csrc import ops
    g = torch.Generator().manual_seed(dk)
    lens = [9, 1, 30]                     # three requests in one batch, in slots 2, 0, 3 of 4
    slots = [2, 0, 3]
    T = sum(lens)
    row = 2 * H * dk + 2 * H * dv + rank
    proj = torch.randn(T, row, generator=g).to(TORCH[dtype])
    w2 = torch.randn(H * dk, rank, generator=g).to(TORCH[dtype])
    bias = torch.randn(H * dk, generator=g)
    x = proj.double()
    a_off = 2 * H * dk + 2 * H * dv
    z = x[:, a_off:] @ w2.double().T + bias.double()
    alpha = torch.sigmoid(z).pow(1 / 4.0).view(T, H, dk)
    dks, dvs = ops.gla_prepared_row(dk, dv)
    prepare = lambda x_in: ops.gla_prepare(x_in, 0, H * dk, 2 * H * dk, a_off, dev(w2), dev(bias), heads=H, key_dim=dk,
                                           value_dim=dv, tau=4.0, q_scale=dk ** -0.5)
    prep = prepare(dev(proj))
    qs = x[:, :H * dk].view(T, H, dk) * dk ** -0.5
    ks = x[:, H * dk:2 * H * dk].view(T, H, dk)
    vs = x[:, 2 * H * dk:2 * H * dk + H * dv].view(T, H, dv)
    pieces, values = ops.gla_prepared_views(prep, H, dk, dv)
    pieces = pieces.permute(1, 0, 3, 2, 4).reshape(T, H, 3, dks)          # [token, head, q / k / alpha, channel]
    values = values.permute(1, 0, 2)
    close(pieces[:, :, 0, :dk], qs, "float32")
    close(pieces[:, :, 1, :dk], ks, "float32")
    close(pieces[:, :, 2, :dk], alpha, "float32")
    close(values[..., :dv], vs, "float32")
    assert not pieces[..., dk:].any() and not values[..., dv:].any()      # the padding to 16 bytes is zero
    # parts of a split product give the same
    halves = dev(torch.stack([proj.float() * 0.5, proj.float() * 0.5]))
    assert torch.equal(prepare(halves), prep)
    state0 = torch.randn(4, H, dk, dv, generator=g)
    state = dev(state0.clone())
    starts = [0, lens[0], lens[0] + lens[1]]
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    rows = [dev(torch.tensor(v, dtype=torch.int32)) for v in (starts, lens, slots)]
    o = ops.gla_scan(prep, state, *rows, err)
    assert err.cpu().tolist()[0] == 0
    alpha32 = pieces[:, :, 2, :dk].cpu().double()
    for s, n, slot in zip(starts, lens, slots):
        want_o, want_s = plain.gla_recurrence(qs[s:s + n], ks[s:s + n], vs[s:s + n], alpha32[s:s + n], state0[slot].double())
        close(o[s:s + n], want_o, "float32", scale=10.0)
        close(state[slot], want_s, "float32", scale=10.0)
    assert torch.equal(state[1].cpu(), state0[1])          # a slot of no request is left alone
    for cols in (32, 16, 8):                               # every split of the columns over blocks, bit for bit
        again = dev(state0.clone())
        o2 = ops.gla_scan(prep, again, *rows, err, cols=cols)
        assert torch.equal(o2, o) and torch.equal(again, state)
    w = 1 + 0.2 * torch.randn(dv, generator=g)
    y = ops.gla_out(o, dev(proj), 2 * H * dk + H * dv, dev(w), 1e-5, TORCH[dtype])
    gate = x[:, 2 * H * dk + H * dv:a_off].view(T, H, dv)
    want = plain.rms_norm(o.cpu().double(), w.double(), 1e-5) * gate * torch.sigmoid(gate)
    close(y, want.reshape(T, H * dv), dtype, scale=3.0)


def test_gla_recurrence_is_bit_equal_however_the_tokens_are_cut():
    from tokamak_b200.csrc import ops
    H, dk, dv, T = 2, 48, 40, 67
    g = torch.Generator().manual_seed(5)
    pieces = torch.randn(H, T, dk // 4, 3, 4, generator=g)
    pieces[..., 2, :] = torch.exp(-torch.rand(H, T, dk // 4, 4, generator=g) * 0.3)
    values = torch.randn(H, T, dv, generator=g)

    def prepared(at, n):       # the layout of gla_prepare for the tokens at .. at + n
        return dev(torch.cat([pieces[:, at:at + n].reshape(-1), values[:, at:at + n].reshape(-1)]))
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    i32 = lambda *v: dev(torch.tensor(v, dtype=torch.int32))

    def run(cuts, cols=0):
        state = torch.zeros(1, H, dk, dv, device="cuda")
        outs, at = [], 0
        for n in cuts:
            outs.append(ops.gla_scan(prepared(at, n), state, i32(0), i32(n), i32(0), err, cols=cols))
            at += n
        return torch.cat(outs), state
    o1, s1 = run([T])
    for cols in (0, 8, 16, 32):
        o2, s2 = run([2, 7, 1, 1, 16, 8, 9, 23], cols)
        assert torch.equal(o1, o2) and torch.equal(s1, s2)
    assert err.cpu().tolist()[0] == 0


# ======================================================================= whole models

LENGTHS = {"KA": [5, 17, 33, 70, 130, 96, 41, 128], "KB": [1, 7, 31, 64, 100, 143, 52, 90],
           "KC": [3, 40, 77, 150, 64, 110, 25, 95]}


def requests_for(tag):
    vocab = kc.ALL[tag][0]["vocab"]
    return {f"r{i}": random_tokens(vocab, n, seed=100 * i + n) for i, n in enumerate(LENGTHS[tag])}


def make_core(tag, dtype, max_tokens, max_live=4):
    from tokamak_b200.engine.replay import build_core
    return build_core(folder_of(tag, dtype), dtype, max_tokens, page_size=kc.ALL[tag][2], max_live=max_live)


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
@pytest.mark.parametrize("tag", ["KA", "KB", "KC"])
def test_whole_prompts(tag, dtype):
    replay(tag, dtype, traces.whole, max_tokens=192)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", ["KA", "KB", "KC"])
def test_tail_decoded_one_by_one_across_every_window(tag, dtype):
    replay(tag, dtype, traces.tail_one_by_one, max_tokens=192, tail=60)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", ["KA", "KB", "KC"])
def test_portions_of_changing_size(tag, dtype):
    replay(tag, dtype, traces.portions, max_tokens=192)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", ["KA", "KB", "KC"])
def test_mixed_batches_with_pages_and_slots_used_again(tag, dtype):
    replay(tag, dtype, traces.mixed, max_tokens=384, poison=True, seed=7)
    assert sum(LENGTHS[tag]) > 384


@pytest.mark.parametrize("seed", [1, 2])
@pytest.mark.parametrize("tag,dtype", [("KA", "float32"), ("KB", "bfloat16"), ("KC", "bfloat16")])
def test_mixed_batches_in_other_orders_with_two_slots(tag, dtype, seed):
    replay(tag, dtype, traces.mixed, max_tokens=320, poison=True, seed=seed, max_live=2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_long_decode(dtype):
    """Positions 0, 1, 2 one by one, then 220 more decoded one by one: over many pages, past every
    window, with a state that has been carried through every one of them."""
    from tokamak_b200.engine.replay import run_trace
    tag = "KA"
    reqs = {"long": random_tokens(kc.ALL[tag][0]["vocab"], 224, seed=5)}
    records, rows = traces.tail_one_by_one(reqs, tail=223)
    results = run_trace(make_core(tag, dtype, 256), records)
    check_rows(results, rows, reqs, folder_of(tag, dtype), dtype, f"long/{dtype}")


def test_same_logits_however_cut_float32():
    from tokamak_b200.engine.replay import run_trace
    tag = "KB"
    reqs = requests_for(tag)
    got = {}
    for name, builder in (("whole", traces.whole), ("portions", traces.portions)):
        records, rows = builder(reqs)
        res = run_trace(make_core(tag, "float32", 192), records)
        got[name] = {rp: res[s][i] for s in rows for i, rp in enumerate(rows[s])}
    for rp, a in got["whole"].items():
        b = got["portions"][rp]
        assert np.abs(a - b).max() <= 2e-5 * max(1.0, np.abs(a).max()), rp


def test_residual_stream_after_every_layer_float32():
    """Layer by layer: what each block leaves, joined to the stream, against the plain implementation."""
    from tokamak_b200.engine.step import StepEntry
    tag = "KA"
    core = make_core(tag, "float32", 64)
    caught = []
    for block in core.model.blocks.values():
        def wrapped(resid, pending, step, view, fwd=block.forward):
            r, p = fwd(resid, pending, step, view)
            x = p.x.float() if p.x.dim() == 2 else p.x.sum(0)
            caught.append(r.double().cpu() + (plain.rms_norm(x.double().cpu(), p.weight.double().cpu(), p.eps)
                                              * p.layer_scale.double().cpu()))
            return r, p
        block.forward = wrapped
    toks = random_tokens(kc.ALL[tag][0]["vocab"], 40, seed=9)
    core.step.run([StepEntry("a", toks, [39])])
    cfg, w = plain.load_folder(folder_of(tag, "float32"))
    want, _ = plain.forward_hidden(cfg, w, toks)
    assert len(caught) == want.shape[0]
    for i, got in enumerate(caught):
        err = (got - want[i]).abs().max().item()
        assert err <= 2e-4 * max(1.0, want[i].abs().max().item()), f"layer {i} is off by {err:.3e}"


@pytest.mark.parametrize("tag", ["KA", "KB"])
def test_greedy_generation_through_the_entry_point_float32(tag):
    """LLM.generate with its scheduler: prompts in portions beside decoding requests, fewer slots
    than requests, a pool that is used again; the tokens are the plain implementation's."""
    from tokamak_b200 import LLM, SamplingParams
    folder = folder_of(tag, "float32")
    llm = LLM(folder, dtype="float32", block_size=kc.ALL[tag][2], max_seq_len=128, kv_pool_tokens=256,
              prefill_chunk=24, max_num_batched_tokens=40, max_batch_size=3)
    vocab = kc.ALL[tag][0]["vocab"]
    prompts = [random_tokens(vocab, n, seed=7 * n + 1) for n in (5, 33, 1, 61, 18)]
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0.0, max_new_tokens=10))
    assert llm.last_stats["mixed_steps"] > 0
    cfg, w = plain.load_folder(folder)
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == plain.greedy_generate(cfg, w, p, 10), len(p)


def test_greedy_generation_bfloat16_picks_a_top_token():
    from tokamak_b200 import LLM, SamplingParams
    tag = "KC"
    folder = folder_of(tag, "bfloat16")
    llm = LLM(folder, dtype="bfloat16", block_size=kc.ALL[tag][2], max_seq_len=128, max_batch_size=4)
    prompts = [random_tokens(kc.ALL[tag][0]["vocab"], n, seed=n) for n in (9, 40, 70)]
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0.0, max_new_tokens=12))
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.output_token_ids:
            logits = truth(folder, seq)[-1]
            assert logits[tok] >= logits.max() - 0.05 * logits.std(), (len(p), len(seq))
            seq.append(tok)


def test_trace_run_program_on_this_design(tmp_path):
    tag, dtype = "KB", "float32"
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
    vocab = kc.ALL[tag][0]["vocab"]
    results = {s: np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, vocab) for s in rows}
    check_rows(results, rows, reqs, folder, dtype, "trace_run")


def test_generation_from_the_command_line(capsys):
    """The command line on a folder of this design: greedy tokens for a seeded random prompt, the same
    at every call."""
    from tokamak_b200.cli import main
    folder = folder_of("KA", "float32")
    argv = ["--model", str(folder), "--dtype", "float32", "--prompt-len", "21", "--temperature", "0",
            "--max-new-tokens", "9", "--ignore-eos", "--block-size", "16", "--max-seq-len", "64", "--kv-pool-tokens", "256"]
    assert main(argv) == 0
    first = capsys.readouterr().out
    assert main(argv) == 0
    assert capsys.readouterr().out == first and first.strip()
