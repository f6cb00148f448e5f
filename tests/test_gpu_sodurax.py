"""Sodurax on the device against the plain implementation: every mechanism alone, then whole models under
four ways of cutting and batching, long decoding past the window, pages used again, and generation."""
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import configs_sodurax as cs
import plain_sodurax as ps
import trace_tools as tt

pytestmark = pytest.mark.gpu

# the error of a logits row: root mean square of the difference (its mean taken off) over that of the row
TOL = {"float32": 5e-5, "bfloat16": 0.03}
LENGTHS = {"a": [7, 130, 1, 64, 33, 97, 2, 65], "b": [40, 1, 23, 64, 81, 5, 17, 50], "c": [48, 3, 150, 31, 80]}


def row_error(got, ref):
    d = np.asarray(got, dtype=np.float64) - np.asarray(ref, dtype=np.float64)
    r = np.asarray(ref, dtype=np.float64)
    return float(np.sqrt(np.mean((d - d.mean()) ** 2)) / np.sqrt(np.mean((r - r.mean()) ** 2)))


def compare(rows, ref, tol, what, margins=None):
    """Every row within ``tol``.  With ``margins`` (bfloat16 runs): where a router's choice in the plain model hangs on
    less than the run's rounding can move, the run may choose another expert; such a row is not held to ``tol``,
    and since a token that chose otherwise is a slightly different key for the tokens after it, of the others
    nine in ten must be within ``tol`` and their median within a third of it."""
    worst, errs = 0.0, []
    for (rid, pos), row in sorted(rows.items()):
        assert np.isfinite(row).all(), f"{what}: request {rid} position {pos}: non-finite logits"
        e = row_error(row, ref[rid][pos])
        if margins is not None:
            if float(margins[rid][pos]) >= CLEAR_MARGIN:
                errs.append(e)
            continue
        worst = max(worst, e)
        assert e <= tol, f"{what}: request {rid} position {pos} of {len(ref[rid])}: error {e:.3e} > {tol:.1e} (first bad place)"
    if margins is not None:
        errs = np.sort(np.asarray(errs))
        assert len(errs) >= len(rows) // 2, f"{what}: too few rows with a clear routing"
        inside = float((errs <= tol).mean())
        assert inside >= 0.9 and errs[len(errs) // 2] <= tol / 3, \
            f"{what}: {inside:.2%} of {len(errs)} rows within {tol}, median {errs[len(errs) // 2]:.3e}"
        worst = float(errs[int(0.9 * (len(errs) - 1))])
    return worst


CLEAR_MARGIN = 0.01


@pytest.fixture(scope="module")
def sdx_dirs(tmp_path_factory):
    out = {}
    for name, (cfg, seed) in cs.SDX.items():
        d = str(tmp_path_factory.mktemp(f"sdx_{name}"))
        ps.write_model(d, cfg, seed)
        out[name] = d
    return out


@pytest.fixture(scope="module")
def plain(sdx_dirs):
    models = {n: ps.PlainSodurax.from_dir(d) for n, d in sdx_dirs.items()}
    cache = {}

    def get(name):
        if name not in cache:
            reqs = tt.make_requests(cs.SDX[name][0]["vocab"], LENGTHS[name], seed=50 + len(name))
            cache[name] = (reqs, [models[name].logits(t).numpy() for t in reqs])
            margins[name] = [models[name].margins(t).numpy() for t in reqs]
        return cache[name]
    margins = {}
    get.models = models
    get.margins = lambda name, dtype: margins[name] if dtype == "bfloat16" else None
    return get


@pytest.fixture(scope="module")
def loaded(sdx_dirs):
    import gesso_b200
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = gesso_b200.load(sdx_dirs[name], dtype=dtype, max_positions=1024)
        return cache[(name, dtype)]
    return get


SCHEDULES = {
    "whole": lambda reqs: tt.trace_whole(reqs),
    "tail_decode": lambda reqs: tt.trace_tail_decode(reqs, tail=60),       # the window passes over decoded tokens
    "portions": lambda reqs: tt.trace_portions(reqs),
    "mixed": lambda reqs: tt.trace_mixed(reqs, seed=5),
}


# ---- mechanisms alone ------------------------------------------------------------------------------------
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [64, 50])
def test_dyt_add_norm_kernel(width, out_dtype):
    from gesso_b200 import ops
    dev = "cuda"
    N = 37
    h = torch.randn(N, width, device=dev)
    d = torch.randn(N, width, device=dev) * 3
    mk = lambda a: ops.DytParams(a, torch.randn(width, device=dev), torch.randn(width, device=dev))
    post, pre = mk(0.6), mk(1.3)
    f = lambda p, x: torch.tanh(p.alpha * x.double()) * p.weight.double() + p.bias.double()
    want_h = h.double() + f(post, d)
    want = f(pre, want_h)
    tol = 1e-6 if out_dtype == torch.float32 else 1e-2
    for delta in (d, d.to(torch.bfloat16)):
        hh = h.clone()
        got = ops.add_dyt(hh, delta, None, post, pre, out_dtype)
        wh = h.double() + f(post, delta)
        assert torch.allclose(hh.double(), wh, atol=1e-6) and torch.allclose(got.double(), f(pre, wh), atol=tol, rtol=tol)
    hh = h.clone()                                   # a row list: only those rows, the stream stays
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device=dev)
    got = ops.add_dyt(hh, d, None, post, pre, out_dtype, rows)
    assert torch.equal(hh, h) and torch.allclose(got.double(), want[rows.long()], atol=tol, rtol=tol)
    hh = h.clone()                                   # a plain add, and a norm with nothing to add
    got = ops.add_dyt(hh, d, None, None, pre, out_dtype)
    assert torch.allclose(hh.double(), h.double() + d.double(), atol=1e-6)
    got = ops.add_dyt(hh, None, None, None, pre, torch.float32)
    assert torch.allclose(got.double(), f(pre, hh), atol=1e-6)


def _pages(k, v, page_size, order):
    """K [T, G, D] and V [T, G, Vd] laid into pages handed out in ``order``; returns pages and the block table."""
    T, G, D = k.shape
    Vd = v.shape[2]
    n = (T + page_size - 1) // page_size
    kp = torch.full((len(order) + 1, G, page_size, D), float("nan"), dtype=k.dtype, device=k.device)
    vp = torch.full((len(order) + 1, G, Vd, page_size), float("nan"), dtype=k.dtype, device=k.device)
    for p in range(n):
        lo, hi = p * page_size, min(T, (p + 1) * page_size)
        kp[order[p], :, :hi - lo] = k[lo:hi].transpose(0, 1)
        vp[order[p], :, :, :hi - lo] = v[lo:hi].permute(1, 2, 0)
        vp[order[p], :, :, hi - lo:] = 0          # the writer's invariant: zeros behind the last position of a block
    bt = torch.full((1, len(order)), -1, dtype=torch.int32, device=k.device)
    bt[0, :n] = torch.tensor(order[:n], dtype=torch.int32)
    return kp, vp, bt


def _plain_attention(q, k, v, scale, window, keep, gate):
    T, H, D = q.shape
    G = k.shape[1]
    vis = ps.visibility(T, {"size": window, "keep_first": keep} if window else None)
    out = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        s = (q[:, h].double().cpu() @ k[:, h // (H // G)].double().cpu().T) * scale
        out[:, h] = torch.softmax(s.masked_fill(~vis, -math.inf), -1) @ v[:, h // (H // G)].double().cpu()
    out = out.reshape(T, -1)
    return out * torch.sigmoid(gate.double().cpu()) if gate is not None else out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,Vd,window,keep", [(4, 2, 32, 32, 40, 3), (6, 1, 24, 40, 11, 0), (2, 2, 64, 64, 50, 20),
                                                  (3, 3, 16, 8, 23, 1), (8, 2, 96, 96, 37, 17), (4, 4, 128, 128, 64, 16),
                                                  (2, 1, 32, 32, None, 0), (8, 2, 64, 64, 45, 5), (6, 2, 64, 64, 130, 140)])
@pytest.mark.parametrize("split", [False, True])
def test_attention_edges_stand_out(H, G, D, Vd, window, keep, dtype, split):
    """One sequence in pages handed out of order.  Keys just inside and just outside the window, the last kept
    key and the first one that is not kept are made to stand out for the queries that test them (their
    score is raised far above the rest), so a mask that is one key off changes the result by a lot.  The
    queries run as one prompt portion and one by one as single tokens, with a gate and a scale of its own.
    ``split``: the attention weights act in two bfloat16 pieces (the mma.sync kernels); without it head size 64
    with several query heads per kv head takes the tcgen05 kernel for the portion."""
    if split and dtype == torch.float32:
        pytest.skip("float32 weights are not split")
    from gesso_b200.engine import attention_dispatch
    from gesso_b200.engine.model import PagedView, Runtime
    dev, T, page = "cuda", 150, 16
    scale = 0.17
    q = torch.randn(T, H, D, device=dev)
    k = torch.randn(T, G, D, device=dev)
    v = torch.randn(T, G, Vd, device=dev)
    gate = torch.randn(T, H * Vd + 8, device=dev)          # a view into a wider row
    for i in (T - 1, 100, 77):                             # the queries that test edges
        if window is None:
            edges = [0, i // 2]
        else:
            edges = [i - window + 1, i - window] + ([keep - 1, keep] if keep else [0])
        for n, j in enumerate(edges):
            if 0 <= j <= i:
                k[j] = (q[i, :: H // G] / q[i, :: H // G].norm(dim=-1, keepdim=True)) * (10.0 + 2 * n) / scale / q[i, 0].norm()
    q, k, v, gate = (t.to(dtype) for t in (q, k, v, gate))
    order = [7, 2, 9, 0, 4, 1, 8, 3, 6, 5]
    kp, vp, bt = _pages(k, v, page, order)
    g = gate[:, :H * Vd]
    want = _plain_attention(q, k, v, scale, window, keep, g)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    rt = Runtime(dev, dtype, 1024)

    class Ctx:
        pass
    # one prompt portion
    c = Ctx()
    c.decode_only, c.n_segs, c.max_kv_len = False, 1, T
    c.positions = torch.arange(T, dtype=torch.int32, device=dev)
    c.seg_of_token = torch.zeros(T, dtype=torch.int32, device=dev)
    c.seg_start = torch.tensor([0, T], dtype=torch.int32, device=dev)
    c.seg_pos0 = torch.zeros(1, dtype=torch.int32, device=dev)
    tiles = (T + 63) // 64
    c.tile_seg = torch.zeros(tiles, dtype=torch.int32, device=dev)
    c.tile_q0 = torch.arange(tiles, dtype=torch.int32, device=dev) * 64
    c.kv_span = torch.tensor([T, T], dtype=torch.int32, device=dev)
    view = PagedView(kp, vp, bt, True)
    got = attention_dispatch.paged_attention(rt, q, view, c, window, scale, keep, g, split).double().cpu()
    from gesso_b200 import ops
    ops.check_tc_status()
    err = (got - want).abs().max() / want.abs().max()
    assert err <= tol, f"portion: {float(err):.3e}"
    # token by token (pages behind the window given back, the kept ones not)
    for i in (T - 1, 100, 77, 0, 16, 15):
        c = Ctx()
        c.decode_only, c.n_segs, c.max_kv_len = True, 1, i + 1
        c.positions = torch.tensor([i], dtype=torch.int32, device=dev)
        c.seg_of_token = torch.zeros(1, dtype=torch.int32, device=dev)
        c.kv_span = torch.tensor([i + 1, i + 1], dtype=torch.int32, device=dev)
        bt_i = bt.clone()
        if window:
            dead = max(0, i - window + 1) // page
            bt_i[0, (keep + page - 1) // page:dead] = -1
        got = attention_dispatch.paged_attention(rt, q[i:i + 1].contiguous(), PagedView(kp, vp, bt_i, True), c, window, scale,
                                                 keep, g[i:i + 1], split).double().cpu()
        err = (got[0] - want[i]).abs().max() / want.abs().max()
        assert err <= tol, f"single token at {i}: {float(err):.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_projection_bias_partial_rotation_and_store(dtype):
    from gesso_b200 import ops
    from gesso_b200.parts.rope import rope_tables
    dev, T, H, G, D, Vd, page = "cuda", 21, 3, 1, 24, 40, 16
    rot = {"base": 100.0, "dims": 8, "scaling": {"factor": 3.0}}
    width = (H + G) * D + G * Vd
    row = torch.randn(T, width + H * Vd, device=dev).to(dtype)           # q, k, v, then columns the kernel leaves alone
    bias = torch.randn(width, device=dev)
    cos, sin = (t.to(dev) for t in rope_tables(rot["base"], rot["dims"], 64, 3.0))
    pos = torch.arange(5, 5 + T, dtype=torch.int32, device=dev)
    bt = torch.tensor([[3, 0, 2, 1]], dtype=torch.int32, device=dev)
    kp = torch.zeros(5, G, page, D, dtype=dtype, device=dev)
    vp = torch.zeros(5, G, Vd, page, dtype=dtype, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    q = ops.qk_norm_rope_store(row, None, None, 0.0, cos, sin, pos, torch.zeros(T, dtype=torch.int32, device=dev), bt, kp, vp,
                               H, G, D, True, status, rot_dim=8, bias=bias, v_head_dim=Vd)
    x = row.double().cpu()[:, :width] + bias.double().cpu()
    ang = ps.rotation_angles(64, rot)[5:5 + T]
    want_q = ps.rotate(x[:, :H * D].view(T, H, D), ang, 8)
    want_k = ps.rotate(x[:, H * D:(H + G) * D].view(T, G, D), ang, 8)
    want_v = x[:, (H + G) * D:].view(T, G, Vd)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(q.double().cpu(), want_q, atol=tol, rtol=tol) and int(status.item()) == 0
    for t in range(T):
        p = 5 + t
        page_id, slot = int(bt[0, p // page]), p % page
        assert torch.allclose(kp[page_id, :, slot].double().cpu(), want_k[t], atol=tol, rtol=tol)
        assert torch.allclose(vp[page_id, :, :, slot].double().cpu(), want_v[t], atol=tol, rtol=tol)


@pytest.mark.parametrize("D,rot_dims", [(64, 16), (32, 32), (128, 8), (64, 64)])
def test_rotation_and_store_by_tiles(D, rot_dims):
    """Prompt portions in bfloat16 take the kernel that works by 64-token tiles: partly rotated heads, biases and
    gate columns behind the v heads, two requests whose portions start in the middle of a page."""
    from gesso_b200 import ops
    from gesso_b200.parts.rope import rope_tables
    dev, H, G, page = "cuda", 4, 2, 16
    lens, pos0 = [70, 9], [21, 40]
    T = sum(lens)
    rot = {"base": 1000.0, "dims": rot_dims, "scaling": {"factor": 2.0}}
    width = (H + 2 * G) * D
    row = torch.randn(T, width + H * D, device=dev).to(torch.bfloat16)
    bias = torch.randn(width, device=dev)
    cos, sin = (t.to(dev) for t in rope_tables(rot["base"], rot_dims, 128, 2.0))
    pos = torch.cat([torch.arange(p, p + n) for p, n in zip(pos0, lens)]).to(torch.int32).to(dev)
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).to(torch.int32).to(dev)
    bt = torch.tensor([[3, 0, 2, 1, 8, 9, -1], [4, 7, 6, 5, -1, -1, -1]], dtype=torch.int32, device=dev)
    seg_start = torch.tensor([0, 70, 79], dtype=torch.int32, device=dev)
    seg_pos0 = torch.tensor(pos0, dtype=torch.int32, device=dev)
    tile_seg = torch.tensor([0, 0, 1], dtype=torch.int32, device=dev)
    tile_q0 = torch.tensor([0, 64, 0], dtype=torch.int32, device=dev)
    outs = []
    for tiles in (None, (seg_start, seg_pos0, tile_seg, tile_q0)):
        kp = torch.zeros(10, G, page, D, dtype=torch.bfloat16, device=dev)
        vp = torch.zeros(10, G, D, page, dtype=torch.bfloat16, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        q = ops.qk_norm_rope_store(row, None, None, 0.0, cos, sin, pos, seg, bt, kp, vp, H, G, D, True, status, tiles=tiles,
                                   rot_dim=rot_dims, bias=bias)
        assert int(status.item()) == 0
        outs.append((q, kp, vp))
    x = row.double().cpu()[:, :width] + bias.double().cpu()
    ang = ps.rotation_angles(128, rot)[pos.long().cpu()]
    want_q = ps.rotate(x[:, :H * D].view(T, H, D), ang, rot_dims)
    assert torch.allclose(outs[1][0].double().cpu(), want_q, atol=3e-2, rtol=3e-2)
    for a, b in zip(outs[0], outs[1]):                   # the per-token kernel and the tile kernel write the same
        assert torch.allclose(a.float(), b.float(), atol=1e-6, rtol=2.0 ** -7)


@pytest.mark.parametrize("E,top,groups,keep", [(8, 2, 4, 2), (6, 1, 1, 1), (16, 3, 8, 5), (12, 4, 3, 3), (64, 8, 8, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_against_plain(E, top, groups, keep, dtype):
    from gesso_b200 import ops
    dev, T, W = "cuda", 200, 72
    x = torch.randn(T, W, device=dev).to(dtype)
    wr = (torch.randn(E, W, device=dev) * 0.3).to(torch.bfloat16).to(dtype)      # the run's own matrix type
    corr = (torch.randn(E, device=dev) * 0.5 - 0.6)                    # most choice scores are negative
    idx, w = ops.moe_route(x, wr, corr, top, groups, keep)
    Wd = {"p.router": wr.double().cpu(), "p.correction": corr.double().cpu()}
    r = {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}
    want_idx, want_w = ps.route(x.double().cpu(), Wd, "p.", r)
    # a close call may fall either way in 32 bit: compare where the plain choice is clear
    s = torch.sigmoid(x.double().cpu() @ Wd["p.router"].T) + Wd["p.correction"]
    clear = 0
    for t in range(T):
        srt = s[t].sort(descending=True).values
        if (srt[:-1] - srt[1:]).min() < 1e-4:
            continue
        clear += 1
        assert idx[t].tolist() == want_idx[t].tolist(), f"token {t}"
        assert torch.allclose(w[t].double().cpu(), want_w[t], atol=2e-6)
    assert clear > T // 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W,F,E,top", [(5, 64, 48, 8, 2), (70, 96, 40, 6, 1), (300, 128, 32, 16, 3), (33, 72, 100, 4, 4),
                                         (200, 96, 40, 6, 2), (150, 192, 64, 16, 4), (260, 200, 72, 12, 3),
                                         (700, 512, 256, 32, 4), (129, 64, 8, 3, 1)])
def test_experts_against_plain(T, W, F, E, top, dtype):
    """Both ways the experts run: pair by pair, and grouped by expert where the step takes that path."""
    from gesso_b200 import ops
    dev = "cuda"
    x = torch.randn(T, W, device=dev).to(dtype)
    wu = (torch.randn(E, F, W, device=dev) / math.sqrt(W)).to(dtype)
    wd = (torch.randn(E, W, F, device=dev) / math.sqrt(F)).to(dtype)
    idx = torch.stack([torch.randperm(E, device=dev)[:top] for _ in range(T)]).to(torch.int32)
    if T > 20:
        idx[:, 0] = torch.where(torch.arange(T, device=dev) % 3 == 0, idx[:, 0], idx[0, 0])      # uneven loads, an idle expert
    w = torch.rand(T, top, device=dev)
    Wd = {}
    for e in range(E):
        Wd[f"p.e{e}.up"], Wd[f"p.e{e}.down"] = wu[e].double().cpu(), wd[e].double().cpu()
    want = ps.experts(x.double().cpu(), Wd, "p.", idx.cpu(), w.double().cpu())
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    got = ops.moe_experts_pairs(x, wu, wd, idx, w)
    assert (got.double().cpu() - want).abs().max() <= tol * want.abs().max()
    if ops.moe_grouped_takes(x, wu, wd, top):
        got = ops.moe_experts_grouped(x, wu, wd, idx, w)
        ops.check_tc_status()
        assert (got.double().cpu() - want).abs().max() <= tol * want.abs().max()
    else:
        assert dtype == torch.float32 or T * top <= ops.MOE_PAIR_MAX_ROWS or F % 8 != 0


# ---- whole models ------------------------------------------------------------------------------------------
def test_layer_streams_float32(sdx_dirs, loaded, plain):
    """The stream after every layer run, layer by layer, in float32 (a hook on the blocks)."""
    from gesso_b200.engine.batch import StepEntry
    from gesso_b200.engine.trace import make_engine
    for name in cs.SDX:
        model = loaded(name, "float32")
        toks = tt.make_requests(cs.SDX[name][0]["vocab"], [29], seed=3)[0]
        want = plain.models[name].stream(toks)
        eng = make_engine(model, 64, use_graphs=False)
        seen = []
        olds = []
        for blk in model.blocks:
            old = blk.forward
            olds.append(old)

            def hooked(h, pending, ctx, cache, old=old):
                out = old(h, pending, ctx, cache)
                hh = h.clone()
                out[0].add_into(hh)
                seen.append(hh.double().cpu())
                return out
            blk.forward = hooked
        try:
            eng.admit("r")
            eng.step([StepEntry("r", toks, [len(toks) - 1])])
        finally:
            for blk, old in zip(model.blocks, olds):
                blk.forward = old
        assert len(seen) == len(want)
        for i, (a, b) in enumerate(zip(seen, want)):
            assert (a - b).abs().max() <= 2e-5 * b.abs().max(), f"{name}: layer run {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", list(SCHEDULES))
@pytest.mark.parametrize("name", list(cs.SDX))
def test_replay_matches_plain(name, schedule, dtype, loaded, plain, tmp_path):
    reqs, ref = plain(name)
    tb, max_tokens = SCHEDULES[schedule](reqs)
    model = loaded(name, dtype)
    tt.run_in_process(model, tb, max_tokens, str(tmp_path))
    rows = tt.read_rows(tb, str(tmp_path), model.vocab_size)
    worst = compare(rows, ref, TOL[dtype], f"{name}/{schedule}/{dtype}", plain.margins(name, dtype))
    print(f"worst error {name}/{schedule}/{dtype}: {worst:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(cs.SDX))
def test_pages_and_slots_used_again(name, dtype, loaded, plain, tmp_path):
    """Every free page filled with NaN before a mixed replay on a pool made for the live requests only, and
    with graphs off and on."""
    reqs, ref = plain(name)
    tb, max_tokens = SCHEDULES["mixed"](reqs)
    model = loaded(name, dtype)
    for graphs in (False, True):
        d = tmp_path / f"g{int(graphs)}"
        tt.run_in_process(model, tb, max_tokens, str(d), prepare=tt.poison_free_memory, use_graphs=graphs)
        compare(tt.read_rows(tb, str(d), model.vocab_size), ref, TOL[dtype], f"poisoned {name}/{dtype}",
                plain.margins(name, dtype))


def test_schedules_agree_float32(loaded, plain, tmp_path):
    reqs, _ = plain("c")
    model = loaded("c", "float32")
    got = {}
    for sched, make in SCHEDULES.items():
        tb, max_tokens = make(reqs)
        tt.run_in_process(model, tb, max_tokens, str(tmp_path / sched))
        got[sched] = tt.read_rows(tb, str(tmp_path / sched), model.vocab_size)
    for sched, rows in got.items():
        for key, row in rows.items():
            assert row_error(row, got["whole"][key]) <= 2e-5, (sched, key)


def test_long_decoding_gives_pages_back_and_keeps_the_first(loaded, plain):
    """Token by token far past the window: the pool stays small, the kept first tokens stay readable."""
    from gesso_b200.engine.batch import StepEntry
    from gesso_b200.engine.engine import Engine
    name = "c"                                                   # window 50 / 33, 20 / 2 kept tokens
    model = loaded(name, "float32")
    toks = tt.make_requests(cs.SDX[name][0]["vocab"], [400], seed=9)[0]
    want = plain.models[name].logits(toks).numpy()
    eng = Engine(model, max_positions=512, page_size=16, num_pages=8, max_requests=2)     # 128 positions of pages
    eng.admit("r")
    eng.step([StepEntry("r", toks[:40], [])])
    for p in range(40, 400):
        lg = eng.step([StepEntry("r", [toks[p]], [0])])
        if p % 37 == 0 or p > 390:
            assert row_error(lg[0].cpu().numpy(), want[p]) <= TOL["float32"], p
    assert max(eng.cache.pages_in_use()) <= 2 + 5
    eng.release("r")
    eng.cache.check_invariants()


@pytest.mark.parametrize("name", list(cs.SDX))
def test_greedy_generation_through_the_session(name, loaded, plain):
    import gesso_b200
    model = loaded(name, "float32")
    s = gesso_b200.Session(model, context_length=256, page_size=16, max_batch=4)
    prompts = tt.make_requests(cs.SDX[name][0]["vocab"], [9, 1, 60, 2], seed=21)
    for p in prompts:
        assert s.generate(p, max_new_tokens=6) == plain.models[name].greedy(p, 6)
    res = s.run_batch([gesso_b200.BatchRequest(p, max_new_tokens=6) for p in prompts])
    for p, r in zip(prompts, res):
        assert list(r.ids) == plain.models[name].greedy(p, 6)
    assert all(n == 0 for n in s.engine.cache.pages_in_use())


def random_sodurax_config(seed):
    """Seeded random configurations: head sizes the tensor-core kernels take and others, values wider or narrower than
    keys, any grouping of heads and experts, windows shorter and longer than the prompts, layers without a
    feed-forward, layers that borrow tensors (with the same or other constants)."""
    import random
    rng = random.Random(seed)
    dim = rng.choice([16, 24, 32, 48, 64, 64, 80, 96, 128])
    kv = rng.choice([1, 2, 3])
    heads = kv * rng.choice([1, 2, 4])
    vdim = dim if rng.random() < 0.7 else rng.choice([8, 16, 40, 72])
    width = rng.choice([48, 64, 72, 96, 128, 200, 256])
    gsz = rng.choice([1, 2, 3, 4])
    count = rng.choice([1, 2, 3, 4, 6])
    experts = gsz * count
    keep = rng.randint(1, count)
    top = rng.randint(1, min(4, gsz * keep))

    def mixer():
        rot_dims = rng.choice([d for d in (2, 4, 8, 12, 16, 24, 32, 64, dim) if d <= dim])
        m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": rng.choice([0.08, 0.15, dim ** -0.5]),
             "rot": {"base": rng.choice([100.0, 1e4, 5e5]), "dims": rot_dims}, "mask": None}
        if rng.random() < 0.7:
            m["rot"]["scaling"] = {"factor": rng.choice([1.5, 2.0, 8.0])}
        if rng.random() < 0.85:
            m["mask"] = {"size": rng.choice([3, 9, 16, 17, 31, 50, 64, 200]), "keep_first": rng.choice([0, 1, 2, 5, 16, 19])}
        return m

    def mlp():
        if rng.random() < 0.15:
            return None
        return {"kind": "moe", "expert": {"ff": rng.choice([8, 24, 40, 64, 100])},
                "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}
    layers = []
    for i in range(rng.randint(2, 4)):
        if i > 0 and rng.random() < 0.35:
            src = rng.randrange(i)
            while "weights_of" in layers[src]:
                src = layers[src]["weights_of"]
            L = dict(layers[src], weights_of=src)
            if rng.random() < 0.3 and L["mixer"]["mask"]:
                L["mixer"] = dict(L["mixer"], mask={"size": rng.choice([5, 40]), "keep_first": rng.choice([0, 3])})
            layers.append(L)
        else:
            layers.append({"type": "attention", "mixer": mixer(), "mlp": mlp()})
    cfg = {"architecture": "Sodurax", "vocab": rng.choice([97, 256, 503]), "width": width, "norm": {"eps": 1e-6}, "layers": layers}
    return cfg, [rng.choice([1, 2, 5, 17, 33, 64, 65, 70, 97, 130]) for _ in range(4)]


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8, 11, 12, 29, 34])
def test_random_configuration_replays_like_plain(seed, tmp_path):
    import gesso_b200
    cfg, lengths = random_sodurax_config(seed)
    d = str(tmp_path / "model")
    ps.write_model(d, cfg, seed)
    plain_model = ps.PlainSodurax.from_dir(d)
    reqs = tt.make_requests(cfg["vocab"], lengths, seed=seed)
    ref = [plain_model.logits(t).numpy() for t in reqs]
    margins = [plain_model.margins(t).numpy() for t in reqs]
    for dtype in ("float32", "bfloat16"):
        model = gesso_b200.load(d, dtype=dtype, max_positions=256)
        for name, make in SCHEDULES.items():
            tb, max_tokens = make(reqs)
            out = str(tmp_path / f"{dtype}_{name}")
            tt.run_in_process(model, tb, max_tokens, out)
            compare(tt.read_rows(tb, out, cfg["vocab"]), ref, TOL[dtype], f"seed {seed} {name} {dtype} {cfg}",
                    margins if dtype == "bfloat16" else None)
        del model


def test_trace_program_on_a_model_folder(sdx_dirs, plain, tmp_path):
    reqs, ref = plain("b")
    tb, max_tokens = tt.trace_mixed(reqs, seed=2)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", sdx_dirs["b"], "--dtype", "bfloat16",
                        "--out", str(out), "--max-tokens", str(max_tokens)], input=tb.text(), capture_output=True, text=True,
                       timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    compare(tt.read_rows(tb, str(out), cs.SDX_B["vocab"]), ref, TOL["bfloat16"], "trace program b/mixed",
            plain.margins("b", "bfloat16"))
