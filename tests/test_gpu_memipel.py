"""Memipel on the device against the plain implementation: every mechanism alone (with inputs made so that a key
that is one off, a lost state or a sink left out shows), then whole models under four ways of cutting and
batching, pages and slots used again, long decoding past every window, and generation through the session."""
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import configs_memipel as cm
import plain_memipel as pm
import trace_tools as tt

pytestmark = pytest.mark.gpu

DEV = "cuda"
# the error of a logits row: root mean square of the difference (its mean taken off) over that of the row
TOL = {"float32": 5e-5, "bfloat16": 0.04}
LENGTHS = {"a": [7, 130, 1, 64, 33, 97, 2, 65], "b": [40, 1, 23, 64, 150, 5, 17, 50], "c": [48, 3, 150, 31, 80]}
CLEAR_MARGIN = 0.15


def row_error(got, ref):
    d = np.asarray(got, dtype=np.float64) - np.asarray(ref, dtype=np.float64)
    r = np.asarray(ref, dtype=np.float64)
    return float(np.sqrt(np.mean((d - d.mean()) ** 2)) / np.sqrt(np.mean((r - r.mean()) ** 2)))


def compare(rows, ref, tol, what, margins=None):
    """Every row within ``tol``.  With ``margins`` (bfloat16 runs): a row whose routing in the plain model hangs on
    less than the run's rounding can move is not held to ``tol``; of the others nine in ten must be within it
    and their median within a third of it (a token that chose otherwise is a slightly different key or state
    for the tokens after it)."""
    errs = []
    for (rid, pos), row in sorted(rows.items()):
        assert np.isfinite(row).all(), f"{what}: request {rid} position {pos}: non-finite logits"
        e = row_error(row, ref[rid][pos])
        if margins is None:
            assert e <= tol, f"{what}: request {rid} position {pos} of {len(ref[rid])}: error {e:.3e} > {tol:.1e} (first bad place)"
        elif float(margins[rid][pos]) >= CLEAR_MARGIN:
            errs.append(e)
    if margins is not None:
        errs = np.sort(np.asarray(errs))
        assert len(errs) >= len(rows) // 3, f"{what}: too few rows with a clear routing"
        inside = float((errs <= tol).mean())
        assert inside >= 0.9 and errs[len(errs) // 2] <= tol / 3, \
            f"{what}: {inside:.2%} of {len(errs)} rows within {tol}, median {errs[len(errs) // 2]:.3e}"


@pytest.fixture(scope="module")
def mmp_dirs(tmp_path_factory):
    out = {}
    for name, (cfg, seed) in cm.MMP.items():
        d = str(tmp_path_factory.mktemp(f"mmp_{name}"))
        pm.write_model(d, cfg, seed)
        out[name] = d
    return out


@pytest.fixture(scope="module")
def plain(mmp_dirs):
    models = {n: pm.PlainMemipel.from_dir(d) for n, d in mmp_dirs.items()}
    cache, margins = {}, {}

    def get(name):
        if name not in cache:
            reqs = tt.make_requests(cm.MMP[name][0]["vocab"], LENGTHS[name], seed=70 + len(name))
            cache[name] = (reqs, [models[name].logits(t).numpy() for t in reqs])
            margins[name] = [models[name].margins(t).numpy() for t in reqs]
        return cache[name]
    get.models = models
    get.margins = lambda name, dtype: margins[name] if dtype == "bfloat16" else None
    return get


@pytest.fixture(scope="module")
def loaded(mmp_dirs):
    import gesso_b200
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = gesso_b200.load(mmp_dirs[name], dtype=dtype, max_positions=1024)
        return cache[(name, dtype)]
    return get


SCHEDULES = {
    "whole": lambda reqs: tt.trace_whole(reqs),
    "tail_decode": lambda reqs: tt.trace_tail_decode(reqs, tail=60),       # every window passes over decoded tokens
    "portions": lambda reqs: tt.trace_portions(reqs),
    "mixed": lambda reqs: tt.trace_mixed(reqs, seed=5),
}


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def segments(lens):
    """Flat-axis metadata of a step whose segments have these lengths."""
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).to(torch.int32).to(DEV)
    start = i32(np.concatenate([[0], np.cumsum(lens)]).tolist())
    return seg, start


# ---- mechanisms alone ------------------------------------------------------------------------------------
@pytest.mark.parametrize("width,rows", [(64, 5), (50, 37), (512, 300), (96, 260)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_norm_adds_two_deltas(width, rows, out_dtype):
    from gesso_b200 import ops
    h = torch.randn(rows, width, device=DEV)
    d1 = torch.randn(rows, width, device=DEV).to(out_dtype)
    d2 = torch.randn(rows, width, device=DEV)
    bias, w = torch.randn(width, device=DEV), torch.randn(width, device=DEV)
    want_h = h.double() + d1.double() + bias.double() + d2.double()
    want = pm.norm_offset(want_h, w.double() - 1.0, 1e-5)
    hh = h.clone()
    got = ops.add_rmsnorm(hh, d1, bias, w, 1e-5, out_dtype, delta2=d2)
    tol = 1e-5 if out_dtype == torch.float32 else 2e-2
    assert torch.allclose(hh.double(), want_h, atol=1e-5)
    assert torch.allclose(got.double(), want, atol=tol, rtol=tol)
    sel = i32([rows - 1, 0, rows // 2])
    hh = h.clone()
    got = ops.add_rmsnorm(hh, d1, bias, w, 1e-5, out_dtype, rows=sel, delta2=d2)
    assert torch.equal(hh, h) and torch.allclose(got.double(), want[sel.long()], atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("L", [1, 2, 3, 4, 8])
def test_causal_conv_across_steps(L, dtype):
    """Two requests whose rows come in portions of many sizes (down to one token, shorter than the taps): the
    state carries what a cut hides.  A third, interleaved request must not disturb them.  Values are mixed on a
    column range."""
    from gesso_b200 import ops
    C, stride, T = 44, 52, 62
    taps = torch.randn(C, L, device=DEV)
    bias = torch.randn(C, device=DEV)
    u = [torch.randn(T, stride, device=DEV).to(dtype) for _ in range(2)]
    first = [torch.randn(T, 12, device=DEV).to(dtype) for _ in range(2)]
    lam, c0 = 0.37, 20
    want = []
    for r in range(2):
        y = pm.causal_conv(u[r][:, :C].double().cpu() + bias.double().cpu(), taps.double().cpu())
        y[:, c0:c0 + 12] = (1 - lam) * y[:, c0:c0 + 12] + lam * first[r].double().cpu()
        want.append(y)
    state = torch.full((4, max(L - 1, 0), C), float("nan"), device=DEV)
    state[1].zero_()
    state[3].zero_()
    cuts = [1, 1, 2, 1, 5, 3, 1, 17, 2, 9, 1, 1, 8, 10]
    assert sum(cuts) == T
    got = [[], []]
    at = 0
    for k, n in enumerate(cuts):
        # request 0 on slot 3, request 1 on slot 1, in changing order inside the step
        order = [0, 1] if k % 2 == 0 else [1, 0]
        rows = torch.cat([u[r][at:at + n] for r in order])
        fr = torch.cat([first[r][at:at + n] for r in order])
        seg, start = segments([n, n])
        slots = i32([3 if r == 0 else 1 for r in order])
        y = ops.causal_conv(rows, C, bias, taps, state, seg, start, slots, 2, mix=(fr, c0, 12, lam))
        for j, r in enumerate(order):
            got[r].append(y[j * n:(j + 1) * n].double().cpu())
        at += n
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    for r in range(2):
        g = torch.cat(got[r])
        assert torch.allclose(g, want[r], atol=tol, rtol=tol), f"request {r}: {float((g - want[r]).abs().max()):.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_norm_store_and_headwise_products(dtype):
    from gesso_b200 import ops
    T, Rq, R, page, H, D = 21, 24, 40, 16, 3, 10
    proj = torch.randn(T, Rq + R, device=DEV) * 3
    wq, wkv = torch.randn(Rq, device=DEV), torch.randn(R, device=DEV)
    pos = torch.arange(5, 5 + T, dtype=torch.int32, device=DEV)
    bt = i32([[3, 0, 2, 1]])
    kp = torch.zeros(5, 1, page, R, dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    cq = ops.latent_norm_store(proj, Rq, R, wq, wkv, 1e-5, dtype, pos, torch.zeros(T, dtype=torch.int32, device=DEV), bt, kp,
                               True, status)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    p = proj.double().cpu()
    assert int(status.item()) == 0
    assert torch.allclose(cq.double().cpu(), pm.norm_plain(p[:, :Rq], wq.double().cpu(), 1e-5), atol=tol, rtol=tol)
    want_c = pm.norm_plain(p[:, Rq:], wkv.double().cpu(), 1e-5)
    for t in range(T):
        q = 5 + t
        assert torch.allclose(kp[int(bt[0, q // page]), 0, q % page].double().cpu(), want_c[t], atol=tol, rtol=tol)
    x = torch.randn(T, H, D, device=DEV).to(dtype)
    w = torch.randn(H, D, R, device=DEV).to(dtype)
    for out_dtype in (torch.float32, dtype):
        got = ops.headwise_linear(x, w, out_dtype).double().cpu()
        want = torch.einsum("nhi,hio->nho", x.double().cpu(), w.double().cpu())
        assert torch.allclose(got, want, atol=tol * 5, rtol=tol)
    if dtype == torch.bfloat16:             # the tensor-core form: many rows, matrices output-major
        for N, Hh, I, O in ((64, 2, 16, 8), (333, 3, 48, 72), (2048, 4, 128, 64), (70, 1, 32, 200)):
            x = torch.randn(N, Hh, I, device=DEV).to(dtype)
            wt = torch.randn(Hh, O, I, device=DEV).to(dtype)
            assert ops.headwise_linear_tc_takes(N, x.dtype, wt, dtype)
            got = ops.headwise_linear_tc(x, wt).double().cpu()
            want = torch.einsum("nhi,hoi->nho", x.double().cpu(), wt.double().cpu())
            assert torch.allclose(got, want, atol=0.15, rtol=2e-2), float((got - want).abs().max())


def _pages(k, v, page_size, order):
    T, G, D = k.shape
    n = (T + page_size - 1) // page_size
    kp = torch.full((len(order) + 1, G, page_size, D), float("nan"), dtype=k.dtype, device=k.device)
    vp = None
    if v is not None:
        vp = torch.full((len(order) + 1, G, v.shape[2], page_size), float("nan"), dtype=k.dtype, device=k.device)
    for p in range(n):
        lo, hi = p * page_size, min(T, (p + 1) * page_size)
        kp[order[p], :, :hi - lo] = k[lo:hi].transpose(0, 1)
        if v is not None:
            vp[order[p], :, :, :hi - lo] = v[lo:hi].permute(1, 2, 0)
    bt = torch.full((1, len(order)), -1, dtype=torch.int32, device=k.device)
    bt[0, :n] = torch.tensor(order[:n], dtype=torch.int32)
    return kp, vp, bt


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,H,G,D,Vd,window", [("latent", 4, 1, 40, 40, 37), ("latent", 1, 1, 96, 96, None),
                                                  ("latent", 6, 1, 130, 130, 64), ("biased", 4, 2, 16, 24, 33),
                                                  ("biased", 3, 3, 48, 8, 16), ("biased", 8, 2, 64, 64, None),
                                                  ("biased", 2, 1, 32, 32, 200)])
def test_attention_sink_bias_and_edges_stand_out(kind, H, G, D, Vd, window, dtype):
    """One sequence in pages handed out of order, free pages full of NaN.  For the queries that test them, the key
    just inside the window, the key just outside it and a key far back are made to stand out (their score is raised
    far above the rest), so a window that is one key off, a far key that is lost or a distance bias of the wrong
    sign changes the result by a lot; the sink of one head is so large that leaving it out, scaling it or counting
    it per key shows.  ``latent``: float32 queries, values that are the keys, a sink.  ``biased``: a distance
    bias per head, values of another width.  The queries run as one portion and one by one."""
    from gesso_b200 import ops
    T, page, scale = 150, 16, 0.17
    latent = kind == "latent"
    q = torch.randn(T, H, D, device=DEV)
    k = torch.randn(T, G, D, device=DEV)
    v = None if latent else torch.randn(T, G, Vd, device=DEV)
    slopes = None if latent else pm.alibi_slopes(H).float().to(DEV)
    sink = torch.randn(H, device=DEV) if latent else None
    if latent:
        sink[0] = 9.0
    for i in (T - 1, 100, 77):
        edges = [0, i // 2] if window is None else [i - window + 1, i - window, max(0, i - window - 40)]
        for n, j in enumerate(edges):
            if 0 <= j <= i:
                k[j] = (q[i, :: H // G] / q[i, :: H // G].norm(dim=-1, keepdim=True)) * (10.0 + 2 * n) / scale / q[i, 0].norm()
    k = k.to(dtype)
    v = None if v is None else v.to(dtype)
    qq = q if latent else q.to(dtype)               # latent attention feeds float32 queries
    order = [7, 2, 9, 0, 4, 1, 8, 3, 6, 5]
    kp, vp, bt = _pages(k, v, page, order)
    kd, vd_ = k.double().cpu(), (k if latent else v).double().cpu()
    want = pm.attend_fast(qq.double().cpu(), kd, vd_, scale, window, sink=None if sink is None else sink.cpu(),
                          slopes=None if slopes is None else slopes.double().cpu(), group=H // G)
    lone = pm.attend(qq.double().cpu()[:20], kd[:20], vd_[:20], scale, window, sink=None if sink is None else sink.cpu(),
                     slopes=None if slopes is None else slopes.double().cpu(), group=H // G)
    assert torch.allclose(lone, want[:20], atol=1e-9)           # the two plain forms agree
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    seg = torch.zeros(T, dtype=torch.int32, device=DEV)
    vpages = vp if vp is not None else kp[:, :, :0]
    got = ops.paged_attention_generic(qq, kp, vpages, bt, pos, seg, window, scale, sink=sink, slopes=slopes,
                                      values_are_keys=latent).double().cpu()
    err = (got - want).abs().max() / want.abs().max()
    assert err <= tol, f"portion: {float(err):.3e}"
    for i in (T - 1, 100, 77, 0, 16, 15):
        bt_i = bt.clone()
        if window:
            bt_i[0, :max(0, i - window + 1) // page] = -1          # pages behind the window are given back
        got = ops.paged_attention_generic(qq[i:i + 1].contiguous(), kp, vpages, bt_i, pos[i:i + 1], seg[:1], window, scale,
                                          sink=sink, slopes=slopes, values_are_keys=latent).double().cpu()
        err = (got[0] - want[i]).abs().max() / want.abs().max()
        assert err <= tol, f"single token at {i}: {float(err):.3e}"


@pytest.mark.parametrize("H,G,D,window", [(8, 2, 64, 45), (4, 4, 128, 64), (4, 2, 32, None), (6, 2, 96, 37), (16, 1, 64, 130),
                                          (32, 2, 64, 50)])
@pytest.mark.parametrize("what", ["bias", "sink"])
def test_distance_bias_and_sink_on_the_tensor_core_kernels(H, G, D, window, what):
    """The sizes whose bfloat16 steps take the mma.sync kernels (a portion; single tokens with the keys cut into
    pieces or not): the same stand-out keys as above, through the engine's own choice of kernel, with a distance
    bias per head or with sinks (one of them far above every score)."""
    from gesso_b200.engine import attention_dispatch
    from gesso_b200.engine.model import PagedView, Runtime
    T, page, scale = 330, 16, 0.17
    q = torch.randn(T, H, D, device=DEV)
    k = torch.randn(T, G, D, device=DEV)
    v = torch.randn(T, G, D, device=DEV)
    slopes = pm.alibi_slopes(H).float().to(DEV) if what == "bias" else None
    sink = None
    if what == "sink":
        sink = torch.randn(H, device=DEV)
        sink[0] = 9.0
    tests = (T - 1, 100, 77)
    for i in tests:
        edges = [0, i // 2] if window is None else [i - window + 1, i - window]
        for n, j in enumerate(edges):
            if 0 <= j <= i:
                k[j] = (q[i, :: H // G] / q[i, :: H // G].norm(dim=-1, keepdim=True)) * (10.0 + 2 * n) / scale / q[i, 0].norm()
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    order = list(range(21))[::-1]
    kp, vp, bt = _pages(k, v, page, order)
    vp = torch.nan_to_num(vp)                       # the cache writer keeps the tail of a request's last block zero
    want = pm.attend_fast(q.double().cpu(), k.double().cpu(), v.double().cpu(), scale, window,
                          sink=None if sink is None else sink.cpu(), slopes=None if slopes is None else slopes.double().cpu(),
                          group=H // G)
    rt = Runtime(DEV, torch.bfloat16, 1024)

    class Ctx:
        pass
    c = Ctx()
    c.decode_only, c.n_segs, c.max_kv_len = False, 1, T
    c.positions = torch.arange(T, dtype=torch.int32, device=DEV)
    c.seg_of_token = torch.zeros(T, dtype=torch.int32, device=DEV)
    c.seg_start, c.seg_pos0 = i32([0, T]), i32([0])
    tiles = (T + 63) // 64
    c.tile_seg = torch.zeros(tiles, dtype=torch.int32, device=DEV)
    c.tile_q0 = torch.arange(tiles, dtype=torch.int32, device=DEV) * 64
    c.kv_span = i32([T, T])
    got = attention_dispatch.paged_attention(rt, q, PagedView(kp, vp, bt, True), c, window, scale, slopes=slopes, sink=sink,
                                             split_weights=True).double().cpu()
    err = (got - want).abs().max() / want.abs().max()
    assert err <= 2e-2, f"portion: {float(err):.3e}"
    for i in tests + (0, 16, 15, 300):
        c = Ctx()
        c.decode_only, c.n_segs, c.max_kv_len = True, 1, i + 1
        c.positions, c.seg_of_token, c.kv_span = i32([i]), i32([0]), i32([i + 1, i + 1])
        bt_i = bt.clone()
        if window:
            bt_i[0, :max(0, i - window + 1) // page] = -1
        got = attention_dispatch.paged_attention(rt, q[i:i + 1].contiguous(), PagedView(kp, vp, bt_i, True), c, window, scale,
                                                 slopes=slopes, sink=sink, split_weights=True).double().cpu()
        err = (got[0] - want[i]).abs().max() / want.abs().max()
        assert err <= 2e-2, f"single token at {i}: {float(err):.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,Dv", [(2, 16, 24), (3, 40, 8), (1, 64, 64), (2, 128, 20), (1, 200, 33), (4, 7, 5)])
def test_lightning_recurrence_portions_and_single_tokens(H, D, Dv, dtype):
    """Decays of one, near one and near zero over 300 positions: a head that forgets nothing keeps the first token
    visible to the last (made large so that losing it shows).  The same rows run as one portion, token by token,
    and in uneven portions beside another request; the state slot carries everything between steps."""
    from gesso_b200 import ops
    T = 300
    stride = 2 * H * D + H * Dv + 16
    decay = [1.0, 0.97, 0.05, 0.999][:H]
    rows = [torch.randn(T, stride, device=DEV).to(dtype) for _ in range(2)]
    rows[0][0, 2 * H * D:2 * H * D + H * Dv] = 6.0          # the first token's values stand out
    dd = torch.tensor(decay, dtype=torch.float32, device=DEV)
    silu = torch.nn.functional.silu
    want = []
    for r in rows:
        x = r.double().cpu()
        q = silu(x[:, :H * D]).view(T, H, D)
        k = silu(x[:, H * D:2 * H * D]).view(T, H, D)
        v = silu(x[:, 2 * H * D:2 * H * D + H * Dv]).view(T, H, Dv)
        o = torch.zeros(T, H, Dv, dtype=torch.float64)
        for h in range(H):
            S = torch.zeros(D, Dv, dtype=torch.float64)
            for t in range(T):
                S = decay[h] * S + torch.outer(k[t, h], v[t, h])
                o[t, h] = S.T @ q[t, h]
        want.append(o.reshape(T, H * Dv))
    tol = 3e-5 if dtype == torch.float32 else 2e-2

    def check(got, r, what):
        err = (got - want[r]).abs().max() / want[r].abs().max()
        assert err <= tol, f"{what}: {float(err):.3e}"
    state = torch.full((3, H, Dv, D), float("nan"), device=DEV)
    state[0].zero_()
    seg_start = i32([0, T])
    check(ops.lightning_attention(rows[0], state, dd, seg_start, i32([0]), 1, H, D, Dv).double().cpu(), 0, "one portion")
    state[2].zero_()
    out = [ops.lightning_attention(rows[0][t:t + 1], state, dd, i32([0, 1]), i32([2]), 1, H, D, Dv) for t in range(T)]
    check(torch.cat(out).double().cpu(), 0, "token by token")
    state[0].zero_()
    state[1].zero_()
    cuts = [1, 2, 17, 1, 64, 3, 100, 2, 45, 65]
    assert sum(cuts) == T
    got, at = [[], []], 0
    for kk, n in enumerate(cuts):
        order = [0, 1] if kk % 2 else [1, 0]
        both = torch.cat([rows[r][at:at + n] for r in order])
        _, start = segments([n, n])
        y = ops.lightning_attention(both, state, dd, start, i32([1 if r == 0 else 0 for r in order]), 2, H, D, Dv)
        for j, r in enumerate(order):
            got[r].append(y[j * n:(j + 1) * n].double().cpu())
        at += n
    for r in range(2):
        check(torch.cat(got[r]), r, f"portions, request {r}")
    if not ops.lightning_chunked_takes(10 ** 6, D, Dv):
        return
    # the same by 64-token tiles side by side: one portion; then uneven portions of two requests, with the tile list
    # of a padded step (its last tile repeated)
    def tiles(lens, extra=0):
        ts = [(i, q0) for i, n in enumerate(lens) for q0 in range(0, n, 64)] + [(len(lens) - 1, 0)] * extra
        return i32([t[0] for t in ts]), i32([t[1] for t in ts])
    state[0].zero_()
    tseg, tq0 = tiles([T])
    check(ops.lightning_attention_chunked(rows[0], state, dd, seg_start, i32([0]), tseg, tq0, 1, H, D, Dv).double().cpu(), 0,
          "one portion by tiles")
    assert torch.allclose(state[0], state[2], atol=1e-4, rtol=1e-4), "the state a portion leaves, by tiles and token by token"
    state[0].zero_()
    state[1].zero_()
    got, at = [[], []], 0
    for kk, n in enumerate([130, 1, 64, 65, 40]):
        order = [0, 1] if kk % 2 else [1, 0]
        both = torch.cat([rows[r][at:at + n] for r in order])
        _, start = segments([n, n])
        tseg, tq0 = tiles([n, n], extra=kk % 3)
        y = ops.lightning_attention_chunked(both, state, dd, start, i32([1 if r == 0 else 0 for r in order]), tseg, tq0, 2,
                                            H, D, Dv)
        for j, r in enumerate(order):
            got[r].append(y[j * n:(j + 1) * n].double().cpu())
        at += n
    for r in range(2):
        check(torch.cat(got[r]), r, f"portions by tiles, request {r}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_norm_and_activations(dtype):
    from gesso_b200 import ops
    N, W = 37, 88
    o = torch.randn(N, W, device=DEV) * 5
    w = torch.randn(W, device=DEV)
    wide = torch.randn(N, W + 24, device=DEV).to(dtype)
    gate = wide[:, 8:8 + W]
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    got = ops.gated_rmsnorm(o, w, 1e-6, gate, dtype).double().cpu()
    want = pm.norm_plain(o.double().cpu(), w.double().cpu(), 1e-6) * torch.sigmoid(gate.double().cpu())
    assert torch.allclose(got, want, atol=tol, rtol=tol)
    x = (torch.randn(N, 56, device=DEV) * 3).to(dtype)
    assert torch.allclose(ops.gelu_erf(x).double().cpu(), pm.gelu_erf(x.double().cpu()), atol=tol, rtol=tol)
    F, limit = 24, 1.3
    gu = (torch.randn(N, 2 * F, device=DEV) * 2).to(dtype)
    g, u = gu.double().cpu()[:, :F], gu.double().cpu()[:, F:]
    g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    want = g * torch.sigmoid(1.702 * g) * (u + 1)
    assert torch.allclose(ops.glu_clamped(gu, limit).double().cpu(), want, atol=tol, rtol=tol)
    packed = torch.stack([gu[:, :F].reshape(N, F // 8, 8), gu[:, F:].reshape(N, F // 8, 8)], dim=2).reshape(N, 2 * F).contiguous()
    assert torch.allclose(ops.glu_clamped(packed, limit, packed=True).double().cpu(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("E,top,groups,keep", [(6, 2, 3, 2), (4, 4, 1, 1), (16, 3, 8, 5), (8, 1, 4, 1), (5, 2, 5, 3)])
def test_softmax_router_with_groups_scored_by_their_best(E, top, groups, keep):
    from gesso_b200 import ops
    T, W = 200, 72
    x = torch.randn(T, W, device=DEV)
    wr = (torch.randn(E, W, device=DEV) * 0.4).to(torch.bfloat16).float()
    idx, w = ops.moe_route(x, wr, None, top, groups, keep, group_top=1, score="softmax")
    z = x.double().cpu() @ wr.double().cpu().T
    clear = 0
    for t in range(T):
        if pm.route_margin(z[t], top, groups, keep) < 1e-3:
            continue
        clear += 1
        chosen, weights = pm.route(z[t], top, groups, keep)
        assert sorted(idx[t].tolist()) == sorted(chosen), f"token {t}"
        got = dict(zip(idx[t].tolist(), w[t].tolist()))
        assert all(abs(got[e] - we) <= 2e-6 for e, we in zip(chosen, weights))
    assert clear > T // 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W,F,E,top", [(5, 64, 24, 6, 2), (70, 96, 20, 4, 4), (300, 128, 32, 16, 3), (33, 72, 100, 4, 1),
                                         (260, 200, 72, 12, 3), (129, 64, 8, 3, 1), (500, 256, 48, 8, 2)])
def test_gated_experts_pairwise_and_grouped(T, W, F, E, top, dtype):
    """The clamped gated unit in both ways the experts run (pair by pair; grouped by expert on the tensor cores where
    the step takes that path), in both layouts of the gate and up rows, added to a shared expert's output."""
    from gesso_b200 import ops
    limit = 1.1
    x = torch.randn(T, W, device=DEV).to(dtype)
    wg = (torch.randn(E, F, W, device=DEV) * 2 / math.sqrt(W)).to(dtype)
    wu = (torch.randn(E, F, W, device=DEV) * 2 / math.sqrt(W)).to(dtype)
    wd = (torch.randn(E, W, F, device=DEV) / math.sqrt(F)).to(dtype)
    idx = torch.stack([torch.randperm(E, device=DEV)[:top] for _ in range(T)]).to(torch.int32)
    if T > 20:
        idx[:, 0] = torch.where(torch.arange(T, device=DEV) % 3 == 0, idx[:, 0], idx[0, 0])      # uneven loads
    w = torch.rand(T, top, device=DEV)
    base = torch.randn(T, W, device=DEV)
    want = base.double().cpu().clone()
    xd = x.double().cpu()
    for t in range(T):
        for kk in range(top):
            e = int(idx[t, kk])
            want[t] += float(w[t, kk]) * pm.expert(xd[t:t + 1], wg[e].double().cpu(), wu[e].double().cpu(), wd[e].double().cpu(), limit)[0]
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    plain_rows = torch.cat([wg, wu], dim=1).contiguous()
    got = ops.moe_experts_pairs(x, plain_rows, wd, idx, w, "glu_clamped", limit, False, add_to=base.clone())
    assert (got.double().cpu() - want).abs().max() <= tol * want.abs().max()
    if F % 8 == 0:
        packed = torch.stack([ops.pack_gate_up(wg[e], wu[e]) for e in range(E)]).contiguous()
        got = ops.moe_experts_pairs(x, packed, wd, idx, w, "glu_clamped", limit, True, add_to=base.clone())
        assert (got.double().cpu() - want).abs().max() <= tol * want.abs().max()
        if ops.moe_grouped_takes(x, packed, wd, top, "glu_clamped", True):
            got = ops.moe_experts_grouped(x, packed, wd, idx, w, "glu_clamped", limit, add_to=base.clone())
            ops.check_tc_status()
            assert (got.double().cpu() - want).abs().max() <= tol * want.abs().max()
        else:
            assert dtype == torch.float32 or T * top <= ops.MOE_PAIR_MAX_ROWS


# ---- whole models ------------------------------------------------------------------------------------------
def test_layer_streams_float32(loaded, plain):
    """The stream after every layer, layer by layer, in float32 (a hook on the blocks)."""
    from gesso_b200 import ops
    from gesso_b200.engine.batch import StepEntry
    from gesso_b200.engine.trace import make_engine
    for name in cm.MMP:
        model = loaded(name, "float32")
        toks = tt.make_requests(cm.MMP[name][0]["vocab"], [29], seed=3)[0]
        want = plain.models[name].stream(toks)
        eng = make_engine(model, 64, use_graphs=False)
        seen, olds = [], []
        for blk in model.blocks:
            old = blk.forward
            olds.append(old)

            def hooked(h, pending, ctx, cache, old=old):
                d, b = old(h, pending, ctx, cache)
                hh = h.double().clone()
                parts = [d.first, d.second] if isinstance(d, ops.SummedDeltas) else [d]
                for p in parts:
                    hh += p.double()
                if b is not None:
                    hh += b.double()
                seen.append(hh.cpu())
                return d, b
            blk.forward = hooked
        try:
            eng.admit("r")
            eng.step([StepEntry("r", toks, [len(toks) - 1])])
        finally:
            for blk, old in zip(model.blocks, olds):
                blk.forward = old
        assert len(seen) == len(want)
        for i, (a, b) in enumerate(zip(seen, want)):
            assert (a - b).abs().max() <= 2e-5 * b.abs().max(), f"{name}: layer {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", list(SCHEDULES))
@pytest.mark.parametrize("name", list(cm.MMP))
def test_replay_matches_plain(name, schedule, dtype, loaded, plain, tmp_path):
    reqs, ref = plain(name)
    tb, max_tokens = SCHEDULES[schedule](reqs)
    model = loaded(name, dtype)
    tt.run_in_process(model, tb, max_tokens, str(tmp_path))
    rows = tt.read_rows(tb, str(tmp_path), model.vocab_size)
    compare(rows, ref, TOL[dtype], f"{name}/{schedule}/{dtype}", plain.margins(name, dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(cm.MMP))
def test_pages_and_slots_used_again(name, dtype, loaded, plain, tmp_path):
    """Every free page and slot filled with NaN before a mixed replay on a pool made for the live requests only,
    with graphs off and on."""
    reqs, ref = plain(name)
    tb, max_tokens = SCHEDULES["mixed"](reqs)
    model = loaded(name, dtype)
    for graphs in (False, True):
        d = tmp_path / f"g{int(graphs)}"
        tt.run_in_process(model, tb, max_tokens, str(d), prepare=tt.poison_free_memory, use_graphs=graphs)
        compare(tt.read_rows(tb, str(d), model.vocab_size), ref, TOL[dtype], f"poisoned {name}/{dtype}",
                plain.margins(name, dtype))


@pytest.mark.parametrize("name", ["a", "c"])
def test_lightning_by_chunks_inside_the_engine(name, loaded, plain, tmp_path, monkeypatch):
    """Every step with a portion takes the chunked form of the recurrence (the tests' prompts are shorter than the
    length from which the engine chooses it by itself), in whole prompts, uneven portions and mixed, padded steps."""
    from gesso_b200 import ops
    monkeypatch.setattr(ops, "LIGHTNING_CHUNK_MIN_TOKENS", 2)
    reqs, ref = plain(name)
    model = loaded(name, "float32")
    for sched in ("whole", "portions", "mixed"):
        tb, max_tokens = SCHEDULES[sched](reqs)
        for graphs in (False, True):
            d = str(tmp_path / f"{sched}{int(graphs)}")
            tt.run_in_process(model, tb, max_tokens, d, prepare=tt.poison_free_memory, use_graphs=graphs)
            compare(tt.read_rows(tb, d, model.vocab_size), ref, TOL["float32"], f"chunked {name}/{sched}/graphs={graphs}")


def test_schedules_agree_float32(loaded, plain, tmp_path):
    reqs, _ = plain("a")
    model = loaded("a", "float32")
    got = {}
    for sched, make in SCHEDULES.items():
        tb, max_tokens = make(reqs)
        tt.run_in_process(model, tb, max_tokens, str(tmp_path / sched))
        got[sched] = tt.read_rows(tb, str(tmp_path / sched), model.vocab_size)
    for sched, rows in got.items():
        for key, row in rows.items():
            assert row_error(row, got["whole"][key]) <= 2e-5, (sched, key)


@pytest.mark.parametrize("name", ["a", "c"])
def test_long_decoding_gives_pages_back(name, loaded, plain):
    """Token by token far past every window: the pool stays small, the states carry on."""
    from gesso_b200.engine.batch import StepEntry
    from gesso_b200.engine.engine import Engine
    model = loaded(name, "float32")
    toks = tt.make_requests(cm.MMP[name][0]["vocab"], [330], seed=9)[0]
    want = plain.models[name].logits(toks).numpy()
    eng = Engine(model, max_positions=512, page_size=16, num_pages=8, max_requests=2)     # 128 positions of pages
    eng.admit("r")
    eng.step([StepEntry("r", toks[:40], [])])
    for p in range(40, 330):
        lg = eng.step([StepEntry("r", [toks[p]], [0])])
        if p % 37 == 0 or p > 320:
            assert row_error(lg[0].cpu().numpy(), want[p]) <= TOL["float32"], p
    assert max(eng.cache.pages_in_use()) <= 6
    eng.release("r")
    eng.cache.check_invariants()


@pytest.mark.parametrize("name", list(cm.MMP))
def test_greedy_generation_through_the_session(name, loaded, plain):
    import gesso_b200
    model = loaded(name, "float32")
    s = gesso_b200.Session(model, context_length=256, page_size=16, max_batch=4)
    prompts = tt.make_requests(cm.MMP[name][0]["vocab"], [9, 1, 60, 2], seed=21)
    for p in prompts:
        assert s.generate(p, max_new_tokens=6) == plain.models[name].greedy(p, 6)
    res = s.run_batch([gesso_b200.BatchRequest(p, max_new_tokens=6) for p in prompts])
    for p, r in zip(prompts, res):
        assert list(r.ids) == plain.models[name].greedy(p, 6)
    assert all(n == 0 for n in s.engine.cache.pages_in_use())


def random_memipel_config(seed):
    """Seeded random configurations: any order of the three mixers, any head layout, windows shorter and longer than
    the prompts, any number of taps, feed-forwards of every kind and none, groups or none, a shared expert or none."""
    import random
    rng = random.Random(seed)
    width = rng.choice([48, 64, 72, 96, 128, 200])
    v_width = rng.choice([16, 24, 32, 48])             # kv_heads * vdim of the layers that mix values

    def mlp():
        x = rng.random()
        if x < 0.15:
            return None
        if x < 0.35:
            return {"kind": "dense", "ff": rng.choice([24, 40, 100])}
        gsz, count = rng.choice([1, 2, 3, 4]), rng.choice([1, 2, 3, 4])
        keep = rng.randint(1, count)
        m = {"kind": "moe", "expert": {"ff": rng.choice([8, 20, 24, 40, 64]), "limit": rng.choice([0.7, 1.5, 3.0])},
             "router": {"experts": gsz * count, "top": rng.randint(1, min(4, gsz * keep))}}
        if rng.random() < 0.8:
            m["router"]["groups"] = {"count": count, "keep": keep}
        elif m["router"]["top"] > gsz * count:
            m["router"]["top"] = gsz * count
        if "groups" not in m["router"]:
            m["router"]["top"] = min(m["router"]["top"], gsz * count)
        if rng.random() < 0.6:
            m["shared"] = {"ff": rng.choice([8, 20, 48]), "limit": rng.choice([1.0, 2.0])}
        return m

    def mask():
        return {"size": rng.choice([1, 3, 9, 16, 17, 31, 50, 64, 200])} if rng.random() < 0.85 else None

    layers = []
    for _ in range(rng.randint(2, 5)):
        kind = rng.choice(["latent_attention", "attention", "lightning"])
        heads = rng.choice([1, 2, 3, 4, 6])
        if kind == "latent_attention":
            dim = rng.choice([8, 16, 24, 32, 64])
            m = {"heads": heads, "dim": dim, "vdim": rng.choice([8, dim, 40]), "q_rank": rng.choice([8, 24, 48]),
                 "kv_rank": rng.choice([8, 32, 40, 96, 144]), "scale": rng.choice([0.1, 0.2, dim ** -0.5])}
            if (mk := mask()) is not None:
                m["mask"] = mk
        elif kind == "attention":
            kv = rng.choice([d for d in (1, 2, 3, 4, 6) if heads % d == 0])
            dim = rng.choice([8, 16, 32, 48, 64])
            v_mix = rng.random() < 0.6 and v_width % kv == 0
            m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": v_width // kv if v_mix else rng.choice([8, dim, 24]),
                 "scale": rng.choice([0.1, 0.25, dim ** -0.5]), "conv": rng.choice([1, 2, 3, 4]), "v_mix": v_mix}
            if (mk := mask()) is not None:
                m["mask"] = mk
        else:
            m = {"heads": heads, "dim": rng.choice([8, 16, 24, 32, 64, 72]), "vdim": rng.choice([8, 16, 40, 64]),
                 "decay": [rng.choice([1.0, 0.999, 0.97, 0.8, 0.3]) for _ in range(heads)]}
        layers.append({"type": kind, "mixer": m, "mlp": mlp()})
    cfg = {"architecture": "Memipel", "vocab": rng.choice([97, 256, 503]), "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5])},
           "layers": layers}
    return cfg, [rng.choice([1, 2, 5, 17, 33, 64, 65, 70, 97, 130]) for _ in range(4)]


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 13, 15, 17])
def test_random_configuration_replays_like_plain(seed, tmp_path):
    import gesso_b200
    cfg, lengths = random_memipel_config(seed)
    d = str(tmp_path / "model")
    pm.write_model(d, cfg, seed)
    plain_model = pm.PlainMemipel.from_dir(d)
    reqs = tt.make_requests(cfg["vocab"], lengths, seed=seed)
    ref = [plain_model.logits(t).numpy() for t in reqs]
    margins = [plain_model.margins(t).numpy() for t in reqs] if seed % 2 else None      # bfloat16 for every other seed
    for dtype in ("float32", "bfloat16") if margins is not None else ("float32",):
        model = gesso_b200.load(d, dtype=dtype, max_positions=256)
        for name, make in SCHEDULES.items():
            tb, max_tokens = make(reqs)
            out = str(tmp_path / f"{dtype}_{name}")
            tt.run_in_process(model, tb, max_tokens, out)
            compare(tt.read_rows(tb, out, cfg["vocab"]), ref, TOL[dtype], f"seed {seed} {name} {dtype} {cfg}",
                    margins if dtype == "bfloat16" else None)
        del model


@pytest.mark.parametrize("which", ["MMP_ONLY_STATE", "MMP_ONLY_PAGES"])
def test_stacks_of_one_kind_of_cache(which, tmp_path):
    """A model without any pages and one without any state go through the same engine, in both run types."""
    import gesso_b200
    cfg = getattr(cm, which)
    d = str(tmp_path / "model")
    pm.write_model(d, cfg, 4)
    plain_model = pm.PlainMemipel.from_dir(d)
    reqs = tt.make_requests(cfg["vocab"], [33, 1, 70, 18], seed=8)
    ref = [plain_model.logits(t).numpy() for t in reqs]
    for dtype in ("float32", "bfloat16"):
        model = gesso_b200.load(d, dtype=dtype, max_positions=256)
        for name, make in SCHEDULES.items():
            tb, max_tokens = make(reqs)
            out = str(tmp_path / f"{dtype}_{name}")
            tt.run_in_process(model, tb, max_tokens, out)
            compare(tt.read_rows(tb, out, cfg["vocab"]), ref, TOL[dtype], f"{which} {name} {dtype}")
        del model


def test_layer_widths_of_a_real_model():
    """Width 1,024, 16 heads, a latent of 128, 16 experts: a prompt of 1,300 tokens takes the paths that only large
    steps take (tcgen05 products, experts grouped by expert, lightning by chunks, the tensor-core attention kernels
    with a sink and with a distance bias, per-head products on the tensor cores).  Cut into portions the float32
    engine gives the same logits as in one step; the bfloat16 engine agrees with the float32 one within rounding
    (the median row well within a hundredth; single rows may sit on a router's close call)."""
    import gesso_b200
    from gesso_b200.engine.batch import StepEntry
    from gesso_b200.engine.trace import make_engine
    moe = {"kind": "moe", "expert": {"ff": 512, "limit": 7.0}, "router": {"experts": 16, "top": 4, "groups": {"count": 4, "keep": 2}},
           "shared": {"ff": 512, "limit": 7.0}}
    layers = [cm.lightning(16, 64, 64, [1.0 - 2.0 ** -(1 + h / 2) for h in range(16)], {"kind": "dense", "ff": 2048}),
              cm.latent(16, 64, 64, 384, 128, 0.125, 1024, moe),
              cm.attention(16, 4, 64, 64, 0.125, 3, 1024, True, moe),
              cm.lightning(16, 64, 64, [1.0 - 2.0 ** -(1 + h / 2) for h in range(16)], moe),
              cm.attention(16, 4, 64, 64, 0.125, 3, 1024, True, moe)]
    cfg = {"architecture": "Memipel", "vocab": 1024, "width": 1024, "norm": {"eps": 1e-6}, "layers": layers}
    T = 1300
    toks = tt.make_requests(1024, [T], seed=1)[0]
    want = list(range(0, T, 37)) + [T - 1]
    res = {}
    for dtype in ("float32", "bfloat16"):
        model = gesso_b200.random_model(cfg, seed=0, dtype=dtype, max_positions=2048, style="fan_in")
        for mode, cuts in (("whole", [T]), ("portions", [1100, 2, 64, 100, 1, 1, 30, 2])):
            eng = make_engine(model, 2048)
            eng.admit("a")
            rows, at = [], 0
            for c in cuts:
                w = [p - at for p in want if at <= p < at + c]
                lg = eng.step([StepEntry("a", toks[at:at + c], w)])
                if w:
                    rows.append(lg.float().cpu().numpy().copy())
                at += c
            eng.check_status()
            eng.release("a")
            res[(dtype, mode)] = np.concatenate(rows, 0)
        del model
        torch.cuda.empty_cache()
    ref = res[("float32", "whole")]
    errs = lambda a: np.array([row_error(x, y) for x, y in zip(a, ref)])
    assert errs(res[("float32", "portions")]).max() <= 2e-5
    for mode in ("whole", "portions"):
        e = errs(res[("bfloat16", mode)])
        assert np.median(e) <= 0.012 and np.percentile(e, 80) <= 0.03, (mode, float(np.median(e)), float(e.max()))


def test_trace_program_on_a_model_folder(mmp_dirs, plain, tmp_path):
    reqs, ref = plain("b")
    tb, max_tokens = tt.trace_mixed(reqs, seed=2)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", mmp_dirs["b"], "--dtype", "bfloat16",
                        "--out", str(out), "--max-tokens", str(max_tokens)], input=tb.text(), capture_output=True, text=True,
                       timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    compare(tt.read_rows(tb, str(out), cm.MMP_B["vocab"]), ref, TOL["bfloat16"], "trace program b/mixed",
            plain.margins("b", "bfloat16"))
