"""Tiny Memipel configurations of the tests.  They differ in every size and option."""


def _moe(ff, limit, experts, top, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def lightning(heads, dim, vdim, decay, mlp):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}


def latent(heads, dim, vdim, q_rank, kv_rank, scale, window, mlp):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def attention(heads, kv, dim, vdim, scale, conv, window, v_mix, mlp):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if conv is not None:
        m["conv"] = conv
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": mlp}


# every kind of layer; two value-mixing layers of different head layouts but equal value width (2 x 16 = 1 x 32),
# windows 20 (longer than a page), 37 and 9 (shorter than a page), 6 experts in 3 groups (2 kept), a shared expert,
# a dense layer, a layer without a feed-forward.
MMP_A = {"architecture": "Memipel", "vocab": 131, "width": 64, "norm": {"eps": 1e-5}, "layers": [
    lightning(2, 16, 24, [0.7, 0.995], _dense(80)),
    latent(4, 16, 8, 24, 32, 0.3, 20, _moe(24, 1.5, 6, 2, (3, 2), (16, 1.0))),
    attention(4, 2, 16, 16, 0.25, 3, 37, True, _moe(24, 1.5, 6, 2, (3, 2), (16, 1.0))),
    attention(2, 1, 32, 32, 0.2, 2, 9, True, _dense(40)),
    lightning(2, 16, 24, [0.9, 0.5], None),
]}

# sizes that are no multiples of 8 or powers of two: an odd head size, values wider than keys, a convolution of four taps, a window
# longer than most prompts, latent attention over all keys with one head, decays of exactly one and near zero,
# experts without groups and without a shared expert (every expert chosen: top = experts), expert width 20.
MMP_B = {"architecture": "Memipel", "vocab": 257, "width": 96, "norm": {"eps": 1e-6}, "layers": [
    attention(3, 3, 9, 40, 0.4, 4, 130, False, _moe(20, 0.8, 4, 4)),
    latent(1, 48, 48, 8, 80, 0.15, None, _dense(72)),
    lightning(3, 40, 8, [1.0, 0.05, 0.97], _moe(20, 2.5, 5, 2, (5, 3))),
]}

# sizes the tensor-core paths take (widths in multiples of 16, many (token, expert) pairs): 16 experts in 8 pairs
# (5 kept), top 3, a shared expert wider than the routed ones; a window that is a whole number of pages; one
# value-mixing layer alone (a source that nobody mixes with); a convolution of one tap.
MMP_C = {"architecture": "Memipel", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "layers": [
    latent(8, 32, 32, 48, 64, 0.18, 64, _moe(32, 2.0, 16, 3, (8, 5), (64, 1.2))),
    lightning(2, 64, 64, [0.999, 0.8], _moe(32, 2.0, 16, 3, (8, 5), (64, 1.2))),
    attention(4, 2, 64, 64, 0.125, 1, 48, True, _moe(48, 1.0, 8, 1, (4, 1))),
]}

# stacks of one kind of mixer only: no pages at all (every layer keeps a state), no state at all (every layer keeps
# pages), a latent wider than 256
MMP_ONLY_STATE = {"architecture": "Memipel", "vocab": 90, "width": 48, "norm": {"eps": 1e-6}, "layers": [
    lightning(3, 8, 16, [0.9, 0.99, 0.5], _dense(32)), lightning(1, 24, 8, [0.95], None)]}
MMP_ONLY_PAGES = {"architecture": "Memipel", "vocab": 90, "width": 48, "norm": {"eps": 1e-6}, "layers": [
    latent(2, 8, 8, 16, 272, 0.3, 25, None), latent(5, 16, 24, 8, 24, 0.2, None, _dense(64))]}

# name -> (config, seed)
MMP = {"a": (MMP_A, 21), "b": (MMP_B, 22), "c": (MMP_C, 23)}
