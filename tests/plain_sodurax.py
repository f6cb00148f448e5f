"""A plain, slow implementation of the Sodurax design in float64, one function per mechanism.

It shares no code with the engine: it reads a configuration object and a dictionary of tensors under
their checkpoint names, runs whole sequences without any cache, and is what the engine is held to.

Notation: ``h`` the stream [T, W]; a layer does ``h += N1b(mixer(N1(h)))`` then ``h += N2b(ff(N2(h)))``
with ``N(x) = tanh(a x) * g + c`` (scalar ``a``, vectors ``g``, ``c``).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def dyt(x, W, name):
    """tanh(a x) g + c."""
    return torch.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def rotation_angles(n_pos: int, rot) -> torch.Tensor:
    """[positions, dims/2]: position p, pair i -> p * base^(-2i/dims) / factor."""
    d = rot["dims"]
    i = torch.arange(d // 2, dtype=F64)
    f = float(rot["base"]) ** (-2.0 * i / d)
    if rot.get("scaling"):
        f = f / float(rot["scaling"]["factor"])
    return torch.arange(n_pos, dtype=F64)[:, None] * f[None, :]


def rotate(x, ang, dims):
    """x [T, heads, D]: feature i is paired with i + dims/2 for i < dims/2; the rest pass unchanged."""
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visibility(T: int, mask) -> torch.Tensor:
    """[T, T] bool: query i sees key j if j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    vis = j <= i
    if mask:
        vis = vis & ((i - j < mask["size"]) | (j < mask.get("keep_first", 0)))
    return vis


def attention(x, W, p, m):
    T = x.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
    q = (x @ W[p + "q"].T + W[p + "q.b"]).view(T, H, D)
    k = (x @ W[p + "k"].T + W[p + "k.b"]).view(T, G, D)
    v = (x @ W[p + "v"].T + W[p + "v.b"]).view(T, G, V)
    if m.get("rot"):
        ang = rotation_angles(T, m["rot"])
        q, k = rotate(q, ang, m["rot"]["dims"]), rotate(k, ang, m["rot"]["dims"])
    vis = visibility(T, m.get("mask"))
    out = torch.zeros(T, H, V, dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~vis, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    gated = out.reshape(T, H * V) * torch.sigmoid(x @ W[p + "g"].T)
    return gated @ W[p + "o"].T


def route(x, W, p, r):
    """Chosen experts [T, top] (best first) and their weights: the scores WITHOUT the correction."""
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    gc, gk = groups["count"], groups["keep"]
    s = torch.sigmoid(x @ W[p + "router"].T)
    c = s + W[p + "correction"]
    T = x.shape[0]
    cg = c.view(T, gc, E // gc)
    gscore = cg.topk(min(2, E // gc), dim=-1).values.sum(-1)
    kept = torch.zeros(T, gc, dtype=torch.bool)
    kept.scatter_(1, gscore.topk(gk, dim=-1).indices, True)
    c_open = cg.masked_fill(~kept[:, :, None], -math.inf).reshape(T, E)
    idx = c_open.topk(top, dim=-1).indices
    return idx, s.gather(1, idx)


def route_margin(x, W, p, r):
    """How clear the choice is, per token: the smaller of the gap between the last kept and the first shut-out
    group and the gap between the last chosen and the first unchosen open expert.  A run in lower precision
    may choose otherwise where this is tiny."""
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    gc, gk = groups["count"], groups["keep"]
    c = torch.sigmoid(x @ W[p + "router"].T) + W[p + "correction"]
    T = x.shape[0]
    cg = c.view(T, gc, E // gc)
    gscore = cg.topk(min(2, E // gc), dim=-1).values.sum(-1)
    gs = gscore.sort(dim=-1, descending=True).values
    margin = gs[:, gk - 1] - gs[:, gk] if gk < gc else torch.full((T,), math.inf, dtype=F64)
    kept = torch.zeros(T, gc, dtype=torch.bool)
    kept.scatter_(1, gscore.topk(gk, dim=-1).indices, True)
    srt = cg.masked_fill(~kept[:, :, None], -math.inf).reshape(T, E).sort(dim=-1, descending=True).values
    if top < E:
        gap = srt[:, top - 1] - srt[:, top]
        margin = torch.minimum(margin, torch.where(torch.isfinite(gap), gap, torch.full_like(gap, math.inf)))
    return margin


def experts(x, W, p, idx, w):
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for k in range(idx.shape[1]):
            e = int(idx[t, k])
            a = torch.relu(W[f"{p}e{e}.up"] @ x[t]) ** 2
            out[t] += w[t, k] * (W[f"{p}e{e}.down"] @ a)
    return out


def moe(x, W, p, m):
    idx, w = route(x, W, p, m["router"])
    return experts(x, W, p, idx, w)


class PlainSodurax:
    def __init__(self, cfg: dict, tensors: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.W = {k: v.to(F64) for k, v in tensors.items()}

    @staticmethod
    def from_dir(model_dir: str) -> "PlainSodurax":
        from gesso_b200.weights.safetensors_io import read_safetensors_file
        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
        return PlainSodurax(cfg, read_safetensors_file(os.path.join(model_dir, "model.safetensors")))

    def stream(self, tokens: List[int], margins: Optional[List[torch.Tensor]] = None) -> List[torch.Tensor]:
        """The stream after every layer run (and, into ``margins``, how clear every router's choice was)."""
        W = self.W
        h = W["embed"][torch.tensor(tokens)]
        out = []
        for i, L in enumerate(self.cfg["layers"]):
            p = f"l{L.get('weights_of', i)}."
            h = h + dyt(attention(dyt(h, W, p + "norm1"), W, p + "mix.", L["mixer"]), W, p + "norm1b")
            if L.get("mlp"):
                x = dyt(h, W, p + "norm2")
                if margins is not None:
                    margins.append(route_margin(x, W, p + "mlp.", L["mlp"]["router"]))
                h = h + dyt(moe(x, W, p + "mlp.", L["mlp"]), W, p + "norm2b")
            out.append(h)
        return out

    def margins(self, tokens: List[int]) -> torch.Tensor:
        """Per position, the least clear router choice over all layer runs."""
        m: List[torch.Tensor] = []
        self.stream(tokens, m)
        return torch.stack(m).min(dim=0).values if m else torch.full((len(tokens),), math.inf, dtype=F64)

    def logits(self, tokens: List[int]) -> torch.Tensor:
        h = self.stream(tokens)[-1]
        return dyt(h, self.W, "final.norm") @ self.W["embed"].T

    def greedy(self, prompt: List[int], n_new: int) -> List[int]:
        ids = list(prompt)
        for _ in range(n_new):
            ids.append(int(self.logits(ids)[-1].argmax()))
        return ids


# ---- random models for the tests ------------------------------------------------------------------------
def random_tensors(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Tensors under their checkpoint names, rounded to bfloat16 (so that every run type sees the same
    numbers), drawn so that nothing is flat: projections N(0, 1/fan_in) scaled up, biases and corrections
    of order 0.1 to 0.5 (some choice scores negative), norm gains near 1, alphas near 0.7."""
    g = torch.Generator().manual_seed(seed)
    W: Dict[str, torch.Tensor] = {}

    def rnd(*shape, std=1.0):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    def norm(name, width):
        W[name] = (1 + 0.2 * torch.randn(width, generator=g)).to(torch.bfloat16)
        W[name + ".b"] = rnd(width, std=0.1)
        W[name + ".alpha"] = (0.7 + 0.2 * torch.rand((), generator=g)).to(torch.bfloat16)

    Wd, V = cfg["width"], cfg["vocab"]
    W["embed"] = rnd(V, Wd, std=1.0)
    norm("final.norm", Wd)
    for i, L in enumerate(cfg["layers"]):
        if "weights_of" in L:
            continue
        p, m = f"l{i}.", L["mixer"]
        H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
        norm(p + "norm1", Wd)
        norm(p + "norm1b", Wd)
        for n, rows in (("q", H * D), ("k", G * D), ("v", G * Vd)):
            W[p + "mix." + n] = rnd(rows, Wd, std=1.5 / math.sqrt(Wd))
            W[p + "mix." + n + ".b"] = rnd(rows, std=0.3)
        W[p + "mix.g"] = rnd(H * Vd, Wd, std=1.5 / math.sqrt(Wd))
        W[p + "mix.o"] = rnd(Wd, H * Vd, std=1.5 / math.sqrt(H * Vd))
        if L.get("mlp"):
            r, F = L["mlp"]["router"], L["mlp"]["expert"]["ff"]
            norm(p + "norm2", Wd)
            norm(p + "norm2b", Wd)
            W[p + "mlp.router"] = rnd(r["experts"], Wd, std=2.0 / math.sqrt(Wd))
            W[p + "mlp.correction"] = (torch.randn(r["experts"], generator=g) * 0.5 - 0.4).to(torch.bfloat16)
            for e in range(r["experts"]):
                W[f"{p}mlp.e{e}.up"] = rnd(F, Wd, std=1.5 / math.sqrt(Wd))
                W[f"{p}mlp.e{e}.down"] = rnd(Wd, F, std=1.5 / math.sqrt(F))
    return W


def write_model(model_dir: str, cfg: dict, seed: int) -> None:
    from gesso_b200.weights.safetensors_io import write_safetensors_file
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors_file(os.path.join(model_dir, "model.safetensors"), random_tensors(cfg, seed))
