"""A plain, slow Memipel in float64 on the CPU: one function per mechanism, a loop over positions where that
is the clearest way to say it.  It shares no code with the engine and is what the engine's tests compare with.

Notation: ``x`` [T, W] the residual stream of ONE sequence, ``n`` the normed rows, ``P`` a dict of the layer's
tensors by their checkpoint names without the ``l<i>.`` prefix, ``m`` the mixer's object of config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_offset(x, w, eps):
    """The layer norm of the design: the tensor holds the scale minus one."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def visible(i: int, j: int, window: Optional[int]) -> bool:
    return 0 <= i - j and (window is None or i - j < window)


# ---- mixers ------------------------------------------------------------------------------------------
def causal_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, L]: y[t] = sum_j taps[:, j] * u[t - (L - 1) + j], zeros before the start."""
    T, C = u.shape
    L = taps.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(L):
            s = t - (L - 1) + j
            if s >= 0:
                y[t] += taps[:, j] * u[s]
    return y


def softmax_rows_with_sink(scores: List[float], sink: Optional[float]) -> List[float]:
    mx = max(scores + ([sink] if sink is not None else []))
    e = [math.exp(s - mx) for s in scores]
    den = sum(e) + (math.exp(sink - mx) if sink is not None else 0.0)
    return [v / den for v in e]


def attend(q, k, v, scale: float, window: Optional[int], sink=None, slopes=None, group: int = 1):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H * Dv]; head h reads kv head h // group.
    ``sink`` [H]: one more term exp(sink_h) in the denominator.  ``slopes`` [H]: slope_h * (i - j) is taken off
    the score."""
    T, H, D = q.shape
    Dv = v.shape[2]
    out = torch.zeros((T, H, Dv), dtype=F64)
    for h in range(H):
        g = h // group
        for i in range(T):
            js = [j for j in range(T) if visible(i, j, window)]
            sc = []
            for j in js:
                s = float(q[i, h] @ k[j, g]) * scale
                if slopes is not None:
                    s -= float(slopes[h]) * (i - j)
                sc.append(s)
            p = softmax_rows_with_sink(sc, None if sink is None else float(sink[h]))
            for w, j in zip(p, js):
                out[i, h] += w * v[j, g]
    return out.reshape(T, H * Dv)


def attend_fast(q, k, v, scale, window, sink=None, slopes=None, group: int = 1):
    """The same numbers as :func:`attend` by whole matrices (for long sequences in tests)."""
    T, H, D = q.shape
    G, Dv = k.shape[1], v.shape[2]
    kk = k.repeat_interleave(group, dim=1)
    vv = v.repeat_interleave(group, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    dist = (i - j).to(F64)
    if slopes is not None:
        s = s - slopes.to(F64)[:, None, None] * dist[None]
    mask = (i - j >= 0)
    if window is not None:
        mask = mask & (i - j < window)
    s = s.masked_fill(~mask[None], -math.inf)
    if sink is not None:
        s = torch.cat([s, sink.to(F64)[:, None, None].expand(H, T, 1)], dim=2)
    p = torch.softmax(s, dim=2)[:, :, :T]
    return torch.einsum("hij,jhd->ihd", p, vv).reshape(T, H * Dv)


def alibi_slopes(H: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=F64)


def mixer_latent(n, P, m, eps, fast=True):
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    T = n.shape[0]
    cq = norm_plain(n @ P["mix.dq"].T, P["mix.dq.norm"], eps)
    q = (cq @ P["mix.uq"].T).reshape(T, H, D)
    c = norm_plain(n @ P["mix.dkv"].T, P["mix.dkv.norm"], eps)
    k = (c @ P["mix.uk"].T).reshape(T, H, D)
    v = (c @ P["mix.uv"].T).reshape(T, H, Dv)
    window = m["mask"]["size"] if m.get("mask") else None
    f = attend_fast if fast else attend
    o = f(q, k, v, float(m["scale"]), window, sink=P["mix.sink"])
    return o @ P["mix.o"].T


def mixer_attention(n, P, m, eps, shared: Dict, fast=True):
    """``shared`` carries the values of the first value-mixing layer from layer to layer."""
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = n.shape[0]
    q = n @ P["mix.q"].T + P["mix.q.b"]
    k = n @ P["mix.k"].T + P["mix.k.b"]
    v = n @ P["mix.v"].T + P["mix.v.b"]
    if m.get("conv"):
        q, k, v = causal_conv(q, P["mix.q.conv"]), causal_conv(k, P["mix.k.conv"]), causal_conv(v, P["mix.v.conv"])
    if m.get("v_mix"):
        if "v_first" not in shared:
            shared["v_first"] = v
        else:
            lam = P["mix.vmix"]
            v = (1.0 - lam) * v + lam * shared["v_first"]
    window = m["mask"]["size"] if m.get("mask") else None
    f = attend_fast if fast else attend
    o = f(q.reshape(T, H, D), k.reshape(T, G, D), v.reshape(T, G, Dv), float(m["scale"]), window,
          slopes=alibi_slopes(H), group=H // G)
    return o @ P["mix.o"].T + P["mix.o.b"]


def mixer_lightning(n, P, m, eps):
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    T = n.shape[0]
    silu = torch.nn.functional.silu
    q = silu(n @ P["mix.q"].T).reshape(T, H, D)
    k = silu(n @ P["mix.k"].T).reshape(T, H, D)
    v = silu(n @ P["mix.v"].T).reshape(T, H, Dv)
    decay = [float(d) for d in m["decay"]]
    o = torch.zeros((T, H, Dv), dtype=F64)
    for h in range(H):
        S = torch.zeros((D, Dv), dtype=F64)
        for t in range(T):
            S = decay[h] * S + torch.outer(k[t, h], v[t, h])
            o[t, h] = S.T @ q[t, h]
    y = norm_plain(o.reshape(T, H * Dv), P["mix.norm"], eps) * torch.sigmoid(n @ P["mix.g"].T)
    return y @ P["mix.o"].T


# ---- feed-forwards ------------------------------------------------------------------------------------
def ff_dense(n, P):
    return gelu_erf(n @ P["mlp.up"].T) @ P["mlp.down"].T


def expert(n, gate, up, down, limit: float):
    g = torch.clamp(n @ gate.T, max=limit)
    u = torch.clamp(n @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(z: torch.Tensor, top: int, groups: int, keep: int):
    """z [E] router logits of one token -> (chosen experts, their weights)."""
    E = z.shape[0]
    s = torch.softmax(z, dim=0)
    per = E // groups
    gscore = [float(s[g * per:(g + 1) * per].max()) for g in range(groups)]
    kept = sorted(range(groups), key=lambda g: -gscore[g])[:keep]
    allowed = [e for e in range(E) if e // per in kept]
    chosen = sorted(allowed, key=lambda e: -float(s[e]))[:top]
    return chosen, [float(s[e]) for e in chosen]


def ff_moe(n, P, mlp):
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    groups = r["groups"]["count"] if r.get("groups") else 1
    keep = r["groups"]["keep"] if r.get("groups") else 1
    limit = float(mlp["expert"]["limit"])
    z = n @ P["mlp.router"].T
    out = torch.zeros((n.shape[0], P["mlp.e0.down"].shape[0]), dtype=F64)
    for t in range(n.shape[0]):
        chosen, w = route(z[t], top, groups, keep)
        for e, we in zip(chosen, w):
            out[t] += we * expert(n[t:t + 1], P[f"mlp.e{e}.gate"], P[f"mlp.e{e}.up"], P[f"mlp.e{e}.down"], limit)[0]
    if mlp.get("shared"):
        out = out + expert(n, P["mlp.shared.gate"], P["mlp.shared.up"], P["mlp.shared.down"], float(mlp["shared"]["limit"]))
    return out


# ---- the model ---------------------------------------------------------------------------------------
def layer_tensors(tensors: Dict[str, torch.Tensor], i: int) -> Dict[str, torch.Tensor]:
    p = f"l{i}."
    return {k[len(p):]: v.to(F64) for k, v in tensors.items() if k.startswith(p)}


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens, fast=True, return_layers=False):
    """Logits [T, vocab] of one sequence (float64); with ``return_layers`` also the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    emb = tensors["embed"].to(F64)
    x = emb[torch.as_tensor(list(tokens), dtype=torch.long)]
    shared: Dict = {}
    after = []
    for i, L in enumerate(cfg["layers"]):
        P = layer_tensors(tensors, i)
        n = norm_offset(x, P["norm1"], eps)
        kind, m = L["type"], L["mixer"]
        if kind == "latent_attention":
            d = mixer_latent(n, P, m, eps, fast)
        elif kind == "attention":
            d = mixer_attention(n, P, m, eps, shared, fast)
        elif kind == "lightning":
            d = mixer_lightning(n, P, m, eps)
        else:
            raise ValueError(kind)
        mlp = L.get("mlp")
        if mlp is not None:
            d = d + (ff_dense(n, P) if mlp["kind"] == "dense" else ff_moe(n, P, mlp))
        x = x + d
        after.append(x.clone())
    logits = norm_offset(x, tensors["final.norm"].to(F64), eps) @ emb.T
    return (logits, torch.stack(after)) if return_layers else logits
