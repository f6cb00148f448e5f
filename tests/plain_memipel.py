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


def route_margin(z: torch.Tensor, top: int, groups: int, keep: int) -> float:
    """How clear the choice of one token is, in units of the router's logits: the gap between the last group that
    is kept and the first that is not, and between the last expert that is chosen and the best one that could
    have been chosen instead (softmax keeps the order of the logits, so the gaps are taken there; a run in 16
    bits may choose otherwise where this is tiny)."""
    E = z.shape[0]
    per = E // groups
    gaps = [math.inf]
    gz = torch.stack([z[g * per:(g + 1) * per].max() for g in range(groups)])
    order = gz.sort(descending=True)
    if keep < groups:
        gaps.append(float(order.values[keep - 1] - order.values[keep]))
    kept = set(order.indices[:keep].tolist())
    allowed = torch.stack([z[e] for e in range(E) if e // per in kept]).sort(descending=True).values
    if top < allowed.shape[0]:
        gaps.append(float(allowed[top - 1] - allowed[top]))
    return min(gaps)


class PlainMemipel:
    def __init__(self, cfg: dict, tensors: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.W = {k: v.to(F64) for k, v in tensors.items()}

    @staticmethod
    def from_dir(model_dir: str) -> "PlainMemipel":
        import json
        import os
        from gesso_b200.weights.safetensors_io import read_safetensors_file
        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
        return PlainMemipel(cfg, read_safetensors_file(os.path.join(model_dir, "model.safetensors")))

    def logits(self, tokens) -> torch.Tensor:
        return forward(self.cfg, self.W, tokens)

    def stream(self, tokens) -> torch.Tensor:
        return forward(self.cfg, self.W, tokens, return_layers=True)[1]

    def margins(self, tokens) -> torch.Tensor:
        """Per position, the least clear router choice over all layers with routed experts."""
        eps = float(self.cfg["norm"]["eps"])
        x = self.W["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
        layers = forward(self.cfg, self.W, tokens, return_layers=True)[1]
        out = torch.full((len(tokens),), math.inf, dtype=F64)
        for i, L in enumerate(self.cfg["layers"]):
            mlp = L.get("mlp")
            if mlp is not None and mlp["kind"] == "moe":
                n = norm_offset(x, self.W[f"l{i}.norm1"], eps)
                z = n @ self.W[f"l{i}.mlp.router"].T
                r = mlp["router"]
                groups = r["groups"]["count"] if r.get("groups") else 1
                keep = r["groups"]["keep"] if r.get("groups") else 1
                for t in range(len(tokens)):
                    out[t] = min(float(out[t]), route_margin(z[t], r["top"], groups, keep))
            x = layers[i]
        return out

    def greedy(self, prompt, n_new: int):
        ids = list(prompt)
        for _ in range(n_new):
            ids.append(int(self.logits(ids)[-1].argmax()))
        return ids


# ---- random models for the tests -----------------------------------------------------------------------
def random_tensors(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Tensors under their checkpoint names, rounded to bfloat16 (every run type sees the same numbers), drawn so
    that nothing is flat: projections N(0, 1/fan_in) scaled up, norm offsets around zero, biases, taps and sinks
    of order 0.3 to 1, mixing weights between 0.2 and 0.8."""
    g = torch.Generator().manual_seed(seed)
    W: Dict[str, torch.Tensor] = {}

    def rnd(*shape, std=1.0):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    def mat(rows, cols, gain=1.5):
        return rnd(rows, cols, std=gain / math.sqrt(cols))

    Wd, V = cfg["width"], cfg["vocab"]
    W["embed"] = rnd(V, Wd)
    W["final.norm"] = rnd(Wd, std=0.2)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        W[p + "norm1"] = rnd(Wd, std=0.2)
        H, D = m["heads"], m["dim"]
        Dv = m.get("vdim", D)
        if L["type"] == "latent_attention":
            Rq, R = m["q_rank"], m["kv_rank"]
            W[p + "mix.dq"], W[p + "mix.dkv"] = mat(Rq, Wd), mat(R, Wd)
            W[p + "mix.dq.norm"] = (1 + 0.2 * torch.randn(Rq, generator=g)).to(torch.bfloat16)
            W[p + "mix.dkv.norm"] = (1 + 0.2 * torch.randn(R, generator=g)).to(torch.bfloat16)
            W[p + "mix.uq"], W[p + "mix.uk"], W[p + "mix.uv"] = mat(H * D, Rq), mat(H * D, R), mat(H * Dv, R)
            W[p + "mix.sink"] = rnd(H, std=1.5)
            W[p + "mix.o"] = mat(Wd, H * Dv)
        elif L["type"] == "attention":
            G = m.get("kv_heads", H)
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                W[p + "mix." + n] = mat(rows, Wd)
                W[p + "mix." + n + ".b"] = rnd(rows, std=0.3)
                if m.get("conv"):
                    W[p + "mix." + n + ".conv"] = rnd(rows, m["conv"], std=0.7)
            if m.get("v_mix"):
                W[p + "mix.vmix"] = (0.2 + 0.6 * torch.rand((), generator=g)).to(torch.bfloat16)
            W[p + "mix.o"] = mat(Wd, H * Dv)
            W[p + "mix.o.b"] = rnd(Wd, std=0.3)
        else:
            W[p + "mix.q"], W[p + "mix.k"] = mat(H * D, Wd), mat(H * D, Wd)
            W[p + "mix.v"], W[p + "mix.g"] = mat(H * Dv, Wd), mat(H * Dv, Wd)
            W[p + "mix.norm"] = (1 + 0.2 * torch.randn(H * Dv, generator=g)).to(torch.bfloat16)
            W[p + "mix.o"] = mat(Wd, H * Dv)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            W[p + "mlp.up"], W[p + "mlp.down"] = mat(mlp["ff"], Wd), mat(Wd, mlp["ff"])
        else:
            F = mlp["expert"]["ff"]
            W[p + "mlp.router"] = mat(mlp["router"]["experts"], Wd, 3.0)
            names = [f"e{e}" for e in range(mlp["router"]["experts"])]
            sizes = [F] * len(names)
            if mlp.get("shared"):
                names.append("shared")
                sizes.append(mlp["shared"]["ff"])
            for n, f in zip(names, sizes):      # gains that make the clamps bite now and then
                W[f"{p}mlp.{n}.gate"], W[f"{p}mlp.{n}.up"] = mat(f, Wd, 2.0), mat(f, Wd, 2.0)
                W[f"{p}mlp.{n}.down"] = mat(Wd, f)
    return W


def write_model(model_dir: str, cfg: dict, seed: int) -> None:
    import json
    import os
    from gesso_b200.weights.safetensors_io import write_safetensors_file
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors_file(os.path.join(model_dir, "model.safetensors"), random_tensors(cfg, seed))
