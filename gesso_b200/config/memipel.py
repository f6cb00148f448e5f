"""Typed Memipel configuration, read from the architecture's own config.json keys.

Memipel is a decoder-only stack of *parallel* layers: one RMS norm per layer (its weight tensor holds the offset from one: scale
``1 + w``) whose output both the mixer and the feed-forward read, ``x += mixer(n) + ff(n)``.  A layer's mixer is one
of three kinds, chosen per layer by ``type``:

* ``latent_attention``: queries and keys/values through low-rank latents, no positions, a sliding window and a
  learned sink per head in the softmax denominator; only the key/value latent is cached;
* ``attention``: grouped-query attention with biased projections, a short causal convolution over time on q, k and
  v, a linear distance bias per head instead of a rotation, a sliding window, and value mixing: the earliest layer
  that mixes is the source, every later one blends its own values of a token with the source's for that token;
* ``lightning``: linear attention with a fixed decay per head, a float32 state per request, a norm over the
  concatenated heads and a sigmoid gate.

The feed-forward is dense (exact gelu between two matrices), a mixture of experts (softmax router, group-limited
top-k with a group scored by its best expert, weights not renormalized, experts and a shared expert that are gated
units with clamped inputs), or absent.  The output head is the embedding table behind the model's norm.

config.json::

    {"architecture": "Memipel", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "latent_attention", "mixer": {"heads", "dim", "vdim", "q_rank", "kv_rank", "scale",
                                                        "mask": {"size"}},
                 "mlp": {...} | null},
                {"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "conv", "v_mix",
                                                 "mask": {"size"}}, "mlp": ...},
                {"type": "lightning", "mixer": {"heads", "dim", "vdim", "decay": [per head]}, "mlp": ...}]}
    mlp: {"kind": "dense", "ff"}  |  {"kind": "moe", "expert": {"ff", "limit"},
                                      "router": {"experts", "top", "groups": {"count", "keep"}},
                                      "shared": {"ff", "limit"}}

Every size and constant comes from there; nothing is assumed equal between layers.  Checkpoint names: ``embed``,
``final.norm``, ``l<i>.norm1``, ``l<i>.mix.*`` and ``l<i>.mlp.*`` (see ``to_spec``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from ..errors import invalid
from .registry import register_architecture
from .spec import BlockSpec, ModelSpec, PartSpec, default_schedule

ARCHITECTURE = "Memipel"
MODEL_TYPE = "memipel"

DISTANCE_BIAS = 8.0      # head h of H takes slope 2 ** (-8 (h + 1) / H) off the score per position of distance
GROUP_TOP = 1            # a group of experts is scored by its single best expert


def _obj(v, what: str) -> Mapping[str, Any]:
    if not isinstance(v, Mapping):
        raise invalid(f"Memipel config: {what} must be an object, got {v!r}")
    return v


def _int(d: Mapping[str, Any], key: str, what: str, minimum: int = 1, default: Optional[int] = None) -> int:
    if key not in d or d[key] is None:
        if default is not None:
            return default
        raise invalid(f"Memipel config: {what} misses {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise invalid(f"Memipel config: {what}.{key} must be an integer, got {v!r}")
    if v < minimum:
        raise invalid(f"Memipel config: {what}.{key} must be >= {minimum}, got {v}")
    return v


def _num(d: Mapping[str, Any], key: str, what: str, default: Optional[float] = None) -> float:
    if key not in d or d[key] is None:
        if default is not None:
            return default
        raise invalid(f"Memipel config: {what} misses {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise invalid(f"Memipel config: {what}.{key} must be a number, got {v!r}")
    return float(v)


def _window(m: Mapping[str, Any], what: str) -> Optional[int]:
    if m.get("mask") is None:
        return None
    return _int(_obj(m["mask"], what + ".mask"), "size", what + ".mask")


@dataclass(frozen=True)
class MemipelLatent:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int]

    @staticmethod
    def from_json(m, what):
        dim = _int(m, "dim", what)
        return MemipelLatent(_int(m, "heads", what), dim, _int(m, "vdim", what, default=dim), _int(m, "q_rank", what),
                             _int(m, "kv_rank", what), _num(m, "scale", what, default=float(dim) ** -0.5),
                             _window(m, what))


@dataclass(frozen=True)
class MemipelAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: Optional[int]
    window: Optional[int]
    v_mix: bool

    @staticmethod
    def from_json(m, what):
        heads = _int(m, "heads", what)
        kv = _int(m, "kv_heads", what, default=heads)
        if heads % kv != 0:
            raise invalid(f"Memipel config: {what}: {heads} heads are not a multiple of {kv} kv_heads")
        dim = _int(m, "dim", what)
        conv = None if m.get("conv") is None else _int(m, "conv", what)
        v_mix = m.get("v_mix", False)
        if not isinstance(v_mix, bool):
            raise invalid(f"Memipel config: {what}.v_mix must be true or false, got {v_mix!r}")
        return MemipelAttention(heads, kv, dim, _int(m, "vdim", what, default=dim),
                                _num(m, "scale", what, default=float(dim) ** -0.5), conv, _window(m, what), v_mix)


@dataclass(frozen=True)
class MemipelLightning:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    @staticmethod
    def from_json(m, what):
        heads, dim = _int(m, "heads", what), _int(m, "dim", what)
        decay = m.get("decay")
        if isinstance(decay, (int, float)) and not isinstance(decay, bool):
            decay = [decay] * heads                      # one number for all heads
        if not isinstance(decay, list) or len(decay) != heads or \
                any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
            raise invalid(f"Memipel config: {what}.decay must list one number per head")
        return MemipelLightning(heads, dim, _int(m, "vdim", what, default=dim), tuple(float(d) for d in decay))


@dataclass(frozen=True)
class MemipelDense:
    ff: int


@dataclass(frozen=True)
class MemipelMoE:
    ff: int
    limit: float
    experts: int
    top: int
    groups: int
    keep_groups: int
    shared_ff: Optional[int]
    shared_limit: float

    @staticmethod
    def from_json(m, what):
        ex = _obj(m.get("expert"), what + ".expert")
        r = _obj(m.get("router"), what + ".router")
        experts, top = _int(r, "experts", what + ".router"), _int(r, "top", what + ".router")
        groups, keep = 1, 1
        if r.get("groups") is not None:
            g = _obj(r["groups"], what + ".router.groups")
            groups = _int(g, "count", what + ".router.groups")
            keep = _int(g, "keep", what + ".router.groups", default=groups)
        if experts % groups != 0:
            raise invalid(f"Memipel config: {what}: {experts} experts do not form {groups} equal groups")
        if keep > groups or top > (experts // groups) * keep:
            raise invalid(f"Memipel config: {what}: {keep} of {groups} groups cannot give {top} experts")
        shared_ff, shared_limit = None, 0.0
        if m.get("shared") is not None:
            sh = _obj(m["shared"], what + ".shared")
            shared_ff, shared_limit = _int(sh, "ff", what + ".shared"), _num(sh, "limit", what + ".shared")
        return MemipelMoE(_int(ex, "ff", what + ".expert"), _num(ex, "limit", what + ".expert"), experts, top, groups,
                          keep, shared_ff, shared_limit)


def _mlp_from_json(m, what):
    if m is None:
        return None
    m = _obj(m, what)
    kind = m.get("kind")
    if kind == "dense":
        return MemipelDense(_int(m, "ff", what))
    if kind == "moe":
        return MemipelMoE.from_json(m, what)
    raise invalid(f"Memipel config: {what}.kind {kind!r}; known kinds: ['dense', 'moe']")


MIXERS = {"latent_attention": MemipelLatent, "attention": MemipelAttention, "lightning": MemipelLightning}


@dataclass(frozen=True)
class MemipelLayer:
    kind: str
    mixer: Any
    mlp: Any


@dataclass(frozen=True)
class MemipelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[MemipelLayer, ...]
    raw: Any = None

    @staticmethod
    def from_json(cfg: Mapping[str, Any]) -> "MemipelConfig":
        vocab, width = _int(cfg, "vocab", "config"), _int(cfg, "width", "config")
        eps = _num(_obj(cfg.get("norm"), "norm"), "eps", "norm")
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise invalid("Memipel config: 'layers' must be a non-empty list")
        layers: List[MemipelLayer] = []
        for i, L in enumerate(raw_layers):
            L = _obj(L, f"layers[{i}]")
            kind = L.get("type")
            if kind not in MIXERS:
                raise invalid(f"Memipel config: layers[{i}].type {kind!r}; known mixers: {sorted(MIXERS)}")
            mixer = MIXERS[kind].from_json(_obj(L.get("mixer"), f"layers[{i}].mixer"), f"layers[{i}].mixer")
            layers.append(MemipelLayer(kind, mixer, _mlp_from_json(L.get("mlp"), f"layers[{i}].mlp")))
        mixing = [L.mixer for L in layers if L.kind == "attention" and L.mixer.v_mix]
        if len({a.kv_heads * a.vdim for a in mixing}) > 1:
            raise invalid("Memipel config: layers that mix values must have values of one width (kv_heads * vdim)")
        return MemipelConfig(vocab, width, eps, tuple(layers), raw=dict(cfg))

    def to_json(self) -> dict:
        if self.raw is not None:
            return dict(self.raw)
        raise invalid("Memipel config: no source object to write")

    # ---- the model this configuration describes ---------------------------------------------------
    def _mixer_spec(self, L: MemipelLayer, mix_role: Optional[str]) -> PartSpec:
        m = L.mixer
        if L.kind == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": self.width, "n_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "window": m.window, "sink": True,
                "norm_eps": self.norm_eps})
        if L.kind == "attention":
            return PartSpec("gqa_attention", {
                "hidden_size": self.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim,
                "v_head_dim": m.vdim, "qk_norm_eps": None, "window": m.window, "scale": m.scale, "qkv_bias": True,
                "o_bias": True, "f32_output": True, "conv_taps": m.conv, "distance_bias": DISTANCE_BIAS,
                "value_mix": mix_role, "position": PartSpec("none", {})})
        return PartSpec("lightning_attention", {
            "hidden_size": self.width, "n_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim,
            "decay": m.decay, "norm_eps": self.norm_eps})

    def _mlp_spec(self, mlp) -> Optional[PartSpec]:
        if mlp is None:
            return None
        if isinstance(mlp, MemipelDense):
            return PartSpec("mlp", {"hidden_size": self.width, "ff_dim": mlp.ff, "activation": "gelu_erf"})
        shared = None
        if mlp.shared_ff is not None:
            shared = PartSpec("glu_clamped", {"hidden_size": self.width, "ff_dim": mlp.shared_ff,
                                              "limit": mlp.shared_limit})
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "ff_dim": mlp.ff, "n_experts": mlp.experts, "top_k": mlp.top,
            "n_groups": mlp.groups, "keep_groups": mlp.keep_groups, "group_top": GROUP_TOP, "score": "softmax",
            "correction": False, "renormalize": False, "activation": "glu_clamped", "limit": mlp.limit,
            "shared": shared})

    def to_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "unit_offset": True})
        names: Dict[str, Tuple[str, ...]] = {"embedding.weight": ("embed",), "final_norm.weight": ("final.norm",)}
        blocks: List[BlockSpec] = []
        seen_mix = False
        for i, L in enumerate(self.layers):
            p, ck = f"layers.{i}.", f"l{i}."
            role = None
            if L.kind == "attention" and L.mixer.v_mix:
                role, seen_mix = ("mix" if seen_mix else "source"), True
            blocks.append(BlockSpec("parallel", self._mixer_spec(L, role), self._mlp_spec(L.mlp), norm, None, p))
            names[p + "mixer_norm.weight"] = (ck + "norm1",)
            mx = p + "mixer."
            if L.kind == "latent_attention":
                for ours, theirs in (("dq.weight", "dq"), ("dq_norm.weight", "dq.norm"), ("uq.weight", "uq"),
                                     ("dkv.weight", "dkv"), ("dkv_norm.weight", "dkv.norm"), ("uk.weight", "uk"),
                                     ("uv.weight", "uv"), ("sink", "sink"), ("o_proj.weight", "o")):
                    names[mx + ours] = (ck + "mix." + theirs,)
            elif L.kind == "attention":
                for t in ("q", "k", "v"):
                    names[mx + f"{t}_proj.weight"] = (ck + f"mix.{t}",)
                    names[mx + f"{t}_proj.bias"] = (ck + f"mix.{t}.b",)
                    names[mx + f"{t}_conv.weight"] = (ck + f"mix.{t}.conv",)
                names[mx + "value_mix.weight"] = (ck + "mix.vmix",)
                names[mx + "o_proj.weight"] = (ck + "mix.o",)
                names[mx + "o_proj.bias"] = (ck + "mix.o.b",)
            else:
                for t in ("q", "k", "v", "g", "o"):
                    names[mx + f"{t}_proj.weight"] = (ck + f"mix.{t}",)
                names[mx + "norm.weight"] = (ck + "mix.norm",)
            ff = p + "feed_forward."
            if isinstance(L.mlp, MemipelDense):
                names[ff + "up.weight"] = (ck + "mlp.up",)
                names[ff + "down.weight"] = (ck + "mlp.down",)
            elif isinstance(L.mlp, MemipelMoE):
                names[ff + "router.weight"] = (ck + "mlp.router",)
                for e in range(L.mlp.experts):
                    for t in ("gate", "up", "down"):
                        names[ff + f"experts.{e}.{t}.weight"] = (ck + f"mlp.e{e}.{t}",)
                if L.mlp.shared_ff is not None:
                    for t in ("gate", "up", "down"):
                        names[ff + f"shared.{t}.weight"] = (ck + f"mlp.shared.{t}",)
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks),
            schedule=default_schedule(len(blocks)), final_norm=norm, tie_embedding=True, tensor_names=names,
            source=self)


def memipel_adapter(cfg: Mapping[str, Any]) -> ModelSpec:
    return MemipelConfig.from_json(cfg).to_spec()


memipel_adapter.model_type = MODEL_TYPE
register_architecture(ARCHITECTURE, memipel_adapter, replace=True)
