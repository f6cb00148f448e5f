"""Typed Sodurax configuration, read from the architecture's own config.json keys.

Sodurax is a decoder-only stack whose every layer norms before AND after each sublayer with
Dynamic Tanh norms (``x += norm1b(mixer(norm1(x)))``, ``x += norm2b(ff(norm2(x)))``), whose mixer is
grouped-query attention with biased projections, a partial rotary encoding with linear scaling, a
configured score scale, a sliding window that also keeps the first tokens of the sequence visible and a
sigmoid output gate, and whose feed-forward is a mixture of experts (sigmoid router with a choice
correction, group-limited top-k, squared-relu experts, weights not renormalized).  The output head is
the embedding table.  A layer may run with another layer's weights (``weights_of``) on a cache of its own.

config.json::

    {"architecture": "Sodurax", "vocab": V, "width": H, "norm": {"eps": e},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale",
                           "rot": {"base", "dims", "scaling": {"factor"}},
                           "mask": {"size", "keep_first"}},
                 "mlp": {"kind": "moe", "expert": {"ff"},
                         "router": {"experts", "top", "groups": {"count", "keep"}}} | null,
                 "weights_of": j (optional)}, ...]}

Every size and constant comes from there; nothing is assumed equal between layers.  Checkpoint names:
``embed``; ``l<i>.norm1|norm1b|norm2|norm2b`` (+ ``.b``, ``.alpha``); ``l<i>.mix.q|k|v`` (+ ``.b``),
``l<i>.mix.g``, ``l<i>.mix.o``; ``l<i>.mlp.router``, ``l<i>.mlp.correction``, ``l<i>.mlp.e<k>.up|down``;
``final.norm`` (+ ``.b``, ``.alpha``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from ..errors import invalid
from .registry import register_architecture
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Sodurax"
MODEL_TYPE = "sodurax"

GROUP_TOP = 2       # a group's score is the sum of this many of its largest choice scores (fixed by the design)


def _obj(v, what: str) -> Mapping[str, Any]:
    if not isinstance(v, Mapping):
        raise invalid(f"Sodurax config: {what} must be an object, got {v!r}")
    return v


def _int(d: Mapping[str, Any], key: str, what: str, minimum: int = 1, default: Optional[int] = None) -> int:
    if key not in d or d[key] is None:
        if default is not None:
            return default
        raise invalid(f"Sodurax config: {what} misses {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise invalid(f"Sodurax config: {what}.{key} must be an integer, got {v!r}")
    if v < minimum:
        raise invalid(f"Sodurax config: {what}.{key} must be >= {minimum}, got {v}")
    return v


def _num(d: Mapping[str, Any], key: str, what: str, default: Optional[float] = None) -> float:
    if key not in d or d[key] is None:
        if default is not None:
            return default
        raise invalid(f"Sodurax config: {what} misses {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise invalid(f"Sodurax config: {what}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class SoduraxAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int                 # 0: no rotation
    rot_base: float
    rot_factor: float             # linear scaling: every frequency is divided by it
    window: Optional[int]         # None: every earlier key is visible
    keep_first: int

    @staticmethod
    def from_json(m: Mapping[str, Any], what: str) -> "SoduraxAttention":
        heads, kv = _int(m, "heads", what), _int(m, "kv_heads", what)
        if heads % kv != 0:
            raise invalid(f"Sodurax config: {what}: {heads} heads are not a multiple of {kv} kv_heads")
        dim = _int(m, "dim", what, 2)
        if dim % 2 != 0:
            raise invalid(f"Sodurax config: {what}.dim {dim} must be even")
        vdim = _int(m, "vdim", what, 1, default=dim)
        scale = _num(m, "scale", what, default=float(dim) ** -0.5)
        rot_dims, base, factor = 0, 10000.0, 1.0
        if m.get("rot") is not None:
            rot = _obj(m["rot"], what + ".rot")
            rot_dims = _int(rot, "dims", what + ".rot", 2)
            if rot_dims % 2 != 0 or rot_dims > dim:
                raise invalid(f"Sodurax config: {what}.rot.dims {rot_dims} must be even and at most dim {dim}")
            base = _num(rot, "base", what + ".rot")
            if rot.get("scaling") is not None:
                factor = _num(_obj(rot["scaling"], what + ".rot.scaling"), "factor", what + ".rot.scaling")
            if not (base > 0 and factor > 0):
                raise invalid(f"Sodurax config: {what}.rot: base and scaling factor must be positive")
        window, keep = None, 0
        if m.get("mask") is not None:
            mask = _obj(m["mask"], what + ".mask")
            window = _int(mask, "size", what + ".mask")
            keep = _int(mask, "keep_first", what + ".mask", 0, default=0)
        return SoduraxAttention(heads, kv, dim, vdim, scale, rot_dims, base, factor, window, keep)


@dataclass(frozen=True)
class SoduraxMoE:
    ff: int
    experts: int
    top: int
    groups: int
    keep_groups: int

    @staticmethod
    def from_json(m: Mapping[str, Any], what: str) -> "SoduraxMoE":
        kind = m.get("kind", "moe")
        if kind != "moe":
            raise invalid(f"Sodurax config: {what}.kind {kind!r}; known kinds: ['moe']")
        ff = _int(_obj(m.get("expert"), what + ".expert"), "ff", what + ".expert")
        r = _obj(m.get("router"), what + ".router")
        experts, top = _int(r, "experts", what + ".router"), _int(r, "top", what + ".router")
        groups, keep = 1, 1
        if r.get("groups") is not None:
            g = _obj(r["groups"], what + ".router.groups")
            groups = _int(g, "count", what + ".router.groups")
            keep = _int(g, "keep", what + ".router.groups", default=groups)
        if experts % groups != 0:
            raise invalid(f"Sodurax config: {what}: {experts} experts do not form {groups} equal groups")
        if keep > groups or top > (experts // groups) * keep:
            raise invalid(f"Sodurax config: {what}: {keep} of {groups} groups cannot give {top} experts")
        return SoduraxMoE(ff, experts, top, groups, keep)


@dataclass(frozen=True)
class SoduraxLayer:
    mixer: SoduraxAttention
    mlp: Optional[SoduraxMoE]
    weights_of: Optional[int]       # the layer whose tensors this one runs with (resolved: that layer owns them)


@dataclass(frozen=True)
class SoduraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[SoduraxLayer, ...]
    raw: Any = None

    @staticmethod
    def from_json(cfg: Mapping[str, Any]) -> "SoduraxConfig":
        vocab, width = _int(cfg, "vocab", "config"), _int(cfg, "width", "config")
        eps = _num(_obj(cfg.get("norm", {}), "norm"), "eps", "norm", default=1e-6)   # the norm of this design has no eps in its formula
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise invalid("Sodurax config: 'layers' must be a non-empty list")
        layers: List[SoduraxLayer] = []
        for i, L in enumerate(raw_layers):
            L = _obj(L, f"layers[{i}]")
            kind = L.get("type")
            if kind != "attention":
                raise invalid(f"Sodurax config: layers[{i}].type {kind!r}; known mixers: ['attention']")
            mixer = SoduraxAttention.from_json(_obj(L.get("mixer"), f"layers[{i}].mixer"), f"layers[{i}].mixer")
            mlp = None if L.get("mlp") is None else SoduraxMoE.from_json(_obj(L["mlp"], f"layers[{i}].mlp"),
                                                                         f"layers[{i}].mlp")
            wo = L.get("weights_of")
            if wo is not None:
                if isinstance(wo, bool) or not isinstance(wo, int) or not (0 <= wo < len(raw_layers)) or wo == i:
                    raise invalid(f"Sodurax config: layers[{i}].weights_of must name another layer, got {wo!r}")
            layers.append(SoduraxLayer(mixer, mlp, wo))
        # a layer may name a layer that itself borrows: follow to the owner
        resolved = []
        for i, L in enumerate(layers):
            j, seen = L.weights_of, {i}
            while j is not None and layers[j].weights_of is not None:
                if j in seen:
                    raise invalid(f"Sodurax config: layers[{i}].weights_of runs in a circle")
                seen.add(j)
                j = layers[j].weights_of
            resolved.append(SoduraxLayer(L.mixer, L.mlp, j))
        for i, L in enumerate(resolved):
            if L.weights_of is not None:
                o = resolved[L.weights_of]
                if (o.mlp is None) != (L.mlp is None):
                    raise invalid(f"Sodurax config: layers[{i}] borrows the tensors of layer {L.weights_of}, which "
                                  "has another set of sublayers")
        return SoduraxConfig(vocab, width, eps, tuple(resolved), raw=dict(cfg))

    def to_json(self) -> dict:
        if self.raw is not None:
            return dict(self.raw)
        raise invalid("Sodurax config: no source object to write")

    # ---- the model this configuration describes ---------------------------------------
    def _mixer_spec(self, a: SoduraxAttention) -> PartSpec:
        position = (PartSpec("rope", {"theta": a.rot_base, "rotary_dim": a.rot_dims, "scaling_factor": a.rot_factor})
                    if a.rot_dims else PartSpec("none", {}))
        return PartSpec("gqa_attention", {
            "hidden_size": self.width, "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim,
            "v_head_dim": a.vdim, "qk_norm_eps": None, "window": a.window, "keep_first": a.keep_first,
            "scale": a.scale, "qkv_bias": True, "output_gate": True, "f32_output": True, "f32_weights": True,
            "position": position})

    def _mlp_spec(self, m: SoduraxMoE) -> PartSpec:
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "ff_dim": m.ff, "n_experts": m.experts, "top_k": m.top,
            "n_groups": m.groups, "keep_groups": m.keep_groups, "group_top": GROUP_TOP, "score": "sigmoid",
            "correction": True, "renormalize": False, "activation": "relu2"})

    def to_spec(self) -> ModelSpec:
        norm = PartSpec("dyt", {"size": self.width, "bias": True})
        names: Dict[str, Tuple[str, ...]] = {"embedding.weight": ("embed",)}
        for ours, theirs in (("weight", ""), ("bias", ".b"), ("alpha", ".alpha")):
            names[f"final_norm.{ours}"] = ("final.norm" + theirs,)
        blocks: List[BlockSpec] = []
        block_of: Dict[int, int] = {}      # config layer -> index into blocks
        schedule: List[ScheduleEntry] = []

        def add_block(i: int, src: int) -> int:
            """A block with layer i's sizes whose tensors carry layer src's checkpoint names."""
            L = self.layers[i]
            p, ck = f"layers.{i}.", f"l{src}."
            has_ff = L.mlp is not None
            blocks.append(BlockSpec("sandwich", self._mixer_spec(L.mixer), self._mlp_spec(L.mlp) if has_ff else None,
                                    norm, norm if has_ff else None, p, mixer_post_norm=norm,
                                    ff_post_norm=norm if has_ff else None))
            norms = [("mixer_norm", "norm1"), ("mixer_post_norm", "norm1b")]
            if has_ff:
                norms += [("ff_norm", "norm2"), ("ff_post_norm", "norm2b")]
            for ours, theirs in norms:
                names[p + ours + ".weight"] = (ck + theirs,)
                names[p + ours + ".bias"] = (ck + theirs + ".b",)
                names[p + ours + ".alpha"] = (ck + theirs + ".alpha",)
            for ours, theirs in (("q_proj", "q"), ("k_proj", "k"), ("v_proj", "v")):
                names[p + f"mixer.{ours}.weight"] = (ck + "mix." + theirs,)
                names[p + f"mixer.{ours}.bias"] = (ck + "mix." + theirs + ".b",)
            names[p + "mixer.g_proj.weight"] = (ck + "mix.g",)
            names[p + "mixer.o_proj.weight"] = (ck + "mix.o",)
            if has_ff:
                names[p + "feed_forward.router.weight"] = (ck + "mlp.router",)
                names[p + "feed_forward.correction"] = (ck + "mlp.correction",)
                for e in range(L.mlp.experts):
                    names[p + f"feed_forward.experts.{e}.up.weight"] = (ck + f"mlp.e{e}.up",)
                    names[p + f"feed_forward.experts.{e}.down.weight"] = (ck + f"mlp.e{e}.down",)
            return len(blocks) - 1

        for i, L in enumerate(self.layers):
            if L.weights_of is None:
                block_of[i] = add_block(i, i)
        for i, L in enumerate(self.layers):
            if L.weights_of is None:
                schedule.append(ScheduleEntry(block_of[i]))
                continue
            o = self.layers[L.weights_of]
            if (o.mixer, o.mlp) == (L.mixer, L.mlp):
                schedule.append(ScheduleEntry(block_of[L.weights_of]))     # the same bound parts, a cache of its own
            else:
                # other constants on the same tensors (another window, say): parts of its own, bound to
                # the owner's checkpoint tensors
                schedule.append(ScheduleEntry(add_block(i, L.weights_of)))
        # a layer without a feed-forward may still carry the unused norms in a checkpoint
        ignorable = tuple(rf"^l{i}\.norm2b?(\.b|\.alpha)?$" for i, L in enumerate(self.layers) if L.mlp is None)
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width,
            blocks=tuple(blocks), schedule=tuple(schedule), final_norm=norm, tie_embedding=True,
            tensor_names=names, ignorable_tensors=ignorable, source=self)


def sodurax_adapter(cfg: Mapping[str, Any]) -> ModelSpec:
    return SoduraxConfig.from_json(cfg).to_spec()


sodurax_adapter.model_type = MODEL_TYPE
register_architecture(ARCHITECTURE, sodurax_adapter, replace=True)
