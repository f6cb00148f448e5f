"""Grouped-query attention over the paged cache, with per-head q/k RMSNorm and a position part.

``q = x Wq^T`` (nh heads), ``k, v = x Wk^T, x Wv^T`` (nkv heads), features head-major
(src/Inference/Inference.jl:1573-1583).  q and k are normed per head over ``head_dim``
before the rotation (:2401-2416); the cache holds normed, rotated K and raw V (:2417-2421).
Scores are ``q.k / sqrt(head_dim)`` (:1201-1205), causal, optionally limited to the last
``window`` positions (:1206-1207); query head h reads kv head ``h // (nh/nkv)`` (:1398).
``out = merge(heads) Wo^T`` (:2494, 2508).

Parameters (all from the part spec): hidden_size, n_heads, n_kv_heads, head_dim,
qk_norm_eps (``None``: no q/k norm), window (``None``: all keys), position (a position
part spec).  The three projections are fused into one matrix at bind time.

Options, all off by default, each a parameter so that any architecture can turn it on:
``v_head_dim`` (values of another width than queries and keys; the output projection then reads
``n_heads * v_head_dim`` features); ``qkv_bias`` (bias vectors ``q_proj.bias``, ``k_proj.bias``,
``v_proj.bias``, added in the projection, before rotation); ``scale`` (the score scale, instead of
``1/sqrt(head_dim)``); ``keep_first`` (with a window: position i sees j if ``j <= i`` and
``(i - j < window or j < keep_first)``; the kept tokens keep their true positions for the rotation,
and the cache manager keeps their pages); ``output_gate`` (a fourth projection ``g_proj`` of the
mixer's input, ``n_heads * v_head_dim`` wide: the concatenated heads are multiplied element by
element with ``sigmoid(g)`` before the output projection; it rides in the fused matrix and the
attention kernels apply it as they store); ``f32_output`` (the output projection's result in
float32, for arrangements that norm it before the add); ``f32_weights`` (the softmax weights act
on the values in 32-bit precision: the tensor-core kernels then feed each weight to the product
as two bfloat16 pieces); ``conv_taps`` (a short causal convolution over time on every channel of q, k and v,
directly behind the projection and its bias: tensors ``q_conv.weight`` [channels, taps] and likewise for k and v,
no bias; the last ``taps - 1`` projected rows of a request are a float32 state beside its pages); ``distance_bias``
(a number b: ``slope_h * (i - j)`` with ``slope_h = 2 ** (-b * (h + 1) / n_heads)`` is taken off the score of key
j for the query at i); ``value_mix`` (``"source"``: this layer's values, as they go into the cache, are left for
later layers of the step; ``"mix"``: ``v <- (1 - lambda) v + lambda v_source`` with the scalar tensor
``value_mix.weight`` and the source layer's values of the same token, before v is cached; both declare the tensor);
``o_bias`` (a bias vector ``o_proj.bias`` on the output projection).  A layer with ``conv_taps``, ``distance_bias``
or ``value_mix`` does not rotate (its position part must be ``none``).
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from .. import ops
from ..errors import invalid
from .base import Mixer, PagedNeed, ParamDecl, StateNeed
from .registry import build_position, register_mixer


class GQAttention(Mixer):
    accepts_lazy_norm = True
    fuses_residual = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["n_heads"])
        self.nkv = int(spec["n_kv_heads"])
        self.hd = int(spec["head_dim"])
        self.eps = spec.get("qk_norm_eps")
        self.window = spec.get("window")
        self.vd = int(spec.get("v_head_dim") or self.hd)
        self.qkv_bias = bool(spec.get("qkv_bias", False))
        self.output_gate = bool(spec.get("output_gate", False))
        self.keep_first = int(spec.get("keep_first") or 0)
        self.f32_output = bool(spec.get("f32_output", False))
        self.f32_weights = bool(spec.get("f32_weights", False))
        self.conv_taps = spec.get("conv_taps")
        self.distance_bias = spec.get("distance_bias")
        self.value_mix = spec.get("value_mix")
        self.o_bias = bool(spec.get("o_bias", False))
        if self.conv_taps is not None and not (1 <= int(self.conv_taps) <= 8):
            raise invalid(f"attention: conv_taps {self.conv_taps} must be between 1 and 8")
        if self.value_mix not in (None, "source", "mix"):
            raise invalid(f"attention: value_mix {self.value_mix!r}; known: 'source', 'mix'")
        # the projection's rows pass through a kernel of their own (bias, convolution, value mixing) before
        # they are cached
        self.row_pass = self.conv_taps is not None or self.value_mix is not None
        if (self.row_pass or self.distance_bias is not None) and spec["position"].kind != "none":
            raise invalid("attention: conv_taps, distance_bias and value_mix go with the position part 'none'")
        if (self.row_pass or self.distance_bias is not None or self.o_bias) and \
                (self.output_gate or self.eps is not None):
            raise invalid("attention: conv_taps, distance_bias, value_mix and o_bias do not combine with an output "
                          "gate or per-head q/k norms")
        if self.vd < 1 or self.vd > 256:
            raise invalid(f"attention: v_head_dim {self.vd} must be between 1 and 256")
        if self.keep_first < 0:
            raise invalid("attention: keep_first must be >= 0")
        if self.nh < 1 or self.nkv < 1 or self.nh % self.nkv != 0:
            raise invalid(f"attention: {self.nh} heads are not a multiple of {self.nkv} kv heads")
        rotates_or_norms = spec["position"].kind != "none" or self.eps is not None
        if self.hd < 1 or self.hd > 256 or (rotates_or_norms and self.hd % 2 != 0):
            raise invalid(f"attention: head_dim {self.hd} must be at most 256, and even where heads are rotated or normed")
        if self.window is not None and int(self.window) < 1:
            raise invalid("attention: window must be >= 1")
        self.position = build_position(spec["position"])
        self.position.check_head_dim(self.hd)
        # 1/sqrt(hd) rounded once from float64 (exact when sqrt(hd) is a power of two,
        # src/Inference/Inference.jl:1209-1232)
        self.scale = 1.0 / math.sqrt(self.hd) if spec.get("scale") is None else float(spec["scale"])

    def param_decls(self) -> Dict[str, ParamDecl]:
        q, kv, v, o = self.nh * self.hd, self.nkv * self.hd, self.nkv * self.vd, self.nh * self.vd
        d = {
            "q_proj.weight": ParamDecl((q, self.hidden), fan_in=self.hidden),
            "k_proj.weight": ParamDecl((kv, self.hidden), fan_in=self.hidden),
            "v_proj.weight": ParamDecl((v, self.hidden), fan_in=self.hidden),
            "o_proj.weight": ParamDecl((self.hidden, o), fan_in=o),
        }
        if self.qkv_bias:
            d["q_proj.bias"] = ParamDecl((q,), role="vector", init="zeros")
            d["k_proj.bias"] = ParamDecl((kv,), role="vector", init="zeros")
            d["v_proj.bias"] = ParamDecl((v,), role="vector", init="zeros")
        if self.output_gate:
            d["g_proj.weight"] = ParamDecl((o, self.hidden), fan_in=self.hidden)
        if self.conv_taps is not None:
            L = int(self.conv_taps)
            d["q_conv.weight"] = ParamDecl((q, L), role="vector", fan_in=L)
            d["k_conv.weight"] = ParamDecl((kv, L), role="vector", fan_in=L)
            d["v_conv.weight"] = ParamDecl((v, L), role="vector", fan_in=L)
        if self.value_mix is not None:
            d["value_mix.weight"] = ParamDecl((), role="vector", init="zeros", alt_shapes=((1,),))
        if self.o_bias:
            d["o_proj.bias"] = ParamDecl((self.hidden,), role="vector", init="zeros")
        if self.eps is not None:
            d["q_norm.weight"] = ParamDecl((self.hd,), role="vector", init="ones")
            d["k_norm.weight"] = ParamDecl((self.hd,), role="vector", init="ones")
        return d

    def cache_need(self):
        windowed = self.window is not None
        pages = PagedNeed(self.nkv, self.hd, int(self.window) if windowed else None,
                          self.keep_first if windowed else 0, None if self.vd == self.hd else self.vd)
        if self.conv_taps is not None and int(self.conv_taps) > 1:
            # the last taps - 1 projected rows (q, k and v channels side by side), float32
            return [pages, StateNeed((int(self.conv_taps) - 1, self._channels()))]
        return pages

    def _channels(self) -> int:
        return (self.nh + self.nkv) * self.hd + self.nkv * self.vd

    def bind(self, tensors, rt) -> None:
        ws = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        gate = [tensors["g_proj.weight"]] if self.output_gate else []
        common = torch.float32 if any(w.dtype == torch.float32 for w in ws + gate) else ws[0].dtype
        # the fused rows: q heads, k heads, v heads, then the gate's columns; an entry that reads another
        # entry's cache projects q (and the gate) only
        self.w_q = torch.cat([w.to(common) for w in ws[:1] + gate], dim=0).contiguous()
        self.w_qkv = torch.cat([w.to(common) for w in ws + gate], dim=0).contiguous()
        self.b_q = self.b_qkv = None
        if self.qkv_bias:
            bs = [tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]]
            self.b_q = bs[0].float().contiguous()
            self.b_qkv = torch.cat([b.float() for b in bs]).contiguous()
        self.w_o = tensors["o_proj.weight"]
        self.b_o = tensors["o_proj.bias"].float().contiguous() if self.o_bias else None
        self.taps = self.slopes = None
        self.mix_lambda = 0.0
        if self.row_pass:
            C = self._channels()
            if self.conv_taps is not None:
                self.taps = torch.cat([tensors["q_conv.weight"], tensors["k_conv.weight"],
                                       tensors["v_conv.weight"]], dim=0).float().contiguous()
            else:                                       # no convolution: one tap of weight one
                self.taps = torch.ones((C, 1), dtype=torch.float32, device=rt.device)
            if self.value_mix == "mix":
                self.mix_lambda = float(tensors["value_mix.weight"].reshape(-1)[0].item())
        if self.distance_bias is not None:
            b = float(self.distance_bias)
            self.slopes = torch.tensor([2.0 ** (-b * (h + 1) / self.nh) for h in range(self.nh)],
                                       dtype=torch.float64).to(device=rt.device, dtype=torch.float32)
        self.q_norm = tensors.get("q_norm.weight")
        self.k_norm = tensors.get("k_norm.weight")
        self.position.bind({}, rt)
        self.rt = rt

    def fold_input_scale(self, scale) -> bool:
        self.w_q = ops.fold_norm_weight(self.w_q, scale)
        self.w_qkv = ops.fold_norm_weight(self.w_qkv, scale)
        return True

    def _row_pass(self, qkv, ctx, conv_state):
        """Bias, convolution over time and value mixing on the fused projection's rows (one kernel)."""
        v0, nv = (self.nh + self.nkv) * self.hd, self.nkv * self.vd
        mix = None
        if self.value_mix == "mix":
            first = ctx.shared.get("attention.value_mix.source")
            if first is None or first.shape[1] != nv:
                raise invalid("attention: value_mix 'mix' needs an earlier 'source' layer with values of the same width")
            mix = (first, v0, nv, self.mix_lambda)
        if conv_state is None:       # a single tap keeps no history
            state = torch.empty((1, 0, self._channels()), dtype=torch.float32, device=qkv.device)
            slots = ctx.slots
        else:
            state, slots = conv_state.state, conv_state.slots
        y = ops.causal_conv(qkv, self._channels(), self.b_qkv, self.taps, state, ctx.seg_of_token, ctx.seg_start,
                            slots, ctx.n_segs, mix)
        if self.value_mix == "source":
            ctx.shared["attention.value_mix.source"] = y[:, v0:v0 + nv]
        return y

    def forward(self, x, ctx, cache, residual=None):
        conv_state = None
        if isinstance(cache, tuple):
            cache, conv_state = cache
        writes = cache.writes
        if self.row_pass and not writes:
            raise invalid("attention: a layer with conv_taps or value_mix owns its cache")
        qkv = ops.linear(x, self.w_qkv if writes else self.w_q, out_dtype=x.dtype)
        bias = self.b_qkv if writes else self.b_q
        if self.row_pass:
            qkv, bias = self._row_pass(qkv, ctx, conv_state), None
        cos, sin = self.position.tables()
        # a position part without layout() rotates the whole head by halves
        rot_dim, interleaved = self.position.layout() if hasattr(self.position, "layout") else (self.hd, False)
        q = ops.qk_norm_rope_store(qkv, self.q_norm, self.k_norm, self.eps if self.eps is not None else 0.0,
                                   cos, sin, ctx.positions, ctx.seg_of_token, cache.block_table,
                                   cache.k_pages, cache.v_pages, self.nh, self.nkv, self.hd, writes, ctx.status,
                                   tiles=None if ctx.decode_only else (ctx.seg_start, ctx.seg_pos0, ctx.tile_seg,
                                                                       ctx.tile_q0),
                                   rot_dim=rot_dim or None, interleaved=interleaved,
                                   bias=bias, v_head_dim=self.vd)
        gate = None
        if self.output_gate:          # the gate's columns of the fused projection, behind q (, k and v)
            g0 = (self.nh + self.nkv) * self.hd + self.nkv * self.vd if writes else self.nh * self.hd
            gate = qkv[:, g0:g0 + self.nh * self.vd]
        o = self.rt.attention(q, cache, ctx, self.window, self.scale, keep_first=self.keep_first, gate=gate,
                              split_weights=self.f32_weights, slopes=self.slopes)
        if residual is not None:
            d = ops.linear_residual(o, self.w_o, residual, self.b_o)
            return (None, None) if d is None else (d, self.b_o)
        return ops.linear(o, self.w_o, out_dtype=torch.float32 if self.f32_output else x.dtype), self.b_o


register_mixer("gqa_attention", GQAttention, replace=True)
