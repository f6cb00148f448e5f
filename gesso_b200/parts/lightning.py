"""Linear attention with a fixed decay per head ("lightning attention"), as a recurrence over a per-request state.

With the mixer's input ``x`` and ``silu(z) = z / (1 + exp(-z))``, per head h::

    q_t = silu(W_q x_t)[h],  k_t = silu(W_k x_t)[h]   (``head_dim`` features),   v_t = silu(W_v x_t)[h]  (``v_head_dim``)
    S_t = decay_h * S_{t-1} + k_t v_t^T               (S_0 = 0; no other scale)
    o_t = S_t^T q_t

The heads of a token are then normed *together*, gated and projected::

    y_t = (o_t / sqrt(mean(o_t^2) + eps)) * w * sigmoid(W_g x_t),      out_t = W_o y_t

The state S (``n_heads x head_dim x v_head_dim`` float32 numbers per request and layer) is all a request keeps; it
is carried from token to token inside a portion and from step to step in the request's state slot.  A step with a
long portion computes the same sums by 64-token chunks side by side (a chunk's own key-value sum, a walk over the
chunks that hands each its starting state, then each chunk's outputs).  The
recurrence, the decays and the norm are float32 whatever the run type; the four projections are one fused matrix.

Parameters: hidden_size, n_heads, head_dim, v_head_dim, decay (one number per head), norm_eps.  Tensors:
``q_proj.weight``, ``k_proj.weight`` [H * head_dim, hidden], ``v_proj.weight``, ``g_proj.weight`` [H * v_head_dim,
hidden], ``norm.weight`` [H * v_head_dim], ``o_proj.weight`` [hidden, H * v_head_dim].
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..errors import invalid
from .base import Mixer, ParamDecl, StateNeed
from .registry import register_mixer


class LightningAttention(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["n_heads"])
        self.hd = int(spec["head_dim"])
        self.vd = int(spec.get("v_head_dim") or self.hd)
        self.decay = [float(d) for d in spec["decay"]]
        self.eps = float(spec["norm_eps"])
        if min(self.nh, self.hd, self.vd) < 1:
            raise invalid("lightning attention: sizes must be positive")
        if len(self.decay) != self.nh:
            raise invalid(f"lightning attention: {len(self.decay)} decays for {self.nh} heads")
        if self.hd > 512:
            raise invalid(f"lightning attention: head_dim {self.hd} is above 512, the most the recurrence kernel takes")

    def param_decls(self) -> Dict[str, ParamDecl]:
        H, D, Dv, W = self.nh, self.hd, self.vd, self.hidden
        return {
            "q_proj.weight": ParamDecl((H * D, W), fan_in=W),
            "k_proj.weight": ParamDecl((H * D, W), fan_in=W),
            "v_proj.weight": ParamDecl((H * Dv, W), fan_in=W),
            "g_proj.weight": ParamDecl((H * Dv, W), fan_in=W),
            "norm.weight": ParamDecl((H * Dv,), role="vector", init="ones"),
            "o_proj.weight": ParamDecl((W, H * Dv), fan_in=H * Dv),
        }

    def cache_need(self):
        return StateNeed((self.nh, self.vd, self.hd), "float32")       # a value column's features are contiguous

    def bind(self, tensors, rt) -> None:
        ws = [tensors[n + "_proj.weight"] for n in ("q", "k", "v", "g")]
        common = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_in = torch.cat([w.to(common) for w in ws], dim=0).contiguous()
        self.w_norm = tensors["norm.weight"]
        self.w_o = tensors["o_proj.weight"]
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float64).to(device=rt.device, dtype=torch.float32)

    def forward(self, x, ctx, cache):
        H, D, Dv = self.nh, self.hd, self.vd
        proj = ops.linear(x, self.w_in, out_dtype=x.dtype)
        if not ctx.decode_only and ops.lightning_chunked_takes(ctx.max_seg_len, D, Dv):
            # long prompt portions: the step's 64-token tiles side by side instead of token after token
            o = ops.lightning_attention_chunked(proj, cache.state, self.decay_dev, ctx.seg_start, cache.slots,
                                                ctx.tile_seg, ctx.tile_q0, ctx.n_segs, H, D, Dv)
        else:
            o = ops.lightning_attention(proj, cache.state, self.decay_dev, ctx.seg_start, cache.slots, ctx.n_segs, H, D, Dv)
        g0 = 2 * H * D + H * Dv
        y = ops.gated_rmsnorm(o, self.w_norm, self.eps, proj[:, g0:g0 + H * Dv], x.dtype)
        return ops.linear(y, self.w_o, out_dtype=torch.float32), None


register_mixer("lightning_attention", LightningAttention, replace=True)
