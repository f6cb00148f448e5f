"""Latent attention: queries, keys and values that go through low-rank latents; only the key/value latent is cached.

With the mixer's input ``x`` (own notation; ``N(.; w)`` is an RMS norm with a plain weight)::

    c_q = N(W_dq x; w_q)          q_h = W_uq[h] c_q                       (H heads of ``head_dim``)
    c   = N(W_dkv x; w_kv)        k_h = W_uk[h] c,   v_h = W_uv[h] c      (``kv_rank`` numbers per position)
    score_h(i, j) = scale * q_h(i) . k_h(j)   for 0 <= i - j < window
    p = softmax over the visible keys, with one more term exp(sink_h) in the denominator (``sink``)
    out = W_o concat_h( sum_j p_h(i, j) v_h(j) )

There are no positions in it.  The cache holds ``c`` alone: one "kv head" of ``kv_rank`` features per position.
The engine evaluates the *absorbed* form, which reads the cached latent directly::

    q'_h = W_uk[h]^T q_h                    (carried into the latent space: kv_rank features, float32)
    a_h  = sum_j p_h(i, j) c(j)             (scores q'_h . c(j); keys and values are the same rows)
    o_h  = W_uv[h] a_h

so that a step never expands keys and values of cached positions, whether it decodes or reads a prompt.

In bfloat16 runs whose sizes the tensor-core attention kernels take (``kv_rank`` 32, 64, 96 or 128, at most 16
heads) the latent is cached twice, as rows and transposed (the two layouts those kernels read keys and values
from; still ``2 kv_rank`` numbers per position against ``H (head_dim + v_head_dim)`` of expanded keys and values),
q' is rounded to bfloat16 as their operand, and the attention weights act on the latents as two bfloat16 pieces.
Every other size and the float32 run keep one copy (no value pages) and take the FP32-arithmetic kernel with float32
q'.  The two per-head products run on the tensor cores for bfloat16 steps of 64 rows and more, else on FP32 FMAs.

Parameters: hidden_size, n_heads, head_dim, v_head_dim, q_rank, kv_rank, scale, window (``None``: all keys), sink
(default true), norm_eps.  Tensors: ``dq.weight`` [q_rank, hidden], ``dq_norm.weight`` [q_rank], ``uq.weight`` [H *
head_dim, q_rank], ``dkv.weight`` [kv_rank, hidden], ``dkv_norm.weight`` [kv_rank], ``uk.weight`` [H * head_dim,
kv_rank], ``uv.weight`` [H * v_head_dim, kv_rank], ``sink`` [H], ``o_proj.weight`` [hidden, H * v_head_dim].

What is 32-bit whatever the run type: both latent norms (on the float32 sums of the down projection), the scores, the
softmax with its sink, and the weights' action on the latents (float32 products, or two bfloat16 pieces per weight).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..errors import invalid
from .base import Mixer, PagedNeed, ParamDecl
from .registry import register_mixer


class LatentAttention(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["n_heads"])
        self.hd = int(spec["head_dim"])
        self.vd = int(spec.get("v_head_dim") or self.hd)
        self.q_rank = int(spec["q_rank"])
        self.kv_rank = int(spec["kv_rank"])
        self.scale = float(spec["scale"]) if spec.get("scale") is not None else float(self.hd) ** -0.5
        self.window = spec.get("window")
        self.has_sink = bool(spec.get("sink", True))
        self.eps = float(spec["norm_eps"])
        if min(self.nh, self.hd, self.vd, self.q_rank, self.kv_rank) < 1:
            raise invalid("latent attention: sizes must be positive")
        if self.kv_rank > 512:
            raise invalid(f"latent attention: kv_rank {self.kv_rank} is above 512, the most the attention kernel takes")
        if self.window is not None and int(self.window) < 1:
            raise invalid("latent attention: window must be >= 1")
        self.mirror = False       # decided when the weights are bound (the run type decides)

    def param_decls(self) -> Dict[str, ParamDecl]:
        H, D, Dv, Rq, R, W = self.nh, self.hd, self.vd, self.q_rank, self.kv_rank, self.hidden
        d = {
            "dq.weight": ParamDecl((Rq, W), fan_in=W),
            "dq_norm.weight": ParamDecl((Rq,), role="vector", init="ones"),
            "uq.weight": ParamDecl((H * D, Rq), fan_in=Rq),
            "dkv.weight": ParamDecl((R, W), fan_in=W),
            "dkv_norm.weight": ParamDecl((R,), role="vector", init="ones"),
            "uk.weight": ParamDecl((H * D, R), fan_in=R),
            "uv.weight": ParamDecl((H * Dv, R), fan_in=R),
            "o_proj.weight": ParamDecl((W, H * Dv), fan_in=H * Dv),
        }
        if self.has_sink:
            d["sink"] = ParamDecl((H,), role="vector", init="zeros")
        return d

    def cache_need(self):
        # one latent per position: a single kv head of kv_rank features; no value pages, or (for the tensor-core
        # kernels) the same latent once more, transposed
        return PagedNeed(1, self.kv_rank, int(self.window) if self.window is not None else None, 0,
                         None if self.mirror else 0)

    def bind(self, tensors, rt) -> None:
        H, D, Dv, R = self.nh, self.hd, self.vd, self.kv_rank
        ws = [tensors["dq.weight"], tensors["dkv.weight"]]
        common = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_down = torch.cat([w.to(common) for w in ws], dim=0).contiguous()          # [Rq + R, hidden]
        self.w_dq = ws[0].contiguous()
        self.wn_q, self.wn_kv = tensors["dq_norm.weight"], tensors["dkv_norm.weight"]
        self.w_uq = tensors["uq.weight"]
        # per head, input-major: q' = W_uk[h]^T q ([D, R] as stored), o = W_uv[h] a ([R, Dv]: transposed once)
        self.w_absorb = tensors["uk.weight"].reshape(H, D, R).contiguous()
        self.w_expand = tensors["uv.weight"].reshape(H, Dv, R).transpose(1, 2).contiguous()
        # the same two output-major, for the tensor-core product that steps of many rows take
        self.w_absorb_t = self.w_absorb.transpose(1, 2).contiguous()                   # [H, R, D]
        self.w_expand_t = tensors["uv.weight"].reshape(H, Dv, R).contiguous()          # [H, Dv, R]
        self.sink = tensors["sink"].float().contiguous() if self.has_sink else None
        self.w_o = tensors["o_proj.weight"]
        self.rt = rt
        self.mirror = (rt.dtype == torch.bfloat16 and self.kv_rank in (32, 64, 96, 128) and self.nh <= 16
                       and ops.LATENT_TENSOR_CORES)

    @staticmethod
    def _per_head(x, w_in_major, w_out_major, out_dtype):
        if ops.headwise_linear_tc_takes(x.shape[0], x.dtype, w_out_major, out_dtype):
            return ops.headwise_linear_tc(x, w_out_major)
        return ops.headwise_linear(x, w_in_major, out_dtype)

    def forward(self, x, ctx, cache):
        writes = cache.writes
        Rq, R = self.q_rank, self.kv_rank
        proj = ops.linear(x, self.w_down if writes else self.w_dq, out_dtype=torch.float32)
        cq = ops.latent_norm_store(proj, Rq, R if writes else 0, self.wn_q, self.wn_kv, self.eps, x.dtype,
                                   ctx.positions, ctx.seg_of_token, cache.block_table, cache.k_pages, writes, ctx.status,
                                   v_pages=cache.v_pages if self.mirror else None)
        q = ops.linear(cq, self.w_uq, out_dtype=x.dtype).view(-1, self.nh, self.hd)
        if self.mirror:
            q_lat = self._per_head(q, self.w_absorb, self.w_absorb_t, x.dtype)            # [N, H, R], an operand
            a = self.rt.attention(q_lat, cache, ctx, self.window, self.scale, sink=self.sink, split_weights=True)
        else:
            q_lat = ops.headwise_linear(q, self.w_absorb, torch.float32)                  # [N, H, R]
            a = self.rt.attention(q_lat, cache, ctx, self.window, self.scale, sink=self.sink, values_are_keys=True)
        o = self._per_head(a.view(-1, self.nh, R), self.w_expand, self.w_expand_t, x.dtype)   # [N, H, Dv]
        return ops.linear(o.view(-1, self.nh * self.vd), self.w_o, out_dtype=torch.float32), None


register_mixer("latent_attention", LatentAttention, replace=True)
