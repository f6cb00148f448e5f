"""Tiny Sodurax configurations of the tests.  They differ in every size and option."""


def _layer(heads, kv, dim, vdim, scale, rot, mask, mlp, weights_of=None):
    L = {"type": "attention",
         "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot, "mask": mask},
         "mlp": mlp}
    if weights_of is not None:
        L["weights_of"] = weights_of
    return L


def _moe(ff, experts, top, count, keep):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


# 4 layer runs on 2 sets of tensors; width 64, 4 heads on 2 kv heads of 32 (the tensor-core attention sizes),
# 16 of 32 features rotate at half speed, window 40 with 3 kept tokens, 8 experts in 4 groups (2 kept), top 2.
_A = _layer(4, 2, 32, 32, 0.2, {"base": 10000.0, "dims": 16, "scaling": {"factor": 2.0}},
            {"size": 40, "keep_first": 3}, _moe(48, 8, 2, 4, 2))
SDX_A = {"architecture": "Sodurax", "vocab": 131, "width": 64, "norm": {"eps": 1e-5},
         "layers": [_A, _A, dict(_A, weights_of=0), dict(_A, weights_of=1)]}

# values narrower and wider than keys, one kv head, a whole-head rotation without scaling, a window shorter
# than a page and no kept tokens, one group, top 1, a layer without a feed-forward, windows that differ.
_B0 = _layer(6, 1, 24, 40, 0.31, {"base": 500000.0, "dims": 24}, {"size": 11, "keep_first": 0}, _moe(40, 6, 1, 1, 1))
_B1 = _layer(3, 3, 16, 8, 0.25, {"base": 100.0, "dims": 4, "scaling": {"factor": 1.5}}, {"size": 23, "keep_first": 1}, None)
SDX_B = {"architecture": "Sodurax", "vocab": 257, "width": 96, "norm": {"eps": 1e-6}, "layers": [_B0, _B1, _B0]}
SDX_B["layers"][2] = dict(_B0, weights_of=0)

# two query heads per kv head of 64 (the tcgen05 attention sizes), 20 kept tokens (more than a page), 16 experts
# in 8 pairs (5 kept), top 3; the second run of the tensors has another window (parts of its own on the same tensors).
_C = _layer(4, 2, 64, 64, 0.125, {"base": 1000.0, "dims": 8, "scaling": {"factor": 8.0}},
            {"size": 50, "keep_first": 20}, _moe(32, 16, 3, 8, 5))
_C2 = _layer(4, 2, 64, 64, 0.125, {"base": 1000.0, "dims": 8, "scaling": {"factor": 8.0}},
             {"size": 33, "keep_first": 2}, _moe(32, 16, 3, 8, 5), weights_of=0)
SDX_C = {"architecture": "Sodurax", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "layers": [_C, _C2]}

# name -> (config, seed)
SDX = {"a": (SDX_A, 11), "b": (SDX_B, 12), "c": (SDX_C, 13)}
