"""Memipel without a device: the configuration reader, the model spec it makes, the checkpoint binding, and the plain
implementation's own mechanisms against closed forms."""
import copy
import math

import pytest
import torch

import configs_memipel as cm
import plain_memipel as pm
from gesso_b200.config import spec_from_config
from gesso_b200.config.memipel import MemipelConfig
from gesso_b200.engine.model import CachePlan
from gesso_b200.errors import GessoError
from gesso_b200.parts.base import PagedNeed, StateNeed
from gesso_b200.parts.registry import build_block
from gesso_b200.weights.loader import bind_tensors


@pytest.mark.parametrize("name", list(cm.MMP))
def test_spec_parts_and_names(name):
    cfg, seed = cm.MMP[name]
    spec = spec_from_config(cfg)
    assert spec.architecture == "Memipel" and spec.tie_embedding and len(spec.blocks) == len(cfg["layers"])
    kinds = {"latent_attention": "latent_attention", "attention": "gqa_attention", "lightning": "lightning_attention"}
    roles = []
    for L, b in zip(cfg["layers"], spec.blocks):
        assert b.arrangement == "parallel" and b.mixer.kind == kinds[L["type"]]
        assert (b.feed_forward is None) == (L["mlp"] is None)
        assert b.mixer_norm.get("unit_offset") is True and b.mixer_norm["eps"] == cfg["norm"]["eps"]
        if L["type"] == "attention":
            roles.append(b.mixer.get("value_mix"))
            assert b.mixer["window"] == (L["mixer"]["mask"]["size"] if "mask" in L["mixer"] else None)
        if L["mlp"] and L["mlp"]["kind"] == "moe":
            assert b.feed_forward["score"] == "softmax" and b.feed_forward["group_top"] == 1
            assert (b.feed_forward["shared"] is None) == ("shared" not in L["mlp"])
    mixing = [r for r in roles if r]
    assert mixing == (["source"] + ["mix"] * (len(mixing) - 1) if mixing else [])     # the first mixing layer is the source
    bound = bind_tensors(spec, pm.random_tensors(cfg, seed))          # every tensor finds its place, none is left over
    assert "embedding.weight" in bound


def test_cache_plan_pages_and_states():
    spec = spec_from_config(cm.MMP_A)
    plan = CachePlan(spec, [build_block(b) for b in spec.blocks])
    needs = [need for need, _ in plan.paged_groups]
    assert PagedNeed(1, 32, 20, 0, 0) in needs                        # the latent alone, no value pages (parts not bound)
    assert PagedNeed(2, 16, 37, 0, None) in needs and PagedNeed(1, 32, 9, 0, None) in needs
    states = [need for need, _ in plan.state_entries]
    assert StateNeed((2, 24, 16), "float32") in states                # heads x value size x key size
    assert StateNeed((2, 4 * 16 + 2 * 16 + 2 * 16), "float32") in states and StateNeed((1, 2 * 32 + 32 + 32), "float32") in states


def test_refusals_name_the_key():
    def broken(change):
        cfg = copy.deepcopy(cm.MMP_A)
        change(cfg)
        with pytest.raises(GessoError) as e:
            MemipelConfig.from_json(cfg)
        return str(e.value)
    assert "type" in broken(lambda c: c["layers"][0].update(type="mamba"))
    assert "decay" in broken(lambda c: c["layers"][0]["mixer"].update(decay=[0.5]))
    assert "kv_heads" in broken(lambda c: c["layers"][2]["mixer"].update(kv_heads=3))
    assert "kind" in broken(lambda c: c["layers"][0]["mlp"].update(kind="glu"))
    assert "groups" in broken(lambda c: c["layers"][1]["mlp"]["router"].update(groups={"count": 4, "keep": 2}))
    assert "one width" in broken(lambda c: c["layers"][3]["mixer"].update(vdim=8))
    assert "q_rank" in broken(lambda c: c["layers"][1]["mixer"].pop("q_rank"))
    assert "eps" in broken(lambda c: c.update(norm={}))
    tensors = pm.random_tensors(cm.MMP_B, 1)
    del tensors["l1.mix.sink"]
    tensors["l0.mix.vmix"] = torch.zeros(())                          # this layer does not mix values
    with pytest.raises(GessoError) as e:
        bind_tensors(spec_from_config(cm.MMP_B), tensors)
    assert "l1.mix.sink" in str(e.value) and "l0.mix.vmix" in str(e.value)


def test_plain_attention_forms_agree_and_edges():
    T, H, G, D = 40, 4, 2, 8
    q, k, v = torch.randn(T, H, D, dtype=pm.F64), torch.randn(T, G, D, dtype=pm.F64), torch.randn(T, G, 5, dtype=pm.F64)
    sink, slopes = torch.randn(H, dtype=pm.F64), pm.alibi_slopes(H)
    for window in (None, 1, 7, 16):
        a = pm.attend(q, k, v, 0.3, window, sink=sink, slopes=slopes, group=2)
        b = pm.attend_fast(q, k, v, 0.3, window, sink=sink, slopes=slopes, group=2)
        assert torch.allclose(a, b, atol=1e-12)
    # a window of w keys: the key at distance w - 1 counts, the one at distance w does not
    v2 = torch.zeros(T, G, 1, dtype=pm.F64)
    v2[10] = 1.0
    out = pm.attend(torch.zeros(T, H, D, dtype=pm.F64), k, v2, 1.0, 7, group=2).view(T, H)
    assert out[16, 0] > 0 and out[17, 0] == 0 and out[9, 0] == 0 and abs(float(out[10, 0]) - 1 / 7) < 1e-12
    # the sink: with equal scores over n keys the weights are 1 / (n + exp(sink))
    out = pm.attend(torch.zeros(T, H, D, dtype=pm.F64), k, v2, 1.0, None, sink=torch.full((H,), math.log(3.0), dtype=pm.F64),
                    group=2).view(T, H)
    assert abs(float(out[10, 0]) - 1 / (11 + 3)) < 1e-12
    # the distance bias: nearer keys weigh more, by exp(-slope * distance)
    out = pm.attend(torch.zeros(3, 1, D, dtype=pm.F64), k[:3, :1], torch.eye(3, dtype=pm.F64).view(3, 1, 3), 1.0, None,
                    slopes=torch.tensor([0.5], dtype=pm.F64)).view(3, 3)
    assert abs(float(out[2, 0] / out[2, 2]) - math.exp(-1.0)) < 1e-12


def test_plain_conv_router_and_recurrence():
    u = torch.arange(12, dtype=pm.F64).view(6, 2)
    taps = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=pm.F64)
    y = pm.causal_conv(u, taps)
    assert y[0].tolist() == [0.0, 1.0] and y[2, 0] == 0 * 1 + 2 * 10 + 4 * 100 and y[5, 1] == 11
    # groups scored by their best expert: the group of the single largest logit is always kept
    z = torch.tensor([0.1, 0.2, 3.0, -1.0, 1.0, 1.1], dtype=pm.F64)
    chosen, w = pm.route(z, 2, 3, 1)
    assert sorted(chosen) == [2, 3] and abs(sum(w) - float(torch.softmax(z, 0)[[2, 3]].sum())) < 1e-12
    chosen, _ = pm.route(z, 2, 3, 2)
    assert sorted(chosen) == [2, 5]
    # the recurrence against its sum form
    m = {"heads": 1, "dim": 3, "vdim": 2, "decay": [0.8]}
    W = 4
    P = {"mix.q": torch.randn(3, W, dtype=pm.F64), "mix.k": torch.randn(3, W, dtype=pm.F64), "mix.v": torch.randn(2, W, dtype=pm.F64),
         "mix.g": torch.randn(2, W, dtype=pm.F64), "mix.norm": torch.ones(2, dtype=pm.F64), "mix.o": torch.eye(2, dtype=pm.F64)}
    n = torch.randn(9, W, dtype=pm.F64)
    silu = torch.nn.functional.silu
    q, k, v = silu(n @ P["mix.q"].T), silu(n @ P["mix.k"].T), silu(n @ P["mix.v"].T)
    o = torch.stack([sum(0.8 ** (t - s) * float(q[t] @ k[s]) * v[s] for s in range(t + 1)) for t in range(9)])
    want = pm.norm_plain(o, P["mix.norm"], 1e-6) * torch.sigmoid(n @ P["mix.g"].T)
    assert torch.allclose(pm.mixer_lightning(n, P, m, 1e-6), want, atol=1e-12)
