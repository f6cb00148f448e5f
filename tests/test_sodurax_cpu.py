"""Sodurax on the CPU: the configuration reader, the names of its tensors, the cache manager's kept first
pages, and the plain implementation's own mechanisms on hand-made cases."""
import copy
import math

import pytest
import torch

import configs_sodurax as cs
import plain_sodurax as ps
from gesso_b200.cache.manager import CacheManager, FREED, PagedGroupSpec
from gesso_b200.config import SoduraxConfig, spec_from_config
from gesso_b200.errors import GessoError
from gesso_b200.weights.loader import bind_tensors, model_param_decls


def test_every_size_comes_from_the_configuration():
    c = SoduraxConfig.from_json(cs.SDX_B)
    assert (c.vocab, c.width, len(c.layers)) == (257, 96, 3)
    m0, m1 = c.layers[0].mixer, c.layers[1].mixer
    assert (m0.heads, m0.kv_heads, m0.dim, m0.vdim, m0.scale) == (6, 1, 24, 40, 0.31)
    assert (m0.rot_dims, m0.rot_base, m0.rot_factor, m0.window, m0.keep_first) == (24, 500000.0, 1.0, 11, 0)
    assert (m1.rot_dims, m1.rot_factor, m1.window, m1.keep_first) == (4, 1.5, 23, 1)
    assert c.layers[1].mlp is None and c.layers[2].weights_of == 0
    e = c.layers[0].mlp
    assert (e.ff, e.experts, e.top, e.groups, e.keep_groups) == (40, 6, 1, 1, 1)


def test_layers_that_borrow_tensors_become_schedule_entries():
    s = spec_from_config(cs.SDX_A)
    assert len(s.blocks) == 2 and [e.layer for e in s.schedule] == [0, 1, 0, 1]
    assert all(e.cache_of is None for e in s.schedule)          # a cache of its own each
    mixer = s.blocks[0].mixer
    assert mixer.kind == "gqa_attention" and mixer["keep_first"] == 3 and mixer["window"] == 40
    assert mixer["position"]["scaling_factor"] == 2.0 and mixer["position"]["rotary_dim"] == 16
    # other constants on the same tensors: parts of its own, bound to the owner's checkpoint names
    s = spec_from_config(cs.SDX_C)
    assert len(s.blocks) == 2 and [e.layer for e in s.schedule] == [0, 1]
    assert s.blocks[1].mixer["window"] == 33
    assert s.external_names("layers.1.mixer.q_proj.weight") == ("l0.mix.q",)
    assert s.external_names("layers.1.feed_forward.experts.3.up.weight") == ("l0.mlp.e3.up",)


def test_tensor_names_and_shapes_bind():
    for name, (cfg, seed) in cs.SDX.items():
        spec = spec_from_config(cfg)
        bound = bind_tensors(spec, ps.random_tensors(cfg, seed))
        assert set(bound) == set(model_param_decls(spec))
    spec = spec_from_config(cs.SDX_B)
    W = ps.random_tensors(cs.SDX_B, 1)
    assert tuple(bound_shape for bound_shape in bind_tensors(spec, W)["layers.0.mixer.o_proj.weight"].shape) == (96, 240)
    del W["l0.mix.g"]
    W["l1.mlp.router"] = torch.zeros(2, 2)
    with pytest.raises(GessoError) as e:
        bind_tensors(spec, W)
    assert "l0.mix.g" in str(e.value) and "l1.mlp.router" in str(e.value)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].__setitem__("type", "recurrent"), "type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 5), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 34), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("experts", 7), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 5), "cannot give"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 2), "weights_of"),
    (lambda c: c.__delitem__("vocab"), "vocab"),
])
def test_bad_configurations_are_refused(change, word):
    cfg = copy.deepcopy(cs.SDX_A)
    change(cfg)
    with pytest.raises(GessoError) as e:
        SoduraxConfig.from_json(cfg)
    assert word in str(e.value)


def test_optional_parts_of_the_configuration():
    cfg = copy.deepcopy(cs.SDX_A)
    m = cfg["layers"][0]["mixer"]
    m["mask"] = None
    m["rot"]["scaling"] = None
    del cfg["layers"][0]["mlp"]["router"]["groups"]
    c = SoduraxConfig.from_json(cfg).layers[0]
    assert c.mixer.window is None and c.mixer.keep_first == 0 and c.mixer.rot_factor == 1.0
    assert (c.mlp.groups, c.mlp.keep_groups) == (1, 1)


# ---- cache manager: the pages of the first positions stay ---------------------------------------------
def test_kept_first_positions_keep_their_pages():
    m = CacheManager([PagedGroupSpec("all"), PagedGroupSpec("win", window=6, keep_first=5)], page_size=4,
                     num_pages=[16, 16], num_slots=2, max_positions=64)
    m.admit("r")
    m.reserve("r", 30)
    m.commit("r", 30)
    # next query at 30 reads keys >= 25 and keys 0..4: pages 0 and 1 stay, pages 2..5 (positions 8..23) go
    row = m.block_table("r", 1)
    assert FREED not in row[:2] and row[2:6] == [FREED] * 4 and FREED not in row[6:]
    for _ in range(20):
        m.reserve("r", 1)
        m.commit("r", 1)
        m.check_invariants()
    row = m.block_table("r", 1)
    assert FREED not in row[:2] and m.pages_in_use()[1] <= 2 + 3
    m.release("r")
    assert m.pages_in_use() == [0, 0]
    # a freed page is handed out again
    m.admit("s")
    m.reserve("s", 8)
    m.check_invariants()


# ---- the plain implementation's mechanisms on hand-made cases -----------------------------------------
def test_plain_visibility_edges():
    vis = ps.visibility(12, {"size": 4, "keep_first": 2})
    assert vis[10].tolist() == [True, True] + [False] * 5 + [True] * 4 + [False]
    assert vis[3].tolist() == [True] * 4 + [False] * 8           # everything earlier is inside the window
    assert vis[7, 1] and not vis[7, 2] and not vis[7, 3] and vis[7, 4] and not vis[7, 8]


def test_plain_rotation_is_partial_and_scaled():
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0}}
    ang = ps.rotation_angles(3, rot)
    assert torch.allclose(ang[2], torch.tensor([2 * 1.0 / 2, 2 * 100.0 ** -0.5 / 2], dtype=torch.float64))
    x = torch.arange(6, dtype=torch.float64).view(1, 1, 6) + 1
    y = ps.rotate(x.expand(3, 1, 6), ang, 4)
    assert torch.equal(y[:, :, 4:], x.expand(3, 1, 6)[:, :, 4:])          # features beyond dims pass
    a = float(ang[1, 0])
    assert math.isclose(float(y[1, 0, 0]), 1 * math.cos(a) - 3 * math.sin(a))
    assert math.isclose(float(y[1, 0, 2]), 3 * math.cos(a) + 1 * math.sin(a))


def test_plain_router_group_limit_and_weights():
    # 6 experts in 3 groups of 2, keep 2 groups, top 2.  z chosen so that the best single expert sits in a
    # group whose SUM of two is the smallest, and corrections push choice scores below zero.
    W = {"p.router": torch.eye(6, dtype=torch.float64), "p.correction": torch.tensor([-2., -2., -2., -2., -2., -2.], dtype=torch.float64)}
    x = torch.tensor([[3.0, -9.0, 1.0, 1.0, 0.5, 0.9]], dtype=torch.float64)
    idx, w = ps.route(x, W, "p.", {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}})
    # group sums of (sigmoid - 2): g0 = .953+.0001-4, g1 = .731*2-4, g2 = .622+.711-4 -> g1, g2 kept, g0 shut out
    assert sorted(idx[0].tolist()) == [2, 3]
    assert torch.allclose(w[0], torch.sigmoid(torch.tensor([1.0, 1.0], dtype=torch.float64)))   # without the correction
