"""Bifusun without a GPU: config to parts, tensor names and shapes, the cache plan of mixers that keep pages and a state, config
errors, and the plain statement's own pieces."""

import copy

import pytest
import torch

import bifusun_util as BU
from plain import bifusun_plain as BP


def _model(cfg):
    from oxr_inference_b200.weights.random_init import shape_only_model

    return shape_only_model(cfg)


def test_tensor_names_and_shapes():
    m = _model(BU.MODEL_P)
    named = {k: tuple(v[2].shape) for k, v in m.named_parameters().items()}
    assert named["embed"] == (131, 48) and named["head"] == (131, 48) and named["final.norm"] == (48,)
    assert named["l0.mix.q"] == (64, 48) and named["l0.mix.k"] == (32, 48) and named["l0.mix.v"] == (48, 48)
    assert named["l0.mix.q.b"] == (64,) and named["l0.mix.o.b"] == (48,) and named["l0.mix.v.conv"] == (48, 3)
    assert named["l0.mix.vmix"] == () and named["l2.mix.vmix"] == () and "l3.mix.vmix" not in named
    assert named["l1.mix.g"] == (48, 48) and named["l1.mix.i"] == (2, 48) and named["l1.mix.f.b"] == (2,) and named["l1.mix.norm"] == (48,)
    assert named["l1.mlp.router"] == (8, 48) and named["l1.mlp.e7.up"] == (16, 48) and named["l1.mlp.e7.down"] == (48, 16)
    assert not any(k.startswith(("l2.mlp", "l2.norm2", "l5.mlp")) for k in named)       # layers without a feed-forward
    assert "l3.mix.q.conv" in named and "l3.mix.q.b" in named


def test_blending_layers_keep_then_blend():
    m = _model(BU.MODEL_P)
    kinds = [getattr(b.mixer, "value_mix", "-") for b in m.blocks]
    assert kinds == ["keep", "-", "blend", None, "blend", "-"]


def test_cache_plan_gives_pages_and_a_state_to_one_mixer():
    from oxr_inference_b200.parts.base import PagedKVNeed, StateNeed

    m = _model(BU.MODEL_P)
    plan = m.cache_plan
    e0, e1, e3 = plan.entries[0], plan.entries[1], plan.entries[3]
    assert e0.group is not None and e0.state is not None          # attention: pages, and the filter's tail
    assert e1.group is None and e1.state is not None              # mlstm: a state only
    assert plan.states[e0.state] == StateNeed(((64 + 32 + 48) * 2,), torch.float32)
    assert plan.states[e1.state] == StateNeed((2 * 16 * 24 + 2 * 16 + 2,), torch.float32)
    # keys and values of one size: the plain need, shared with nobody else here
    assert plan.groups[e3.group].need == PagedKVNeed(4, 16, 0)
    assert plan.entries[2].group == e0.group and plan.entries[2].layer_in_group == 1
    # a filter of one tap keeps nothing
    q = _model(BU.MODEL_Q)
    assert q.cache_plan.entries[2].state is None and q.cache_plan.entries[1].state is not None


def test_a_pair_of_needs_is_planned_and_a_wrong_one_refused():
    from oxr_inference_b200.cache.plan import make_cache_plan
    from oxr_inference_b200.parts.base import PagedKVNeed, StateNeed

    paged, state = PagedKVNeed(2, 16), StateNeed((5,))
    plan = make_cache_plan([(paged, state), paged, state, None, (state, paged)], [None] * 5)
    assert [(e.group, e.layer_in_group, e.state) for e in plan.entries] == [(0, 0, 0), (0, 1, None), (None, 0, 1), (None, 0, None), (0, 2, 2)]
    with pytest.raises(TypeError):
        make_cache_plan([(paged, paged)], [None])
    with pytest.raises(TypeError):
        make_cache_plan(["pages"], [None])


@pytest.mark.parametrize("change,words", [
    (lambda c: c["layers"][0].update(type="retention"), "is not one of"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "lacks 'scale'"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "not a multiple"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=8), "blends its values"),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0.0), "gate_cap"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "do not fit"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "do not fit"),
    (lambda c: c.pop("norm"), "lacks 'norm'"),
])
def test_config_errors(change, words):
    from oxr_inference_b200.config.model_config import ConfigError
    from oxr_inference_b200.config.registry import resolve_architecture

    cfg = copy.deepcopy(BU.MODEL_P)
    change(cfg)
    with pytest.raises(ConfigError, match=words):
        resolve_architecture(cfg).config_from_dict(cfg, None)


def test_plain_filter_and_temperature():
    u = torch.arange(10, dtype=torch.float64).view(5, 2)
    taps = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 2.0]], dtype=torch.float64)
    y = BP.short_convolution(u, taps)
    assert y[0].tolist() == [0.0, 2.0] and y[1].tolist() == [200.0, 6.0] and y[4].tolist() == [1 * 4 + 10 * 6 + 100 * 8, 18.0]
    t = BP.query_temperature(9, 0.5, 4, torch.float64)
    assert t[0] == t[2] == 1.0 and abs(t[3] - (1 + 0.5 * 0.6931471805599453)) < 1e-12 and t[7] > t[6] == t[3]


def test_plain_router_keeps_groups_and_normalises():
    z = torch.tensor([[5.0, 4.0, -9.0, -9.0, 4.5, -9.0, 3.0, 3.0]], dtype=torch.float64)
    # groups of two: scores (5+4), (-,-), (4.5,-), (3+3): the best two groups are 0 and 3, so expert 4 cannot be chosen
    chosen, weight = BP.route(z, {"experts": 8, "top": 3, "scale": 2.0, "groups": {"count": 4, "keep": 2}})
    assert sorted(chosen[0].tolist()) == [0, 1, 6] or sorted(chosen[0].tolist()) == [0, 1, 7]
    assert abs(weight.sum().item() - 2.0) < 1e-9
    chosen, _ = BP.route(z, {"experts": 8, "top": 3, "scale": 2.0})
    assert sorted(chosen[0].tolist()) == [0, 1, 4]


def test_plain_matrix_memory_matches_its_own_decoding():
    """The recurrence over a whole sequence equals the same recurrence fed the sequence's prefixes (nothing looks ahead)."""
    cfg = BU.model_config([BU.mlstm_layer()])
    torch.manual_seed(0)
    w = {name: torch.randn(info.shape, dtype=torch.float64) * 0.3 for name, (_, _, info) in _model(cfg).named_parameters().items()}
    ids = BU.tokens(cfg, 12, seed=1)
    whole = BP.forward(cfg, w, ids)
    for n in (1, 5, 12):
        assert torch.allclose(BP.forward(cfg, w, ids[:n])[-1], whole[n - 1], atol=1e-10)


def test_unused_tensors_of_a_layer_may_be_present(tmp_path):
    """A checkpoint that also stores a blending weight for a layer that blends nothing, and the second norm of a layer without a
    feed-forward, still fits the model; any other stray tensor does not."""
    import re

    spec = _model(BU.MODEL_P).spec
    allowed = [re.compile(p + "$") for p in spec.ignored_tensors]
    assert any(r.match("l3.mix.vmix") for r in allowed) and any(r.match("l12.norm2") for r in allowed)
    assert not any(r.match(name) for r in allowed for name in ("l3.mix.q.conv", "l3.mix.vmixer", "xl3.norm2", "l3.norm21", "head"))
