"""Radapel on the host: config.json to parts, tensor names, the schedule of a repeated stretch, the cache plan, the distance
buckets, and the cache manager's handling of chunked groups. No GPU."""

import math

import pytest
import torch

import radapel_util as RU
from oxr_inference_b200.cache import CacheManager, RELEASED
from oxr_inference_b200.config import ConfigError, resolve_architecture
from oxr_inference_b200.parts.base import PagedKVNeed, StateNeed
from oxr_inference_b200.parts.masked_attention import bias_by_distance, distance_bucket
from oxr_inference_b200.weights import shape_only_model
from plain import radapel_plain as RP


def test_architecture_is_found_by_its_single_name():
    assert resolve_architecture(RU.MODEL_X).name == "Radapel"
    with pytest.raises(ConfigError):
        resolve_architecture({"architecture": "NoSuchDesign"})


def test_tensor_names_and_shapes():
    named = {k: tuple(v[2].shape) for k, v in shape_only_model(RU.MODEL_X).named_parameters().items()}
    assert named["embed"] == (131, 48) and named["head"] == (131, 48) and named["final.norm"] == (48,)
    assert named["loop.in"] == (48, 96) and named["loop.step"] == (3, 48)
    # mamba2, no feed-forward: one pair of norms only
    assert named["l0.mix.in"] == (2 * 32 + 2 * 2 * 16 + 4, 48) and named["l0.mix.conv"] == (32 + 64, 3) and named["l0.mix.o"] == (48, 32)
    assert "l0.norm1" in named and "l0.norm1b" in named and "l0.norm2" not in named and "l0.mlp.gate" not in named
    assert named["l1.mix.q"] == (64, 48) and named["l1.mix.k"] == (32, 48) and named["l1.mix.v"] == (48, 48) and named["l1.mix.rel"] == (12, 4)
    assert named["l1.mix.o"] == (48, 96) and named["l1.mlp.gate"] == (40, 48) and named["l1.mlp.down"] == (48, 40)
    assert named["l2.mix.q"] == (2 * 24, 48) and named["l2.mix.dkv"] == (32, 48) and named["l2.mix.dkv.norm"] == (24,)
    assert named["l2.mix.uk"] == (32, 24) and named["l2.mix.uv"] == (24, 24) and named["l2.mix.sink"] == (2,) and named["l2.mix.o"] == (48, 24)
    assert named["l3.mix.rel"] == (6, 4)
    assert not [k for k in shape_only_model(RU.MODEL_Y).named_parameters() if k.startswith("loop.") or k.endswith(".rel")]


def test_bias_table_height_comes_from_the_tensor():
    arch = resolve_architecture(RU.MODEL_X)
    spec = arch.spec_for(arch.config_from_dict(RU.MODEL_X, None), {"l1.mix.rel": (18, 4)})
    assert spec.layers[1].mixer.params["bias_rows"] == 18 and spec.layers[3].mixer.params["bias_rows"] == 6


def test_schedule_of_a_repeated_stretch_and_its_caches():
    model = shape_only_model(RU.MODEL_X)
    runs = [(e.layer, e.joint, e.joint_arg) for e in model.schedule]
    assert runs == [(0, None, 0), (1, 0, 0), (2, None, 0), (1, 0, 1), (2, None, 1), (1, 0, 2), (2, None, 2), (3, None, 0)]
    assert RP.layer_runs(RU.MODEL_X) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    plan = model.cache_plan
    # every pass has a cache of its own: three runs of the chunked layer share one pool as three layers of it
    chunked = [g for g in plan.groups if g.need.chunk == 10]
    assert len(chunked) == 1 and chunked[0].num_layers == 3 and chunked[0].need == PagedKVNeed(2, 16, 0, value_dim=24, chunk=10)
    latent = [g for g in plan.groups if g.need.value_dim == 0]
    assert len(latent) == 1 and latent[0].num_layers == 3 and latent[0].need.head_dim == 24 + 8 and latent[0].need.num_kv_heads == 1
    assert plan.states == (StateNeed((4 * 8 * 16 + (32 + 64) * 2,), torch.float32),)
    assert len({(e.group, e.layer_in_group, e.state) for e in plan.entries}) == len(plan.entries)


def test_config_errors_are_named():
    bad = RU.model_config([RU.attention_layer()])
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError, match="type"):
        resolve_architecture(bad).config_from_dict(bad, None)
    bad = RU.model_config([RU.attention_layer()], loop=(0, 2, 2))
    with pytest.raises(ConfigError, match="loop"):
        resolve_architecture(bad).config_from_dict(bad, None)
    bad = RU.model_config([RU.attention_layer()])
    del bad["layers"][0]["mixer"]["scale"]
    arch = resolve_architecture(bad)
    with pytest.raises(ConfigError, match="scale"):
        arch.spec_for(arch.config_from_dict(bad, None))


@pytest.mark.parametrize("rows,far", [(32, 120.0), (12, 40.0), (6, 9.5), (20, 100.0), (16, 1024.0)])
def test_distance_buckets(rows, far):
    half = rows // 2
    got = [distance_bucket(n, rows, far) for n in range(int(far) + 50)]
    assert got == [RP.distance_bucket(n, rows, far) for n in range(int(far) + 50)]
    assert got[:half] == list(range(half)) and got[half] == half
    assert all(a <= b for a, b in zip(got, got[1:])) and got[-1] == rows - 1
    assert all(b == rows - 1 for n, b in enumerate(got) if n >= far)
    first_last = got.index(rows - 1)
    assert half * (far / half) ** ((rows - 1 - half) / (rows - half)) <= first_last + 1e-9
    table = torch.arange(rows * 3, dtype=torch.float32).view(rows, 3)
    wide = bias_by_distance(table, far)
    assert wide.shape[0] == max(half, math.ceil(far)) + 1
    assert torch.equal(wide, table[torch.tensor(got[:wide.shape[0]])])
    with pytest.raises(ValueError):
        bias_by_distance(table, float(half))


def test_pages_before_the_chunk_are_given_back_and_used_again():
    model = shape_only_model(RU.model_config([RU.attention_layer(chunk=10)]))
    m = CacheManager(model.cache_plan, page_size=4, num_pages=9, max_requests=2, scratch=True)
    a = m.open("a")
    assert m.reserve(a, 9)
    m.advance(a, 9)          # the next query (position 9) still sees 0..9
    assert a.tables[0] == sorted(a.tables[0]) and RELEASED not in a.tables[0]
    assert m.reserve(a, 10)
    m.advance(a, 10)         # the next query sits at 10: chunk 10..19 begins in page 2
    assert a.tables[0][:2] == [RELEASED, RELEASED] and a.tables[0][2] != RELEASED
    m.check()
    assert m.reserve(a, 23)
    m.advance(a, 23)         # next query at 23: chunk 20..29 begins in page 5
    assert a.tables[0][:5] == [RELEASED] * 5 and all(p != RELEASED for p in a.tables[0][5:])
    held = [p for p in a.tables[0] if p != RELEASED]
    b = m.open("b")
    assert m.reserve(b, 20)  # five pages: only possible with what a gave back
    assert not set(b.tables[0]) & set(held)
    m.check()
    m.close(a)
    m.close(b)
    assert m.free_pages == m.usable_pages and m.free_slots == 2
