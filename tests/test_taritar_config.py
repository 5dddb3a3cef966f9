"""Taritar on the host: reading config.json, the plan's tensors, cache groups of layers that share keys and values,
pages that a window gives back while the first keys stay, and the plain statement's own mechanisms."""
import copy
import json

import pytest
import torch

import plain_taritar as plain
from taritar_configs import CONFIGS, ONE, PLAIN, WIDE
from wllm_b200.cache import CacheGroupSpec, CacheManager
from wllm_b200.config import ConfigError, TaritarConfig, resolve_architecture
from wllm_b200.engine import ComposedModel


def model_of(raw):
    cfg = TaritarConfig.from_dict(raw)
    return cfg, ComposedModel(resolve_architecture("Taritar").make_plan(cfg), torch.float32)


def test_a_round_trip_through_a_dictionary_keeps_everything():
    for raw in CONFIGS.values():
        cfg = TaritarConfig.from_dict(raw)
        assert TaritarConfig.from_dict(cfg.to_dict()) == cfg
        assert json.loads(json.dumps(cfg.to_dict()))["architecture"] == "Taritar"


@pytest.mark.parametrize("damage,word", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].__setitem__("type", "retention"), "type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), "size"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("dim", 8), "dim"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 3), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 5), "top"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "experts"), "kind"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
])
def test_a_bad_config_is_refused_with_the_key_named(damage, word):
    raw = copy.deepcopy(WIDE)
    damage(raw)
    with pytest.raises(ConfigError, match=word):
        TaritarConfig.from_dict(raw)


def test_a_layer_cannot_read_a_layer_that_reads_another():
    raw = copy.deepcopy(WIDE)
    raw["layers"].append(copy.deepcopy(raw["layers"][2]))
    raw["layers"][4]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError, match="kv_from"):
        TaritarConfig.from_dict(raw)


def test_the_plan_names_every_tensor_once_and_no_keys_for_a_layer_that_borrows_them():
    _, model = model_of(WIDE)
    names = [p.name for p in model.param_specs()]
    assert len(names) == len(set(names))
    assert {"embed", "pos", "head", "final.norm", "l0.hc1.in", "l0.hc2.mix", "l1.mlp.router", "l1.mlp.e7.down", "l1.mlp.shared.sg",
            "l2.mix.q", "l2.mix.o", "l3.mlp.e4.up"} <= set(names)
    assert not {"l2.mix.k", "l2.mix.v", "l2.norm2", "l2.hc2.in", "l3.mlp.shared.gate", "l3.mlp.e5.gate"} & set(names)
    shapes = {p.name: tuple(p.shape) for p in model.param_specs()}
    assert shapes["l0.mix.v"] == (2 * 24, 64) and shapes["l0.mix.o"] == (64, 4 * 24) and shapes["l0.hc1.mix"] == (3, 3)
    assert shapes["pos"] == (400, 64) and shapes["l1.mlp.shared.sg"] == (1, 64)
    _, bare = model_of(PLAIN)
    assert not [n for n in (p.name for p in bare.param_specs()) if ".hc" in n]


def test_cache_groups_keep_what_the_widest_reader_sees():
    _, model = model_of(WIDE)
    groups = {g.name: g for g in model.group_specs}
    # layer 1 (window 24) is read by layer 2 (window 70, 17 kept): its pages serve both
    assert sorted((g.window or 0, g.keep_first, g.layers) for g in groups.values()) == [(0, 0, 1), (40, 5, 1), (70, 17, 1)]
    refs = model.cache_refs
    assert (refs[2].group, refs[2].layer, refs[2].writes) == (refs[1].group, refs[1].layer, False) and refs[1].writes
    _, one = model_of(ONE)
    assert sorted((g.window, g.keep_first) for g in one.group_specs) == [(13, 1), (16, 33)]
    assert model.graph_safe and one.graph_safe


def test_a_window_gives_pages_back_but_not_those_of_the_kept_first_keys():
    cache = CacheManager([CacheGroupSpec("w", 1, 1, 8, window=20, keep_first=17)], page_size=16, num_pages=12, max_requests=2)
    rc = cache.open("a")
    for n in (40, 1, 30, 60):
        cache.reserve([(rc, n)])
        cache.commit(rc, n)
        cache.check()
    table = rc.tables[0]
    first_needed = rc.num_tokens - 20 + 1
    assert table[0] >= 0 and table[1] >= 0                      # keys 0..16 live on pages 0 and 1
    assert all(p == -1 for p in table[2:first_needed // 16]) and all(p >= 0 for p in table[first_needed // 16:])
    cache.close(rc)
    assert cache.free_pages() == [12]


def test_visibility_of_the_plain_mask():
    v = plain.visible(12, size=4, keep_first=2)
    assert v[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert v[3].tolist() == [True] * 4 + [False] * 8 and v[5].tolist() == [True, True, True, True, True, True] + [False] * 6
    assert plain.visible(5, size=5, keep_first=0).tolist() == torch.tril(torch.ones(5, 5)).bool().tolist()


def test_the_plain_router_keeps_to_the_best_groups():
    s = torch.tensor([[0.05, 0.30, 0.20, 0.02, 0.25, 0.01, 0.10, 0.07]])
    assert plain.route(s, top=3, groups=4, keep=2).tolist() == [[1, 4, 0]]          # groups (0,1) and (4,5) stay
    assert plain.route(s, top=3, groups=1, keep=1).tolist() == [[1, 4, 2]]
    assert plain.route(s, top=2, groups=2, keep=1).tolist() == [[1, 2]]
