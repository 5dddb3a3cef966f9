"""Pesanex on the host: reading config.json, the order of layer runs, the plan's tensors, caches and state."""
import copy
import json
import os

import pytest
import torch

from pesanex_configs import CONFIGS, MIX, ONCE, PLAIN, write_folder
from wllm_b200.config import ConfigError, PesanexConfig, config_from_folder
from wllm_b200.engine import ComposedModel


def plan_of(raw):
    from wllm_b200.config import resolve_architecture
    cfg = PesanexConfig.from_dict(raw)
    return cfg, resolve_architecture("Pesanex").make_plan(cfg)


def test_the_order_of_runs_follows_the_loop():
    assert PesanexConfig.from_dict(MIX).order() == [0, 1, 2, 1, 2, 1, 2]
    assert PesanexConfig.from_dict(PLAIN).order() == [0, 1, 2]
    assert PesanexConfig.from_dict(ONCE).order() == [0, 1]
    raw = copy.deepcopy(MIX)
    raw["loop"] = {"start": 0, "stop": 1, "times": 2}
    assert PesanexConfig.from_dict(raw).order() == [0, 0, 1, 2]
    raw["loop"] = {"start": 3, "stop": 3, "times": 5}
    assert PesanexConfig.from_dict(raw).order() == [0, 1, 2]


def test_a_round_trip_through_a_dictionary_keeps_everything():
    for raw in CONFIGS.values():
        cfg = PesanexConfig.from_dict(raw)
        assert PesanexConfig.from_dict(cfg.to_dict()) == cfg
        assert json.loads(json.dumps(cfg.to_dict()))["architecture"] == "Pesanex"


@pytest.mark.parametrize("damage,word", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.9]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "rot"),
    (lambda c: c["layers"][2]["mixer"].pop("tau"), "tau"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "experts"), "mlp"),
    (lambda c: c.__setitem__("loop", {"start": 2, "stop": 1, "times": 2}), "loop"),
])
def test_a_bad_config_is_refused_with_the_key_named(damage, word):
    raw = copy.deepcopy(MIX)
    damage(raw)
    with pytest.raises(ConfigError, match=word):
        PesanexConfig.from_dict(raw)


def test_the_plan_lists_the_checkpoint_tensors_of_every_layer_once():
    cfg, plan = plan_of(MIX)
    model = ComposedModel(plan, torch.float32)
    names = {ps.name: ps.shape for ps in model.param_specs()}
    assert names["embed"] == (211, 96) and names["head"] == (211, 96) and names["final.norm"] == (96,)
    assert names["l0.mix.left.q"] == (128, 96) and names["l0.mix.left.k"] == (64, 96) and names["l0.mix.left.v"] == (32, 96)
    assert names["l0.mix.left.o"] == (96, 64) and names["l0.mix.left.sink"] == (4,)
    assert names["l0.mix.right.a1"] == (8, 96) and names["l0.mix.right.a2"] == (72, 8) and names["l0.mix.right.a2.b"] == (72,)
    assert names["l0.mix.right.norm"] == (40,) and names["l0.mix.left.out"] == (96,) and names["l0.mix.right.out"] == (96,)
    assert names["l1.mix.g"] == (96, 96) and "l1.mix.norm" not in names and "l1.mix.a1" not in names
    assert names["l1.mlp.gate"] == (72, 96) and names["l1.norm2b"] == (96,)
    assert "l2.norm2" not in names and "l2.mlp.up" not in names and names["l2.norm1b"] == (96,)
    assert len(names) == len(model.param_specs())


@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_test_configuration_builds_and_gets_seeded_weights(name, tmp_path):
    folder = write_folder(str(tmp_path / name), name)
    arch, cfg = config_from_folder(folder)
    model = ComposedModel(arch.make_plan(cfg), torch.bfloat16)
    from safetensors.torch import load_file
    held = load_file(os.path.join(folder, "model.safetensors"))
    assert set(held) == {ps.name for ps in model.param_specs()}
    assert len(model.plan.runs) == len(cfg.order()) and len(model.state_specs) >= 1


def test_a_rank_that_the_configuration_leaves_out_is_an_open_size():
    raw = copy.deepcopy(PLAIN)
    del raw["layers"][2]["mixer"]["rank"]
    _, plan = plan_of(raw)
    names = {ps.name: ps.shape for ps in ComposedModel(plan, torch.float32).param_specs()}
    assert names["l2.mix.a1"] == (None, 64) and names["l2.mix.a2"] == (32, None)
    from wllm_b200.weights import random_tensors
    with pytest.raises(ValueError, match="only a checkpoint gives"):
        random_tensors(raw, 1)


def test_every_run_has_its_own_pages_and_state():
    _, plan = plan_of(MIX)
    model = ComposedModel(plan, torch.bfloat16)
    # the attention of layer 0 runs once: one cache layer, keys of 32 and values of 16
    assert [(g.name, g.layers, g.kv_heads, g.head_dim, g.v_head_dim) for g in model.group_specs] == [("all-2x32v16", 1, 2, 32, 16)]
    assert [s.name for s in model.state_specs] == ["run0.right.state", "run1.state", "run2.state", "run3.state", "run4.state",
                                                   "run5.state", "run6.state"]
    shapes = {s.name: s.shape for s in model.state_specs}
    assert shapes["run0.right.state"] == (3, 24, 40) and shapes["run1.state"] == (2, 24, 48) and shapes["run2.state"] == (2, 40, 24)
    assert all(s.dtype == torch.float32 for s in model.state_specs)
    _, plan = plan_of(PLAIN)
    model = ComposedModel(plan, torch.bfloat16)
    assert [(g.name, g.layers, g.v_head_dim) for g in model.group_specs] == [("all-2x64", 1, None)]


def test_a_folder_is_found_by_its_single_architecture_name(tmp_path):
    folder = write_folder(str(tmp_path / "m"), "once")
    arch, cfg = config_from_folder(folder)
    assert arch.name == "Pesanex" and cfg.width == 48 and cfg.layers[1]["mixer"]["left"].get("rot") is None
    from safetensors.torch import load_file
    assert load_file(os.path.join(folder, "model.safetensors"))["l1.mix.left.sink"].shape == (1,)


def test_value_heads_of_their_own_size_get_pools_of_their_own():
    from wllm_b200.cache import CacheGroupSpec, CacheManager
    cache = CacheManager([CacheGroupSpec("g", 2, 2, 32, None, 16)], page_size=16, num_pages=4, max_requests=2,
                         dtype=torch.float32, device="cpu", poison=True)
    g = cache.groups[0]
    assert g.keys(1).shape == (4, 2, 16, 32) and g.values(1).shape == (4, 2, 16, 16) and g.bytes_per_token() == 2 * 2 * 48 * 4
    rc = cache.open("a")
    cache.reserve([(rc, 20)])
    g.keys(0)[rc.tables[0][0]] = 1.0
    g.values(1)[rc.tables[0][1]] = 2.0
    cache.commit(rc, 20)
    cache.close(rc)
    assert torch.isnan(g.key_pages).all() and torch.isnan(g.value_pages).all()
