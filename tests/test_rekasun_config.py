"""What needs no GPU of the Rekasun decoder: its configuration, the order its layers run in,
the model spec built from it, and the cache manager's kept first pages."""
from __future__ import annotations

import copy

import numpy as np
import pytest
import torch

import plain_rekasun
from helix_runtime_b200.cache import CacheManager, KvNeed
from helix_runtime_b200.config import ConfigError, RekasunConfig, architecture_for
from helix_runtime_b200.models import DecoderModel, build_rekasun_spec
from rekasun_configs import CONFIGS

CPU = torch.device("cpu")


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_configuration_round_trip_and_spec(name):
    document = CONFIGS[name]
    entry = architecture_for(document)
    assert entry.name == "Rekasun"
    config = entry.config_from_dict(document)
    assert RekasunConfig.from_dict(config.to_dict()) == config
    spec = entry.build_spec(config)
    runs = plain_rekasun.layer_runs(len(document["layers"]), document.get("loop"))
    assert [(e.block, e.add_embedding) for e in spec.schedule] == runs
    model = DecoderModel(spec)
    names = {request.name: tuple(request.shape) for request in model.tensor_requests()}
    width = document["width"]
    assert names["embed"] == (document["vocab"], width) and names["head"] == (document["vocab"], width)
    for index, layer in enumerate(document["layers"]):
        mixer = layer["mixer"]
        assert names[f"l{index}.mix.q"] == (mixer["heads"] * mixer["dim"], width)
        assert names[f"l{index}.mix.v"] == (mixer["kv_heads"] * mixer["vdim"], width)
        assert names[f"l{index}.mix.o"] == (width, mixer["heads"] * mixer["vdim"])
        assert names[f"l{index}.mix.g"] == (mixer["heads"] * mixer["vdim"], width)
        assert (f"l{index}.mix.k.conv" in names) == (mixer["conv"] > 1)
        if mixer["conv"] > 1:
            assert names[f"l{index}.mix.k.conv"] == (mixer["kv_heads"] * mixer["dim"], mixer["conv"])
        assert (f"l{index}.mlp.gate" in names) == (layer["mlp"] is not None)
        assert names[f"l{index}.norm1.b"] == (width,)
    # every run of a layer owns a cache: one need per schedule entry
    kv, state = model.cache_needs()
    assert sorted(kv) == list(range(len(runs)))
    assert sorted(state) == [i for i, (layer, _) in enumerate(runs)
                             if document["layers"][layer]["mixer"]["conv"] > 1]


def test_order_of_layer_runs():
    config = RekasunConfig.from_dict(CONFIGS["mixed"])
    assert config.layer_runs() == ((0, False), (1, False), (0, True), (1, False), (0, True),
                                   (1, False), (2, False))
    document = copy.deepcopy(CONFIGS["mixed"])
    document["loop"] = {"start": 1, "stop": 3, "times": 1}
    assert RekasunConfig.from_dict(document).layer_runs() == ((0, False), (1, False), (2, False))
    del document["loop"]
    assert RekasunConfig.from_dict(document).layer_runs() == ((0, False), (1, False), (2, False))


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].__setitem__("type", "recurrent"), "type"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("heads", 3), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda d: d["layers"][0]["mlp"].__setitem__("kind", "routed"), "dense"),
    (lambda d: d.__setitem__("loop", {"start": 2, "stop": 1, "times": 2}), "loop"),
    (lambda d: d.__setitem__("loop", {"start": 0, "stop": 9, "times": 2}), "loop"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d.__setitem__("width", -4), "width"),
])
def test_configurations_that_are_refused(change, message):
    document = copy.deepcopy(CONFIGS["mixed"])
    change(document)
    with pytest.raises(ConfigError, match=message):
        RekasunConfig.from_dict(document)


def test_kept_first_pages_stay_while_the_window_gives_the_rest_back():
    # window 6, 5 kept keys, pages of 4: pages 0 and 1 hold kept keys
    needs = {0: KvNeed(2, 8, window=6, keep_first=5), 1: KvNeed(2, 8)}
    cache = CacheManager(needs, {}, 4, 16, 2, 64, torch.float32, CPU)
    windowed = next(group for group in cache.groups if group.need.window)
    assert cache.kept_pages(windowed) == 2
    cache.admit("a")
    for length in range(1, 41):
        cache.extend("a", length)
        cache.commit("a", length)
        cache.check()
        table = list(windowed.host_tables[cache.slot("a")][:-(-length // 4)])
        first_seen = max(0, length - 6 + 1) // 4       # the next query sits at `length`
        for page, entry in enumerate(table):
            assert (entry >= 0) == (page < 2 or page >= first_seen), (length, page, table)
    assert windowed.pool.pages_in_use <= 2 + 3
    # a request that could never fit is known from the page arithmetic: kept + window + a page
    assert cache.pages_needed_alone(1000)[windowed.index] == -(-(6 + 4 + 2 * 4) // 4)
    cache.release("a")
    cache.check()
    assert windowed.pool.free_pages == 16


def test_random_lives_with_kept_pages_lose_nothing():
    rng = np.random.default_rng(0)
    needs = {0: KvNeed(1, 8, window=9, keep_first=3), 1: KvNeed(1, 8, window=4, keep_first=0)}
    cache = CacheManager(needs, {}, 4, 24, 3, 128, torch.float32, CPU)
    lengths = {}
    for step in range(400):
        name = f"r{rng.integers(0, 5)}"
        if name not in lengths:
            if cache.free_slots == 0:
                continue
            cache.admit(name)
            lengths[name] = 0
        elif rng.random() < 0.15:
            cache.release(name)
            del lengths[name]
        else:
            grow = int(rng.integers(1, 9))
            if cache.max_extend(name, grow) < grow:
                continue
            cache.extend(name, lengths[name] + grow)
            if rng.random() < 0.2:
                cache.rollback(name)
            else:
                lengths[name] += grow
                cache.commit(name, lengths[name])
        cache.check()
