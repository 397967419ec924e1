"""The Zuzadra configuration: reading, refusing, writing back, the sizes that only a
checkpoint gives, and the parts its model is assembled from.  No GPU."""
from __future__ import annotations

import copy

import pytest

from helix_runtime_b200.config import ConfigError, ZuzadraConfig, architecture_for
from helix_runtime_b200.models import DecoderModel
from zuzadra_configs import CONFIGS, DECAY_RANK, tensors_for


def with_rank(name):
    document = copy.deepcopy(CONFIGS[name])
    for layer in document["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["right"]["rank"] = DECAY_RANK[name]
    return document


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_round_trip_and_registry(name):
    document = with_rank(name)
    entry = architecture_for(document)
    assert entry.name == "Zuzadra"
    config = entry.config_from_dict(document)
    assert ZuzadraConfig.from_dict(config.to_dict()) == config
    spec = entry.build_spec(config)
    loop = document.get("loop")
    runs = len(document["layers"]) + ((loop["stop"] - loop["start"]) * (loop["times"] - 1) if loop else 0)
    assert len(spec.schedule) == runs and spec.streams == (document.get("streams") or 1)
    assert all(block.arrangement == "streams" for block in spec.blocks)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_model_binds_exactly_the_checkpoint_tensors(name):
    import torch
    document = CONFIGS[name]
    entry = architecture_for(document)
    tensors = tensors_for(document, 1, torch.float32, DECAY_RANK[name])
    config = entry.sizes_from_checkpoint(entry.config_from_dict(document),
                                         {key: tuple(value.shape) for key, value in tensors.items()})
    model = DecoderModel(entry.build_spec(config))
    requests = {request.name: tuple(request.shape) for request in model.tensor_requests()}
    assert requests == {key: tuple(value.shape) for key, value in tensors.items()}
    kv, state = model.cache_needs()
    parallel_runs = [index for index, entry_ in enumerate(model.schedule)
                     if document["layers"][entry_.block]["type"] == "parallel"]
    assert sorted(kv) == parallel_runs and sorted(state) == list(range(len(model.schedule)))
    for index in parallel_runs:
        left = document["layers"][model.schedule[index].block]["mixer"]["left"]
        assert kv[index].window == left["mask"]["size"] and kv[index].kv_heads == left["kv_heads"]


def test_the_decay_rank_comes_from_the_checkpoint_or_the_configuration():
    document = CONFIGS["streams3"]
    entry = architecture_for(document)
    config = entry.config_from_dict(document)
    with pytest.raises(ConfigError, match="rank"):
        entry.build_spec(config)
    sized = entry.sizes_from_checkpoint(config, {"l1.mix.right.w1": (11, 64)})
    assert sized.layers[1].mixer.right.rank == 11
    assert entry.config_from_dict(with_rank("streams3")).layers[1].mixer.right.rank == 8


def test_without_streams_there_are_no_connection_weights():
    entry = architecture_for(CONFIGS["single"])
    model = DecoderModel(entry.build_spec(entry.config_from_dict(with_rank("single"))))
    names = {request.name for request in model.tensor_requests()}
    assert not any(".hc" in name for name in names) and "l0.ls1" in names and model.streams == 1


@pytest.mark.parametrize("change,complaint", [
    (lambda d: d["layers"][0].update(type="conv"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(groups=3), "groups"),
    (lambda d: d["layers"][0]["mixer"].update(norm_groups=7), "norm_groups"),
    (lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=5), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(layout="spiral"), "layout"),
    (lambda d: d["layers"][1]["mixer"]["left"]["mask"].update(size=0), "mask.size"),
    (lambda d: d["layers"][1]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][1]["mixer"].pop("right"), "right"),
    (lambda d: d.update(streams=0), "streams"),
    (lambda d: d.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
    (lambda d: d["layers"][0]["mlp"].update(kind="experts"), "kind"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_what_the_configuration_refuses(change, complaint):
    document = with_rank("streams3")
    change(document)
    with pytest.raises(ConfigError, match=complaint):
        ZuzadraConfig.from_dict(document)
