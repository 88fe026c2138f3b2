"""The Medolorn configuration: reading, refusing, writing back, the order its layers run in,
and the parts its model is assembled from.  No GPU."""
from __future__ import annotations

import copy

import pytest

from helix_runtime_b200.config import ConfigError, architecture_for
from helix_runtime_b200.config.medolorn import MedolornConfig
from helix_runtime_b200.models import DecoderModel
from medolorn_configs import CONFIGS, tensors_for


def runs_of(document):
    loop = document.get("loop")
    count = len(document["layers"])
    if loop is None:
        return list(range(count))
    body = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + body * loop["times"] + list(range(loop["stop"], count))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_round_trip_and_registry(name):
    document = CONFIGS[name]
    entry = architecture_for(document)
    assert entry.name == "Medolorn"
    config = entry.config_from_dict(document)
    assert MedolornConfig.from_dict(config.to_dict()) == config
    spec = entry.build_spec(config)
    assert [run.block for run in spec.schedule] == runs_of(document)
    loop = document.get("loop")
    starts = [index for index, run in enumerate(spec.schedule) if run.before is not None]
    if loop is None:
        assert starts == []
    else:
        span = loop["stop"] - loop["start"]
        assert starts == [loop["start"] + turn * span for turn in range(loop["times"])]
        assert [spec.schedule[index].before["index"] for index in starts] == list(range(loop["times"]))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_model_binds_exactly_the_checkpoint_tensors(name):
    import torch
    document = CONFIGS[name]
    entry = architecture_for(document)
    tensors = tensors_for(document, 1, torch.float32)
    model = DecoderModel(entry.build_spec(entry.config_from_dict(document)))
    requests = {request.name: tuple(request.shape) for request in model.tensor_requests()}
    assert requests == {key: tuple(value.shape) for key, value in tensors.items()}
    kv, state = model.cache_needs()
    runs = runs_of(document)
    latent_runs = [index for index, layer in enumerate(runs)
                   if document["layers"][layer]["type"] == "latent_attention"]
    # every run of a layer owns its pages and its state row, a looped layer once per pass
    assert sorted(kv) == latent_runs
    taps = document["canon"]["taps"]
    for index, layer in enumerate(runs):
        mixer = document["layers"][layer]["mixer"]
        if index in latent_runs:
            assert kv[index].window == mixer["mask"]["size"] and kv[index].kv_heads == 1
            assert kv[index].head_dim >= mixer["kv_rank"] + mixer["rot_dim"]
            assert (index in state) == (taps > 1)
        else:
            assert index in state and state[index].dtype == torch.float32
            held = state[index].shape[0]
            assert held >= (taps - 1) * document["width"] + mixer["heads"] * mixer["dim"] * mixer["vdim"]


def test_a_loop_may_be_absent_or_run_once():
    document = copy.deepcopy(CONFIGS["plain"])
    assert MedolornConfig.from_dict(document).layer_runs() == ((0, None), (1, None), (2, None))
    document["loop"] = {"start": 0, "stop": 3, "times": 1}
    assert MedolornConfig.from_dict(document).layer_runs() == ((0, 0), (1, None), (2, None))
    document["loop"] = {"start": 2, "stop": 3, "times": 3}
    assert MedolornConfig.from_dict(document).layer_runs() == \
        ((0, None), (1, None), (2, 0), (2, 1), (2, 2))


@pytest.mark.parametrize("change,complaint", [
    (lambda d: d["layers"][0].update(type="conv"), "type"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda d: d["layers"][1]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda d: d["layers"][2]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda d: d["layers"][0]["mlp"].pop("expert"), "expert"),
    (lambda d: d.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
    (lambda d: d.update(loop={"start": 0, "stop": 4, "times": 2}), "loop"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d.pop("canon"), "canon"),
    (lambda d: d.update(layers=[]), "layers"),
])
def test_what_the_configuration_refuses(change, complaint):
    document = copy.deepcopy(CONFIGS["looped"])
    change(document)
    with pytest.raises(ConfigError, match=complaint):
        MedolornConfig.from_dict(document)
