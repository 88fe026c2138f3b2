"""The Rorovik configuration: reading, refusing, writing back, and the parts its model is
assembled from.  No GPU."""
from __future__ import annotations

import copy

import pytest

from helix_runtime_b200.config import ConfigError, architecture_for
from helix_runtime_b200.config.rorovik import RorovikConfig
from helix_runtime_b200.models import DecoderModel
from rorovik_configs import CONFIGS, tensors_for


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_round_trip_and_registry(name):
    document = CONFIGS[name]
    entry = architecture_for(document)
    assert entry.name == "Rorovik"
    config = entry.config_from_dict(document)
    assert RorovikConfig.from_dict(config.to_dict()) == config
    spec = entry.build_spec(config)
    assert [run.block for run in spec.schedule] == list(range(len(document["layers"])))
    side = document.get("token_side")
    for index, run in enumerate(spec.schedule):
        assert run.before is None and (run.after is not None) == (side is not None)
        if side is not None:
            assert run.after["offset"] == index * side["dim"] and run.after["dim"] == side["dim"]
            block = spec.blocks[index]
            last = block.feed_forward_connection or block.mixer_connection
            assert last.get("cast_to") == run.after["reads"]


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_model_binds_exactly_the_checkpoint_tensors(name):
    import torch
    document = CONFIGS[name]
    entry = architecture_for(document)
    tensors = tensors_for(document, 1, torch.float32)
    model = DecoderModel(entry.build_spec(entry.config_from_dict(document)))
    requests = {request.name: tuple(request.shape) for request in model.tensor_requests()
                if not request.optional or request.name in tensors}
    assert requests == {key: tuple(value.shape) for key, value in tensors.items()}
    kv, state = model.cache_needs()
    assert not state and sorted(kv) == list(range(len(document["layers"])))
    for index, layer in enumerate(document["layers"]):
        mixer = layer["mixer"]
        if layer["type"] == "attention":
            assert kv[index].window == (mixer.get("mask") or {}).get("size")
            assert kv[index].kv_heads == mixer["kv_heads"]
            assert kv[index].head_dim >= max(mixer["dim"], mixer["vdim"])
        else:
            assert kv[index].window is None and kv[index].kv_heads == 1
            assert kv[index].head_dim >= mixer["kv_rank"] + mixer["rot_dim"]


def test_the_first_value_mixing_layer_keeps_and_the_later_ones_blend():
    entry = architecture_for(CONFIGS["mixed"])
    spec = entry.build_spec(entry.config_from_dict(CONFIGS["mixed"]))
    modes = [block.mixer.get("value_mix") for block in spec.blocks]
    assert modes == ["source", None, "mix", None]
    slopes = spec.blocks[0].mixer["distance_slopes"]
    assert slopes == tuple(2.0 ** (-8.0 * (head + 1) / 4) for head in range(4))
    entry = architecture_for(CONFIGS["plain"])
    spec = entry.build_spec(entry.config_from_dict(CONFIGS["plain"]))
    assert [block.mixer.get("value_mix") for block in spec.blocks] == [None, None, None]


def test_optional_keys_may_be_left_out():
    document = copy.deepcopy(CONFIGS["plain"])
    config = RorovikConfig.from_dict(document)
    assert config.side_dim is None and config.residual_mult == 1.0
    attention = config.layers[1].mixer
    assert attention.temp_every is None and not attention.v_mix and attention.window == 7
    assert config.layers[0].mixer.scaling is None
    del document["layers"][1]["mixer"]["mask"]
    del document["layers"][1]["mixer"]["kv_heads"]
    del document["layers"][1]["mixer"]["vdim"]
    relaxed = RorovikConfig.from_dict(document).layers[1].mixer
    assert relaxed.window is None and relaxed.kv_heads == relaxed.heads and relaxed.vdim == relaxed.dim


@pytest.mark.parametrize("change,complaint", [
    (lambda d: d["layers"][0].update(type="conv"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda d: d["layers"][0]["mixer"]["q_temp"].update(every=0), "q_temp.every"),
    (lambda d: d["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda d: d["layers"][0]["mlp"].pop("ff"), "ff"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=8), "top"),
    (lambda d: d["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda d: d["layers"][1]["mlp"].pop("expert"), "expert"),
    (lambda d: d["layers"][2]["mixer"].update(vdim=16), "kv_heads \\* vdim"),
    (lambda d: d.update(token_side={"dim": 0}), "token_side.dim"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d.update(layers=[]), "layers"),
])
def test_what_the_configuration_refuses(change, complaint):
    document = copy.deepcopy(CONFIGS["mixed"])
    change(document)
    with pytest.raises(ConfigError, match=complaint):
        RorovikConfig.from_dict(document)
