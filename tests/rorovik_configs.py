"""Small Rorovik configurations for the tests and how their model folders are made.

They differ in every size and constant, and inside a model the layers differ too:

* ``mixed``: a value-mixing attention layer with a dense feed-forward, a latent attention layer
  with routed experts and identity outputs, a second value-mixing layer (other head count, same
  value row) with experts, a latent layer without a feed-forward; window 21 over pages of 8,
  query temperature that changes every 16 positions, stretched rotary frequencies whose
  original length (24) the prompts pass.
* ``plain``: no token input, no value mixing, no query temperature, no frequency stretching,
  residual factor 1, equal query and key/value heads, a window (7) smaller than a page, a
  router without identity outputs that uses one expert, values wider than keys.
* ``fast``: shapes the tensor-core kernels take (width 256, heads of 64, a cached row of 128),
  sharp attention over a window of 44, prompts of hundreds of tokens, a window-less attention
  layer.
* ``odd``: sizes no fast kernel takes: width 72, an odd vocabulary, heads of 10 with values of
  6, three query heads on one key/value head, a cached row of 26, 5 router outputs of which 3
  are identities and 4 are used, a token input of 3 numbers, a negative residual factor.

Weights are drawn so that nothing is trivial: attention is sharp, sinks matter, biases and norm
weights are neither zero nor one, router corrections change choices.
"""
from __future__ import annotations

import math
import os

import numpy as np
import torch

from helix_runtime_b200.weights.random_init import write_model_folder


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, limit, experts, identity, top):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "identity": identity, "top": top}}


def _attention(heads, kv_heads, dim, vdim, window, temp, v_mix, mlp, sharp=2.0):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
             "scale": sharp / math.sqrt(dim), "v_mix": v_mix}
    if window is not None:
        mixer["mask"] = {"size": window}
    if temp is not None:
        mixer["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base, scaling, mlp, sharp=2.0):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
                      "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": sharp / math.sqrt(dim + rot_dim), "rot": rot}}


CONFIGS = {
    "mixed": {
        "architecture": "Rorovik", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
        "residual_mult": 0.4, "token_side": {"dim": 8},
        "layers": [_attention(4, 2, 24, 16, 21, (0.4, 16), True, _dense(80)),
                   _latent(3, 16, 8, 24, 40, 24, 10000.0, (4.0, 24, 8.0, 1.0),
                           _moe(32, 1.2, 5, 2, 3)),
                   _attention(2, 1, 16, 32, 21, (0.7, 5), True, _moe(40, 0.8, 4, 1, 2)),
                   _latent(2, 8, 16, 8, 24, 48, 300.0, (2.0, 16, 4.0, 0.5), None)],
    },
    "plain": {
        "architecture": "Rorovik", "vocab": 300, "width": 128, "norm": {"eps": 1e-6},
        "layers": [_latent(4, 32, 16, 16, 48, 64, 300.0, None, _moe(24, 2.0, 8, 0, 1)),
                   _attention(4, 4, 16, 32, 7, None, False, _dense(48)),
                   _attention(2, 2, 32, 32, 12, None, False, _moe(64, 1.0, 3, 0, 3))],
    },
    "fast": {
        "architecture": "Rorovik", "vocab": 512, "width": 256, "norm": {"eps": 1e-5},
        "residual_mult": 0.5, "token_side": {"dim": 16},
        "layers": [_attention(4, 2, 64, 64, 44, (0.25, 64), True, _moe(128, 1.25, 8, 2, 2),
                              sharp=6.0),
                   _latent(4, 64, 48, 64, 80, 96, 500000.0, (6.0, 128, 16.0, 2.0),
                           _dense(256), sharp=6.0),
                   _attention(4, 1, 64, 128, None, (0.4, 100), True, _moe(128, 2.5, 4, 4, 2),
                              sharp=4.0)],
    },
    "odd": {
        "architecture": "Rorovik", "vocab": 101, "width": 72, "norm": {"eps": 1e-4},
        "residual_mult": -0.6, "token_side": {"dim": 3},
        "layers": [_attention(3, 1, 10, 6, 33, (1.5, 1), False, _moe(20, 0.5, 2, 3, 4)),
                   _latent(5, 10, 6, 6, 20, 14, 77.0, (3.0, 10, 2.0, 0.25), _dense(30))],
    },
}
PAGE_SIZE = {"mixed": 8, "plain": 16, "fast": 16, "odd": 8}
SEED = {"mixed": 61, "plain": 62, "fast": 63, "odd": 64}


def tensors_for(config: dict, seed: int, storage_dtype: torch.dtype):
    rng = np.random.default_rng(seed)
    width = config["width"]

    def store(values):
        return torch.tensor(np.asarray(values), dtype=torch.float32).to(storage_dtype)

    def matrix(rows, columns, gain=1.0):
        return store(rng.normal(size=(rows, columns)) * gain / math.sqrt(columns))

    def vector(size, mean, spread):
        return store(mean + spread * rng.normal(size=size))

    tensors = {"embed": matrix(config["vocab"], width, math.sqrt(width)),
               "embed.norm": vector(width, 1.0, 0.2),
               "final.norm": vector(width, 1.0, 0.2), "head": matrix(config["vocab"], width)}
    side = (config.get("token_side") or {}).get("dim")
    if side:
        tensors["side.embed"] = store(rng.normal(size=(config["vocab"], side * len(config["layers"]))))
    for index, layer in enumerate(config["layers"]):
        prefix, mixer = f"l{index}", layer["mixer"]
        for name in ("norm1", "norm1b") + (("norm2", "norm2b") if layer["mlp"] else ()):
            tensors[f"{prefix}.{name}"] = vector(width, 1.0, 0.2)
        if layer["type"] == "attention":
            heads, kv_heads, dim, vdim = (mixer[k] for k in ("heads", "kv_heads", "dim", "vdim"))
            for name, rows in (("q", heads * dim), ("k", kv_heads * dim), ("v", kv_heads * vdim)):
                tensors[f"{prefix}.mix.{name}"] = matrix(rows, width, 1.5)
                tensors[f"{prefix}.mix.{name}.b"] = vector(rows, 0.0, 0.3)
            tensors[f"{prefix}.mix.q.norm"] = vector(heads * dim, 1.0, 0.3)
            tensors[f"{prefix}.mix.k.norm"] = vector(kv_heads * dim, 1.0, 0.3)
            if mixer.get("v_mix"):
                tensors[f"{prefix}.mix.vmix"] = store(rng.uniform(0.2, 0.7))
            tensors[f"{prefix}.mix.sink"] = vector(heads, 0.5, 1.0)
            tensors[f"{prefix}.mix.g"] = matrix(heads, width, 2.0)
            tensors[f"{prefix}.mix.o"] = matrix(width, heads * vdim, 0.7)
        else:
            heads, dim, rot, vdim = (mixer[k] for k in ("heads", "dim", "rot_dim", "vdim"))
            tensors[f"{prefix}.mix.dq"] = matrix(mixer["q_rank"], width)
            tensors[f"{prefix}.mix.dq.norm"] = vector(mixer["q_rank"], 1.0, 0.2)
            tensors[f"{prefix}.mix.uq"] = matrix(heads * (dim + rot), mixer["q_rank"], 1.5)
            tensors[f"{prefix}.mix.dkv"] = matrix(mixer["kv_rank"] + rot, width, 1.2)
            tensors[f"{prefix}.mix.dkv.norm"] = vector(mixer["kv_rank"], 1.0, 0.2)
            tensors[f"{prefix}.mix.uk"] = matrix(heads * dim, mixer["kv_rank"], 1.5)
            tensors[f"{prefix}.mix.uv"] = matrix(heads * vdim, mixer["kv_rank"])
            tensors[f"{prefix}.mix.sink"] = vector(heads, 0.5, 1.0)
            tensors[f"{prefix}.mix.o"] = matrix(width, heads * vdim, 0.7)
        mlp = layer["mlp"]
        if mlp is not None and mlp["kind"] == "dense":
            ff = mlp["ff"]
            for name, rows, columns in (("gate", ff, width), ("up", ff, width), ("down", width, ff)):
                tensors[f"{prefix}.mlp.{name}"] = matrix(rows, columns, 1.5)
                tensors[f"{prefix}.mlp.{name}.b"] = vector(rows, 0.0, 0.3)
        elif mlp is not None:
            ff, router = mlp["expert"]["ff"], mlp["router"]
            outputs = router["experts"] + router["identity"]
            # router sums spread by about two: scores differ clearly, choices change with the
            # token, and the corrections are large enough to change some of them
            tensors[f"{prefix}.mlp.router"] = matrix(outputs, width, 2.0)
            tensors[f"{prefix}.mlp.correction"] = vector(outputs, 0.0, 0.15)
            for e in range(router["experts"]):
                tensors[f"{prefix}.mlp.e{e}.gate"] = matrix(ff, width, 2.0)
                tensors[f"{prefix}.mlp.e{e}.up"] = matrix(ff, width, 2.0)
                tensors[f"{prefix}.mlp.e{e}.down"] = matrix(width, ff, 0.7)
        if side:
            tensors[f"{prefix}.side.gate"] = matrix(side, width, 1.5)
            tensors[f"{prefix}.side.proj"] = matrix(width, side)
            tensors[f"{prefix}.side.norm"] = vector(width, 1.0, 0.2)
    return tensors


def make_folder(directory: str, name: str, storage_dtype: str = "float32") -> str:
    path = os.path.join(directory, f"rorovik_{name}_{storage_dtype}")
    if not os.path.exists(os.path.join(path, "model.safetensors")):
        dtype = torch.bfloat16 if storage_dtype == "bfloat16" else torch.float32
        write_model_folder(path, CONFIGS[name], tensors_for(CONFIGS[name], SEED[name], dtype))
    return path
