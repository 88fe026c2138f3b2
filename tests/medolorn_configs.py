"""Small Medolorn configurations for the tests and how their model folders are made.

They differ in every size and constant, and inside a model the layers differ too:

* ``looped``: a retention layer (rotation over part of the head, three decays), a latent
  attention layer (window 21 over pages of 8, queries' latent smaller than the cached one) and
  a delta layer without a feed-forward (two query/key heads for four value heads, a filter of
  two taps); the first two layers run twice, so a recurrent layer and a windowed cache each
  exist once per pass.
* ``plain``: no loop key; a delta layer whose query/key heads equal its value heads, latent
  attention whose window (7) is smaller than a page, a retention layer with values wider than
  keys; one router uses all of its experts, another a single one; input filter of two taps.
* ``fast``: the shapes the tensor-core kernels take (width 256, a cached row of 128, heads of
  64), sharp attention over a window of 44, prompts of hundreds of tokens, an input filter and
  a delta filter of ONE tap, a loop that runs once.
* ``odd``: sizes no fast kernel takes: width 72, an odd vocabulary, a cached row of 26, heads
  of 10 with values of 6, a single retention head that turns 4 of 20 coordinates, three delta
  heads on one query/key head, five taps, 33 experts of which 5 are used.

Weights are drawn so that nothing is trivial: attention is sharp, learned decays run from
slow to fast, filters and gate biases are not zero, norm weights are not zero, the steps added
before the passes differ.
"""
from __future__ import annotations

import math
import os

import numpy as np
import torch

from helix_runtime_b200.weights.random_init import write_model_folder


def _moe(ff, experts, top, scale):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "scale": scale}}


def _delta(heads, kv_heads, dim, vdim, conv, mlp):
    return {"type": "delta", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, base, mlp, sharp=2.0):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
                      "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": sharp / math.sqrt(dim + rot_dim), "mask": {"size": window},
                      "rot": {"base": base, "dims": rot_dim}}}


def _retention(heads, dim, vdim, decay, rot_dims, base, mlp):
    return {"type": "retention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay),
                      "rot": {"base": base, "dims": rot_dims}}}


CONFIGS = {
    "looped": {
        "architecture": "Medolorn", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
        "canon": {"taps": 3},
        "layers": [_retention(3, 24, 16, (0.9, 0.97, 0.995), 16, 5000.0, _moe(40, 5, 2, 0.8)),
                   _latent(3, 16, 8, 24, 40, 24, 21, 10000.0, _moe(32, 6, 3, 1.25)),
                   _delta(4, 2, 16, 24, 2, None)],
        "loop": {"start": 0, "stop": 2, "times": 2},
    },
    "plain": {
        "architecture": "Medolorn", "vocab": 300, "width": 128, "norm": {"eps": 1e-6},
        "canon": {"taps": 2},
        "layers": [_delta(2, 2, 32, 32, 4, _moe(48, 3, 3, 1.0)),
                   _latent(4, 32, 16, 16, 48, 64, 7, 300.0, _moe(24, 8, 1, 2.0)),
                   _retention(2, 16, 48, (0.96875, 0.9990234375), 16, 1000000.0,
                              _moe(64, 4, 2, 1.0))],
    },
    "fast": {
        "architecture": "Medolorn", "vocab": 512, "width": 256, "norm": {"eps": 1e-5},
        "canon": {"taps": 1},
        "layers": [_delta(4, 2, 64, 64, 1, _moe(128, 8, 2, 1.5)),
                   _latent(4, 64, 32, 64, 96, 128, 44, 500000.0, _moe(128, 8, 2, 1.5), sharp=6.0),
                   _retention(4, 64, 64, (0.9375, 0.984375, 0.99609375, 0.9990234375), 64,
                              10000.0, _moe(256, 4, 1, 1.0))],
        "loop": {"start": 1, "stop": 2, "times": 1},
    },
    "odd": {
        "architecture": "Medolorn", "vocab": 101, "width": 72, "norm": {"eps": 1e-4},
        "canon": {"taps": 5},
        "layers": [_latent(5, 10, 6, 6, 20, 14, 33, 77.0, _moe(24, 33, 5, 0.7)),
                   _retention(1, 20, 12, (0.98,), 4, 50.0, None),
                   _delta(3, 1, 12, 10, 5, _moe(20, 2, 1, 1.0))],
        "loop": {"start": 1, "stop": 3, "times": 3},
    },
}
PAGE_SIZE = {"looped": 8, "plain": 16, "fast": 16, "odd": 8}
SEED = {"looped": 41, "plain": 42, "fast": 43, "odd": 44}


def tensors_for(config: dict, seed: int, storage_dtype: torch.dtype):
    rng = np.random.default_rng(seed)
    width = config["width"]
    canon = config["canon"]["taps"]

    def store(values):
        return torch.tensor(np.asarray(values), dtype=torch.float32).to(storage_dtype)

    def matrix(rows, columns, gain=1.0):
        return store(rng.normal(size=(rows, columns)) * gain / math.sqrt(columns))

    def vector(size, mean, spread):
        return store(mean + spread * rng.normal(size=size))

    def uniform(size, low, high):
        return store(rng.uniform(low, high, size=size))

    def taps(channels, count, spread):
        return store(rng.normal(size=(channels, count)) * spread)

    tensors = {"embed": matrix(config["vocab"], width, math.sqrt(width)),
               "embed.norm": vector(width, 0.0, 0.2),
               "final.norm": vector(width, 0.0, 0.2), "head": matrix(config["vocab"], width)}
    loop = config.get("loop")
    if loop is not None:
        tensors["loop.in"] = store(np.concatenate(
            [0.8 * np.eye(width) + 0.3 * rng.normal(size=(width, width)) / math.sqrt(width),
             0.4 * np.eye(width) + 0.3 * rng.normal(size=(width, width)) / math.sqrt(width)], axis=1))
        tensors["loop.step"] = store(0.3 * rng.normal(size=(loop["times"], width)))
    for index, layer in enumerate(config["layers"]):
        prefix, mixer = f"l{index}", layer["mixer"]
        for which in (1, 2):
            if which == 2 and layer["mlp"] is None:
                continue
            tensors[f"{prefix}.norm{which}"] = vector(width, 0.0, 0.2)
            tensors[f"{prefix}.rg{which}"] = matrix(width, width, 1.5)
            tensors[f"{prefix}.rg{which}.b"] = vector(width, 0.5, 0.5)
        tensors[f"{prefix}.canon1"] = taps(width, canon, 0.4)
        if layer["type"] == "delta":
            heads, kv_heads, dim, vdim = (mixer[k] for k in ("heads", "kv_heads", "dim", "vdim"))
            for name, rows in (("q", kv_heads * dim), ("k", kv_heads * dim), ("v", heads * vdim)):
                tensors[f"{prefix}.mix.{name}"] = matrix(rows, width, 1.5)
                filter_taps = rng.normal(size=(rows, mixer["conv"])) * 0.4
                filter_taps[:, -1] += 1.0
                tensors[f"{prefix}.mix.{name}.conv"] = store(filter_taps)
            tensors[f"{prefix}.mix.b"] = matrix(heads, width, 2.0)
            tensors[f"{prefix}.mix.a"] = matrix(heads, width, 1.0)
            # decays from about 0.999 per token to 0.3
            tensors[f"{prefix}.mix.A_log"] = uniform(heads, math.log(0.02), math.log(2.0))
            tensors[f"{prefix}.mix.dt_bias"] = uniform(heads, -3.0, 0.5)
            tensors[f"{prefix}.mix.norm"] = vector(vdim, 1.0, 0.2)
            tensors[f"{prefix}.mix.g"] = matrix(heads * vdim, width)
            tensors[f"{prefix}.mix.o"] = matrix(width, heads * vdim, 0.7)
        elif layer["type"] == "latent_attention":
            heads, dim, rot, vdim = (mixer[k] for k in ("heads", "dim", "rot_dim", "vdim"))
            tensors[f"{prefix}.mix.dq"] = matrix(mixer["q_rank"], width)
            tensors[f"{prefix}.mix.dq.norm"] = vector(mixer["q_rank"], 1.0, 0.2)
            tensors[f"{prefix}.mix.uq"] = matrix(heads * (dim + rot), mixer["q_rank"], 1.5)
            tensors[f"{prefix}.mix.dkv"] = matrix(mixer["kv_rank"] + rot, width, 1.2)
            tensors[f"{prefix}.mix.dkv.norm"] = vector(mixer["kv_rank"], 1.0, 0.2)
            tensors[f"{prefix}.mix.uk"] = matrix(heads * dim, mixer["kv_rank"], 1.5)
            tensors[f"{prefix}.mix.uv"] = matrix(heads * vdim, mixer["kv_rank"])
            tensors[f"{prefix}.mix.g"] = matrix(heads * vdim, width, 1.5)
            tensors[f"{prefix}.mix.o"] = matrix(width, heads * vdim, 0.7)
        else:
            heads, dim, vdim = (mixer[k] for k in ("heads", "dim", "vdim"))
            tensors[f"{prefix}.mix.q"] = matrix(heads * dim, width, 1.5)
            tensors[f"{prefix}.mix.k"] = matrix(heads * dim, width, 1.5)
            tensors[f"{prefix}.mix.v"] = matrix(heads * vdim, width)
            tensors[f"{prefix}.mix.g"] = matrix(heads * vdim, width)
            tensors[f"{prefix}.mix.o"] = matrix(width, heads * vdim, 0.7)
        if layer["mlp"] is not None:
            ff, router = layer["mlp"]["expert"]["ff"], layer["mlp"]["router"]
            # router sums spread by about two: scores differ clearly, choices change with the token
            tensors[f"{prefix}.mlp.router"] = matrix(router["experts"], width, 2.0)
            for e in range(router["experts"]):
                tensors[f"{prefix}.mlp.e{e}.gate"] = matrix(ff, width, 1.5)
                tensors[f"{prefix}.mlp.e{e}.up"] = matrix(ff, width, 1.5)
                tensors[f"{prefix}.mlp.e{e}.down"] = matrix(width, ff, 0.7)
    return tensors


def make_folder(directory: str, name: str, storage_dtype: str = "float32") -> str:
    path = os.path.join(directory, f"medolorn_{name}_{storage_dtype}")
    if not os.path.exists(os.path.join(path, "model.safetensors")):
        dtype = torch.bfloat16 if storage_dtype == "bfloat16" else torch.float32
        write_model_folder(path, CONFIGS[name], tensors_for(CONFIGS[name], SEED[name], dtype))
    return path
