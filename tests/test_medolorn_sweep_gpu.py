"""Randomly drawn Medolorn configurations through the engine against the plain implementation:
the order and number of layers, loops (none, once, several passes), every size of the three
mixers (heads, grouped query/key heads, head and value sizes up to 256, filters of 1 to 6
taps; latents smaller and larger than a head, cached rows beyond what the tensor-core
attention takes, windows of 1 to 300, rotated parts of 2 to 64; decays, partly rotated heads),
routers of 1 to 40 experts that use 1 to all of them, expert sizes the tensor-core products do
not take, widths likewise, and every model is replayed as mixed batches over a pool made for
its live requests only."""
from __future__ import annotations

import math
import os

import numpy as np
import pytest
import torch

import plain_medolorn
import traces
from conftest import random_tokens
from engine_harness import Harness, assert_close
from helix_runtime_b200.weights.random_init import write_model_folder
from medolorn_configs import tensors_for

pytestmark = pytest.mark.gpu


def draw_config(seed: int):
    rng = np.random.default_rng(3000 + seed)
    pick = lambda values: values[int(rng.integers(0, len(values)))]
    width = pick([40, 64, 72, 100, 128, 136, 256])

    def mlp():
        if rng.random() < 0.2:
            return None
        experts = pick([1, 2, 3, 8, 16, 40])
        return {"kind": "moe", "expert": {"ff": pick([8, 20, 48, 64, 100, 128])},
                "router": {"experts": experts, "top": int(rng.integers(1, min(experts, 6) + 1)),
                           "scale": float(pick([1.0, 0.5, 2.5]))}}

    layers = []
    for _ in range(int(rng.integers(1, 5))):
        kind = pick(["delta", "latent_attention", "retention"])
        if kind == "delta":
            kv_heads = pick([1, 2, 3])
            mixer = {"heads": kv_heads * pick([1, 2, 4]), "kv_heads": kv_heads,
                     "dim": pick([4, 8, 20, 32, 64, 100, 128, 256]),
                     "vdim": pick([4, 8, 24, 32, 64, 136]), "conv": pick([1, 2, 3, 4, 6])}
        elif kind == "latent_attention":
            dim, rot = pick([8, 16, 24, 64, 128]), pick([2, 4, 8, 16, 32, 64])
            mixer = {"heads": pick([1, 2, 3, 4, 6, 16]), "dim": dim, "rot_dim": rot,
                     "vdim": pick([8, 16, 32, 64, 80]),
                     "kv_rank": pick([8, 20, 32, 64, 96, 192, 272]),
                     "q_rank": pick([8, 24, 64, 128]),
                     "scale": pick([1.0, 2.0, 4.0]) / math.sqrt(dim + rot),
                     "mask": {"size": pick([1, 2, 5, 16, 17, 31, 40, 64, 90, 300])},
                     "rot": {"base": float(pick([100.0, 10000.0, 500000.0])), "dims": rot}}
        else:
            heads, dim = pick([1, 2, 3, 6]), pick([4, 8, 16, 32, 64, 128])
            mixer = {"heads": heads, "dim": dim, "vdim": pick([4, 8, 16, 32, 64, 136]),
                     "decay": [float(1.0 - 2.0 ** -pick([2, 4, 6, 9, 11])) for _ in range(heads)],
                     "rot": {"base": float(pick([50.0, 10000.0, 1000000.0])),
                             "dims": pick([d for d in (0, 2, 4, dim // 2, dim) if d % 2 == 0])}}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp()})
    config = {"architecture": "Medolorn", "vocab": pick([97, 256, 300]), "width": width,
              "norm": {"eps": float(pick([1e-6, 1e-5, 1e-3]))},
              "canon": {"taps": pick([1, 2, 3, 4, 5])}, "layers": layers}
    if rng.random() < 0.7:
        start = int(rng.integers(0, len(layers)))
        stop = int(rng.integers(start + 1, len(layers) + 1))
        config["loop"] = {"start": start, "stop": stop, "times": int(rng.integers(1, 4))}
    return config


def relative_error(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Per row: the root mean square of the difference (its mean taken off) over the spread of
    the wanted logits."""
    difference = got.astype(np.float64) - want
    difference -= difference.mean(axis=-1, keepdims=True)
    spread = want - want.mean(axis=-1, keepdims=True)
    return np.sqrt((difference ** 2).mean(axis=-1)) / np.sqrt((spread ** 2).mean())


@pytest.mark.parametrize("seed", range(int(os.environ.get("HELIX_SWEEP_SEEDS", "12"))))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configuration_in_mixed_batches(seed, dtype, model_root):
    config = draw_config(seed)
    folder = os.path.join(model_root, f"medolorn_sweep_{seed}_{dtype}")
    storage = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    write_model_folder(folder, config, tensors_for(config, 90 + seed, storage))
    model = plain_medolorn.PlainMedolorn.from_folder(folder)
    precision = "bfloat16" if dtype == "bfloat16" else "float64"
    # every third model also gets a long request fed in long portions
    long_one = seed % 3 == 0
    lengths = (1, 7, 45, 130, 77) + ((400,) if long_one else ())
    requests = {f"r{index}": random_tokens(config["vocab"], length, seed=seed * 10 + index)
                for index, length in enumerate(lengths)}
    expected = {name: model.forward(tokens, precision=precision)
                for name, tokens in requests.items()}
    # bfloat16: a row may differ by some per cent of the logits' spread, by a multiple of what
    # rounding the activations moves the plain logits, and where a router's choice is a close
    # call (with or without rounding) it only has to be finite
    moved, close = {}, {}
    if dtype == "bfloat16":
        for name, tokens in requests.items():
            margins = []
            for how in ("float64", "bfloat16"):
                model.margins = []
                exact = model.forward(tokens, precision=how)
                seen, model.margins = model.margins, None
                margins += seen
                if how == "float64":
                    moved[name] = relative_error(expected[name], exact)
            close[name] = np.min(np.stack(margins), axis=0) < 0.1 if margins else \
                np.zeros(len(tokens), dtype=bool)
    steps = traces.mixed(requests, max_live=3, seed=seed,
                         chunk_choices=(2, 3, 7, 16, 33, 64) + ((300, 129) if long_one else ()))
    page = int(np.random.default_rng(seed).choice([8, 16]))
    pages = -(-traces.live_token_need(steps, round_to=page) // page)
    harness = Harness(folder, dtype, page, num_pages=pages, max_requests=3, max_tokens=1024)
    positions = {}
    for step in steps:
        rows = traces.labels(step, positions)
        out = harness.run([(e["id"], e["tokens"], e["want"]) for e in step["entries"]])
        for name in step["end"]:
            harness.end(name)
        want = np.stack([expected[name][position] for name, position in rows])
        if dtype == "float32":
            assert_close(out, want, f"seed {seed} step {step['step']} rows {rows[:3]}",
                         atol=6e-4, rtol=6e-4)
        else:
            assert np.isfinite(out).all()
            error = relative_error(out, want.astype(np.float64))
            allowed = np.array([np.inf if close[name][position] else
                                max(0.08, 4.0 * moved[name][position]) for name, position in rows])
            bad = np.nonzero(error > allowed)[0]
            assert bad.size == 0, (f"seed {seed} step {step['step']}: row {rows[bad[0]]} differs by "
                                   f"{error[bad[0]]:.3f} of the logits' spread, allowed "
                                   f"{allowed[bad[0]]:.3f}")
    harness.cache.check()
    assert not harness.cache.live_requests()
