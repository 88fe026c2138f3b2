"""Randomly drawn Rorovik configurations through the engine against the plain implementation:
the order and number of layers, every size of the two mixers (heads, grouped key/value heads,
head and value sizes up to 136, windows of 1 to 300 or none, query temperatures, value mixing in
some, all or none of the layers; latents smaller and larger than a head, cached rows beyond what
the tensor-core attention takes, partly rotated parts, stretched frequencies whose original
length the prompts pass or never reach), dense feed-forwards, routers of 1 to 45 outputs with
and without identity outputs that use 1 to 6 of them, layers without a feed-forward, with and
without the per-layer token input, residual factors of either sign, and every model is replayed
as mixed batches over a pool made for its live requests only."""
from __future__ import annotations

import math
import os

import numpy as np
import pytest
import torch

import plain_rorovik
import traces
from conftest import random_tokens
from engine_harness import Harness, assert_close
from helix_runtime_b200.weights.random_init import write_model_folder
from rorovik_configs import tensors_for

pytestmark = pytest.mark.gpu


def draw_config(seed: int):
    rng = np.random.default_rng(7000 + seed)
    pick = lambda values: values[int(rng.integers(0, len(values)))]
    width = pick([40, 64, 72, 100, 128, 136, 256])

    def mlp():
        roll = rng.random()
        if roll < 0.15:
            return None
        if roll < 0.4:
            return {"kind": "dense", "ff": pick([8, 20, 48, 100, 128, 256])}
        experts, identity = pick([1, 2, 3, 8, 16, 40]), pick([0, 0, 1, 2, 5])
        return {"kind": "moe",
                "expert": {"ff": pick([8, 20, 48, 64, 100, 128]),
                           "limit": float(pick([0.4, 1.0, 1.5, 7.0]))},
                "router": {"experts": experts, "identity": identity,
                           "top": int(rng.integers(1, min(experts + identity, 6) + 1))}}

    value_row = pick([16, 32, 48, 64, 128])       # kv_heads * vdim of the value-mixing layers
    layers = []
    for _ in range(int(rng.integers(1, 6))):
        kind = pick(["attention", "attention", "latent_attention"])
        if kind == "attention":
            dim = pick([4, 8, 20, 32, 64, 100, 128])
            v_mix = rng.random() < 0.6
            if v_mix:
                kv_heads = pick([h for h in (1, 2, 4) if value_row % h == 0])
                vdim = value_row // kv_heads
            else:
                kv_heads, vdim = pick([1, 2, 3]), pick([4, 8, 24, 32, 64, 136])
            mixer = {"heads": kv_heads * pick([1, 2, 3, 4]), "kv_heads": kv_heads, "dim": dim,
                     "vdim": vdim, "scale": pick([1.0, 2.0, 3.0]) / math.sqrt(dim), "v_mix": v_mix}
            if rng.random() < 0.85:
                mixer["mask"] = {"size": pick([1, 2, 5, 16, 17, 31, 40, 64, 90, 300])}
            if rng.random() < 0.8:
                mixer["q_temp"] = {"coef": float(pick([0.1, 0.5, 1.0])),
                                   "every": pick([1, 3, 16, 50, 256])}
        else:
            dim, rot = pick([8, 16, 24, 64, 128]), pick([2, 4, 8, 16, 32, 64])
            mixer = {"heads": pick([1, 2, 3, 4, 6, 16]), "dim": dim, "rot_dim": rot,
                     "vdim": pick([8, 16, 32, 64, 80]),
                     "kv_rank": pick([8, 20, 32, 64, 96, 192, 272]),
                     "q_rank": pick([8, 24, 64, 128]),
                     "scale": pick([1.0, 2.0, 4.0]) / math.sqrt(dim + rot),
                     "rot": {"base": float(pick([100.0, 10000.0, 500000.0])),
                             "dims": pick([d for d in (2, rot // 2, rot) if d % 2 == 0 and d > 0])}}
            if rng.random() < 0.75:
                mixer["rot"]["scaling"] = {"factor": float(pick([1.5, 4.0, 8.0, 40.0])),
                                           "original": pick([8, 32, 64, 512]),
                                           "fast": float(pick([1.0, 4.0, 32.0])),
                                           "slow": float(pick([0.25, 1.0, 2.0]))}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp()})
    config = {"architecture": "Rorovik", "vocab": pick([97, 256, 300]), "width": width,
              "norm": {"eps": float(pick([1e-6, 1e-5, 1e-3]))},
              "residual_mult": float(pick([1.0, 0.3, 0.7, -0.5])), "layers": layers}
    if rng.random() < 0.8:
        # (a token input of a few numbers is normed to little more than their signs: where all of
        # its gates are near zero, whatever rounds differently turns it, in any implementation)
        config["token_side"] = {"dim": pick([8, 16, 24, 40])}
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
    folder = os.path.join(model_root, f"rorovik_sweep_{seed}_{dtype}")
    storage = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    write_model_folder(folder, config, tensors_for(config, 90 + seed, storage))
    model = plain_rorovik.PlainRorovik.from_dir(folder, dtype)
    exact_model = plain_rorovik.PlainRorovik.from_dir(folder, "float32")
    # every third model also gets a long request fed in long portions
    long_one = seed % 3 == 0
    lengths = (1, 7, 45, 130, 77) + ((400,) if long_one else ())
    requests = {f"r{index}": random_tokens(config["vocab"], length, seed=seed * 10 + index)
                for index, length in enumerate(lengths)}
    expected = {name: model.forward(tokens) for name, tokens in requests.items()}
    # bfloat16: a row may differ by some per cent of the logits' spread, by a multiple of what
    # rounding the activations moves the plain logits, and from the first position on at which
    # a router's choice is a close call (with or without rounding) a request's rows only have to
    # be finite: there rounding decides which expert runs, and later positions attend to it.
    # The float32 run of the same model holds every row.
    moved, close = {}, {}
    if dtype == "bfloat16":
        for name, tokens in requests.items():
            margins = []
            for which in (exact_model, model):
                logits = which.forward(tokens)
                margins += which.router_margins
                if which is exact_model:
                    moved[name] = relative_error(expected[name], logits)
            # a close call changes the token's own row and, through the attention of the
            # layers behind it, the rows of the positions after it
            close[name] = np.maximum.accumulate(np.min(np.stack(margins), axis=0) < 0.01) \
                if margins else np.zeros(len(tokens), dtype=bool)
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
