"""Edges of the Medolorn mixers, made visible on purpose.  The models here have ONE layer, so
what a position can see is exactly what its mixer lets through: swapping one earlier token
changes a later position's plain logits if and only if the mixer still sees that token.  The
tests look for a swap whose effect is large, check that the plain implementation shows it just
inside the edge and nothing just outside, and ask the engine for the same logits, in prompts,
in portions that end at the edge, and in tokens decoded one by one.
"""
from __future__ import annotations

import os

import numpy as np
import pytest
import torch

import plain_medolorn
from conftest import random_tokens
from engine_harness import Harness, assert_close
from medolorn_configs import _delta, _latent, tensors_for
from helix_runtime_b200.weights.random_init import write_model_folder

pytestmark = pytest.mark.gpu

WINDOW, PAGE = 19, 8
LATENT_ONLY = {
    "architecture": "Medolorn", "vocab": 60, "width": 64, "norm": {"eps": 1e-5},
    "canon": {"taps": 2},
    "layers": [_latent(2, 16, 8, 16, 24, 16, WINDOW, 100.0, None, sharp=12.0)],
}
DELTA_ONLY = {
    "architecture": "Medolorn", "vocab": 60, "width": 64, "norm": {"eps": 1e-5},
    "canon": {"taps": 1},
    "layers": [_delta(2, 1, 24, 16, 3, None)],
}


def folder_for(root: str, name: str, config: dict, adjust=None) -> str:
    path = os.path.join(root, f"medolorn_edge_{name}")
    if not os.path.exists(os.path.join(path, "model.safetensors")):
        tensors = tensors_for(config, 77, torch.float32)
        if adjust is not None:
            adjust(tensors)
        write_model_folder(path, config, tensors)
    return path


def ways_of_feeding(length: int, edge: int):
    """Portions per way: whole; a portion that ends right at ``edge`` and one that starts
    there; two-token portions around it; everything from ``edge - 3`` on decoded one by one."""
    return {
        "whole": [length],
        "cut at the edge": [edge, length - edge],
        "cut behind the edge": [edge + 1, length - edge - 1],
        "pairs": [edge - 3, 2, 2, 2, length - edge - 3],
        "decoded": [edge - 3] + [1] * (length - edge + 3),
    }


def engine_logits(harness: Harness, tokens, portions) -> np.ndarray:
    rows, cursor = [], 0
    for size in portions:
        rows.append(harness.run([("a", tokens[cursor:cursor + size], range(size))]))
        cursor += size
    harness.end("a")
    assert cursor == len(tokens)
    return np.concatenate(rows)


def test_a_key_at_the_windows_edge(model_root):
    folder = folder_for(model_root, "latent", LATENT_ONLY)
    plain = plain_medolorn.PlainMedolorn.from_folder(folder)
    place, length = 11, 11 + WINDOW + 6
    inside, outside = place + WINDOW - 1, place + WINDOW
    best = None
    for seed in range(12):
        tokens = random_tokens(60, length, seed=seed)
        other = list(tokens)
        other[place] = (tokens[place] + 17) % 60
        a, b = plain.forward(tokens), plain.forward(other)
        effect = float(np.abs(a[inside] - b[inside]).max())
        # the filter of two taps reaches one token back, so `place + 1` sees the swap too
        assert np.abs(a[outside + 1:] - b[outside + 1:]).max() == 0.0
        if best is None or effect > best[0]:
            best = (effect, tokens, other, a, b)
    effect, tokens, other, a, b = best
    assert effect > 0.05, "no swap shows at the window's edge; the test would prove nothing"
    harness = Harness(folder, "float32", PAGE, num_pages=16, max_requests=1)
    for way, portions in ways_of_feeding(length, outside).items():
        got_a = engine_logits(harness, tokens, portions)
        got_b = engine_logits(harness, other, portions)
        assert_close(got_a, a, f"{way}", atol=4e-4, rtol=4e-4)
        assert_close(got_b, b, f"{way}, swapped", atol=4e-4, rtol=4e-4)
        # one token further the swapped key is out of sight: the same logits, to rounding
        assert_close(got_a[outside + 1:], got_b[outside + 1:], f"{way}, outside", atol=2e-5, rtol=0.0)


def test_the_first_token_stays_in_a_slow_delta_state(model_root):
    """Heads that hardly decay (what fades the first token is only that later writes replace
    part of it): it still shows 160 tokens later, 120 of them decoded alone."""
    def slow(tensors):
        tensors["l0.mix.A_log"] = torch.tensor([-7.0, -6.0])
        tensors["l0.mix.dt_bias"] = torch.tensor([-2.0, -1.0])
        tensors["l0.mix.b"] = tensors["l0.mix.b"] * 0.2            # writes of about one half
    folder = folder_for(model_root, "delta", DELTA_ONLY, slow)
    plain = plain_medolorn.PlainMedolorn.from_folder(folder)
    length = 160
    tokens = random_tokens(60, length, seed=2)
    other = [(tokens[0] + 9) % 60] + tokens[1:]
    a, b = plain.forward(tokens), plain.forward(other)
    effect = float(np.abs(a[-1] - b[-1]).max())
    assert effect > 3e-3, f"the first token's effect at the end is only {effect:.1e}"
    harness = Harness(folder, "float32", PAGE, num_pages=4, max_requests=1)
    for way, portions in {"whole": [length], "portions": [64, 2, 43, 1, 50],
                          "decoded": [40] + [1] * 120}.items():
        # a tolerance well below the effect
        assert_close(engine_logits(harness, tokens, portions), a, way, atol=2e-4, rtol=1e-4)
        assert_close(engine_logits(harness, other, portions), b, f"{way}, swapped", atol=2e-4, rtol=1e-4)
