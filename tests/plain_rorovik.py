"""Plain, slow implementation of the Rorovik decoder: whole sequences, no cache, NumPy in
double precision, one function per mechanism.  It shares no code with the engine (own
safetensors reader, own order of layers, own masks).

Notation.  ``x [T, W]`` is the residual, ``m`` the residual multiplier, ``norm(x, w) = x /
sqrt(mean(x^2) + eps) * w``.  The token's row of the table passes ``norm(., embed.norm)``.  A
layer is

    x += m * norm(mixer(norm(x, n1)), n1b)
    x += m * norm(ff(norm(x, n2)), n2b)              (when the layer has a feed-forward)
    y = P (gelu_tanh(G x) * side[token, layer's piece]);  x += m * norm(y, ns)

Mixers (``h`` is the normed input):

* ``attention``: ``q = Wq h + bq`` and so on; q and k each pass one norm over the WHOLE
  projection (all heads at once); q times ``1 + coef * ln(floor((p + 1) / every) + 1)`` at
  position ``p``; scores ``q . k * scale - slope_h (i - j)`` with ``slope_h = 2^(-8 (h + 1) /
  H)`` over ``0 <= i - j < window``; the softmax's denominator also holds ``exp(sink_h)``;
  from the second value-mixing layer on ``v <- (1 - l) v + l v_first``; head ``h`` of the
  result times ``sigmoid(Wg h)_h``; the output matrix.
* ``latent_attention``: ``cq = norm(Wdq h, wq)``, ``q = Wuq cq`` (per head ``dim`` plain then
  ``rot_dim`` rotated coordinates); ``Wdkv h = [c' | kr]``, ``c = norm(c', wc)``; per head
  ``k = [Wuk c | rot(kr)]``, ``v = Wuv c``; pairs ``(2i, 2i + 1)`` rotated with stretched
  frequencies and an amplitude; causal; a sink in the denominator; the output matrix.

Feed-forward: dense ``Wd (relu(Wg h + bg) * (Wu h + bu)) + bd``, or routed experts: ``s =
softmax(R h)`` over experts and identity outputs, choice by ``s + correction``, weights ``s`` of
the chosen (not renormed); expert ``Wd (g sigmoid(1.702 g) (u + 1))`` with ``g = min(Wg h, L)``,
``u = clamp(Wu h, -L, L)``; an identity output returns ``h``.

``precision="bfloat16"`` rounds activations to bfloat16 where a bfloat16 engine stores them;
sums, norms, scores and the residual stay in double.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Callable, Dict, List, Optional

import numpy as np


def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    with open(path, "rb") as source:
        (length,) = struct.unpack("<Q", source.read(8))
        header = json.loads(source.read(length).decode("utf-8"))
        payload = source.read()
    header.pop("__metadata__", None)
    tensors = {}
    for name, record in header.items():
        begin, end = record["data_offsets"]
        raw = payload[begin:end]
        if record["dtype"] == "F32":
            value = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif record["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << np.uint32(16)
            value = bits.view(np.float32).astype(np.float64)
        elif record["dtype"] == "I32":
            value = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"unsupported dtype {record['dtype']}")
        tensors[name] = value.reshape(tuple(record["shape"]))
    return tensors


def to_bfloat16(values: np.ndarray) -> np.ndarray:
    """Round to the nearest bfloat16 (ties to even), returned as float64."""
    bits = np.asarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(values))


def identity(values: np.ndarray) -> np.ndarray:
    return values


# ------------------------------------------------------------------- small functions

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * weight


# ------------------------------------------------------------------- mechanisms

def query_temperature(positions: np.ndarray, coef: float, every: int) -> np.ndarray:
    """The factor on the query at each position: ``1 + coef ln(floor((p + 1) / every) + 1)``."""
    return 1.0 + coef * np.log(np.floor((positions + 1) / every) + 1.0)


def head_slopes(heads: int) -> np.ndarray:
    return np.array([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)])


def sink_softmax_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float,
                           sink: np.ndarray, window: Optional[int] = None,
                           slopes: Optional[np.ndarray] = None, first: int = 0) -> np.ndarray:
    """``q [T, H, D]``, ``k [S, H, D]``, ``v [S, H, E]`` (keys already spread over the query
    heads); query ``t`` stands at position ``first + t``, key ``j`` at ``j``.  Returns ``[T, H,
    E]``.  The denominator of every row also holds ``exp(sink_h)``."""
    T, H, _ = q.shape
    out = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        i = first + t
        lo = 0 if window is None else max(0, i - window + 1)
        js = np.arange(lo, i + 1)
        for h in range(H):
            s = (k[js, h] @ q[t, h]) * scale
            if slopes is not None:
                s = s - slopes[h] * (i - js)
            top = max(s.max(), sink[h])
            e = np.exp(s - top)
            out[t, h] = (e @ v[js, h]) / (e.sum() + math.exp(sink[h] - top))
    return out


def stretched_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """Frequencies of the rotated pairs and the amplitude of cos and sin.  Without scaling
    ``f_i = base^(-2i/dims)`` and 1.  With it, pair ``i`` keeps ``f_i`` below ``lo``, takes
    ``f_i / factor`` above ``hi`` and a blend between; ``lo`` and ``hi`` are the pairs whose
    wavelengths fit ``fast`` and ``slow`` times into the original length."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x: np.ndarray, positions: np.ndarray, freq: np.ndarray,
                       amplitude: float) -> np.ndarray:
    """``x [T, ..., D]``: the first ``2 len(freq)`` coordinates in pairs ``(2i, 2i + 1)``."""
    out = np.array(x, dtype=np.float64, copy=True)
    n = 2 * len(freq)
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (len(freq),)
    angle = (positions[:, None] * freq[None, :]).reshape(shape)
    c, s = np.cos(angle) * amplitude, np.sin(angle) * amplitude
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


def attention_mixer(h: np.ndarray, weights: Dict[str, np.ndarray], prefix: str, mixer: dict,
                    eps: float, positions: np.ndarray, rnd: Callable, v_first, state: dict):
    """The ``attention`` mixer over a whole sequence; ``state['v_first']`` carries the first
    value-mixing layer's values to the later ones."""
    w = lambda name: weights[f"{prefix}.mix.{name}"]
    H, G, D, E = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    T = h.shape[0]
    q = h @ w("q").T + w("q.b")
    k = h @ w("k").T + w("k.b")
    v = rnd(h @ w("v").T + w("v.b"))
    q = rms_norm(q, w("q.norm"), eps)
    k = rnd(rms_norm(k, w("k.norm"), eps))
    temp = mixer.get("q_temp")
    if temp:
        q = q * query_temperature(positions, temp["coef"], temp["every"])[:, None]
    q = rnd(q)
    if mixer.get("v_mix"):
        if "v_first" in state:
            lam = float(w("vmix"))
            v = rnd((1.0 - lam) * v + lam * state["v_first"])
        else:
            state["v_first"] = v
    share = H // G
    kh = k.reshape(T, G, D)[:, np.arange(H) // share]
    vh = v.reshape(T, G, E)[:, np.arange(H) // share]
    window = (mixer.get("mask") or {}).get("size")
    o = sink_softmax_attention(q.reshape(T, H, D), kh, vh, mixer["scale"], w("sink"), window,
                               head_slopes(H))
    gate = sigmoid(h @ w("g").T)                       # [T, H]
    o = rnd(rnd(o) * gate[:, :, None]).reshape(T, H * E)
    return o @ w("o").T


def latent_attention_mixer(h: np.ndarray, weights: Dict[str, np.ndarray], prefix: str,
                           mixer: dict, eps: float, positions: np.ndarray, rnd: Callable):
    w = lambda name: weights[f"{prefix}.mix.{name}"]
    H, D, R, E, C = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    T = h.shape[0]
    cq = rnd(rms_norm(h @ w("dq").T, w("dq.norm"), eps))
    q = rnd(cq @ w("uq").T).reshape(T, H, D + R)
    down = h @ w("dkv").T
    c = rnd(rms_norm(down[:, :C], w("dkv.norm"), eps))
    rot = mixer.get("rot") or {}
    freq, amplitude = stretched_frequencies(rot.get("dims", R), rot.get("base", 10000.0),
                                            rot.get("scaling"))
    kr = rnd(rotate_interleaved(down[:, C:], positions, freq, amplitude))
    qr = rotate_interleaved(q[:, :, D:], positions, freq, amplitude)
    keys = (c @ w("uk").T).reshape(T, H, D)
    values = (c @ w("uv").T).reshape(T, H, E)
    full_q = np.concatenate([q[:, :, :D], qr], axis=2)
    full_k = np.concatenate([keys, np.broadcast_to(kr[:, None, :], (T, H, R))], axis=2)
    o = sink_softmax_attention(full_q, full_k, values, mixer["scale"], w("sink"))
    return rnd(o).reshape(T, H * E) @ w("o").T


def dense_feed_forward(h, weights, prefix, rnd):
    w = lambda name: weights[f"{prefix}.mlp.{name}"]
    gate = h @ w("gate").T + w("gate.b")
    up = h @ w("up").T + w("up.b")
    return rnd(np.maximum(gate, 0.0) * up) @ w("down").T + w("down.b")


def router_choice(h, weights, prefix, router: dict):
    """Scores over all router outputs, the chosen indices ``[T, top]`` (largest choice score
    first, the lowest index among equals) and the margin between the last chosen and the best
    one left out."""
    z = h @ weights[f"{prefix}.mlp.router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    choice = s + weights[f"{prefix}.mlp.correction"]
    order = np.argsort(-choice, axis=-1, kind="stable")
    top = router["top"]
    chosen = order[:, :top]
    ranked = np.take_along_axis(choice, order, axis=-1)
    margin = ranked[:, top - 1] - ranked[:, top] if choice.shape[1] > top else \
        np.full(h.shape[0], np.inf)
    return s, chosen, margin


def expert(hrow, weights, prefix, index: int, limit: float, rnd):
    w = lambda name: weights[f"{prefix}.mlp.e{index}.{name}"]
    g = np.minimum(w("gate") @ hrow, limit)
    u = np.clip(w("up") @ hrow, -limit, limit)
    return w("down") @ rnd(g * sigmoid(1.702 * g) * (u + 1.0))


def routed_feed_forward(h, weights, prefix, mlp: dict, rnd, margins: Optional[list] = None):
    router = mlp["router"]
    experts = router["experts"]
    s, chosen, margin = router_choice(h, weights, prefix, router)
    if margins is not None:
        margins.append(margin)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t]:
            if e >= experts:
                out[t] += s[t, e] * h[t]
            else:
                out[t] += s[t, e] * expert(h[t], weights, prefix, int(e), mlp["expert"]["limit"], rnd)
    return out


def token_side_input(x, tokens, weights, prefix, layer: int, dim: int, eps: float, rnd):
    e = weights["side.embed"][tokens, layer * dim:(layer + 1) * dim]
    g = rnd(gelu_tanh(rnd(x) @ weights[f"{prefix}.side.gate"].T) * e)
    y = g @ weights[f"{prefix}.side.proj"].T
    return rms_norm(y, weights[f"{prefix}.side.norm"], eps)


# ------------------------------------------------------------------------- the model

class PlainRorovik:
    def __init__(self, config: dict, weights: Dict[str, np.ndarray], precision: str = "float32"):
        self.config = config
        self.weights = weights
        self.rnd = to_bfloat16 if precision == "bfloat16" else identity
        self.eps = float(config["norm"]["eps"])
        self.m = float(config.get("residual_mult", 1.0))
        self.router_margins: List[np.ndarray] = []

    @classmethod
    def from_dir(cls, path: str, precision: str = "float32") -> "PlainRorovik":
        with open(os.path.join(path, "config.json")) as source:
            config = json.load(source)
        return cls(config, read_safetensors(os.path.join(path, "model.safetensors")), precision)

    def forward(self, tokens, layers_out: Optional[list] = None) -> np.ndarray:
        """Logits ``[T, vocab]`` of a whole sequence; ``layers_out`` collects the residual after
        every layer."""
        w, rnd, eps, m = self.weights, self.rnd, self.eps, self.m
        tokens = np.asarray(tokens, dtype=np.int64)
        positions = np.arange(len(tokens), dtype=np.float64)
        x = rms_norm(w["embed"][tokens], w["embed.norm"], eps)
        state: dict = {}
        side = self.config.get("token_side")
        self.router_margins = []
        for index, layer in enumerate(self.config["layers"]):
            prefix = f"l{index}"
            h = rnd(rms_norm(x, w[f"{prefix}.norm1"], eps))
            if layer["type"] == "attention":
                y = attention_mixer(h, w, prefix, layer["mixer"], eps, positions, rnd, None, state)
            elif layer["type"] == "latent_attention":
                y = latent_attention_mixer(h, w, prefix, layer["mixer"], eps, positions, rnd)
            else:
                raise ValueError(f"unknown mixer {layer['type']!r}")
            x = x + m * rms_norm(y, w[f"{prefix}.norm1b"], eps)
            mlp = layer.get("mlp")
            if mlp is not None:
                h = rnd(rms_norm(x, w[f"{prefix}.norm2"], eps))
                if mlp["kind"] == "dense":
                    y = dense_feed_forward(h, w, prefix, rnd)
                else:
                    y = routed_feed_forward(h, w, prefix, mlp, rnd, self.router_margins)
                x = x + m * rms_norm(y, w[f"{prefix}.norm2b"], eps)
            if side:
                x = x + m * token_side_input(x, tokens, w, prefix, index, int(side["dim"]), eps, rnd)
            if layers_out is not None:
                layers_out.append(x.copy())
        x = rnd(rms_norm(x, w["final.norm"], eps))
        return x @ w["head"].T
