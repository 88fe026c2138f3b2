"""Plain, slow implementation of the Medolorn decoder: whole sequences, no cache, NumPy in
double precision, one function per mechanism.  It shares no code with the engine (own
safetensors reader, own order of layers, own masks, own recurrences written token by token).

Notation.  ``x [T, W]`` is the residual, ``x0`` the embedding's output (token row through the
model's norm).  ``norm(x) = x / sqrt(mean(x^2) + eps) * (1 + w)``.  A layer is

    h = norm1(x);  x += sigmoid(R1 h + r1) * mixer(h + conv(h))
    h = norm2(x);  x += sigmoid(R2 h + r2) * ff(h)

with ``conv`` a causal per-channel filter over time.  Before every pass of the looped layers
``x <- Win [x ; x0] + step[pass]``.

Mixers (``h`` is what the layer hands over):

* ``delta``: q, k (``kv_heads`` heads of ``dim``) and v (``heads`` of ``vdim``) each pass a
  causal filter and silu; q and k become unit vectors (``/ sqrt(sum sq + 1e-6)``), q times
  ``dim^-1/2``; ``beta = sigmoid(Wb h)``, ``g = exp(-exp(A) softplus(Wa h + dt))`` per head;
  ``S <- g S; u = beta (v - S' k); S <- S + k u'; o = S' q``; ``o / rms(o) * w * silu(Wg h)``.
* ``latent_attention``: ``cq = rms(Wdq h) wq``, ``q = Wuq cq`` (per head ``dim`` plain then
  ``rot_dim`` rotated coordinates); ``Wdkv h = [c' | kr]``, ``c = rms(c') wc``; per head
  ``k = [Wuk c | rot(kr)]``, ``v = Wuv c``; softmax over the last ``window`` keys; the heads
  times ``sigmoid(Wg h)``.  Pairs ``(2i, 2i + 1)`` are rotated.
* ``retention``: q, k rotated over their first ``dims`` coordinates in pairs ``(i, i + dims/2)``,
  k times ``dim^-1/2``; ``S <- decay S + k v'; o = S' q``; ``o / rms(o) * silu(Wg h)``.

Feed-forward: ``s = sigmoid(Wr h)``; the ``top`` largest; weights ``s / (sum + 1e-20) * scale``;
experts ``Wdown (silu(Wgate h) * (Wup h))``.

``precision="bfloat16"`` rounds activations to bfloat16 where a bfloat16 engine stores them;
sums, recurrences, norms, scores and the residual stay in double.
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

def softplus(z):
    return np.logaddexp(0.0, z)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x: np.ndarray, eps: float) -> np.ndarray:
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def norm_one_plus(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    return unit_rms(x, eps) * (1.0 + weight)


def norm_plain(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    return unit_rms(x, eps) * weight


# ------------------------------------------------------------------- mechanisms

def causal_filter(u: np.ndarray, taps: np.ndarray) -> np.ndarray:
    """``u [T, C]``, ``taps [C, n]`` with the last column on the token itself, zeros before the
    sequence: ``y[t, c] = sum_j taps[c, j] u[t - (n - 1) + j, c]``."""
    length, n = u.shape[0], taps.shape[1]
    out = np.zeros_like(u, dtype=np.float64)
    for t in range(length):
        for j in range(n):
            source = t - (n - 1) + j
            if source >= 0:
                out[t] += taps[:, j] * u[source]
    return out


def rotate_pairs(x: np.ndarray, positions: np.ndarray, base: float, dims: int,
                 layout: str) -> np.ndarray:
    """``x [T, H, D]``: the first ``dims`` coordinates of every head turned by ``p * f_i``,
    ``f_i = base^(-2i/dims)``; ``layout`` ``interleaved`` pairs ``(2i, 2i+1)``, ``halves`` pairs
    ``(i, i + dims/2)``.  The pair ``(u, v)`` becomes ``(u cos - v sin, v cos + u sin)``."""
    out = np.array(x, dtype=np.float64, copy=True)
    half = dims // 2
    for i in range(half):
        first, second = (2 * i, 2 * i + 1) if layout == "interleaved" else (i, i + half)
        angle = positions.astype(np.float64) * base ** (-2.0 * i / dims)
        cos, sin = np.cos(angle)[:, None], np.sin(angle)[:, None]
        u, v = x[:, :, first], x[:, :, second]
        out[:, :, first] = u * cos - v * sin
        out[:, :, second] = v * cos + u * sin
    return out


def windowed_softmax_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float,
                               window: int) -> np.ndarray:
    """``q, k [T, H, D]``, ``v [T, H, V]``: position ``i`` sees ``j`` with ``0 <= i - j < window``."""
    length, heads = q.shape[0], q.shape[1]
    out = np.zeros((length, heads, v.shape[2]))
    for i in range(length):
        low = max(0, i - window + 1)
        for h in range(heads):
            scores = (k[low:i + 1, h] @ q[i, h]) * scale
            weights = np.exp(scores - scores.max())
            weights /= weights.sum()
            out[i, h] = weights @ v[low:i + 1, h]
    return out


def delta_rule_scan(q: np.ndarray, k: np.ndarray, v: np.ndarray, beta: np.ndarray,
                    decay: np.ndarray) -> np.ndarray:
    """``q, k [T, H, D]``, ``v [T, H, V]``, ``beta, decay [T, H]``, token by token:
    ``S <- g S; u = beta (v - S' k); S <- S + k u'; o = S' q``."""
    length, heads, dim = q.shape
    out = np.zeros((length, heads, v.shape[2]))
    for h in range(heads):
        state = np.zeros((dim, v.shape[2]))
        for t in range(length):
            state = decay[t, h] * state
            u = beta[t, h] * (v[t, h] - state.T @ k[t, h])
            state = state + np.outer(k[t, h], u)
            out[t, h] = state.T @ q[t, h]
    return out


def retention_scan(q: np.ndarray, k: np.ndarray, v: np.ndarray, decay: np.ndarray) -> np.ndarray:
    """``S_t = decay_h S_(t-1) + k_t v_t'``, ``o_t = S_t' q_t``; ``decay [H]``."""
    length, heads, dim = q.shape
    out = np.zeros((length, heads, v.shape[2]))
    for h in range(heads):
        state = np.zeros((dim, v.shape[2]))
        for t in range(length):
            state = decay[h] * state + np.outer(k[t, h], v[t, h])
            out[t, h] = state.T @ q[t, h]
    return out


def router_margins(h: np.ndarray, router: np.ndarray, top: int) -> np.ndarray:
    """Per token, how far the router's sum of the last chosen expert lies above that of the best
    one left out (infinite when every expert is chosen): a small margin is a close call."""
    sums = np.sort(h @ router.T, axis=1)[:, ::-1]
    if top >= sums.shape[1]:
        return np.full(h.shape[0], np.inf)
    return sums[:, top - 1] - sums[:, top]


def routed_experts(h: np.ndarray, router: np.ndarray, experts: List[Dict[str, np.ndarray]],
                   top: int, scale: float, rnd: Callable) -> np.ndarray:
    """Sigmoid scores, the ``top`` largest, normalised to sum one, times ``scale``."""
    scores = sigmoid(h @ router.T)
    out = np.zeros((h.shape[0], experts[0]["down"].shape[0]))
    for t in range(h.shape[0]):
        chosen = np.argsort(-scores[t], kind="stable")[:top]
        weights = scores[t, chosen] / (scores[t, chosen].sum() + 1e-20) * scale
        for weight, e in zip(weights, chosen):
            expert = experts[e]
            act = rnd(silu(h[t] @ expert["gate"].T) * (h[t] @ expert["up"].T))
            out[t] += weight * (act @ expert["down"].T)
    return out


# ------------------------------------------------------------------------ the model

class PlainMedolorn:
    def __init__(self, config: dict, tensors: Dict[str, np.ndarray]) -> None:
        self.c = config
        self.t = tensors
        self.eps = float(config["norm"]["eps"])
        self.width = int(config["width"])
        self.taps = int(config["canon"]["taps"])
        # a list: every run of a feed-forward appends its tokens' router margins
        self.margins: Optional[List[np.ndarray]] = None

    @classmethod
    def from_folder(cls, folder: str) -> "PlainMedolorn":
        with open(os.path.join(folder, "config.json")) as source:
            config = json.load(source)
        return cls(config, read_safetensors(os.path.join(folder, "model.safetensors")))

    # ------------------------------------------------------------------ mixers

    def delta(self, p: str, m: dict, h: np.ndarray, rnd: Callable) -> np.ndarray:
        t = self.t
        heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        length = h.shape[0]

        def filtered(name):
            return rnd(silu(causal_filter(rnd(h @ t[f"{p}.{name}"].T), t[f"{p}.{name}.conv"])))
        q = filtered("q").reshape(length, kv_heads, dim)
        k = filtered("k").reshape(length, kv_heads, dim)
        v = filtered("v").reshape(length, heads, vdim)
        q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
        k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
        share = heads // kv_heads
        q, k = np.repeat(q, share, axis=1), np.repeat(k, share, axis=1)
        beta = sigmoid(rnd(h @ t[f"{p}.b"].T))
        decay = np.exp(-np.exp(t[f"{p}.A_log"]) * softplus(rnd(h @ t[f"{p}.a"].T) + t[f"{p}.dt_bias"]))
        o = delta_rule_scan(q, k, v, beta, decay)
        o = unit_rms(o, self.eps) * t[f"{p}.norm"]
        o = rnd(o.reshape(length, heads * vdim) * silu(rnd(h @ t[f"{p}.g"].T)))
        return o @ t[f"{p}.o"].T

    def latent_attention(self, p: str, m: dict, h: np.ndarray, rnd: Callable) -> np.ndarray:
        t = self.t
        heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        length = h.shape[0]
        positions = np.arange(length)
        base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
        cq = rnd(norm_plain(h @ t[f"{p}.dq"].T, t[f"{p}.dq.norm"], self.eps))
        q = rnd(cq @ t[f"{p}.uq"].T).reshape(length, heads, dim + rot)
        down = h @ t[f"{p}.dkv"].T
        c = rnd(norm_plain(down[:, :rank], t[f"{p}.dkv.norm"], self.eps))
        shared = rnd(down[:, rank:]).reshape(length, 1, rot)
        q_rot = rotate_pairs(q[:, :, dim:], positions, base, dims, "interleaved")
        k_rot = rotate_pairs(shared, positions, base, dims, "interleaved")
        k_plain = rnd(c @ t[f"{p}.uk"].T).reshape(length, heads, dim)
        v = rnd(c @ t[f"{p}.uv"].T).reshape(length, heads, vdim)
        qf = np.concatenate([q[:, :, :dim], rnd(q_rot)], axis=2)
        kf = np.concatenate([k_plain, np.repeat(rnd(k_rot), heads, axis=1)], axis=2)
        o = windowed_softmax_attention(qf, kf, v, float(m["scale"]), int(m["mask"]["size"]))
        o = rnd(rnd(o).reshape(length, heads * vdim) * sigmoid(rnd(h @ t[f"{p}.g"].T)))
        return o @ t[f"{p}.o"].T

    def retention(self, p: str, m: dict, h: np.ndarray, rnd: Callable) -> np.ndarray:
        t = self.t
        heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
        length = h.shape[0]
        positions = np.arange(length)
        base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
        q = rnd(h @ t[f"{p}.q"].T).reshape(length, heads, dim)
        k = rnd(h @ t[f"{p}.k"].T).reshape(length, heads, dim)
        v = rnd(h @ t[f"{p}.v"].T).reshape(length, heads, vdim)
        q = rotate_pairs(q, positions, base, dims, "halves")
        k = rotate_pairs(k, positions, base, dims, "halves") * dim ** -0.5
        o = retention_scan(q, k, v, np.asarray(m["decay"], dtype=np.float64))
        o = unit_rms(o, self.eps).reshape(length, heads * vdim)
        o = rnd(o * silu(rnd(h @ t[f"{p}.g"].T)))
        return o @ t[f"{p}.o"].T

    # ------------------------------------------------------------------- layers

    def feed_forward(self, p: str, m: dict, h: np.ndarray, rnd: Callable) -> np.ndarray:
        router = m["router"]
        experts = [{name: self.t[f"{p}.e{e}.{name}"] for name in ("gate", "up", "down")}
                   for e in range(int(router["experts"]))]
        if self.margins is not None:
            self.margins.append(router_margins(h, self.t[f"{p}.router"], int(router["top"])))
        return routed_experts(h, self.t[f"{p}.router"], experts, int(router["top"]),
                              float(router["scale"]), rnd)

    def layer(self, index: int, x: np.ndarray, rnd: Callable) -> np.ndarray:
        t, p = self.t, f"l{index}"
        layer = self.c["layers"][index]
        h = rnd(norm_one_plus(x, t[f"{p}.norm1"], self.eps))
        gate = sigmoid(h @ t[f"{p}.rg1"].T + t[f"{p}.rg1.b"])
        mixed = rnd(h + causal_filter(h, t[f"{p}.canon1"]))
        y = getattr(self, layer["type"])(f"{p}.mix", layer["mixer"], mixed, rnd)
        x = x + gate * y
        if layer.get("mlp") is not None:
            h = rnd(norm_one_plus(x, t[f"{p}.norm2"], self.eps))
            gate = sigmoid(h @ t[f"{p}.rg2"].T + t[f"{p}.rg2.b"])
            x = x + gate * self.feed_forward(f"{p}.mlp", layer["mlp"], h, rnd)
        return x

    def forward(self, tokens, precision: str = "float64", after_layer=None) -> np.ndarray:
        """Logits ``[T, vocab]`` of one whole sequence."""
        rnd = to_bfloat16 if precision == "bfloat16" else identity
        t = self.t
        x = norm_one_plus(t["embed"][np.asarray(tokens, dtype=np.int64)], t["embed.norm"], self.eps)
        x0 = x
        count = len(self.c["layers"])
        loop = self.c.get("loop")
        runs: List[tuple] = []          # (layer, pass that starts here or None)
        if loop is None:
            runs = [(i, None) for i in range(count)]
        else:
            runs = [(i, None) for i in range(loop["start"])]
            for number in range(loop["times"]):
                for i in range(loop["start"], loop["stop"]):
                    runs.append((i, number if i == loop["start"] else None))
            runs += [(i, None) for i in range(loop["stop"], count)]
        for run, (index, starts) in enumerate(runs):
            if starts is not None:
                joined = np.concatenate([rnd(x), rnd(x0)], axis=1)
                x = joined @ t["loop.in"].T + t["loop.step"][starts]
            x = self.layer(index, x, rnd)
            if after_layer is not None:
                after_layer(run, x)
        x = rnd(norm_one_plus(x, t["final.norm"], self.eps))
        return x @ t["head"].T
