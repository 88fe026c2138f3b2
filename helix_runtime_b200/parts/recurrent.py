"""Recurrent mixers: the selective state-space layer, the time-mixing layer with a decayed
outer-product state, and a mixer that runs several mixers side by side.

All three keep per-request state in ONE float32 row per schedule entry (``StateNeed`` of a flat
shape); a mixer cuts its row into the pieces it needs.  A step brings a portion of each
request's tokens (cut anywhere, one token when decoding); the kernels carry the state from
portion to portion, so the result does not depend on the cut.

:class:`StateSpaceMixer` (``state_space``).  Parameters ``heads``, ``head_width`` (``P``),
``state_size`` (``N``), ``groups`` (``G``), ``filter_taps``, ``norm_groups``, ``eps``.  With
``inner = heads * P``, the input projection's rows are ``[z: inner | x: inner | B: G N | C: G N |
dt: heads]``; ``x, B, C`` pass a causal per-channel filter with bias, then silu;
``d = softplus(dt + dt_bias)``; per head (head ``h`` reads group ``h // (heads / G)``)
``S_t = exp(-exp(A_log) d_t) S_(t-1) + d_t B_t x_t'``, ``y_t = S_t' C_t + D x_t``; ``y silu(z)``
is RMS-normed in ``norm_groups`` equal parts, times ``norm``, then the output projection.
State: the filter's last ``filter_taps - 1`` inputs and the matrices ``S`` (in the scan
kernel's own order, ``ops.scan_state_floats`` floats per head).

:class:`TimeMix` (``time_mix``).  Parameters ``heads``, ``head_dim``, ``decay_rank``, ``eps``.
With ``h'`` the previous token's input, each of r, k, v, g, w reads ``h + (h' - h) mu_s``;
``r, k, v`` are projections of their blends, ``gate = silu(W_g m_g)``,
``w = exp(-exp(W_w2 tanh(W_w1 m_w) + w0))``; per head ``o_t = (S_(t-1) + diag(u) k_t v_t')' r_t``
then ``S_t = diag(w_t) S_(t-1) + k_t v_t'``; each head's ``o`` over its root mean square, times
``norm``, times the gate, then the output projection.  State: ``h'`` and the
matrices ``S`` (``ops.scan_state_floats`` floats per head).

:class:`LinearState` (``linear_state``).  Linear attention with one ``[head_dim, value_dim]``
matrix per head and no softmax.  Parameters ``heads``, ``qk_heads`` (query/key heads; value head
``h`` reads ``h // (heads / qk_heads)``), ``head_dim``, ``value_dim``, ``rule`` (``decay``:
``S <- g S + k v'``; ``delta``: ``S <- g S; u = beta (v - S' k); S <- S + k u'``; then
``o = S' q``), ``decay`` (a list: one constant per head; left out: ``g = exp(-exp(A_log)
softplus(W_a x + dt_bias))``), ``filter_taps`` (a causal per-channel filter with silu on q, k
and v), ``unit_norm`` (q and k divided by ``sqrt(sum x^2 + unit_eps)`` per head), ``rotary``
(``theta``, ``dims``, ``layout``: q and k rotated by their position over their first ``dims``
coordinates), ``q_scale``, ``k_scale``, ``norm_weight`` (the head norm has a weight
``[value_dim]`` shared by the heads), ``eps``.  Each head's ``o`` over its root mean square, times
the weight, times ``silu(W_g x)``, then the output projection.  State: the filter's last inputs
and the matrices.

:class:`InputFilter` (``input_filter``).  Parameters ``taps``, ``mixer`` (a part spec): the inner
mixer reads ``x + conv(x)``, ``conv`` a causal per-channel filter over time (tensor ``filter``
``[hidden, taps]``, the last tap on the token itself); the last ``taps - 1`` inputs are state.

:class:`SideBySide` (``side_by_side``).  Parameters ``mixers`` (part specs) and ``scales``: every
mixer reads the same input and the result is ``sum_i scales[i] * mixer_i(x)``, summed in float32.
"""
from __future__ import annotations

import dataclasses
from typing import List, Mapping, Optional

import torch

from ..cache.manager import KvNeed, StateNeed
from ..config.spec import PartSpec
from ..ops import library as ops
from ..weights.loader import TensorRequest
from .base import LayerCache, Mixer, StepContext, build_part, register_part
from .linear import Weight, project


def _state_piece(cache: LayerCache, offset: int, size: int) -> torch.Tensor:
    """Columns ``[offset, offset + size)`` of the entry's state rows (a view; the kernels take
    its address and the stride between slots)."""
    return cache.state[:, offset:offset + size]


class StateSpaceMixer(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.heads = int(spec["heads"])
        self.head_width = int(spec["head_width"])
        self.state_size = int(spec["state_size"])
        self.groups = int(spec.get("groups", 1))
        self.taps = int(spec.get("filter_taps", 1))
        self.norm_groups = int(spec.get("norm_groups", 1))
        self.eps = float(spec["eps"])
        if self.heads % self.groups:
            raise ValueError("heads must be a multiple of groups")
        self.inner = self.heads * self.head_width
        if self.inner % self.norm_groups:
            raise ValueError("norm_groups must divide heads * head_width")
        if self.taps < 1:
            raise ValueError("filter_taps counts the filter's taps: at least 1")
        self.filtered = self.inner + 2 * self.groups * self.state_size
        self.projected = 2 * self.inner + 2 * self.groups * self.state_size + self.heads
        self.filter_state = (self.taps - 1) * self.filtered
        self.matrix_state = self.heads * ops.scan_state_floats(self.head_width, self.state_size)
        self.names = dict(spec.tensors)
        self.w_in: Optional[Weight] = None
        self.w_o: Optional[Weight] = None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.filter_state + self.matrix_state,), torch.float32)

    def tensor_requests(self) -> List[TensorRequest]:
        h = self.hidden_size
        return [TensorRequest(self.names["in"], (self.projected, h)),
                TensorRequest(self.names["filter"], (self.filtered, self.taps), role="scale"),
                TensorRequest(self.names["filter_bias"], (self.filtered,), role="scale"),
                TensorRequest(self.names["dt_bias"], (self.heads,), role="scale"),
                TensorRequest(self.names["a_log"], (self.heads,), role="scale"),
                TensorRequest(self.names["skip"], (self.heads,), role="scale"),
                TensorRequest(self.names["norm"], (self.inner,), role="scale"),
                TensorRequest(self.names["o"], (h, self.inner))]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        def scale(role: str) -> torch.Tensor:
            return tensors[self.names[role]].to(device=device, dtype=torch.float32).contiguous()
        self.w_in = Weight(tensors[self.names["in"]].to(device=device, dtype=dtype).contiguous())
        self.w_o = Weight(tensors[self.names["o"]].to(device=device, dtype=dtype).contiguous())
        self.filter, self.filter_bias = scale("filter"), scale("filter_bias")
        self.dt_bias, self.a_log, self.skip = scale("dt_bias"), scale("a_log"), scale("skip")
        self.norm = scale("norm")

    def weight_bytes(self) -> int:
        return self.w_in.nbytes() + self.w_o.nbytes()

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        n = ctx.n_tokens
        # a row width that keeps every row of the scratch 16-byte aligned for the products
        wide = -(-self.projected // 8) * 8
        rows = ctx.workspace.get(f"state_space.rows/{wide}", (ctx.capacity, wide), ctx.dtype)
        filtered = ctx.workspace.get(f"state_space.filtered/{self.filtered}",
                                     (ctx.capacity, self.filtered), ctx.dtype)
        y = ctx.workspace.get(f"state_space.y/{self.inner}", (ctx.capacity, self.inner),
                              torch.float32)
        gated = ctx.workspace.get(f"state_space.gated/{self.inner}", (ctx.capacity, self.inner),
                                  ctx.dtype)
        project(x, self.w_in, rows, n, ops.EPI_STORE, ctx.status)
        inner, bc = self.inner, self.groups * self.state_size
        ops.causal_filter(rows[:, inner:inner + self.filtered], filtered, self.filter,
                          self.filter_bias,
                          _state_piece(cache, 0, self.filter_state) if self.taps > 1 else None,
                          n, True, ctx.token_request, ctx.request_slot, ctx.request_start)
        ops.state_space_scan(filtered[:, :inner], filtered[:, inner:inner + bc],
                             filtered[:, inner + bc:inner + 2 * bc],
                             rows[:, inner + self.filtered:inner + self.filtered + self.heads],
                             self.dt_bias, self.a_log, self.skip,
                             _state_piece(cache, self.filter_state, self.matrix_state), y,
                             ctx.request_start, ctx.request_slot, ctx.n_requests, self.heads,
                             self.head_width, self.state_size, self.groups, tokens=n)
        ops.gated_group_norm(y, rows[:, :inner], self.norm, gated, n, self.norm_groups, self.eps,
                             gate_after=False)
        project(gated, self.w_o, residual, n, ops.EPI_ADD_F32, ctx.status, ctx.ordered_sums)


MIXES = ("r", "k", "v", "g", "w")


class TimeMix(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.heads = int(spec["heads"])
        self.head_dim = int(spec["head_dim"])
        self.decay_rank = int(spec["decay_rank"])
        self.eps = float(spec["eps"])
        self.width = self.heads * self.head_dim
        self.matrix_state = self.heads * ops.scan_state_floats(self.head_dim, self.head_dim)
        self.names = dict(spec.tensors)
        self.weights: dict = {}

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.hidden_size + self.matrix_state,), torch.float32)

    def tensor_requests(self) -> List[TensorRequest]:
        h, a = self.hidden_size, self.width
        requests = [TensorRequest(self.names[f"mu_{s}"], (h,), role="scale") for s in MIXES]
        requests += [TensorRequest(self.names[s], (a, h)) for s in ("r", "k", "v", "g")]
        requests += [TensorRequest(self.names["w1"], (self.decay_rank, h)),
                     TensorRequest(self.names["w2"], (a, self.decay_rank)),
                     TensorRequest(self.names["w0"], (a,), role="scale"),
                     TensorRequest(self.names["bonus"], (self.heads, self.head_dim), role="scale"),
                     TensorRequest(self.names["norm"], (a,), role="scale"),
                     TensorRequest(self.names["o"], (h, a))]
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        def scale(role: str) -> torch.Tensor:
            return tensors[self.names[role]].to(device=device, dtype=torch.float32).contiguous()
        for role in ("r", "k", "v", "g", "w1", "w2", "o"):
            self.weights[role] = Weight(tensors[self.names[role]].to(device=device, dtype=dtype)
                                        .contiguous())
        self.mu = torch.stack([scale(f"mu_{s}") for s in MIXES]).contiguous()
        self.w0, self.bonus, self.norm = scale("w0"), scale("bonus"), scale("norm")

    def weight_bytes(self) -> int:
        return sum(weight.nbytes() for weight in self.weights.values())

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        n, h, a, cap = ctx.n_tokens, self.hidden_size, self.width, ctx.capacity
        ws = ctx.workspace
        mixes = ws.get(f"time_mix.mixes/{h}", (len(MIXES), cap, h), ctx.dtype)
        projected = ws.get(f"time_mix.rkvg/{a}", (4, cap, a), ctx.dtype)
        rank = -(-self.decay_rank // 8) * 8
        low_sums = ws.get(f"time_mix.low_sums/{rank}", (cap, rank), torch.float32)
        low = ws.get(f"time_mix.low/{rank}", (cap, rank), ctx.dtype)
        decay_log = ws.get(f"time_mix.decay/{a}", (cap, a), torch.float32)
        o = ws.get(f"time_mix.o/{a}", (cap, a), torch.float32)
        normed = ws.get(f"time_mix.normed/{a}", (cap, a), ctx.dtype)
        ops.token_shift(x, self.mu, mixes, _state_piece(cache, 0, h), n, ctx.token_request,
                        ctx.request_slot, ctx.request_start)
        for index, role in enumerate(("r", "k", "v", "g")):
            project(mixes[index], self.weights[role], projected[index], n, ops.EPI_STORE, ctx.status)
        project(mixes[4], self.weights["w1"], low_sums, n, ops.EPI_STORE_F32, ctx.status)
        ops.biased_activation(low_sums[:, :self.decay_rank], None, low[:, :self.decay_rank], n,
                              ops.ACT_TANH)
        project(low[:, :self.decay_rank], self.weights["w2"], decay_log, n, ops.EPI_STORE_F32,
                ctx.status)
        ops.outer_product_scan(projected[0], projected[1], projected[2], decay_log, self.w0,
                               self.bonus, _state_piece(cache, h, self.matrix_state), o,
                               ctx.request_start, ctx.request_slot, ctx.n_requests, self.heads,
                               self.head_dim, tokens=n)
        ops.gated_group_norm(o, projected[3], self.norm, normed, n, self.heads, self.eps,
                             gate_after=True)
        project(normed, self.weights["o"], residual, n, ops.EPI_ADD_F32, ctx.status,
                ctx.ordered_sums)


def _flat_state(mixer: Mixer) -> int:
    """Floats of an inner mixer's state row (0: none); inner mixers keep one float32 row."""
    need = mixer.state_need()
    if need is None:
        return 0
    if need.dtype != torch.float32 or len(need.shape) != 1:
        raise ValueError("a mixer inside another keeps its state as one float32 row")
    return need.shape[0]


class LinearState(Mixer):
    RULES = ("decay", "delta")

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.heads = int(spec["heads"])
        self.qk_heads = int(spec.get("qk_heads") or self.heads)
        self.head_dim = int(spec["head_dim"])
        self.value_dim = int(spec.get("value_dim") or self.head_dim)
        self.rule = spec.get("rule", "decay")
        if self.rule not in self.RULES:
            raise ValueError(f"unknown rule {self.rule!r}; known: {', '.join(self.RULES)}")
        if self.heads % self.qk_heads:
            raise ValueError("heads must be a multiple of qk_heads")
        decay = spec.get("decay")
        self.fixed_decay = None if decay is None else [float(value) for value in decay]
        if self.fixed_decay is not None and len(self.fixed_decay) != self.heads:
            raise ValueError("a constant decay is given per head")
        # None: q, k and v go into the recurrence as projected; a count (1 too): a causal filter
        # of that many taps and silu come first
        taps = spec.get("filter_taps")
        self.taps = None if taps is None else int(taps)
        if self.taps is not None and self.taps < 1:
            raise ValueError("filter_taps counts the filter's taps: at least 1")
        self.unit_norm = bool(spec.get("unit_norm", False))
        self.unit_eps = float(spec.get("unit_eps", 1e-6))
        self.rotary = spec.get("rotary")
        if self.rotary is not None:
            dims = int(self.rotary["dims"])
            if dims % 2 or not 0 <= dims <= self.head_dim:
                raise ValueError("rotary dims must be even and at most head_dim")
            if self.rotary.get("layout", "halves") not in ops.ROTARY_LAYOUTS:
                raise ValueError(f"unknown rotary layout {self.rotary.get('layout')!r}")
        self.q_scale = float(spec.get("q_scale", 1.0))
        self.k_scale = float(spec.get("k_scale", 1.0))
        self.norm_weight = bool(spec.get("norm_weight", False))
        self.eps = float(spec["eps"])
        self.qk_width = self.qk_heads * self.head_dim
        self.v_width = self.heads * self.value_dim
        self.filtered = 2 * self.qk_width + self.v_width
        # projected rows: q | k | v | gate | beta (delta) | decay input (learned decay)
        self.gate_at = self.filtered
        self.beta_at = self.gate_at + self.v_width
        self.decay_at = self.beta_at + (self.heads if self.rule == "delta" else 0)
        self.projected = self.decay_at + (self.heads if self.fixed_decay is None else 0)
        self.filter_state = ((self.taps or 1) - 1) * self.filtered
        self.matrix_state = self.heads * ops.scan_state_floats(self.value_dim, self.head_dim)
        self.names = dict(spec.tensors)
        self.w_in: Optional[Weight] = None
        self.w_o: Optional[Weight] = None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.filter_state + self.matrix_state,), torch.float32)

    def tensor_requests(self) -> List[TensorRequest]:
        h = self.hidden_size
        requests = [TensorRequest(self.names["q"], (self.qk_width, h)),
                    TensorRequest(self.names["k"], (self.qk_width, h)),
                    TensorRequest(self.names["v"], (self.v_width, h)),
                    TensorRequest(self.names["g"], (self.v_width, h)),
                    TensorRequest(self.names["o"], (h, self.v_width))]
        if self.rule == "delta":
            requests.append(TensorRequest(self.names["beta"], (self.heads, h)))
        if self.fixed_decay is None:
            requests += [TensorRequest(self.names["decay"], (self.heads, h)),
                         TensorRequest(self.names["a_log"], (self.heads,), role="scale"),
                         TensorRequest(self.names["dt_bias"], (self.heads,), role="scale")]
        if self.taps is not None:
            requests += [TensorRequest(self.names[f"{part}_filter"], (rows, self.taps), role="scale")
                         for part, rows in (("q", self.qk_width), ("k", self.qk_width),
                                            ("v", self.v_width))]
        if self.norm_weight:
            requests.append(TensorRequest(self.names["norm"], (self.value_dim,), role="scale"))
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        def scale(role: str) -> torch.Tensor:
            return tensors[self.names[role]].to(device=device, dtype=torch.float32).contiguous()
        fused = [tensors[self.names[role]] for role in ("q", "k", "v", "g")]
        if self.rule == "delta":
            fused.append(tensors[self.names["beta"]])
        if self.fixed_decay is None:
            fused.append(tensors[self.names["decay"]])
        self.w_in = Weight(torch.cat(fused, dim=0).to(device=device, dtype=dtype).contiguous())
        self.w_o = Weight(tensors[self.names["o"]].to(device=device, dtype=dtype).contiguous())
        self.a_log = self.dt_bias = self.decay = self.decay_m1 = None
        if self.fixed_decay is None:
            self.a_log, self.dt_bias = scale("a_log"), scale("dt_bias")
        else:
            exact = torch.tensor(self.fixed_decay, dtype=torch.float64)
            self.decay = exact.to(torch.float32).to(device)
            self.decay_m1 = (exact - 1.0).to(torch.float32).to(device)
        self.filter = None
        if self.taps is not None:
            self.filter = torch.cat([scale("q_filter"), scale("k_filter"), scale("v_filter")],
                                    dim=0).contiguous()
        weight = scale("norm") if self.norm_weight else \
            torch.ones((self.value_dim,), dtype=torch.float32, device=device)
        self.norm = weight.repeat(self.heads).contiguous()
        self.freq = self.freq_exact = None
        self.rotary_dims, self.rotary_layout = 0, 1
        if self.rotary is not None and int(self.rotary["dims"]) > 0:
            dims = int(self.rotary["dims"])
            exponent = -2.0 * torch.arange(dims // 2, dtype=torch.float64) / float(dims)
            exact = torch.pow(torch.tensor(float(self.rotary["theta"]), dtype=torch.float64),
                              exponent)
            self.freq_exact = exact.to(device).contiguous()
            self.freq = exact.to(torch.float32).to(device).contiguous()
            self.rotary_dims = dims
            self.rotary_layout = ops.ROTARY_LAYOUTS[self.rotary.get("layout", "halves")]

    def weight_bytes(self) -> int:
        return self.w_in.nbytes() + self.w_o.nbytes()

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        n = ctx.n_tokens
        wide = -(-self.projected // 8) * 8
        rows = ctx.workspace.get(f"linear_state.rows/{wide}", (ctx.capacity, wide), ctx.dtype)
        o = ctx.workspace.get(f"linear_state.o/{self.v_width}", (ctx.capacity, self.v_width),
                              torch.float32)
        gated = ctx.workspace.get(f"linear_state.gated/{self.v_width}",
                                  (ctx.capacity, self.v_width), ctx.dtype)
        project(x, self.w_in, rows, n, ops.EPI_STORE, ctx.status)
        qkv = rows
        if self.taps is not None:
            qkv = ctx.workspace.get(f"linear_state.filtered/{self.filtered}",
                                    (ctx.capacity, self.filtered), ctx.dtype)
            ops.causal_filter(rows[:, :self.filtered], qkv, self.filter, None,
                              _state_piece(cache, 0, self.filter_state) if self.taps > 1 else None,
                              n, True,
                              ctx.token_request, ctx.request_slot, ctx.request_start)
        learned = self.fixed_decay is None
        ops.linear_state_scan(
            qkv[:, :self.qk_width], qkv[:, self.qk_width:2 * self.qk_width],
            qkv[:, 2 * self.qk_width:self.filtered],
            _state_piece(cache, self.filter_state, self.matrix_state), o, ctx.request_start,
            ctx.request_slot, ctx.n_requests, self.heads, self.qk_heads, self.head_dim,
            self.value_dim, delta=self.rule == "delta",
            decay_in=rows[:, self.decay_at:self.decay_at + self.heads] if learned else None,
            beta_in=rows[:, self.beta_at:self.beta_at + self.heads] if self.rule == "delta" else None,
            a_log=self.a_log, dt_bias=self.dt_bias, fixed_decay=self.decay,
            fixed_decay_m1=self.decay_m1,
            positions=ctx.positions if self.rotary_dims else None, freq=self.freq,
            freq_exact=self.freq_exact, rotary_dim=self.rotary_dims,
            rotary_layout=self.rotary_layout, unit_norm=self.unit_norm, unit_eps=self.unit_eps,
            q_scale=self.q_scale, k_scale=self.k_scale, tokens=n)
        ops.gated_group_norm(o, rows[:, self.gate_at:self.gate_at + self.v_width], self.norm, gated,
                             n, self.heads, self.eps, gate_after=True)
        project(gated, self.w_o, residual, n, ops.EPI_ADD_F32, ctx.status, ctx.ordered_sums)


class InputFilter(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.taps = int(spec["taps"])
        if self.taps < 1:
            raise ValueError("taps counts the filter's taps: at least 1")
        self.inner: Mixer = build_part("mixer", spec["mixer"], hidden_size)
        self.own_state = (self.taps - 1) * hidden_size
        self.inner_state = _flat_state(self.inner)
        self.name = spec.tensors["filter"]
        self.filter: Optional[torch.Tensor] = None

    @property
    def graph_safe(self) -> bool:
        return self.inner.graph_safe

    def kv_need(self) -> Optional[KvNeed]:
        return self.inner.kv_need()

    def state_need(self) -> Optional[StateNeed]:
        total = self.own_state + self.inner_state
        return StateNeed((total,), torch.float32) if total else None

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.name, (self.hidden_size, self.taps), role="scale"),
                *self.inner.tensor_requests()]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        taps = tensors[self.name].to(device=device, dtype=torch.float32).clone()
        taps[:, -1] += 1.0          # x + conv(x): the token's own tap carries the identity
        self.filter = taps.contiguous()
        self.inner.bind(tensors, dtype, device)

    def weight_bytes(self) -> int:
        return self.filter.numel() * 4 + self.inner.weight_bytes()

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        filtered = ctx.workspace.get(f"input_filter.rows/{self.hidden_size}",
                                     (ctx.capacity, self.hidden_size), ctx.dtype)
        ops.causal_filter(x, filtered, self.filter, None,
                          _state_piece(cache, 0, self.own_state) if self.taps > 1 else None,
                          ctx.n_tokens, False, ctx.token_request, ctx.request_slot,
                          ctx.request_start)
        view = cache
        if cache.state is not None:
            view = dataclasses.replace(
                cache, state=cache.state[:, self.own_state:self.own_state + self.inner_state]
                if self.inner_state else None)
        self.inner.forward(ctx, view, filtered, residual)


class SideBySide(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.mixers: List[Mixer] = [build_part("mixer", part, hidden_size)
                                    for part in spec["mixers"]]
        self.scales = [float(scale) for scale in spec["scales"]]
        if len(self.mixers) != len(self.scales) or not 1 <= len(self.mixers) <= 4:
            raise ValueError("side_by_side runs one to four mixers, each with its scale")
        needs = [mixer.kv_need() for mixer in self.mixers]
        if sum(need is not None for need in needs) > 1:
            raise ValueError("at most one of the mixers side by side may keep keys and values")
        self.offsets: List[Optional[int]] = []
        total = 0
        for mixer in self.mixers:
            need = mixer.state_need()
            if need is None:
                self.offsets.append(None)
                continue
            if need.dtype != torch.float32 or len(need.shape) != 1:
                raise ValueError("mixers side by side keep their state as one float32 row each")
            self.offsets.append(total)
            total += need.shape[0]
        self.state_size = total

    @property
    def graph_safe(self) -> bool:
        return all(mixer.graph_safe for mixer in self.mixers)

    def kv_need(self) -> Optional[KvNeed]:
        return next((need for need in (mixer.kv_need() for mixer in self.mixers)
                     if need is not None), None)

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.state_size,), torch.float32) if self.state_size else None

    def tensor_requests(self) -> List[TensorRequest]:
        return [request for mixer in self.mixers for request in mixer.tensor_requests()]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        for mixer in self.mixers:
            mixer.bind(tensors, dtype, device)

    def weight_bytes(self) -> int:
        return sum(mixer.weight_bytes() for mixer in self.mixers)

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        sources = []
        for index, (mixer, offset) in enumerate(zip(self.mixers, self.offsets)):
            # an all-zero float32 buffer per mixer: it sums its output in, the sum below reads
            # and clears it again
            output = ctx.workspace.accumulator(f"side_by_side.{index}/{self.hidden_size}",
                                               (ctx.capacity, self.hidden_size))
            view = cache
            if offset is not None:
                size = mixer.state_need().shape[0]
                view = dataclasses.replace(cache, state=cache.state[:, offset:offset + size])
            mixer.forward(ctx, view, x, output)
            sources.append(output)
        ops.scaled_sum(residual, sources, self.scales, ctx.n_tokens)


register_part("mixer", "state_space", StateSpaceMixer)
register_part("mixer", "time_mix", TimeMix)
register_part("mixer", "side_by_side", SideBySide)
register_part("mixer", "linear_state", LinearState)
register_part("mixer", "input_filter", InputFilter)
