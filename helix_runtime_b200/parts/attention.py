"""Causal multi-head attention over the paged cache.

Parameters: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale`` (default
``1/sqrt(head_dim)``, src/attention/reference.cpp:152), ``window`` (None: all earlier
keys), ``position`` (a position-encoding spec), ``checkpoint_pairing`` (how the
checkpoint's q/k rows are ordered for rotation).  Tensors: ``q``, ``k``, ``v``
``[heads*head_dim, hidden]`` and ``o`` ``[hidden, heads*head_dim]``, all ``[out, in]``.

Optional mechanisms, each a parameter (absent: as if it did not exist):

* ``value_dim``: the size of a value head when it differs from ``head_dim`` (``v`` is then
  ``[kv_heads*value_dim, hidden]``, ``o`` ``[hidden, heads*value_dim]``).  Heads are held in
  rows of ``row_dim``, the kernels' size that holds the larger of the two, with exact zeros in
  the coordinates a head does not have (see the last paragraph).
* ``keep_first`` (with ``window``): position ``i`` sees ``j <= i`` when ``i - j < window`` or
  ``j < keep_first``; the kept keys keep their pages when the window has passed them.
* ``short_conv``: taps of a causal filter over time on every channel of q, k and v, applied
  right after the projection (tensors ``q_conv``, ``k_conv``, ``v_conv`` ``[channels, taps]``,
  the last tap on the token's own value).  The last ``taps - 1`` projected values of a request
  are per-request state (``state_need``).  The filter kernel appends keys and values to the
  pages itself when the position encoding is ``none``.
* rotated values and a query/key norm belong to the position encoding (``computed_rotary``):
  when it has ``restore_values`` the attention output is handed to it before the gate and the
  output projection.
* ``output_gate`` (``"sigmoid"``): the concatenated heads are multiplied by
  ``sigmoid(g x)`` before the output projection (tensor ``g`` ``[heads*value_dim, hidden]``);
  with a filter the gate's projection is part of the fused product.

* ``sinks`` (True): a learned number per head (tensor ``sink`` ``[heads]``) whose exponential
  is one more term of the softmax's denominator; it has no key and no value.
* ``distance_slopes`` (a number per head): the score of key ``j`` for the query at position
  ``i`` is lowered by ``slope_h * (i - j)``.

:class:`NormedProjectionAttention` adds what sits between the projection and the cache for
models without a rotation; :class:`LatentAttention` caches one latent for all heads.

At load the three projections are fused into one ``[(A + 2 Akv) D, H]`` matrix and,
when the checkpoint rotates half-split pairs while the encoding rotates adjacent
pairs, the rows of q and k are permuted per head to ``[0, D/2, 1, D/2+1, ...]``
(the reference's converter does the same, tools/convert_hf_llama.py:535-542).
Steps: fused projection, rotary encoding + cache append, paged attention, output
projection added into the residual (src/model/cpu_llama.cpp:65-91).

A head whose size is no multiple of 16 (100, say; of 32 above 128) is held in rows of the
next multiple (``row_dim``): the projection gets zero rows for the extra coordinates of every head and
the output projection zero columns, so queries, keys and values carry exact zeros there,
scores and outputs are unchanged, and the tensor-core attention kernels, which tile the
head in steps of 16, take the head.  The scale stays ``1/sqrt(head_dim)`` and the rotation
covers the real coordinates only.  This needs a position encoding that takes a row width
of its own (``row_dim``); with one that does not, the head keeps its size and the
CUDA-core attention runs.
"""
from __future__ import annotations

import math
from typing import List, Mapping, Optional

import torch

from ..cache.manager import KvNeed, StateNeed
from ..config.spec import PartSpec
from ..ops import library as ops
from ..weights.loader import TensorRequest
from .base import LayerCache, Mixer, StepContext, build_part, register_part
from .linear import (STREAMING_MAX_TOKENS, Weight, is_weight_stream, project,
                     project_into_accumulator)


TENSOR_CORE_MIN_QUERY = 16


def row_width(head_dim: int) -> int:
    """The head size the tensor-core attention kernels are built for that holds ``head_dim``:
    steps of 16 up to 128, of 32 up to 256; beyond that a head that fits the CUDA-core kernel is
    rounded up to a step of 32 (up to 1,024) and a larger one keeps its size."""
    step = 16 if head_dim <= 128 else 32
    wide = -(-head_dim // step) * step
    return wide if wide <= 1024 else head_dim


def rotary_row_permutation(heads: int, head_dim: int, rotary_dim: int) -> torch.Tensor:
    """Row order that turns half-split rotary rows into adjacent-pair rows, per head."""
    half = rotary_dim // 2
    order: List[int] = []
    for head in range(heads):
        base = head * head_dim
        for frequency in range(half):
            order.extend((base + frequency, base + half + frequency))
        order.extend(range(base + rotary_dim, base + head_dim))
    return torch.tensor(order, dtype=torch.long)


def stretched_frequencies(dims: int, theta: float, scaling: Optional[Mapping[str, float]]):
    """Frequencies of the ``dims / 2`` rotated pairs (float64 tensor) and the factor on sine and
    cosine.  Without ``scaling``: ``f_i = theta^(-2i / dims)`` and 1.  With ``scaling``
    (``factor``, ``original``: the trained length, ``fast`` and ``slow``: turns over that
    length) a pair that turns more often than ``fast`` keeps its frequency, one that turns less
    than ``slow`` takes ``f_i / factor``, and the pairs between are blended linearly in the
    pair's index: with ``pair(t) = dims ln(original / (2 pi t)) / (2 ln theta)``, ``lo =
    max(floor(pair(fast)), 0)``, ``hi = min(ceil(pair(slow)), dims - 1)`` and ``r_i =
    clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` the frequency is ``f_i / factor * r_i + f_i
    (1 - r_i)``; sine and cosine are multiplied by ``0.1 ln(factor) + 1``."""
    index = torch.arange(dims // 2, dtype=torch.float64)
    plain = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * index / float(dims))
    if not scaling:
        return plain, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((index - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return plain / factor * ramp + plain * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class PagedAttention(Mixer):
    pack_heads = False      # subclasses whose heads share few cached rows set this
    pack_always = True      # ... for every step; False: only for steps of single tokens

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.heads = int(spec["num_heads"])
        self.kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        if self.heads % self.kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.scale = float(spec.get("scale") or 1.0 / math.sqrt(float(self.head_dim)))
        window = spec.get("window")
        self.window: Optional[int] = int(window) if window else None
        self.keep_first = int(spec.get("keep_first") or 0) if self.window else 0
        self.value_dim = int(spec.get("value_dim") or self.head_dim)
        self.conv_taps = int(spec.get("short_conv") or 1)
        if self.conv_taps < 1:
            raise ValueError("short_conv counts the filter's taps: at least 1")
        gate = spec.get("output_gate")
        if gate not in (None, "sigmoid"):
            raise ValueError(f"output gate {gate!r} has no kernel; only 'sigmoid'")
        self.gated = gate is not None
        self._init_score_terms(spec)
        self.row_dim = self.head_dim
        self.position = build_part("position", spec["position"], hidden_size)
        wide = row_width(max(self.head_dim, self.value_dim))
        if wide != self.head_dim or self.value_dim != self.head_dim:
            position = spec["position"]
            padded = build_part("position", PartSpec(position.kind,
                                                     {**position.params, "row_dim": wide,
                                                      "value_dim": self.value_dim},
                                                     position.tensors), hidden_size)
            if getattr(padded, "row_dim", None) == wide:
                self.position, self.row_dim = padded, wide
            elif self.value_dim != self.head_dim:
                raise ValueError(f"position encoding {position.kind!r} takes no row width of its "
                                 f"own, which heads of {self.head_dim} with values of "
                                 f"{self.value_dim} need")
        self.checkpoint_pairing = spec.get("checkpoint_pairing", self.position.pairing)
        self.names = dict(spec.tensors)
        # widths of the checkpoint's matrices and of the rows this part computes with
        self.q_rows = self.heads * self.head_dim
        self.kv_rows = self.kv_heads * self.head_dim
        self.v_rows = self.kv_heads * self.value_dim
        self.o_columns = self.heads * self.value_dim
        self.q_size = self.heads * self.row_dim
        self.kv_size = self.kv_heads * self.row_dim
        self.qkv_size = self.q_size + 2 * self.kv_size
        # with a filter the gate's projection rides in the fused product, behind q, k and v
        self.fused_gate = self.gated and self.conv_taps > 1
        self.projected_size = self.qkv_size + (self.q_size if self.fused_gate else 0)
        # the filter kernel appends to the pages itself when nothing comes between
        self.conv_appends = self.conv_taps > 1 and self.position.pairing is None \
            and getattr(self.position, "rotary_dim", None) == 0
        self.dtype = torch.float32
        self.w_qkv: Optional[Weight] = None
        self.w_o: Optional[Weight] = None
        self.w_g: Optional[Weight] = None
        self.conv_filter: Optional[torch.Tensor] = None

    def _init_score_terms(self, spec: PartSpec) -> None:
        """The optional per-head terms of the scores: sinks and distance slopes."""
        self.has_sinks = bool(spec.get("sinks", False))
        slopes = spec.get("distance_slopes")
        if slopes is not None and len(slopes) != self.heads:
            raise ValueError("distance_slopes gives one slope per head")
        self.slope_values = None if slopes is None else tuple(float(v) for v in slopes)
        self.sinks: Optional[torch.Tensor] = None
        self.slopes: Optional[torch.Tensor] = None

    def _score_term_requests(self) -> List[TensorRequest]:
        if not self.has_sinks:
            return []
        return [TensorRequest(self.names["sink"], (self.heads,), role="scale")]

    def _bind_score_terms(self, tensors: Mapping[str, torch.Tensor], device) -> None:
        if self.has_sinks:
            self.sinks = tensors[self.names["sink"]].to(device=device, dtype=torch.float32) \
                .contiguous()
        if self.slope_values is not None:
            self.slopes = torch.tensor(self.slope_values, dtype=torch.float64) \
                .to(torch.float32).to(device).contiguous()

    def kv_need(self) -> Optional[KvNeed]:
        return KvNeed(self.kv_heads, self.row_dim, self.window, self.keep_first)

    def state_need(self) -> Optional[StateNeed]:
        if self.conv_taps <= 1:
            return None
        return StateNeed((self.conv_taps - 1, self.qkv_size), self.dtype)

    def tensor_requests(self) -> List[TensorRequest]:
        h = self.hidden_size
        requests = [
            TensorRequest(self.names["q"], (self.q_rows, h)),
            TensorRequest(self.names["k"], (self.kv_rows, h)),
            TensorRequest(self.names["v"], (self.v_rows, h)),
            TensorRequest(self.names["o"], (h, self.o_columns)),
            *self.position.tensor_requests(),
            *self._score_term_requests(),
        ]
        if self.gated:
            requests.append(TensorRequest(self.names["g"], (self.o_columns, h)))
        if self.conv_taps > 1:
            requests.extend(
                TensorRequest(self.names[name], (rows, self.conv_taps), role="scale")
                for name, rows in (("q_conv", self.q_rows), ("k_conv", self.kv_rows),
                                   ("v_conv", self.v_rows)))
        return requests

    def widen_rows(self, matrix: torch.Tensor, heads: int, head_dim: Optional[int] = None) -> torch.Tensor:
        """``[heads * head_dim, in]`` to ``[heads * row_dim, in]``: zero rows behind each head."""
        head_dim = self.head_dim if head_dim is None else head_dim
        if self.row_dim == head_dim:
            return matrix
        wide = matrix.new_zeros((heads, self.row_dim, matrix.shape[1]))
        wide[:, :head_dim] = matrix.reshape(heads, head_dim, matrix.shape[1])
        return wide.reshape(heads * self.row_dim, matrix.shape[1])

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        q = tensors[self.names["q"]]
        k = tensors[self.names["k"]]
        v = tensors[self.names["v"]]
        if (self.checkpoint_pairing is not None and self.position.pairing is not None
                and self.checkpoint_pairing != self.position.pairing):
            if self.checkpoint_pairing == "half_split" and self.position.pairing == "adjacent":
                rotary = self.position.rotary_dim
                q_order = rotary_row_permutation(self.heads, self.head_dim, rotary)
                k_order = rotary_row_permutation(self.kv_heads, self.head_dim, rotary)
                q = q[q_order.to(q.device)]
                k = k[k_order.to(k.device)]
                if self.conv_taps > 1:      # the filter's channels move with their rows
                    tensors = dict(tensors)
                    for name, order in (("q_conv", q_order), ("k_conv", k_order)):
                        taps = tensors[self.names[name]]
                        tensors[self.names[name]] = taps[order.to(taps.device)]
            else:
                raise ValueError(f"no row permutation from {self.checkpoint_pairing!r} to "
                                 f"{self.position.pairing!r}")
        q, k, v = (self.widen_rows(q, self.heads), self.widen_rows(k, self.kv_heads),
                   self.widen_rows(v, self.kv_heads, self.value_dim))
        o = self.widen_rows(tensors[self.names["o"]].t().contiguous(), self.heads,
                            self.value_dim).t()
        fused = [q, k, v]
        if self.gated:
            g = self.widen_rows(tensors[self.names["g"]], self.heads, self.value_dim)
            if self.fused_gate:
                fused.append(g)
            else:
                self.w_g = Weight(g.to(device=device, dtype=dtype).contiguous())
        self.w_qkv = Weight(torch.cat(fused, dim=0).to(device=device, dtype=dtype).contiguous())
        self.w_o = Weight(o.to(device=device, dtype=dtype).contiguous())
        if self.conv_taps > 1:
            self.conv_filter = torch.cat([
                self.widen_rows(tensors[self.names["q_conv"]], self.heads),
                self.widen_rows(tensors[self.names["k_conv"]], self.kv_heads),
                self.widen_rows(tensors[self.names["v_conv"]], self.kv_heads, self.value_dim),
            ], dim=0).to(device=device, dtype=torch.float32).contiguous()
        self.dtype = dtype
        self.position.bind(tensors, dtype, device)
        self._bind_score_terms(tensors, device)

    @property
    def graph_safe(self) -> bool:
        return self.position.graph_safe

    def weight_bytes(self) -> int:
        return (self.w_qkv.nbytes() + self.w_o.nbytes()
                + (self.w_g.nbytes() if self.w_g is not None else 0))

    def project_filtered(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                         qkv: torch.Tensor) -> Optional[torch.Tensor]:
        """Projection, causal filter over time and cache append.  Leaves the filtered queries
        in ``qkv``.  Returns the float32 accumulator the projection summed into, which is still
        to be cleared (or None), and the buffer whose columns behind q, k and v hold the gate's
        projection when it is fused: the projected rows themselves, or ``qkv`` when the
        projection arrived as sums (the filter kernel then rounds and copies those columns)."""
        n = ctx.n_tokens
        write = cache.owns and cache.keys is not None
        appends = self.conv_appends and write
        accumulator = raw = None
        if is_weight_stream(x, self.w_qkv, n):
            accumulator = ctx.workspace.accumulator(f"attention.projected/{self.projected_size}",
                                                    (STREAMING_MAX_TOKENS, self.projected_size))
            project_into_accumulator(x, self.w_qkv, accumulator, n, ctx.status, ctx.ordered_sums)
        else:
            raw = ctx.workspace.get(f"attention.projected/{self.projected_size}",
                                    (ctx.capacity, self.projected_size), ctx.dtype)
            project(x, self.w_qkv, raw, n, ops.EPI_STORE, ctx.status)
        ops.short_conv_append(raw, accumulator, qkv, self.conv_filter, cache.state, ctx.positions,
                              ctx.token_request, ctx.request_slot, ctx.request_start,
                              cache.block_tables if appends else None,
                              cache.keys if appends else None, cache.values if appends else None,
                              n, self.heads, self.kv_heads, self.row_dim,
                              self.projected_size if raw is None else self.qkv_size,
                              cache.page_size, cache.num_pages, ctx.status)
        if not self.conv_appends:
            self.position.apply(ctx, cache, qkv, self.heads, self.kv_heads)
        return accumulator, (qkv if raw is None else raw)

    def split_keys_for(self, tokens: int, longest: int, limit: int) -> int:
        """Keys per split.  One warp walks one (token, head, split); a step with few tokens
        (decoding) gets narrower splits so that about sixteen warps per SM stream the cache,
        a step with many tokens keeps ``limit``.  Splits are multiples of the 32-key chunk,
        so the choice changes the order of float32 sums only."""
        wanted_warps = ops.sm_count() * 16
        splits = max(1, wanted_warps // max(1, tokens * self.heads))
        keys = -(-longest // splits)
        keys = max(32, -(-keys // 32) * 32)
        return min(keys, max(32, limit))

    def attend(self, ctx: StepContext, cache: LayerCache, qkv: torch.Tensor,
               context: torch.Tensor) -> None:
        """Scores, mask, softmax and weighted sum for the step's rows: queries from ``qkv``
        (``heads`` rows of ``row_dim``), keys and values from the entry's pages, the result into
        ``context``.  Chooses the kernels by the step's make-up."""
        n = ctx.n_tokens
        window = cache.window or 0
        kept = self.keep_first if window else 0
        # prompt portions of at least TENSOR_CORE_MIN_QUERY tokens go to a tensor-core
        # kernel (bfloat16, head sizes it has; with a window the ``mma.sync`` one); the rest,
        # decode tokens above all, to the streaming or the CUDA-core kernel.  A step may need
        # both.
        tensor_cores = (ctx.dtype == torch.bfloat16
                        and ctx.max_query_len >= TENSOR_CORE_MIN_QUERY
                        and ops.prefill_attention_supports(self.row_dim, cache.page_size))
        # many heads on one cached row: the kernel whose rows are a token's heads reads the
        # row once for all of them, decoded tokens included
        if (self.pack_heads and ctx.dtype == torch.bfloat16
                and (self.pack_always or ctx.max_query_len < TENSOR_CORE_MIN_QUERY)
                and ops.prefill_attention_supports(self.row_dim, cache.page_size)
                and ops.prefill_attention_packed_tokens(self.heads, self.kv_heads) > 0):
            ops.prefill_attention(qkv, cache.keys, cache.values, ctx.request_start,
                                  ctx.request_context, ctx.request_slot, cache.block_tables,
                                  context, ctx.n_requests, n, self.heads, self.kv_heads,
                                  self.row_dim, cache.page_size, cache.num_pages, self.scale, 1,
                                  ctx.status, query_lengths=ctx.host_query_lengths,
                                  window=window, keep_first=kept, packed=True,
                                  sinks=self.sinks, slopes=self.slopes)
            return
        if tensor_cores:
            ops.prefill_attention(qkv, cache.keys, cache.values, ctx.request_start,
                                  ctx.request_context, ctx.request_slot, cache.block_tables,
                                  context, ctx.n_requests, n // 64 + ctx.n_requests, self.heads,
                                  self.kv_heads, self.row_dim, cache.page_size, cache.num_pages,
                                  self.scale, TENSOR_CORE_MIN_QUERY, ctx.status,
                                  query_lengths=ctx.host_query_lengths, window=window,
                                  keep_first=kept, sinks=self.sinks, slopes=self.slopes)
        if not tensor_cores or ctx.min_query_len < TENSOR_CORE_MIN_QUERY:
            longest = ctx.max_context_len if not window else \
                min(ctx.max_context_len, window + kept)
            split_keys = self.split_keys_for(n, longest, ctx.attention_split_keys)
            max_splits = max(1, -(-longest // split_keys))
            floats = ops.attention_scratch_floats(n, self.heads, self.row_dim, max_splits,
                                                  ctx.dtype, cache.page_size, window)
            partial = ctx.workspace.at_least("attention.partial", floats, torch.float32)
            arrivals = ctx.workspace.accumulator(f"attention.arrivals/{self.heads}",
                                                 (ctx.capacity * self.heads,), torch.int32)
            ops.paged_attention(qkv, cache.keys, cache.values, ctx.positions, ctx.token_request,
                                ctx.request_slot, cache.block_tables, context, partial, n,
                                self.heads, self.kv_heads, self.row_dim, cache.page_size,
                                cache.num_pages, window, self.scale, split_keys, max_splits,
                                ctx.status, request_start=ctx.request_start,
                                skip_query_len=TENSOR_CORE_MIN_QUERY if tensor_cores else 0,
                                arrivals=arrivals, keep_first=kept, sinks=self.sinks,
                                slopes=self.slopes)

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        n = ctx.n_tokens
        # scratch is named by its width: layers of different sizes each keep their own buffer
        # (a name whose shape changed from layer to layer would be replaced at every call)
        qkv = ctx.workspace.get(f"attention.qkv/{self.projected_size}",
                                (ctx.capacity, self.projected_size), ctx.dtype)
        context = ctx.workspace.get(f"attention.context/{self.q_size}",
                                    (ctx.capacity, self.q_size), ctx.dtype)
        uncleared = gate_rows = None
        if self.conv_taps > 1:
            uncleared, gate_rows = self.project_filtered(ctx, cache, x, qkv)
        elif is_weight_stream(x, self.w_qkv, n):
            # few tokens: split-K into a float32 accumulator that the rotary kernel reads,
            # rounds as the product's store would have, and clears
            accumulator = ctx.workspace.accumulator(f"attention.qkv/{self.qkv_size}",
                                                    (STREAMING_MAX_TOKENS, self.qkv_size))
            project_into_accumulator(x, self.w_qkv, accumulator, n, ctx.status,
                                     ctx.ordered_sums)
            self.position.apply(ctx, cache, qkv, self.heads, self.kv_heads, accum=accumulator)
        elif not self.position.project_and_apply(ctx, cache, x, self.w_qkv, qkv, self.heads,
                                                 self.kv_heads):
            project(x, self.w_qkv, qkv, n, ops.EPI_STORE, ctx.status)
            self.position.apply(ctx, cache, qkv, self.heads, self.kv_heads)

        self.attend(ctx, cache, qkv, context)
        restore = getattr(self.position, "restore_values", None)
        if restore is not None:
            restore(ctx, context, self.heads)
        if self.gated:
            if self.fused_gate:
                gate = gate_rows[:, self.qkv_size:]
            else:
                gate = ctx.workspace.get(f"attention.gate/{self.q_size}",
                                         (ctx.capacity, self.q_size), ctx.dtype)
                project(x, self.w_g, gate, n, ops.EPI_STORE, ctx.status)
            ops.sigmoid_gate(context, gate, n, self.q_size, clear=uncleared)
        elif uncleared is not None:
            uncleared[:n].zero_()
        project(context, self.w_o, residual, n, ops.EPI_ADD_F32, ctx.status, ctx.ordered_sums)


class NormedProjectionAttention(PagedAttention):
    """Attention without a rotation whose projection is worked on as a whole before it is cached.

    On top of :class:`PagedAttention`'s ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``value_dim``, ``scale``, ``window``, ``sinks`` and ``distance_slopes`` (the position encoding
    is ``none``), each optional:

    * ``bias`` (True): q, k and v have biases (tensors ``q_bias``, ``k_bias``, ``v_bias``), added
      to the projection's float32 sums;
    * ``whole_norm`` (``{"eps": ...}``): ONE RMS norm over all of a token's query coordinates and
      one over all of its key coordinates, before they are cut into heads (plain weights
      ``q_norm`` ``[heads * head_dim]`` and ``k_norm`` ``[kv_heads * head_dim]``);
    * ``query_temperature`` (``{"coef": c, "every": n}``): the query at position ``p`` is
      multiplied by ``1 + c ln(floor((p + 1) / n) + 1)``;
    * ``value_mix`` (``"source"`` or ``"mix"``): the first such layer of a model keeps its
      values of the step's tokens (``"source"``), every later one caches and uses ``(1 - l) v +
      l v_source`` with ``l`` the scalar tensor ``value_mix``; the layers agree in ``num_kv_heads *
      value_dim``;
    * ``output_gate`` ``"sigmoid_per_head"``: head ``h`` of the result is multiplied by
      ``sigmoid(G x)_h``, ONE number per head (tensor ``g`` ``[heads, hidden]``).

    ``[q | k | v | g]`` is one product with float32 sums (a weight stream for few tokens); one
    kernel then adds the biases, norms, scales, blends, takes the gates' sigmoid, writes the
    queries in rows of ``row_dim`` and appends keys and values to the token's pages; the paged
    attention with its sinks and slopes, the gate and the output matrix follow.
    """

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        gate = spec.get("output_gate")
        if gate not in (None, "sigmoid_per_head"):
            raise ValueError(f"output gate {gate!r}: this part has 'sigmoid_per_head' only")
        inner = {key: value for key, value in spec.params.items() if key != "output_gate"}
        inner["position"] = PartSpec("none", {"head_dim": int(spec["head_dim"])})
        super().__init__(PartSpec(spec.kind, inner, spec.tensors), hidden_size)
        if self.conv_taps > 1:
            raise ValueError("this part has no filter over time")
        self.spec = spec
        # decoding: query heads that share a key/value head attend side by side in a tile's
        # rows (the streaming kernel would read the shared keys once per query head); steps
        # with prompt portions keep the kernels every attention part uses
        self.pack_heads = self.heads // self.kv_heads >= 2
        self.pack_always = False
        self.head_gated = gate is not None
        self.bias = bool(spec.get("bias", False))
        norm = spec.get("whole_norm")
        self.whole_norm = norm is not None
        self.eps = float(norm["eps"]) if norm else 0.0
        if self.whole_norm and not self.eps > 0.0:
            raise ValueError("the norm over the projection needs a positive eps")
        temperature = spec.get("query_temperature")
        self.temp_coef = float(temperature["coef"]) if temperature else 0.0
        self.temp_every = int(temperature["every"]) if temperature else 0
        if temperature and self.temp_every < 1:
            raise ValueError("query_temperature.every counts positions: at least 1")
        mix = spec.get("value_mix")
        if mix not in (None, "source", "mix"):
            raise ValueError(f"value_mix {mix!r} is neither 'source' nor 'mix'")
        self.value_mix = {None: 0, "source": 1, "mix": 2}[mix]
        self.mix = 0.0
        # the projection's columns as the checkpoint has them: no padding inside a head
        self.projected_size = self.q_rows + self.kv_rows + self.v_rows + \
            (self.heads if self.head_gated else 0)
        self.w_proj: Optional[Weight] = None
        self.q_bias = self.k_bias = self.v_bias = None
        self.q_norm = self.k_norm = None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def tensor_requests(self) -> List[TensorRequest]:
        h = self.hidden_size
        requests = [
            TensorRequest(self.names["q"], (self.q_rows, h)),
            TensorRequest(self.names["k"], (self.kv_rows, h)),
            TensorRequest(self.names["v"], (self.v_rows, h)),
            TensorRequest(self.names["o"], (h, self.o_columns)),
            *self._score_term_requests(),
        ]
        if self.bias:
            requests += [TensorRequest(self.names["q_bias"], (self.q_rows,), role="scale"),
                         TensorRequest(self.names["k_bias"], (self.kv_rows,), role="scale"),
                         TensorRequest(self.names["v_bias"], (self.v_rows,), role="scale")]
        if self.whole_norm:
            requests += [TensorRequest(self.names["q_norm"], (self.q_rows,), role="scale"),
                         TensorRequest(self.names["k_norm"], (self.kv_rows,), role="scale")]
        if "value_mix" in self.names:
            # the blend of a layer that only keeps its values (or does not mix at all) may be in
            # the checkpoint too, unused
            requests.append(TensorRequest(self.names["value_mix"], (), role="scale",
                                          optional=self.value_mix != 2))
        if self.head_gated:
            requests.append(TensorRequest(self.names["g"], (self.heads, h)))
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        def vector(role: str) -> torch.Tensor:
            return tensors[self.names[role]].to(device=device, dtype=torch.float32).contiguous()
        fused = [tensors[self.names[name]] for name in ("q", "k", "v")]
        if self.head_gated:
            fused.append(tensors[self.names["g"]])
        self.w_proj = Weight(torch.cat(fused, dim=0).to(device=device, dtype=dtype).contiguous())
        o = self.widen_rows(tensors[self.names["o"]].t().contiguous(), self.heads,
                            self.value_dim).t()
        self.w_o = Weight(o.to(device=device, dtype=dtype).contiguous())
        if self.bias:
            self.q_bias, self.k_bias, self.v_bias = (vector("q_bias"), vector("k_bias"),
                                                     vector("v_bias"))
        if self.whole_norm:
            self.q_norm, self.k_norm = vector("q_norm"), vector("k_norm")
        if self.value_mix == 2:
            self.mix = float(tensors[self.names["value_mix"]].to(torch.float64).cpu())
        self.dtype = dtype
        self.position.bind(tensors, dtype, device)
        self._bind_score_terms(tensors, device)

    def weight_bytes(self) -> int:
        return self.w_proj.nbytes() + self.w_o.nbytes()

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        n = ctx.n_tokens
        get = ctx.workspace.get
        qkv = get(f"attention.qkv/{self.qkv_size}", (ctx.capacity, self.qkv_size), ctx.dtype)
        context = get(f"attention.context/{self.q_size}", (ctx.capacity, self.q_size), ctx.dtype)
        gates = get(f"attention.head_gates/{self.heads}", (ctx.capacity, self.heads),
                    torch.float32) if self.head_gated else None
        # every value-mixing layer of a model reads and writes the same buffer: the first one's
        # values of this step's tokens
        source = get(f"attention.value_source/{self.v_rows}", (ctx.capacity, self.v_rows),
                     torch.float32) if self.value_mix else None
        write = cache.owns and cache.keys is not None
        if is_weight_stream(x, self.w_proj, n):
            projected = ctx.workspace.accumulator(f"attention.projected/{self.projected_size}",
                                                  (STREAMING_MAX_TOKENS, self.projected_size))
            project_into_accumulator(x, self.w_proj, projected, n, ctx.status, ctx.ordered_sums)
            clear = True
        else:
            projected = get(f"attention.projected_sums/{self.projected_size}",
                            (ctx.capacity, self.projected_size), torch.float32)
            project(x, self.w_proj, projected, n, ops.EPI_STORE_F32, ctx.status)
            clear = False
        ops.biased_normed_rows(projected, clear, qkv, n, self.heads, self.kv_heads, self.head_dim,
                               self.value_dim, self.row_dim, ctx.positions, q_bias=self.q_bias,
                               k_bias=self.k_bias, v_bias=self.v_bias, q_weight=self.q_norm,
                               k_weight=self.k_norm, eps=self.eps, temp_coef=self.temp_coef,
                               temp_every=self.temp_every, value_mix=self.value_mix, mix=self.mix,
                               value_source=source, gates=gates,
                               token_request=ctx.token_request, request_table_row=ctx.request_slot,
                               block_tables=cache.block_tables,
                               k_cache=cache.keys if write else None,
                               v_cache=cache.values if write else None,
                               page_size=cache.page_size, num_pages=cache.num_pages,
                               status=ctx.status)
        if not write:       # nothing of its own to append to: keys and values stay in the rows
            self.position.apply(ctx, cache, qkv, self.heads, self.kv_heads)
        self.attend(ctx, cache, qkv, context)
        if self.head_gated:
            ops.head_gate(context, gates, n, self.heads, self.row_dim)
        project(context, self.w_o, residual, n, ops.EPI_ADD_F32, ctx.status, ctx.ordered_sums)


class LatentAttention(PagedAttention):
    """Attention whose keys and values of all heads are functions of one small latent per
    token, which is all that is cached.

    Parameters: ``num_heads``, ``head_dim`` (the unrotated query/key coordinates of a head),
    ``rotated_dim`` (the rotated ones behind them; the rotated key part is one vector shared by
    all heads), ``value_dim``, ``kv_rank`` (the cached latent), ``q_rank`` (the queries' own
    latent), ``scale``, ``window`` (None: all earlier keys), ``eps`` (of both latents' RMS
    norms, which have plain weights), ``rotary`` (``theta``, ``dims``: the leading rotated
    coordinates that are turned; ``layout`` ``interleaved`` or ``halves``; ``scaling``: see
    :func:`stretched_frequencies`), ``output_gate`` (``"sigmoid"`` or None), ``sinks`` (True:
    tensor ``sink`` ``[heads]``, a term of every head's softmax denominator).  Tensors: ``q_down`` ``[q_rank, hidden]``, ``q_norm``
    ``[q_rank]``, ``q_up`` ``[heads * (head_dim + rotated_dim), q_rank]`` (per head the
    unrotated rows, then the rotated ones), ``kv_down`` ``[kv_rank + rotated_dim, hidden]``,
    ``kv_norm`` ``[kv_rank]``, ``k_up`` ``[heads * head_dim, kv_rank]``, ``v_up``
    ``[heads * value_dim, kv_rank]``, ``g`` ``[heads * value_dim, hidden]``, ``o``
    ``[hidden, heads * value_dim]``.

    With ``c`` the normed latent and ``r`` the rotated shared part, head ``h`` scores
    ``(q_h . Uk_h c + rot(qr_h) . rot(r)) * scale = ([Uk_h' q_h | rot(qr_h)] . [c | rot(r)]) *
    scale``: the keys' up-projection moves to the query's side and every head attends to the
    ONE cached row ``[c | rot(r)]`` (a cache of one key head of ``kv_rank + rotated_dim``
    coordinates); the weighted sum of the value rows ``[c]`` is a latent again, and the head's
    value up-projection ``Uv_h`` follows it.  The attention kernels are those of
    :class:`PagedAttention`, with one key/value head and rows of ``row_dim``.
    """

    pack_heads = True       # every head attends to the one cached row

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        Mixer.__init__(self, spec, hidden_size)
        self.heads = int(spec["num_heads"])
        self.kv_heads = 1
        self.plain_dim = int(spec["head_dim"])
        self.rotated_dim = int(spec.get("rotated_dim") or 0)
        self.value_dim = int(spec.get("value_dim") or self.plain_dim)
        self.kv_rank = int(spec["kv_rank"])
        self.q_rank = int(spec["q_rank"])
        self.scale = float(spec["scale"])
        window = spec.get("window")
        self.window: Optional[int] = int(window) if window else None
        self.keep_first = 0
        self.eps = float(spec["eps"])
        rotary = spec.get("rotary") or {}
        self.rotary_dims = int(rotary.get("dims", self.rotated_dim)) if self.rotated_dim else 0
        if self.rotary_dims % 2 or self.rotary_dims > self.rotated_dim:
            raise ValueError("rotary dims must be even and at most rotated_dim")
        layout = rotary.get("layout", "interleaved")
        if layout not in ops.ROTARY_LAYOUTS:
            raise ValueError(f"unknown rotary layout {layout!r}")
        self.rotary_layout = ops.ROTARY_LAYOUTS[layout]
        self.theta = float(rotary.get("theta", 10000.0))
        self.rotary_scaling = rotary.get("scaling")
        self.amplitude = 1.0
        gate = spec.get("output_gate")
        if gate not in (None, "sigmoid"):
            raise ValueError(f"output gate {gate!r} has no kernel; only 'sigmoid'")
        self.gated = gate is not None
        self._init_score_terms(spec)
        if self.slope_values is not None:
            raise ValueError("latent attention takes no distance slopes")
        self.head_dim = self.kv_rank + self.rotated_dim        # of the one cached key head
        self.row_dim = row_width(self.head_dim)
        self.row_dim += self.row_dim % 2                       # the append moves pairs
        self.q_size = self.heads * self.row_dim
        self.rows_size = self.q_size + 2 * self.row_dim
        self.q_width = self.heads * (self.plain_dim + self.rotated_dim)
        self.o_columns = self.heads * self.value_dim
        self.down_rows = self.q_rank + self.kv_rank + self.rotated_dim
        self.names = dict(spec.tensors)
        self.dtype = torch.float32

    def kv_need(self) -> Optional[KvNeed]:
        return KvNeed(1, self.row_dim, self.window, 0)

    def state_need(self) -> Optional[StateNeed]:
        return None

    @property
    def graph_safe(self) -> bool:
        return True

    def tensor_requests(self) -> List[TensorRequest]:
        h = self.hidden_size
        requests = [
            TensorRequest(self.names["q_down"], (self.q_rank, h)),
            TensorRequest(self.names["q_norm"], (self.q_rank,), role="scale"),
            TensorRequest(self.names["q_up"], (self.q_width, self.q_rank)),
            TensorRequest(self.names["kv_down"], (self.kv_rank + self.rotated_dim, h)),
            TensorRequest(self.names["kv_norm"], (self.kv_rank,), role="scale"),
            TensorRequest(self.names["k_up"], (self.heads * self.plain_dim, self.kv_rank)),
            TensorRequest(self.names["v_up"], (self.o_columns, self.kv_rank)),
            TensorRequest(self.names["o"], (h, self.o_columns)),
            *self._score_term_requests(),
        ]
        if self.gated:
            requests.append(TensorRequest(self.names["g"], (self.o_columns, h)))
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        def matrix(value: torch.Tensor) -> torch.Tensor:
            return value.to(device=device, dtype=dtype).contiguous()

        def scale(role: str) -> torch.Tensor:
            return tensors[self.names[role]].to(device=device, dtype=torch.float32).contiguous()
        heads, plain, rotated = self.heads, self.plain_dim, self.rotated_dim
        self.w_down = Weight(matrix(torch.cat([tensors[self.names["q_down"]],
                                               tensors[self.names["kv_down"]]], dim=0)))
        # the queries' up-projection: every head's unrotated rows first, then the rotated ones
        q_up = tensors[self.names["q_up"]].reshape(heads, plain + rotated, self.q_rank)
        self.w_q_up = Weight(matrix(torch.cat([q_up[:, :plain].reshape(heads * plain, self.q_rank),
                                               q_up[:, plain:].reshape(heads * rotated, self.q_rank)],
                                              dim=0)))
        # per head [kv_rank, head_dim]: the keys' up-projection, transposed
        k_up = tensors[self.names["k_up"]].reshape(heads, plain, self.kv_rank)
        self.w_k_up = matrix(k_up.transpose(1, 2))
        self.w_v_up = matrix(tensors[self.names["v_up"]].reshape(heads, self.value_dim, self.kv_rank))
        self.w_o = Weight(matrix(tensors[self.names["o"]]))
        self.w_g = Weight(matrix(tensors[self.names["g"]])) if self.gated else None
        self.q_norm, self.kv_norm = scale("q_norm"), scale("kv_norm")
        self.freq = self.freq_exact = None
        if self.rotary_dims:
            exact, self.amplitude = stretched_frequencies(self.rotary_dims, self.theta,
                                                          self.rotary_scaling)
            self.freq_exact = exact.to(device).contiguous()
            self.freq = exact.to(torch.float32).to(device).contiguous()
        self._no_angles = torch.zeros((1, 1), dtype=torch.float32, device=device)
        self._bind_score_terms(tensors, device)
        self.dtype = dtype

    def weight_bytes(self) -> int:
        held = [self.w_down, self.w_q_up, self.w_o] + ([self.w_g] if self.gated else [])
        small = self.w_k_up.numel() + self.w_v_up.numel()
        return sum(weight.nbytes() for weight in held) + small * self.w_k_up.element_size()

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        n = ctx.n_tokens
        get = ctx.workspace.get
        down = get(f"latent.down/{self.down_rows}", (ctx.capacity, self.down_rows), torch.float32)
        latent = get(f"latent.query_latent/{self.q_rank}", (ctx.capacity, self.q_rank), ctx.dtype)
        q = get(f"latent.q/{self.q_width}", (ctx.capacity, self.q_width), ctx.dtype)
        rows = get(f"latent.rows/{self.rows_size}", (ctx.capacity, self.rows_size), ctx.dtype)
        context = get(f"attention.context/{self.q_size}", (ctx.capacity, self.q_size), ctx.dtype)
        heads_out = get(f"latent.heads/{self.o_columns}", (ctx.capacity, self.o_columns), ctx.dtype)
        project(x, self.w_down, down, n, ops.EPI_STORE_F32, ctx.status)
        ops.latent_prepare(down, self.q_norm, self.kv_norm, self.eps, ctx.positions, self.freq,
                           self.freq_exact, self.rotary_dims, self.rotary_layout, latent, rows,
                           self.q_size, n, self.q_rank, self.kv_rank, self.rotated_dim,
                           self.row_dim, amplitude=self.amplitude)
        project(latent, self.w_q_up, q, n, ops.EPI_STORE, ctx.status)
        # [Uk_h' q_h | rot(qr_h) | 0] per head
        ops.head_products(q, self.plain_dim, self.w_k_up, rows, self.row_dim, n)
        ops.latent_queries(q, self.heads * self.plain_dim, rows, ctx.positions, self.freq,
                           self.freq_exact, self.rotary_dims, self.rotary_layout, n, self.heads,
                           self.kv_rank, self.rotated_dim, self.row_dim,
                           amplitude=self.amplitude)
        write = cache.owns and cache.keys is not None
        ops.rope_append(rows, ctx.positions, ctx.token_request, ctx.request_slot,
                        cache.block_tables, cache.keys if write else None,
                        cache.values if write else None, self._no_angles, self._no_angles, n,
                        self.heads, 1, self.row_dim, 0, 0, cache.page_size, cache.num_pages,
                        ctx.status)
        self.attend(ctx, cache, rows, context)
        ops.head_products(context, self.row_dim, self.w_v_up, heads_out, self.value_dim, n)
        if self.gated:
            gate = get(f"attention.gate/{self.o_columns}", (ctx.capacity, self.o_columns), ctx.dtype)
            project(x, self.w_g, gate, n, ops.EPI_STORE, ctx.status)
            ops.sigmoid_gate(heads_out, gate, n, self.o_columns)
        project(heads_out, self.w_o, residual, n, ops.EPI_ADD_F32, ctx.status, ctx.ordered_sums)


register_part("mixer", "paged_attention", PagedAttention)
register_part("mixer", "latent_attention", LatentAttention)
register_part("mixer", "normed_projection_attention", NormedProjectionAttention)
