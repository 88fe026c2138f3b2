"""How a sublayer is joined to the residual: several residual streams (hyper-connections)
and a per-channel layer scale.

A model with ``streams`` residual streams ``X[s]`` (all equal to the embedding at the start)
joins a sublayer ``f`` with read weights ``a[s]``, write weights ``b[r]`` and a mixing matrix
``M[s, r]`` (indexed from, to):

    u = sum_s a[s] X[s];   y = f(norm(u));   X[r] <- sum_s M[s, r] X[s] + b[r] * scale * y

for all ``r`` at once from the old streams.  Parameters: ``streams`` (1: the ordinary residual
sum ``x <- x + scale * y``; no read, write or mixing tensors then unless ``weighted``),
``weighted`` (the tensors ``read`` ``[streams]``, ``write`` ``[streams]`` and ``mixing``
``[streams, streams]`` exist), ``layer_scale`` (the tensor ``scale`` ``[hidden]`` exists).
Everything is float32; the streams of a token lie next to each other, ``[rows, streams * hidden]``.

:class:`GatedConnection` (``gated``): one residual, and the sublayer's result is multiplied
element by element by ``sigmoid(G h + b)`` before it is added, ``h`` being the normed input the
sublayer is handed: ``x <- x + sigmoid(G norm(x) + b) * f(norm(x))``.  Tensors ``gate``
``[hidden, hidden]`` and ``gate_bias`` ``[hidden]``.  The gate's sums, the sigmoid, the product
and the residual sum are float32.

:class:`LinearRejoin` (family ``entry``, kind ``linear_rejoin``): run before a schedule entry,
it replaces the residual by ``W [x ; x0] + step[index]`` with ``x0`` the embedding's output,
``W`` ``[hidden, 2 hidden]`` (tensor ``weight``, the residual's columns first) and ``step``
``[steps, hidden]`` (tensor ``step``; parameter ``index`` picks the row).
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..config.spec import PartSpec
from ..ops import library as ops
from ..weights.loader import TensorRequest
from .base import Norm, Part, StepContext, register_part
from .linear import Weight, project


class StreamConnection(Part):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.streams = int(spec.get("streams", 1))
        if self.streams < 1:
            raise ValueError("a model has at least one residual stream")
        self.weighted = bool(spec.get("weighted", self.streams > 1))
        self.layer_scale = bool(spec.get("layer_scale", False))
        self.names = dict(spec.tensors)
        self.read: Optional[torch.Tensor] = None
        self.write: Optional[torch.Tensor] = None
        self.mixing: Optional[torch.Tensor] = None
        self.scale: Optional[torch.Tensor] = None

    def tensor_requests(self) -> List[TensorRequest]:
        s = self.streams
        requests = []
        if self.weighted:
            requests += [TensorRequest(self.names["read"], (s,), role="scale"),
                         TensorRequest(self.names["write"], (s,), role="scale"),
                         TensorRequest(self.names["mixing"], (s, s), role="scale")]
        if self.layer_scale:
            requests.append(TensorRequest(self.names["scale"], (self.hidden_size,), role="scale"))
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        def held(role: str) -> torch.Tensor:
            return tensors[self.names[role]].to(device=device, dtype=torch.float32).contiguous()
        if self.weighted:
            self.read, self.write, self.mixing = held("read"), held("write"), held("mixing")
        if self.layer_scale:
            self.scale = held("scale")

    def weight_bytes(self) -> int:
        return 4 * ((self.streams * (self.streams + 2) if self.weighted else 0)
                    + (self.hidden_size if self.layer_scale else 0))

    def read_normed(self, ctx: StepContext, norm: Norm, streams: torch.Tensor, normed: torch.Tensor,
                    output: torch.Tensor, initial: Optional[torch.Tensor] = None) -> None:
        """``normed[:n] = norm(sum_s a[s] X[s])``; ``output[:n]`` is zeroed for the sublayer, or
        set to ``initial`` (a bias of the sublayer's output, ``[hidden]`` float32)."""
        norm.forward_streams(ctx, streams, self.streams, self.read, normed, clear=output,
                             initial=initial)

    def write_back(self, ctx: StepContext, streams: torch.Tensor, output: torch.Tensor) -> None:
        ops.streams_write(streams, output, self.mixing, self.write, self.scale, self.streams,
                          ctx.n_tokens)


class GatedConnection(Part):
    streams = 1

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.names = dict(spec.tensors)
        self.weight: Optional[Weight] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_requests(self) -> List[TensorRequest]:
        h = self.hidden_size
        return [TensorRequest(self.names["gate"], (h, h)),
                TensorRequest(self.names["gate_bias"], (h,), role="scale")]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.weight = Weight(tensors[self.names["gate"]].to(device=device, dtype=dtype).contiguous())
        self.bias = tensors[self.names["gate_bias"]].to(device=device, dtype=torch.float32) \
            .contiguous()

    def weight_bytes(self) -> int:
        return self.weight.nbytes() + 4 * self.hidden_size

    def _gate(self, ctx: StepContext) -> torch.Tensor:
        return ctx.workspace.get(f"gated_connection.gate/{self.hidden_size}",
                                 (ctx.capacity, self.hidden_size), torch.float32)

    def read_normed(self, ctx: StepContext, norm: Norm, streams: torch.Tensor, normed: torch.Tensor,
                    output: torch.Tensor, initial: Optional[torch.Tensor] = None) -> None:
        """``normed[:n] = norm(x)``; the gate's sums ``G normed`` are taken now, while ``normed``
        holds the sublayer's input; ``output[:n]`` is zeroed for the sublayer."""
        if initial is not None:
            raise ValueError("a gated connection starts the sublayer's output from zero")
        n = ctx.n_tokens
        norm.forward(ctx, streams, normed)
        project(normed, self.weight, self._gate(ctx), n, ops.EPI_STORE_F32, ctx.status)
        output[:n].zero_()

    def write_back(self, ctx: StepContext, streams: torch.Tensor, output: torch.Tensor) -> None:
        ops.gated_residual_add(streams, output, self._gate(ctx), self.bias, ctx.n_tokens)


class LinearRejoin(Part):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.index = int(spec.get("index", 0))
        self.steps = int(spec.get("steps", 1))
        if not 0 <= self.index < self.steps:
            raise ValueError("index names one of the step rows")
        self.names = dict(spec.tensors)
        self.weight: Optional[Weight] = None
        self.step: Optional[torch.Tensor] = None

    def tensor_requests(self) -> List[TensorRequest]:
        h = self.hidden_size
        return [TensorRequest(self.names["weight"], (h, 2 * h)),
                TensorRequest(self.names["step"], (self.steps, h), role="scale")]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.weight = Weight(tensors[self.names["weight"]].to(device=device, dtype=dtype)
                             .contiguous())
        self.step = tensors[self.names["step"]][self.index] \
            .to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.nbytes() + 4 * self.hidden_size

    def forward(self, ctx: StepContext, residual: torch.Tensor, embedded: torch.Tensor) -> None:
        """``residual[:n] = W [residual | embedded] + step`` (the product reads the joined rows
        in the compute dtype and stores float32 sums)."""
        n, h = ctx.n_tokens, self.hidden_size
        joined = ctx.workspace.get(f"linear_rejoin.joined/{h}", (ctx.capacity, 2 * h), ctx.dtype)
        ops.join_rows(residual, embedded, joined, n)
        project(joined, self.weight, residual, n, ops.EPI_STORE_F32, ctx.status)
        ops.add_bias(residual, self.step, n)


register_part("connection", "streams", StreamConnection)
register_part("connection", "gated", GatedConnection)
register_part("entry", "linear_rejoin", LinearRejoin)
