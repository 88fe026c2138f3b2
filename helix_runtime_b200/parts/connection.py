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

:class:`NormedConnection` (``post_norm``): one residual, and the sublayer's result passes an RMS
norm of its own before it is added, times a constant: ``x <- x + scale * norm_b(f(norm(x)))``
(a norm on either side of the sublayer).  Parameters ``eps``, ``scale``, ``cast_to`` (optional:
the name of a scratch buffer that receives the updated residual in the compute type, for a part
that reads the residual itself as a product's input); tensor ``weight`` ``[hidden]``.

:class:`TokenSideInput` (family ``entry``, kind ``token_side``): an input of the layer's own,
looked up by the token's id: with ``e`` the columns ``[offset, offset + dim)`` of the token's
row of a table, ``g = gelu_tanh(G x) * e``, ``y = P g``, ``x <- x + scale * y / sqrt(mean(y^2) +
eps) * w``.  Parameters ``dim``, ``offset``, ``table_columns``, ``vocab_size``, ``eps``,
``scale``, ``reads`` (the scratch buffer that holds ``x`` in the compute type, see ``cast_to``);
tensors ``table`` ``[vocab, table_columns]``, ``gate`` ``[dim, hidden]``, ``proj`` ``[hidden,
dim]``, ``norm`` ``[hidden]``.
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


class NormedConnection(Part):
    streams = 1

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.eps = float(spec["eps"])
        if not self.eps > 0.0:
            raise ValueError("the norm behind a sublayer needs a positive eps")
        self.scale = float(spec.get("scale", 1.0))
        self.cast_to: Optional[str] = spec.get("cast_to")
        self.weight_name = spec.tensors["weight"]
        self.weight: Optional[torch.Tensor] = None

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.weight_name, (self.hidden_size,), role="scale")]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.weight = tensors[self.weight_name].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return 4 * self.hidden_size

    def read_normed(self, ctx: StepContext, norm: Norm, streams: torch.Tensor, normed: torch.Tensor,
                    output: torch.Tensor, initial: Optional[torch.Tensor] = None) -> None:
        """``normed[:n] = norm(x)``; ``output[:n]`` is zeroed for the sublayer, or set to
        ``initial`` (a bias of the sublayer's output)."""
        n = ctx.n_tokens
        norm.forward(ctx, streams, normed)
        if initial is None:
            output[:n].zero_()
        else:
            output[:n].copy_(initial.unsqueeze(0).expand(n, -1))

    def write_back(self, ctx: StepContext, streams: torch.Tensor, output: torch.Tensor) -> None:
        cast = None
        if self.cast_to is not None:
            cast = ctx.workspace.get(self.cast_to, (ctx.capacity, self.hidden_size), ctx.dtype)
        ops.norm_residual_add(streams, output, self.weight, self.eps, self.scale, ctx.n_tokens,
                              cast_out=cast)


class TokenSideInput(Part):
    needs_embedding = False      # it reads the residual, not the embedding's output

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.dim = int(spec["dim"])
        self.offset = int(spec.get("offset", 0))
        self.table_columns = int(spec.get("table_columns", self.offset + self.dim))
        self.vocab_size = int(spec["vocab_size"])
        if self.dim < 1 or self.offset < 0 or self.offset + self.dim > self.table_columns:
            raise ValueError("the layer's piece lies inside the table's row")
        self.eps = float(spec["eps"])
        self.scale = float(spec.get("scale", 1.0))
        self.reads = str(spec["reads"])
        self.names = dict(spec.tensors)
        self.table: Optional[torch.Tensor] = None
        self.w_gate: Optional[Weight] = None
        self.w_proj: Optional[Weight] = None
        self.norm: Optional[torch.Tensor] = None

    def tensor_requests(self) -> List[TensorRequest]:
        h = self.hidden_size
        return [TensorRequest(self.names["table"], (self.vocab_size, self.table_columns),
                              role="embedding"),
                TensorRequest(self.names["gate"], (self.dim, h)),
                TensorRequest(self.names["proj"], (h, self.dim)),
                TensorRequest(self.names["norm"], (h,), role="scale")]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        # the table is one tensor for all layers: held once, every layer reads its columns
        self.table = tensors[self.names["table"]].to(device=device, dtype=dtype).contiguous()
        self.w_gate = Weight(tensors[self.names["gate"]].to(device=device, dtype=dtype).contiguous())
        self.w_proj = Weight(tensors[self.names["proj"]].to(device=device, dtype=dtype).contiguous())
        self.norm = tensors[self.names["norm"]].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.w_gate.nbytes() + self.w_proj.nbytes() + 4 * self.hidden_size

    def forward(self, ctx: StepContext, residual: torch.Tensor, embedded) -> None:
        n, h, get = ctx.n_tokens, self.hidden_size, ctx.workspace.get
        x = get(self.reads, (ctx.capacity, h), ctx.dtype)
        sums = get(f"token_side.sums/{self.dim}", (ctx.capacity, self.dim), torch.float32)
        gated = get(f"token_side.gated/{self.dim}", (ctx.capacity, self.dim), ctx.dtype)
        y = get(f"token_side.output/{h}", (ctx.capacity, h), torch.float32)
        project(x, self.w_gate, sums, n, ops.EPI_STORE_F32, ctx.status)
        ops.token_gate(sums, False, self.table, self.offset, ctx.token_ids, gated, n, self.dim,
                       ctx.status)
        project(gated, self.w_proj, y, n, ops.EPI_STORE_F32, ctx.status)
        ops.norm_residual_add(residual, y, self.norm, self.eps, self.scale, n)


register_part("connection", "streams", StreamConnection)
register_part("connection", "post_norm", NormedConnection)
register_part("entry", "token_side", TokenSideInput)
register_part("connection", "gated", GatedConnection)
register_part("entry", "linear_rejoin", LinearRejoin)
