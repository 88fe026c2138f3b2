"""Gated feed-forward: ``down(act(gate(x)) * up(x))`` (src/model/cpu_llama.cpp:93-98).

Parameters: ``intermediate_size``, ``activation`` (``silu``, or ``gelu_tanh``:
the tanh approximation of GELU, ``z * sigmoid(2 c (z + a z^3))`` with ``c = sqrt(2/pi)``,
``a = 0.044715``; or ``relu``), ``bias`` (True: all three projections have biases, tensors
``gate_bias``, ``up_bias``, ``down_bias``).  Tensors: ``gate``, ``up``
``[intermediate, hidden]`` and ``down`` ``[hidden, intermediate]``.  gate and up are
fused into one ``[2I, H]`` matrix at load so that both products read the input once;
on the tensor cores the gated activation is the epilogue of that product (silu and gelu_tanh
without biases; otherwise the product leaves float32 sums and one kernel adds the biases and
applies the gate).

:class:`DenseMlp` is the plain two-matrix feed-forward ``down(act(up(x) + b)) + b'``.
"""
from __future__ import annotations

import math
from typing import List, Mapping, Optional

import torch

from ..config.spec import PartSpec
from ..ops import library as ops
from ..weights.loader import TensorRequest
from .base import FeedForward, StepContext, register_part
from .linear import Weight, project, project_gated, project_swiglu


class GatedMlp(FeedForward):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.intermediate = int(spec["intermediate_size"])
        activation = spec.get("activation", "silu")
        if activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"activation {activation!r} has no kernel; known: "
                             + ", ".join(sorted(ops.GATE_ACTIVATIONS)))
        if activation == "clamped_sigmoid":
            raise ValueError("the clamped gate belongs to routed experts")
        self.activation = ops.GATE_ACTIVATIONS[activation]
        self.bias = bool(spec.get("bias", False))
        # the product's own epilogue knows silu and gelu_tanh without biases
        self.fused_gate = not self.bias and self.activation in (ops.GATE_SILU, ops.GATE_GELU_TANH)
        self.names = dict(spec.tensors)
        self.w_gate_up: Optional[Weight] = None
        self.w_down: Optional[Weight] = None
        self.gate_bias = self.up_bias = self.down_bias = None

    def tensor_requests(self) -> List[TensorRequest]:
        h, i = self.hidden_size, self.intermediate
        requests = [TensorRequest(self.names["gate"], (i, h)),
                    TensorRequest(self.names["up"], (i, h)),
                    TensorRequest(self.names["down"], (h, i))]
        if self.bias:
            requests += [TensorRequest(self.names["gate_bias"], (i,), role="scale"),
                         TensorRequest(self.names["up_bias"], (i,), role="scale"),
                         TensorRequest(self.names["down_bias"], (h,), role="scale")]
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        fused = torch.cat([tensors[self.names["gate"]], tensors[self.names["up"]]],
                          dim=0).to(device=device, dtype=dtype).contiguous()
        # tiles of 128 rows: the up rows begin on one only when the intermediate size allows
        self.w_gate_up = Weight(fused, tile=self.intermediate % ops.WEIGHT_TILE_ROWS == 0)
        self.w_down = Weight(tensors[self.names["down"]].to(device=device, dtype=dtype).contiguous())
        if self.bias:
            self.gate_bias, self.up_bias, self.down_bias = (
                tensors[self.names[role]].to(device=device, dtype=torch.float32).contiguous()
                for role in ("gate_bias", "up_bias", "down_bias"))

    def weight_bytes(self) -> int:
        return self.w_gate_up.nbytes() + self.w_down.nbytes()

    @property
    def output_bias(self) -> Optional[torch.Tensor]:
        """The bias of the second projection (see :class:`DenseMlp`)."""
        return self.down_bias

    def forward(self, ctx: StepContext, x: torch.Tensor, residual: torch.Tensor,
                bias_in_place: bool = False) -> None:
        n = ctx.n_tokens
        act = ctx.workspace.get(f"mlp.act/{self.intermediate}", (ctx.capacity, self.intermediate),
                                ctx.dtype)
        if self.fused_gate:
            project_swiglu(x, self.w_gate_up, self.intermediate, act, ctx.workspace, ctx.capacity,
                           n, ctx.status, ctx.ordered_sums, self.activation)
        else:
            project_gated(x, self.w_gate_up, self.intermediate, act, ctx.workspace, ctx.capacity,
                          n, ctx.status, ctx.ordered_sums, self.activation, self.gate_bias,
                          self.up_bias)
        if self.down_bias is not None and not bias_in_place:
            ops.add_bias(residual, self.down_bias, n)
        project(act, self.w_down, residual, n, ops.EPI_ADD_F32, ctx.status, ctx.ordered_sums)


class DenseMlp(FeedForward):
    """``down(act(up(x) + b_up)) + b_down`` with biases on both projections (``bias``: False for
    none).  ``activation`` ``xielu``: with the two numbers ``p, q`` of the tensor ``act``,
    ``act(z) = softplus(p) z^2 + z/2`` for ``z > 0`` and ``(1/2 + softplus(q)) (exp(z) - 1 - z) +
    z/2`` otherwise; the sums of the first product, the bias and the activation are float32,
    one rounding into the compute dtype.  Tensors: ``up`` ``[intermediate, hidden]``, ``down``
    ``[hidden, intermediate]``, ``up_bias``, ``down_bias``, ``act`` ``[2]``."""

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.intermediate = int(spec["intermediate_size"])
        activation = spec.get("activation", "xielu")
        if activation != "xielu":
            raise ValueError(f"activation {activation!r} has no kernel here; only 'xielu'")
        self.bias = bool(spec.get("bias", True))
        self.names = dict(spec.tensors)
        self.w_up: Optional[Weight] = None
        self.w_down: Optional[Weight] = None
        self.up_bias: Optional[torch.Tensor] = None
        self.down_bias: Optional[torch.Tensor] = None
        self.constants = (0.0, 0.0)

    def tensor_requests(self) -> List[TensorRequest]:
        h, i = self.hidden_size, self.intermediate
        requests = [TensorRequest(self.names["up"], (i, h)), TensorRequest(self.names["down"], (h, i)),
                    TensorRequest(self.names["act"], (2,), role="scale")]
        if self.bias:
            requests += [TensorRequest(self.names["up_bias"], (i,), role="scale"),
                         TensorRequest(self.names["down_bias"], (h,), role="scale")]
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.w_up = Weight(tensors[self.names["up"]].to(device=device, dtype=dtype).contiguous())
        self.w_down = Weight(tensors[self.names["down"]].to(device=device, dtype=dtype).contiguous())
        if self.bias:
            self.up_bias = tensors[self.names["up_bias"]].to(device=device, dtype=torch.float32).contiguous()
            self.down_bias = tensors[self.names["down_bias"]].to(device=device, dtype=torch.float32).contiguous()
        p, q = (float(v) for v in tensors[self.names["act"]].to(torch.float64).cpu())
        softplus = lambda z: max(z, 0.0) + math.log1p(math.exp(-abs(z)))
        self.constants = (softplus(p), 0.5 + softplus(q))

    def weight_bytes(self) -> int:
        return self.w_up.nbytes() + self.w_down.nbytes()

    @property
    def output_bias(self) -> Optional[torch.Tensor]:
        """The bias of the second projection, ``[hidden]`` float32: a caller that owns the buffer
        this part sums into may let the buffer start from it and say so (``bias_in_place``)."""
        return self.down_bias

    def forward(self, ctx: StepContext, x: torch.Tensor, residual: torch.Tensor,
                bias_in_place: bool = False) -> None:
        n = ctx.n_tokens
        sums = ctx.workspace.get(f"mlp.up/{self.intermediate}", (ctx.capacity, self.intermediate),
                                 torch.float32)
        act = ctx.workspace.get(f"mlp.act/{self.intermediate}", (ctx.capacity, self.intermediate),
                                ctx.dtype)
        project(x, self.w_up, sums, n, ops.EPI_STORE_F32, ctx.status)
        ops.biased_activation(sums, self.up_bias, act, n, ops.ACT_XIELU, *self.constants)
        if self.down_bias is not None and not bias_in_place:
            ops.add_bias(residual, self.down_bias, n)
        project(act, self.w_down, residual, n, ops.EPI_ADD_F32, ctx.status, ctx.ordered_sums)


class RoutedExperts(FeedForward):
    """``experts`` small gated feed-forwards of which every token uses ``top``, chosen by a
    router: ``s = sigmoid(R x)`` (float32 sums and scores), the ``top`` largest scores (the
    lowest index among equals), weights ``s / (sum of the chosen + 1e-20) * scale``, output
    ``sum_k weight_k * down_k(act(gate_k x) * (up_k x))``.  Parameters: ``experts``, ``top``,
    ``intermediate_size`` (of one expert), ``scale``, ``activation``.  Tensors: ``router``
    ``[experts, hidden]`` and, per expert ``e``, ``gate.{e}``, ``up.{e}`` ``[intermediate,
    hidden]`` and ``down.{e}`` ``[hidden, intermediate]``; at load they are stacked into
    ``[experts, 2 * intermediate, hidden]`` and ``[experts, hidden, intermediate]``.
    Nothing is read back to the host, so a step records into a CUDA graph.

    More rules, each a parameter: ``score`` (``sigmoid``, or ``softmax`` over all router
    outputs), ``correction`` (True: the tensor ``correction`` ``[router outputs]`` is added to the
    scores for the CHOICE only, the weights use the scores without it), ``normalize`` (False: the
    weights are the chosen scores times ``scale``, not divided by their sum), ``identity`` (so
    many more router outputs behind the experts that have no matrices: chosen, such an output
    contributes ``weight * x``), ``activation`` ``clamped_sigmoid`` with ``limit`` ``L``:
    ``g = min(gate x, L)``, ``u = clamp(up x, -L, L)``, ``down(g sigmoid(1.702 g) (u + 1))``."""

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.experts = int(spec["experts"])
        self.top = int(spec["top"])
        self.identity = int(spec.get("identity", 0))
        self.router_outputs = self.experts + self.identity
        if self.identity < 0 or not 1 <= self.top <= self.router_outputs:
            raise ValueError("top counts the experts a token uses: between 1 and experts")
        self.intermediate = int(spec["intermediate_size"])
        self.scale = float(spec.get("scale", 1.0))
        score = spec.get("score", "sigmoid")
        if score not in ("sigmoid", "softmax"):
            raise ValueError(f"router score {score!r} is neither 'sigmoid' nor 'softmax'")
        self.softmax = score == "softmax"
        self.corrected = bool(spec.get("correction", False))
        self.normalize = bool(spec.get("normalize", True))
        self.limit = float(spec.get("limit", 0.0))
        self.correction: Optional[torch.Tensor] = None
        activation = spec.get("activation", "silu")
        if activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"activation {activation!r} has no kernel; known: "
                             + ", ".join(sorted(ops.GATE_ACTIVATIONS)))
        self.activation = ops.GATE_ACTIVATIONS[activation]
        self.names = dict(spec.tensors)
        self.w_router: Optional[Weight] = None
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_requests(self) -> List[TensorRequest]:
        h, i = self.hidden_size, self.intermediate
        requests = [TensorRequest(self.names["router"], (self.router_outputs, h))]
        if self.corrected:
            requests.append(TensorRequest(self.names["correction"], (self.router_outputs,),
                                          role="scale"))
        for e in range(self.experts):
            requests += [TensorRequest(self.names[f"gate.{e}"], (i, h)),
                         TensorRequest(self.names[f"up.{e}"], (i, h)),
                         TensorRequest(self.names[f"down.{e}"], (h, i))]
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.w_router = Weight(tensors[self.names["router"]].to(device=device, dtype=dtype)
                               .contiguous())
        self.w_gate_up = torch.stack([
            torch.cat([tensors[self.names[f"gate.{e}"]], tensors[self.names[f"up.{e}"]]], dim=0)
            for e in range(self.experts)]).to(device=device, dtype=dtype).contiguous()
        self.w_down = torch.stack([tensors[self.names[f"down.{e}"]] for e in range(self.experts)]) \
            .to(device=device, dtype=dtype).contiguous()
        if self.corrected:
            self.correction = tensors[self.names["correction"]] \
                .to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.w_router.nbytes() + (self.w_gate_up.numel() + self.w_down.numel()) \
            * self.w_down.element_size()

    def forward(self, ctx: StepContext, x: torch.Tensor, residual: torch.Tensor) -> None:
        n = ctx.n_tokens
        get = ctx.workspace.get
        sums = get(f"experts.router/{self.router_outputs}", (ctx.capacity, self.router_outputs),
                   torch.float32)
        chosen = get(f"experts.chosen/{self.top}", (ctx.capacity, self.top), torch.int32)
        weights = get(f"experts.weights/{self.top}", (ctx.capacity, self.top), torch.float32)
        act = get(f"experts.act/{self.top}x{self.intermediate}",
                  (ctx.capacity * self.top, self.intermediate), ctx.dtype)
        project(x, self.w_router, sums, n, ops.EPI_STORE_F32, ctx.status)
        ops.route_top(sums, chosen, weights, n, self.router_outputs, self.top, self.scale,
                      softmax=self.softmax, correction=self.correction, normalize=self.normalize)
        if self.identity:
            # router outputs behind the experts return the input; the experts' kernels leave
            # such choices out
            ops.expert_identity_add(x, chosen, weights, residual, n, self.top, self.experts)
        if self.grouped(ctx, n):
            self.forward_grouped(ctx, x, chosen, weights, residual)
            return
        ops.expert_gate_up(x, self.w_gate_up, chosen, act, n, self.top, self.activation,
                           self.limit)
        ops.expert_down(act, self.w_down, chosen, weights, residual, n, self.top)

    # Fewer pairs than this and an expert's matrices are read about once anyway: a product
    # per pair streams them; from here on the pairs are sorted by expert.
    GROUPED_FROM_PAIRS = 32

    def grouped(self, ctx: StepContext, tokens: int) -> bool:
        return (ctx.dtype == torch.bfloat16 and tokens * self.top >= self.GROUPED_FROM_PAIRS
                and self.hidden_size % 8 == 0 and self.intermediate % 8 == 0)

    def forward_grouped(self, ctx: StepContext, x: torch.Tensor, chosen: torch.Tensor,
                        weights: torch.Tensor, residual: torch.Tensor) -> None:
        """Pairs sorted by expert, two grouped tensor-core products (the gated activation is the
        first one's epilogue, the second stores float32 sums), and the weighted sum per token
        in the order of its choices."""
        n, get = ctx.n_tokens, ctx.workspace.get
        pairs = n * self.top
        tile = ops.expert_tile(pairs, self.experts)
        tiles = ops.expert_tile_bound(pairs, self.experts, tile)
        # buffers are made once for the largest step: the widest tile pads the most rows
        most = max(ops.expert_tile_bound(ctx.capacity * self.top, self.experts, t) * t
                   for t in ops.GROUPED_TILES)
        pair_row = get(f"experts.pair_row/{self.top}", (ctx.capacity * self.top,), torch.int32)
        tile_group = get(f"experts.tile_group/{self.experts}x{self.top}",
                         (ops.expert_tile_bound(ctx.capacity * self.top, self.experts,
                                                ops.GROUPED_TILES[0]),), torch.int32)
        rows_in = get(f"experts.rows_in/{self.hidden_size}", (most, self.hidden_size), ctx.dtype)
        rows_act = get(f"experts.rows_act/{self.intermediate}", (most, self.intermediate), ctx.dtype)
        rows_out = get(f"experts.rows_out/{self.hidden_size}", (most, self.hidden_size),
                       torch.float32)
        ops.expert_rows(chosen, pair_row, tile_group, pairs, self.experts, tile, tiles)
        ops.expert_gather(x, pair_row, rows_in, n, self.top)
        ops.gemm_tc_grouped(rows_in, self.w_gate_up, rows_act, tiles * tile, self.intermediate,
                            ops.EPI_SWIGLU, self.intermediate, tile, tile_group, ctx.status,
                            gate_activation=self.activation, gate_limit=self.limit)
        ops.gemm_tc_grouped(rows_act, self.w_down, rows_out, tiles * tile, self.hidden_size,
                            ops.EPI_STORE_F32, 0, tile, tile_group, ctx.status)
        ops.expert_combine(rows_out, pair_row, weights, residual, n, self.top, self.hidden_size)


register_part("feed_forward", "gated_mlp", GatedMlp)
register_part("feed_forward", "routed_experts", RoutedExperts)
register_part("feed_forward", "dense_mlp", DenseMlp)
