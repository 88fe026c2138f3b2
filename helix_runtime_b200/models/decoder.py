"""A decoder assembled from a :class:`ModelSpec`: embedding, scheduled blocks, norm, head.

The model owns the parts and the order in which they run; it owns no cache and no
batch.  ``forward`` runs exactly the tokens of the step's context through every
schedule entry and returns float32 logits at the wanted rows.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Mapping, Optional, Sequence

import torch

from ..cache.manager import CacheManager, KvNeed, StateNeed
from ..config.spec import BlockSpec, ModelSpec
from ..ops import library as ops
from ..parts.base import (FeedForward, LayerCache, Mixer, Norm, StepContext, build_part)
from ..weights.loader import TensorRequest


# ----------------------------------------------------------------- arrangements
#
# An arrangement wires the parts of a block: ``run(block, ctx, cache, residual, normed)`` reads
# and updates the float32 residual stream ``residual[:n]`` through the block's parts, with
# ``normed`` as scratch for a norm's output (compute dtype, same rows).  Mixers and
# feed-forwards ADD their output into the residual they are handed.

Arrangement = Callable[["Block", StepContext, LayerCache, torch.Tensor, torch.Tensor], None]
_ARRANGEMENTS: Dict[str, Arrangement] = {}


def register_arrangement(name: str, run: Arrangement) -> None:
    """Make ``name`` usable as ``BlockSpec.arrangement``."""
    _ARRANGEMENTS[name] = run


def _pre_norm(block: "Block", ctx: StepContext, cache: LayerCache, residual: torch.Tensor,
              normed: torch.Tensor) -> None:
    # x += mixer(norm(x)); x += ff(norm(x))   (src/model/cpu_llama.cpp:62-98)
    block.mixer_norm.forward(ctx, residual, normed)
    block.mixer.forward(ctx, cache, normed, residual)
    if block.feed_forward is not None:
        block.feed_forward_norm.forward(ctx, residual, normed)
        block.feed_forward.forward(ctx, normed, residual)


register_arrangement("pre_norm", _pre_norm)


def _parallel(block: "Block", ctx: StepContext, cache: LayerCache, residual: torch.Tensor,
              normed: torch.Tensor) -> None:
    # h = norm(x); x += mixer(h) + ff(h): one norm, both sublayers read its output and add
    # into the float32 residual stream (the sum is taken as (x + mixer) + ff)
    block.mixer_norm.forward(ctx, residual, normed)
    block.mixer.forward(ctx, cache, normed, residual)
    if block.feed_forward is not None:
        block.feed_forward.forward(ctx, normed, residual)


register_arrangement("parallel", _parallel)


def _streams(block: "Block", ctx: StepContext, cache: LayerCache, residual: torch.Tensor,
             normed: torch.Tensor) -> None:
    # residual holds the model's streams side by side per token.  Per sublayer: the connection
    # reads their weighted sum through the norm and clears `output`; the sublayer sums its
    # result into `output`; the connection rewrites all streams from the old ones and `output`.
    output = ctx.workspace.get("model.sublayer_output", (ctx.capacity, block.hidden_size),
                               torch.float32)
    block.mixer_connection.read_normed(ctx, block.mixer_norm, residual, normed, output)
    block.mixer.forward(ctx, cache, normed, output)
    block.mixer_connection.write_back(ctx, residual, output)
    if block.feed_forward is not None:
        # a feed-forward whose output has a bias lets the buffer start from it (output_bias)
        # instead of adding it in a pass of its own
        bias = getattr(block.feed_forward, "output_bias", None)
        block.feed_forward_connection.read_normed(ctx, block.feed_forward_norm, residual, normed,
                                                  output, initial=bias)
        if bias is None:
            block.feed_forward.forward(ctx, normed, output)
        else:
            block.feed_forward.forward(ctx, normed, output, bias_in_place=True)
        block.feed_forward_connection.write_back(ctx, residual, output)


register_arrangement("streams", _streams)


class Block:
    """One decoder layer: its parts, and the arrangement that runs them."""

    def __init__(self, spec: BlockSpec, hidden_size: int) -> None:
        run = _ARRANGEMENTS.get(spec.arrangement)
        if run is None:
            raise ValueError(f"unknown block arrangement {spec.arrangement!r}; known: "
                             + ", ".join(sorted(_ARRANGEMENTS)))
        if (spec.feed_forward is None) != (spec.feed_forward_norm is None) \
                and spec.arrangement == "pre_norm":
            raise ValueError("a pre_norm block has a feed-forward with its norm, or neither")
        if spec.arrangement == "streams" and (
                spec.mixer_connection is None or
                (spec.feed_forward is not None and (spec.feed_forward_connection is None
                                                    or spec.feed_forward_norm is None))):
            raise ValueError("a streams block joins every sublayer with a connection and a norm")
        self.arrangement = spec.arrangement
        self.hidden_size = hidden_size
        self._run = run
        self.mixer_norm: Norm = build_part("norm", spec.mixer_norm, hidden_size)
        self.mixer: Mixer = build_part("mixer", spec.mixer, hidden_size)
        self.feed_forward_norm: Optional[Norm] = None if spec.feed_forward_norm is None else \
            build_part("norm", spec.feed_forward_norm, hidden_size)
        self.feed_forward: Optional[FeedForward] = None if spec.feed_forward is None else \
            build_part("feed_forward", spec.feed_forward, hidden_size)
        self.mixer_connection = None if spec.mixer_connection is None else \
            build_part("connection", spec.mixer_connection, hidden_size)
        self.feed_forward_connection = None if spec.feed_forward_connection is None else \
            build_part("connection", spec.feed_forward_connection, hidden_size)

    def parts(self):
        return tuple(part for part in (self.mixer_norm, self.mixer_connection, self.mixer,
                                       self.feed_forward_norm, self.feed_forward_connection,
                                       self.feed_forward) if part is not None)

    def forward(self, ctx: StepContext, cache: LayerCache, residual: torch.Tensor,
                normed: torch.Tensor) -> None:
        self._run(self, ctx, cache, residual, normed)


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        spec.validate()
        self.spec = spec
        self.hidden_size = spec.hidden_size
        self.vocab_size = spec.vocab_size
        self.max_positions = spec.max_positions
        self.streams = spec.streams
        self.embedding = build_part("embedding", spec.embedding, spec.hidden_size)
        self.blocks: List[Block] = [Block(block, spec.hidden_size) for block in spec.blocks]
        self.schedule = spec.schedule
        # parts that run before a schedule entry, by the entry's index
        self.entry_parts = {index: build_part("entry", entry.before, spec.hidden_size)
                            for index, entry in enumerate(spec.schedule)
                            if entry.before is not None}
        # and behind it
        self.entry_parts_after = {index: build_part("entry", entry.after, spec.hidden_size)
                                  for index, entry in enumerate(spec.schedule)
                                  if entry.after is not None}
        self.final_norm: Norm = build_part("norm", spec.final_norm, spec.hidden_size)
        self.lm_head = build_part("lm_head", spec.lm_head, spec.hidden_size)
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None
        # debugging hook: called with (schedule index, residual rows) after every entry
        self.after_entry: Optional[Callable[[int, torch.Tensor], None]] = None

    # ------------------------------------------------------------------ weights

    def all_parts(self):
        yield self.embedding
        for block in self.blocks:
            yield from block.parts()
        yield from self.entry_parts.values()
        yield from self.entry_parts_after.values()
        yield self.final_norm
        yield self.lm_head

    @property
    def graph_safe(self) -> bool:
        """Whether every part may be recorded into a CUDA graph (see ``Part.graph_safe``)."""
        return all(part.graph_safe for part in self.all_parts())

    def tensor_requests(self) -> List[TensorRequest]:
        requests: List[TensorRequest] = []
        seen = set()
        for part in self.all_parts():
            for request in part.tensor_requests():
                if request.name not in seen:
                    seen.add(request.name)
                    requests.append(request)
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        for part in self.all_parts():
            part.bind(tensors, dtype, device)
        self.dtype = dtype
        self.device = device

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one step reads: every matrix and norm of every scheduled layer once,
        plus the head (the embedding is gathered, not streamed)."""
        total = self.final_norm.weight_bytes() + self.lm_head.weight_bytes()
        for entry in self.schedule:
            total += sum(part.weight_bytes() for part in self.blocks[entry.block].parts())
        total += sum(part.weight_bytes() for part in (*self.entry_parts.values(),
                                                      *self.entry_parts_after.values()))
        return total

    # -------------------------------------------------------------------- cache

    def cache_needs(self):
        """``(kv_needs, state_needs)`` keyed by the schedule entries that own a cache."""
        kv: Dict[int, KvNeed] = {}
        state: Dict[int, StateNeed] = {}
        for index, entry in enumerate(self.schedule):
            if entry.cache_from is not None:
                continue
            mixer = self.blocks[entry.block].mixer
            need = mixer.kv_need()
            if need is not None:
                kv[index] = need
            state_need = mixer.state_need()
            if state_need is not None:
                state[index] = state_need
        for index, entry in enumerate(self.schedule):
            if entry.cache_from is None:
                continue
            own = self.blocks[entry.block].mixer.kv_need()
            other = self.blocks[self.schedule[entry.cache_from].block].mixer.kv_need()
            if own != other:
                raise ValueError(f"schedule entry {index} reads the cache of entry "
                                 f"{entry.cache_from}, whose geometry differs")
        return kv, state

    def layer_cache(self, cache: CacheManager, index: int) -> LayerCache:
        entry = self.schedule[index]
        owner = index if entry.cache_from is None else entry.cache_from
        view = LayerCache(entry=owner, owns=entry.cache_from is None)
        if cache.owns_pages(owner):
            group = cache.group_of(owner)
            view.keys, view.values = cache.layer_storage(owner)
            view.block_tables = group.device_tables
            view.page_size = group.page_size
            view.num_pages = group.pool.num_pages
            view.window = group.need.window
        if owner in cache.states:
            view.state = cache.state(owner)
        return view

    # ------------------------------------------------------------------ forward

    def forward(self, ctx: StepContext, cache: CacheManager, want_rows: Optional[torch.Tensor],
                n_want: int) -> Optional[torch.Tensor]:
        """Run the step's tokens; return logits ``[n_want, vocab]`` float32 for the flattened
        token indices in ``want_rows`` (device int32), or None when nothing is wanted."""
        h = self.hidden_size
        # with several residual streams a token's streams lie side by side in its row
        residual = ctx.workspace.get("model.residual", (ctx.capacity, self.streams * h),
                                     torch.float32)
        normed = ctx.workspace.get("model.normed", (ctx.capacity, h), ctx.dtype)
        embedded = None
        if self.streams > 1:
            # every stream starts as the embedding's output
            first = ctx.workspace.get("model.embedded", (ctx.capacity, h), torch.float32)
            self.embedding.forward(ctx, first)
            ops.streams_spread(first, residual, ctx.n_tokens, self.streams)
        else:
            self.embedding.forward(ctx, residual)
        # an entry part that does not read the embedding's output says so (needs_embedding)
        if any(entry.add_embedding for entry in self.schedule) or any(
                getattr(part, "needs_embedding", True)
                for part in (*self.entry_parts.values(), *self.entry_parts_after.values())):
            if self.streams > 1:
                raise ValueError("adding the embedding back in is defined for one residual stream")
            # the embedding's output is kept for the entries that add it back in
            embedded = ctx.workspace.get("model.embedded", (ctx.capacity, h), torch.float32)
            self.embedding.forward(ctx, embedded)
        for index, entry in enumerate(self.schedule):
            if entry.add_embedding:
                ops.add_rows(residual, embedded, ctx.n_tokens)
            if index in self.entry_parts:
                self.entry_parts[index].forward(ctx, residual, embedded)
            self.blocks[entry.block].forward(ctx, self.layer_cache(cache, index), residual, normed)
            if index in self.entry_parts_after:
                self.entry_parts_after[index].forward(ctx, residual, embedded)
            if self.after_entry is not None:
                rows = residual[:ctx.n_tokens]
                self.after_entry(index, rows if self.streams == 1 else
                                 rows.view(ctx.n_tokens, self.streams, h).sum(dim=1))
        if n_want == 0:
            return None
        wanted = ctx.workspace.get("model.wanted", (ctx.capacity, h), ctx.dtype)
        logits = ctx.workspace.get("model.logits", (ctx.capacity, self.vocab_size), torch.float32)
        if self.streams > 1:
            # the norm of the sum of the streams
            self.final_norm.forward_streams(ctx, residual, self.streams, None, wanted,
                                            rows=want_rows, n_rows=n_want)
        else:
            self.final_norm.forward(ctx, residual, wanted, rows=want_rows, n_rows=n_want)
        self.lm_head.forward(ctx, wanted, logits, n_want)
        return logits[:n_want]
