"""Architecture-neutral description of a decoder: which parts each layer is made of.

An architecture's typed configuration (read from its own ``config.json`` keys) is
translated into a :class:`ModelSpec` by that architecture's ``build_spec``.  The
spec is plain data: every size and constant a part needs is a field of its spec,
the blocks are a list (one :class:`BlockSpec` per distinct layer), and the order
in which layers run is a second list (:class:`ScheduleEntry`), which may name a
block twice or let an entry read the cache written by an earlier entry.

The reference hard-wires this structure into one function
(src/model/cpu_llama.cpp:62-98); here it is data so that a second architecture
only adds a new ``build_spec``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping, Optional, Tuple


@dataclasses.dataclass(frozen=True)
class PartSpec:
    """A part's kind (the key in the part registry) plus its parameters."""

    kind: str
    params: Mapping[str, Any] = dataclasses.field(default_factory=dict)
    # checkpoint tensor names this part binds, keyed by the part's own role names
    tensors: Mapping[str, str] = dataclasses.field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclasses.dataclass(frozen=True)
class BlockSpec:
    """One decoder layer: a mixer and (usually) a feed-forward, each behind its own norm.

    ``arrangement`` names how the parts are wired, a key of the arrangement registry
    (``models.decoder.register_arrangement``); ``pre_norm`` is
    ``x += mixer(norm(x)); x += ff(norm(x))`` (src/model/cpu_llama.cpp:62-98), ``parallel`` is
    ``h = norm(x); x += mixer(h) + ff(h)`` (one norm, both sublayers read its output).  A block whose
    arrangement has no feed-forward, or no second norm, leaves those fields ``None``.
    ``streams`` is the pre-norm order over several residual streams: each sublayer is joined to
    them by a connection part (``mixer_connection``, ``feed_forward_connection``), which reads a
    weighted sum of the streams for the norm and rewrites all streams from the sublayer's output.
    """

    arrangement: str
    mixer_norm: PartSpec
    mixer: PartSpec
    feed_forward_norm: Optional[PartSpec] = None
    feed_forward: Optional[PartSpec] = None
    mixer_connection: Optional[PartSpec] = None
    feed_forward_connection: Optional[PartSpec] = None


@dataclasses.dataclass(frozen=True)
class ScheduleEntry:
    """One executed layer.  ``block`` indexes ``ModelSpec.blocks``.

    ``cache_from`` is the index of an earlier schedule entry whose key/value
    cache (or state) this entry reads instead of owning one; ``None`` means the
    entry owns its cache.  ``add_embedding``: before this entry runs, the embedding's output
    (the residual stream as it stood before the first entry) is added to the residual stream
    once more; models that run a stretch of layers several times feed the input back in at
    the start of every repeat.  ``before``: a part of the family ``entry`` that is run before
    the entry's block on the residual stream and the embedding's output (a model that feeds its
    input back in through a matrix at the start of every repeat names it here).  ``after``: a
    part of the same family that is run behind the entry's block (a model that gives every layer
    an input of its own, looked up by the token's id, names it here).
    """

    block: int
    cache_from: Optional[int] = None
    add_embedding: bool = False
    before: Optional[PartSpec] = None
    after: Optional[PartSpec] = None


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    lm_head: PartSpec
    # residual streams per token (1: one residual row).  With more, every block is of the
    # ``streams`` arrangement, the embedding fills all of them and the final norm reads their sum.
    streams: int = 1

    def validate(self) -> None:
        if not self.blocks or not self.schedule:
            raise ValueError("a model needs at least one block and one schedule entry")
        if self.streams < 1:
            raise ValueError("a model has at least one residual stream")
        if self.streams > 1 and any(block.arrangement != "streams" for block in self.blocks):
            raise ValueError("with several residual streams every block is of the 'streams' "
                             "arrangement")
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.block < len(self.blocks):
                raise ValueError(f"schedule entry {index} names block {entry.block}, "
                                 f"but there are {len(self.blocks)} blocks")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < index:
                    raise ValueError(f"schedule entry {index} reads the cache of entry "
                                     f"{entry.cache_from}, which does not run before it")
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(f"schedule entry {index} reads the cache of entry "
                                     f"{entry.cache_from}, which owns none")
