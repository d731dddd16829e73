"""The architecture-neutral description of an assembled model.

An architecture's builder turns its typed configuration into a :class:`ModelSpec`: which
mixer, feed-forward, norms and position encoding each layer has (chosen layer by layer),
the tensor names they read, and the order in which layers run.  The engine only ever sees
this description; nothing below it knows which architecture it came from.
No torch import here.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """One part, by registered kind, with its sizes and constants as plain parameters."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (``block``) of a mixer, a feed-forward and named norms.

    ``prefix`` is the tensor-name prefix of the layer (``model.layers.3``).  Which norm
    names a block uses is the block's business (the pre-norm residual block uses
    ``pre_mixer`` and ``pre_feed_forward``).
    """

    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norms: dict[str, PartSpec]


@dataclass(frozen=True)
class ScheduleEntry:
    """One step of the run order.  ``layer`` indexes ``ModelSpec.layers`` and may appear
    more than once (every run keeps a cache of its own).  ``cache_from`` is the index of an
    earlier entry of the run order whose cache this run reads instead of keeping one of
    its own (it then writes nothing)."""

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    embedding: PartSpec
    positions: dict[str, PartSpec]
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("the run order is empty")
        for i, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"run order names layer {entry.layer}, which does not exist")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < i:
                    raise ValueError(
                        f"entry {i} of the run order borrows the cache of entry "
                        f"{entry.cache_from}, which is not an earlier entry")
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(
                        f"entry {i} of the run order borrows from entry {entry.cache_from}, "
                        "which has no cache of its own")
