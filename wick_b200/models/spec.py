"""A model described as data.

An architecture's ``build_spec(config)`` returns a :class:`ModelSpec`: which
part (by registered kind, with its sizes and constants as parameters) stands at
each place of each layer, under which tensor-name prefix its weights are
stored, and in which order the layers run.  Nothing here computes anything and
nothing here is specific to one architecture.

The run order is a list of :class:`ScheduleEntry`.  An entry names a layer (the
same layer may be named more than once: its weights are then shared, but each
entry has cache storage of its own) and may say that its mixer reads the cache
that an earlier entry wrote instead of writing one itself.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping, Optional, Tuple


@dataclasses.dataclass(frozen=True)
class PartSpec:
    """``kind`` selects a registered part class of some category; ``params`` are
    the sizes and constants that the class needs (never read from a model)."""

    kind: str
    params: Mapping[str, Any] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (``block``) of a mixer and a feed-forward, each
    with its norm.  ``prefix`` is the layer's tensor-name prefix; ``names`` maps
    each place (``mixer``, ``mixer_norm``, ``ffn``, ``ffn_norm``) to the
    sub-prefix its part's tensors are stored under."""

    block: PartSpec
    mixer: PartSpec
    mixer_norm: PartSpec
    ffn: PartSpec
    ffn_norm: PartSpec
    prefix: str
    names: Mapping[str, str]


@dataclasses.dataclass(frozen=True)
class ScheduleEntry:
    """Run ``layer``.  ``read_cache_of`` is the index (in the schedule) of an
    earlier entry whose cache this entry's mixer reads without writing."""

    layer: int
    read_cache_of: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab: int
    width: int                       # size of the residual stream
    max_position: int
    embedding: PartSpec
    embedding_prefix: str
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    final_norm_prefix: str
    head: PartSpec
    head_prefix: str
    ignore_tensors: Tuple[str, ...] = ()   # fnmatch patterns of names a checkpoint may carry unused
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        n = len(self.layers)
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ValueError(f"schedule[{i}] names layer {e.layer}, model has {n}")
            if e.read_cache_of is not None and not 0 <= e.read_cache_of < i:
                raise ValueError(f"schedule[{i}] reads the cache of entry {e.read_cache_of}, "
                                 f"which does not run before it")
            if e.read_cache_of is not None and self.schedule[e.read_cache_of].read_cache_of is not None:
                raise ValueError(f"schedule[{i}] reads the cache of entry {e.read_cache_of}, "
                                 f"which has none of its own")
