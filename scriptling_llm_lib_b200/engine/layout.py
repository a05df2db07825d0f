"""A model as data: its layers, the order they run in, and what surrounds them.

The reference runs blocks 0..L-1 once each over one cache per block (model_f32.go:371-373). Here
the order is a list of schedule entries; an entry names the layer to run and the cache unit it
uses, so a layer can appear twice (with a unit for each appearance) or read the unit that another
entry wrote (`writes_cache=False`). An entry may also name stream inputs that run right before its layer (`before`,
indices into the layout's `stream_parts`): parts that add to the residual stream between two layers, such as the vector
that opens a pass over a run of layers that is gone through several times with the same weights.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..parts.base import PartSpec
from ..parts.block import LayerSpec


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int
    cache_unit: int
    writes_cache: bool = True
    before: tuple[int, ...] = ()        # stream inputs (ModelLayout.stream_parts) that run right before the layer


@dataclass(frozen=True)
class ModelLayout:
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec                 # resolved through the EMBEDDINGS registry
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec                # NORMS; adds the last pending addend and norms the wanted rows
    head: PartSpec                      # HEADS
    stop_ids: tuple[int, ...] = ()
    ignorable_tensors: tuple[str, ...] = field(default=())   # may be in the file without being used
    stream_parts: tuple[PartSpec, ...] = ()                  # STREAM_INPUTS that schedule entries run before their layers

    def check(self) -> None:
        written: set[int] = set()
        for e in self.schedule:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule names layer {e.layer}; the model has {len(self.layers)}")
            for i in e.before:
                if not 0 <= i < len(self.stream_parts):
                    raise ValueError(f"schedule names stream input {i}; the model has {len(self.stream_parts)}")
            if e.writes_cache:
                if e.cache_unit in written:
                    raise ValueError(f"cache unit {e.cache_unit} is written by two schedule entries")
                written.add(e.cache_unit)
            elif e.cache_unit not in written:
                raise ValueError(f"schedule entry reads cache unit {e.cache_unit} before any entry has written it")


def sequential_schedule(n_layers: int) -> tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(i, i, True) for i in range(n_layers))


def looped_schedule(n_layers: int, start: int, stop: int, times: int, before_pass=None) -> tuple[ScheduleEntry, ...]:
    """The schedule of a model that goes through the run of layers [start, stop) `times` times on one set of weights: the
    layers before the run once, the run again and again, then the layers behind it once. Every appearance of a layer has a
    cache unit of its own, numbered in running order. `before_pass(t)` -> the stream
    inputs (indices) that run right before pass t's first layer."""
    if not 0 <= start <= stop <= n_layers or times < 1:
        raise ValueError(f"a loop over layers {start}..{stop - 1} of {n_layers}, {times} times")
    order = [(i, ()) for i in range(start)]
    for t in range(times):
        order += [(i, tuple(before_pass(t)) if before_pass is not None and i == start else ()) for i in range(start, stop)]
    order += [(i, ()) for i in range(stop, n_layers)]
    return tuple(ScheduleEntry(layer, unit, True, before) for unit, (layer, before) in enumerate(order))
