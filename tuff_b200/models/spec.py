"""The description of a model as data: parts chosen layer by layer, and the
order in which layers run.

`schedule` is a list of `ScheduleEntry`: the layer to run, the cache storage it
uses, and whether it only reads that storage (a layer that runs on another
layer's keys and values).  The default schedule runs every layer once, in
order, each with storage of its own; a schedule may name a layer twice (the
second run has its own storage unless it says otherwise).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

from ..parts.base import PartSpec


@dataclass
class LayerSpec:
    mixer: PartSpec
    ffn: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    block: PartSpec = field(default_factory=lambda: PartSpec("prenorm"))


@dataclass
class ScheduleEntry:
    layer: int
    storage: int            # index of the cache storage this run uses
    reads_only: bool = False


@dataclass
class ModelSpec:
    architecture: str
    d_model: int
    vocab_size: int
    embedding: PartSpec
    layers: List[LayerSpec]
    final_norm: PartSpec
    head: PartSpec
    schedule: List[ScheduleEntry] | None = None
    max_context: int | None = None

    def resolved_schedule(self) -> List[ScheduleEntry]:
        if self.schedule is None:
            return [ScheduleEntry(i, i) for i in range(len(self.layers))]
        for e in self.schedule:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule names layer {e.layer}, the model has {len(self.layers)}")
        return list(self.schedule)
