"""A model as data: which parts, with which constants, run in which order.

``ModelSpec`` is what an architecture's builder returns.  It names parts by
their registry kind and gives each its sizes and constants; nothing in it is
code.  The order in which layers run is data too (``schedule``): a list of
``(layer, cache_layer)`` pairs which may name a layer twice or let a layer
use another layer's cache.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


@dataclass
class PartSpec:
    kind: str                       # key in the part registry
    params: dict = field(default_factory=dict)
    prefix: str = ""                # prepended to the part's tensor names


@dataclass
class LayerSpec:
    block: PartSpec                 # the arrangement (e.g. "pre_norm")
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]      # the norms the arrangement asks for, by role


@dataclass
class ScheduleEntry:
    layer: int                      # which layer's parameters run
    cache_layer: int                # which cache layer (pages / slot state) this run reads and writes;
                                    # cache layers are their own index space: a layer that runs twice
                                    # takes two, two runs that name the same one share it


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_model_len: int
    embedding: PartSpec
    positions: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    # maps a tensor name found in a checkpoint to its canonical name, or None to ignore it
    normalise_name: Optional[Callable[[str], Optional[str]]] = None
    # the inverse: canonical name -> the name a checkpoint of this architecture stores it under
    checkpoint_name: Optional[Callable[[str], str]] = None

    def __post_init__(self):
        if not self.schedule:
            self.schedule = [ScheduleEntry(i, i) for i in range(len(self.layers))]
        for entry in self.schedule:
            if not (0 <= entry.layer < len(self.layers)) or entry.cache_layer < 0:
                raise ValueError("schedule names a layer that does not exist")

    @property
    def num_cache_layers(self) -> int:
        return max(entry.cache_layer for entry in self.schedule) + 1
