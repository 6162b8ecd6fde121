"""A model as data: which parts, with which constants, in which order.

An architecture's registry entry turns its configuration into a
``ModelBlueprint``; ``engine.model.Model`` builds the parts from it.  Nothing
here knows a concrete part or architecture.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class PartSpec:
    """A part to build: registry key (``kind``, ``name``), its constants and
    the prefix of its tensors' names in the checkpoint."""
    kind: str
    name: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass
class LayerSpec:
    """One layer: the arrangement (a ``block`` part) and the four parts it
    arranges.  Different layers of one model may name different mixers and
    feed-forwards."""
    block: str
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    feed_forward: PartSpec


@dataclass
class RunSpec:
    """One entry of the order in which layers run.  ``layer`` indexes
    ``ModelBlueprint.layers`` (a layer may be named by several entries: its
    weights are shared, its cache is not).  ``cache_from``: index of an EARLIER
    entry whose keys/values and state this entry reads instead of keeping its
    own."""
    layer: int
    cache_from: Optional[int] = None


@dataclass
class ModelBlueprint:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    positions: Dict[str, PartSpec]            # shared position encodings, by the name mixers ask for
    layers: List[LayerSpec]
    schedule: List[RunSpec]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int                        # longest sequence the configuration allows

    def validate(self) -> None:
        for i, run in enumerate(self.schedule):
            if not (0 <= run.layer < len(self.layers)):
                raise ValueError(f"schedule entry {i} names layer {run.layer}, the model has {len(self.layers)}")
            if run.cache_from is not None:
                if not (0 <= run.cache_from < i):
                    raise ValueError(f"schedule entry {i} reads the cache of entry {run.cache_from}, "
                                     f"which does not run before it")
                if self.schedule[run.cache_from].cache_from is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {run.cache_from}, "
                                     f"which keeps none of its own")
