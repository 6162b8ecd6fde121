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


class LayerSpec:
    """One layer: the arrangement (a ``block`` part, by its registry name) and
    the parts it arranges, by the names the block class gives them.  The block
    class is built as ``block_cls(**built_parts)``, so which parts a layer has,
    and how many, is the block's business: the pre-norm block takes ``norm1,
    mixer, norm2, feed_forward``; another arrangement may take three norms, one
    norm shared by both sub-layers, or no feed-forward at all.  Different
    layers of one model may name different blocks, mixers and feed-forwards.

    ``LayerSpec("prenorm", norm1=..., mixer=..., norm2=..., feed_forward=...)``
    or ``LayerSpec("prenorm", {"norm1": ..., ...})``; the four parts of the
    pre-norm block may also be given by position, in that order.
    """

    _PRENORM_ORDER = ("norm1", "mixer", "norm2", "feed_forward")

    def __init__(self, block: str, *positional, **named):
        self.block = block
        parts: Dict[str, PartSpec] = {}
        if len(positional) == 1 and isinstance(positional[0], dict):
            parts.update(positional[0])
        elif positional:
            if len(positional) > len(self._PRENORM_ORDER):
                raise ValueError("parts given by position are norm1, mixer, norm2, feed_forward; name any others")
            parts.update(zip(self._PRENORM_ORDER, positional))
        parts.update(named)
        for name, spec in parts.items():
            if not isinstance(spec, PartSpec):
                raise TypeError(f"part {name!r} of a layer must be a PartSpec, got {type(spec).__name__}")
        self.parts = parts

    def __getattr__(self, name: str) -> PartSpec:
        parts = self.__dict__.get("parts", {})
        if name in parts:
            return parts[name]
        raise AttributeError(name)

    def __repr__(self) -> str:
        return f"LayerSpec({self.block!r}, {self.parts!r})"


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
