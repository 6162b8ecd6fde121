"""What a part asks of a checkpoint: one ``TensorSpec`` per tensor."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class TensorSpec:
    """``name``: the tensor's name in the checkpoint.  ``shape``: what the
    configuration implies.  ``kind``: ``matrix`` (operand of a matrix product
    or a lookup table of activations: kept in the compute dtype), ``vector``
    (norm weights, biases: a tensor stored in 32-bit stays so) or ``table``
    (integers: kept as int32).  ``optional``: absence is not an error.
    ``init``: how the random-weights mode draws it: ``normal`` N(0, 0.02),
    ``norm`` 1 + N(0, 0.1), ``bias`` N(0, 0.02), ``zeros``."""

    name: str
    shape: Tuple[int, ...]
    kind: str = "matrix"
    optional: bool = False
    init: str = "normal"
