"""Interfaces of the parts a model is put together from.

A part is built from constants (sizes, eps, theta, ...) given as keyword
parameters, declares the tensors it needs (``tensor_specs``), takes them
(``bind``) and then runs on the tokens of a step (``forward``).  No part knows
which model it is in or what runs before or after it.

Kinds and their ``forward``:

* ``embedding``:    ``forward(ctx, resid)``: resid[T, H] (float32) <- rows of the table
* ``position``:     no forward; mixers read its tables (``prepare(n_positions)``)
* ``norm``:         ``forward(ctx, delta, resid, out, rows=None, write_resid=True)``:
                    resid += delta; out <- norm(resid)  (delta None: plain norm)
* ``mixer``:        ``forward(ctx, x, layer_cache) -> delta [T, H]``; says what
                    it needs cached through ``kv_request`` / ``state_requests``
* ``feed_forward``: ``forward(ctx, x) -> delta [T, H]``
* ``block``:        ``forward(ctx, resid, delta, layer_cache) -> delta``: the
                    arrangement of two norms, a mixer and a feed-forward
* ``head``:         ``forward(ctx, x [n, H]) -> logits [n, V]`` float32

``resid`` is the float32 residual stream of the step; ``delta`` the output of
the previous sub-layer that has not been added to it yet (the deferred add of
engine/model.py:1-45 in davidjoyme/flashdecode-cuda).  A ``delta`` is [T, H]
in the activation dtype.

Partial sums are an agreement between two parts, never a surprise: a mixer or
feed-forward may return float32 partial sums [parts, T, H] (a matrix product
split over K, which the consumer adds up in order while it adds the rest) ONLY
when its caller passes ``parts_ok=True``.  A block passes that for a sub-layer
whose output goes to a norm with ``accepts_parts = True`` (the built-in RMSNorm),
and for its last sub-layer when ``ctx.delta_parts_ok`` says that whoever norms
next - the next block (``Block.accepts_parts``) or the final norm - takes them.
A norm, block or mixer that knows nothing of this gets plain [T, H] tensors.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..cache.paged import KVGroup, StateSpec
from ..weights.spec import TensorSpec


@dataclass
class Runtime:
    """What the parts of one model share on the device."""
    device: torch.device
    dtype: torch.dtype                 # activations, matrices and the cache: float32 or bfloat16
    status: torch.Tensor               # int32[1] status word the kernels set bits in
    sm_count: int = 148


@dataclass
class KVRequest:
    """Paged key/value storage a mixer needs for each sequence."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass
class LayerCache:
    """What one schedule entry sees of the cache."""
    group: Optional[KVGroup]           # None: the mixer keeps no keys
    layer: int                         # index inside the group
    writes: bool                       # False: it reads another entry's keys and state
    states: Dict[str, torch.Tensor]    # per-sequence state buffers [max_slots, ...], by the mixer's own names

    @property
    def k_pool(self) -> torch.Tensor:
        return self.group.k_pool(self.layer)

    @property
    def v_pool(self) -> torch.Tensor:
        return self.group.v_pool(self.layer)


class Part:
    kind = ""
    # False for a part whose forward reads the step's host mirrors (``ctx.h_*``) or
    # otherwise decides on the host: its steps cannot be replayed from a CUDA graph.
    graph_safe = True

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        """Take the declared tensors (already on the device, in their storage
        dtype).  Parts that repack tensors may pop the originals."""
        self.rt = rt

    def weight_bytes(self) -> int:
        """Bytes of weights one step has to read (for the roofline model)."""
        return 0

    def first_weights(self) -> Optional[torch.Tensor]:
        """The weights a decode step of this part streams first, or None.  Whoever runs the parts offers them
        to the part that runs before (``ctx.upcoming``), whose last kernel may ask L2 for their beginning."""
        return None


class Embedding(Part):
    kind = "embedding"


class Position(Part):
    kind = "position"

    def prepare(self, n_positions: int, rt: Runtime) -> None:
        raise NotImplementedError


class Norm(Part):
    kind = "norm"
    # True: ``forward`` takes ``delta`` as float32 partial sums [parts, T, H] as well as [T, H]
    accepts_parts = False


class Mixer(Part):
    kind = "mixer"

    def kv_request(self) -> Optional[KVRequest]:
        return None

    def state_requests(self) -> List[StateSpec]:
        return []


class FeedForward(Part):
    kind = "feed_forward"


class Block(Part):
    """An arrangement of parts in one layer.  Built as ``cls(**parts)`` from the named parts of its
    ``LayerSpec``; ``parts()`` lists them; ``mixer`` (if the block has one) is the part whose
    ``kv_request`` / ``state_requests`` size the layer's share of the cache."""
    kind = "block"
    # True: ``forward`` takes the incoming ``delta`` as float32 partial sums [parts, T, H] too
    accepts_parts = False


class Head(Part):
    kind = "head"
