"""Rotary position encoding with rotate-half pairing (j with j + d/2)."""

from __future__ import annotations

import torch

from ..registry import register_part
from .base import Position, Runtime


@register_part("position", "rotary_half")
class RotaryHalf(Position):
    """cos/sin tables [positions, d/2] in float32.

    inv_freq_j = 1 / theta^(2j/d), angle[p, j] = p * inv_freq_j, both computed
    in float32 exactly as ``build_rope_cache`` of davidjoyme/flashdecode-cuda
    does (engine/ops.py:102-110); its tables repeat the d/2 angles twice, these
    keep one copy.  The table covers the configuration's
    ``max_position_embeddings`` (the reference caps at 8192,
    engine/model.py:82-91); a position beyond it sets a status bit instead of
    reading out of bounds.
    """

    # Tables longer than this many positions are built for what the first cache asks for instead of the
    # configuration's whole max_position_embeddings (8 bytes per position and pair of dims).
    FULL_TABLE_LIMIT = 1 << 18

    def __init__(self, head_dim: int, theta: float, max_positions: int):
        self.head_dim, self.theta, self.max_positions = head_dim, float(theta), max_positions
        self.cos = self.sin = None

    def prepare(self, n_positions: int, rt: Runtime) -> None:
        """Build the tables, once.  They are made for every position the configuration allows (or, beyond
        ``FULL_TABLE_LIMIT`` positions, for what this first cache needs) and never replaced: kernels
        captured into CUDA graphs hold their addresses and their length, so a later, longer cache must
        find the same tensors.  A cache that needs more positions than the tables have is refused."""
        n = min(n_positions, self.max_positions)
        if self.cos is not None:
            if self.cos.shape[0] < n:
                raise ValueError(f"the rotary tables were built for {self.cos.shape[0]} positions and cannot grow "
                                 f"(captured graphs hold their address); a cache of {n} positions needs a model "
                                 f"loaded anew, or a first cache at least as long")
            return
        if self.max_positions <= self.FULL_TABLE_LIMIT:
            n = self.max_positions
        d = self.head_dim
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, d, 2).float() / d))
        freqs = torch.outer(torch.arange(n).float(), inv_freq)
        self.cos = freqs.cos().contiguous().to(rt.device)
        self.sin = freqs.sin().contiguous().to(rt.device)
