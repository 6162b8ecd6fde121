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
    keep one copy.  The table is as long as the cache can hold, capped by the
    configuration's ``max_position_embeddings`` (the reference caps at 8192,
    engine/model.py:82-91); a position beyond it sets a status bit instead of
    reading out of bounds.
    """

    def __init__(self, head_dim: int, theta: float, max_positions: int):
        self.head_dim, self.theta, self.max_positions = head_dim, float(theta), max_positions
        self.cos = self.sin = None

    def prepare(self, n_positions: int, rt: Runtime) -> None:
        n = min(n_positions, self.max_positions)
        if self.cos is not None and self.cos.shape[0] >= n:
            return
        d = self.head_dim
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, d, 2).float() / d))
        freqs = torch.outer(torch.arange(n).float(), inv_freq)
        self.cos = freqs.cos().contiguous().to(rt.device)
        self.sin = freqs.sin().contiguous().to(rt.device)
