"""Choosing the next token of each sequence from its logits, on the device.

davidjoyme/flashdecode-cuda samples greedily only (``logits.argmax(-1)``,
engine/model.py:324,327).  Greedy here is the same argmax (the lowest index
wins a tie); temperature sampling is added as a Gumbel-max draw whose noise is
keyed by (seed, request id, step of the request), so a request's tokens do not
depend on which other requests share its batch or on its row in it.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from .. import kernels as K


@dataclass
class SamplingParams:
    """``temperature`` 0: greedy.  ``seed`` keys the noise of temperature sampling."""
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        if not (self.temperature >= 0.0):
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._out: Optional[torch.Tensor] = None

    def _buf(self, n: int) -> torch.Tensor:
        if self._out is None or self._out.numel() < n:
            self._out = torch.zeros(max(n, 64), dtype=torch.int32, device=self.device)
        return self._out[:n]

    def sample(self, logits: torch.Tensor, temperatures: Optional[Sequence[float]] = None,
               request_ids: Optional[Sequence[int]] = None, steps: Optional[Sequence[int]] = None,
               seed: int = 0) -> torch.Tensor:
        """int32 [n] token ids on the device (a buffer the next call reuses).
        Rows with temperature 0 (or ``temperatures`` None) are greedy."""
        n = logits.shape[0]
        out = self._buf(n)
        if temperatures is None or not any(t > 0.0 for t in temperatures):
            K.sample(logits, out)
            return out
        if request_ids is None or steps is None or len(request_ids) != n or len(steps) != n or len(temperatures) != n:
            raise ValueError("temperature sampling needs one temperature, request id and step per row")
        temp = torch.from_numpy(np.asarray(temperatures, dtype=np.float32)).to(self.device)
        req = torch.from_numpy(np.asarray(request_ids, dtype=np.int64)).to(self.device)
        stp = torch.from_numpy(np.asarray(steps, dtype=np.int32)).to(self.device)
        K.sample(logits, out, temp, req, stp, seed)
        return out
