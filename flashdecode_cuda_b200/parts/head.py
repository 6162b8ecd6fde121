"""Output head: logits at the wanted rows."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import Head, Runtime
from .linear import matmul


@register_part("head", "linear_head")
class LinearHead(Head):
    """logits = x W^T in float32, no bias, no scaling (engine/model.py:229-234
    of davidjoyme/flashdecode-cuda).  ``tied_to``: the name of the embedding
    table to use when the checkpoint keeps no separate head
    (engine/loader.py:39-40)."""

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None):
        self.name = f"{prefix}.weight"
        self.vocab_size, self.hidden_size, self.tied_to = vocab_size, hidden_size, tied_to

    def tensor_specs(self) -> List[TensorSpec]:
        if self.tied_to:
            return []
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), "matrix")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.weight = tensors[self.tied_to or self.name]

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.weight

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        logits = ctx.ws.get("logits", (x.shape[0], self.vocab_size), torch.float32)
        matmul(x, self.weight, None, logits, status=self.rt.status)
        return logits
