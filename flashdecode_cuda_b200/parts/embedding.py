"""Token embedding: the start of the residual stream."""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import Embedding, Runtime


@register_part("embedding", "token_table")
class TokenEmbedding(Embedding):
    """resid[t] = table[token[t]], unscaled (engine/model.py:166,255 of
    davidjoyme/flashdecode-cuda), written as float32."""

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int):
        self.name = f"{prefix}.weight"
        self.vocab_size, self.hidden_size = vocab_size, hidden_size

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), "matrix")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.table = tensors[self.name]

    def forward(self, ctx, resid: torch.Tensor) -> None:
        K.embed(ctx.tokens, self.table, resid, self.rt.status)
