"""RMSNorm fused with the deferred residual add."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import Norm, Runtime


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """resid += delta; out = resid * rsqrt(mean(resid^2) + eps) * weight.

    The formula of ``rmsnorm_residual`` in davidjoyme/flashdecode-cuda
    (engine/ops.py:61-79, kernels/rmsnorm.cu:70-132).  There the sum is rounded
    to bfloat16 before it is squared and kept; here the residual stream stays in
    float32 and everything up to the final store is float32.
    """

    accepts_parts = True        # the kernel adds up to four float partial sums in order while it adds the residual

    def __init__(self, prefix: str, size: int, eps: float):
        self.name = f"{prefix}.weight"
        self.size, self.eps = size, float(eps)

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.size,), "vector", init="norm")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.weight = tensors[self.name]

    def forward(self, ctx, delta: Optional[torch.Tensor], resid: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, n_out: Optional[int] = None,
                write_resid: bool = True, n_parts: int = 1) -> None:
        K.add_rmsnorm(delta, resid, self.weight, self.eps, out, rows=rows, n_out=n_out,
                      write_resid=write_resid, n_parts=n_parts)
