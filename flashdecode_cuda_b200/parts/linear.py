"""Matrix products of the parts: ``out = x w^T (+ bias)`` with ``w [N, K]``.

float32: the library's own FFMA kernel with a fixed summation order (no
tensor cores, no reduced-precision mode).  bfloat16: the hand-written
tensor-core kernels where they take the shape, else cuBLAS through torch,
which is what ``F.linear`` is in davidjoyme/flashdecode-cuda
(engine/model.py:188-190,208,213-216,232).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K


def matmul(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """x [M, K], w [N, K], bias [N] or None, out [M, N] (dtype of x, or
    float32 for logits)."""
    if x.dtype == torch.float32:
        K.gemm_simt(x, w, bias, out)
        return out
    if out.dtype == torch.float32:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
        if bias is not None:
            out.add_(bias)
        return out
    if bias is not None and bias.dtype == out.dtype:
        torch.addmm(bias, x, w.t(), out=out)
    else:
        torch.mm(x, w.t(), out=out)
        if bias is not None:
            out.add_(bias.to(out.dtype))
    return out
