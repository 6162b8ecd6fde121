"""Matrix products of the parts: ``out = x w^T (+ bias)`` with ``w [N, K]``.

float32: the library's own FFMA kernel with a fixed summation order (no
tensor cores, no reduced-precision mode).  bfloat16 with at most 16 rows of x
(decode steps): the weight-streaming ``mma.sync`` kernel (``csrc/gemv_mma.cu``);
17 to 128 rows (larger decode batches, short prompts): the weight-streaming
TMA + tcgen05 kernel (``csrc/gemm_stream_tcgen05.cu``).  More rows (prompts):
the TMA + tcgen05 kernel of ``csrc/gemm_tcgen05.cu`` where its fused epilogues
pay, cuBLAS through torch for the plain products, which is what ``F.linear`` is
in davidjoyme/flashdecode-cuda (engine/model.py:188-190,208,213-216,232).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K


# Which kernel takes the bfloat16 products of prompt steps (more than GEMV_MAX_ROWS rows):
#   "auto":    the library's own TMA + tcgen05 kernel where its fused epilogues pay for themselves
#              (q/k/v with bias + rotation + cache append, gate/up with SiLU), cuBLAS for the plain
#              products, where cuBLAS's 256-wide two-CTA tiles are still ahead (measured on B200);
#   "tcgen05": the library's own kernel everywhere;  "cublas": cuBLAS everywhere.
PROMPT_GEMM = "auto"

# Up to this many rows the weight-streaming kernel beats the library product (measured on
# B200 at the sizes of Qwen2.5-1.5B); above it the rows of x no longer fit the registers' reach.
GEMV_MAX_ROWS = 16
MAX_PARTS = 8           # most partial sums the norm's fast kernel adds up
# Up to this many rows (and above GEMV_MAX_ROWS) the streaming tcgen05 kernel takes the product with
# its fused epilogues: the rows of x are the N side of its MMAs, so nothing is padded to a 128-row tile.
STREAM_MAX_ROWS = 128
# How much of what the step streams next (``ctx.upcoming``) the last kernel of a part asks L2 for in a decode step of up
# to GEMV_MAX_ROWS rows.  It pays for what arrives before it is wanted, in the time the kernels in between leave HBM
# idle; more than that competes with the stream of whoever wants it.  Measured at the sizes of Qwen2.5-1.5B, batch 8
# and 1, for the attention kernel asking for the beginning of the 55 MB gate/up matrix: 8 MB - 1.0 / - 2.1 %, 16 MB
# - 1.9 / - 2.8 %, 24 MB - 1.7 / - 2.6 %, 32 MB - 1.3 / - 1.1 %, 40 MB and more: nothing, or slower.
UPCOMING_BYTES = 16 << 20


def stream_gemm(M: int, N: int, Kd: int) -> bool:
    """Whether a bfloat16 product with M rows of x goes to the streaming tcgen05 kernel."""
    return PROMPT_GEMM == "auto" and GEMV_MAX_ROWS < M <= STREAM_MAX_ROWS and K.gemm_stream_splits(M, N, Kd) > 0


def fused_prompt_gemm(M: int, N: int, Kd: int) -> bool:
    """Whether a product with a fused epilogue goes to the tcgen05 kernel: from one full
    128-row tile on (between GEMV_MAX_ROWS and 128 rows its tiles would be mostly padding)."""
    if PROMPT_GEMM == "cublas" or not K.gemm_tc_supported(M, N, Kd):
        return False
    return PROMPT_GEMM == "tcgen05" or M >= 128


def matmul(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
           target_ctas: int = 0, parts: Optional[torch.Tensor] = None,
           status: Optional[torch.Tensor] = None, upcoming: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K], w [N, K], bias [N] or None, out [M, N] (dtype of x, or
    float32 for logits).  ``target_ctas``: how many CTAs a decode product
    should spread over (it splits K to get there).  ``parts``: float32 memory
    for [splits <= MAX_PARTS, M, N]; when given (no bias) and the product is
    split, the splits' partial sums are returned in it as [splits, M, N] for the
    consumer to add up in order (the next norm does), instead of being added
    inside a thread-block cluster, whose launch and barriers cost more.
    ``status``: the status word for the kernels with bounded waits.  ``upcoming``: what the step
    streams after this product; a decode product asks L2 for its first ``UPCOMING_BYTES``."""
    if x.dtype == torch.float32:
        K.gemm_simt(x, w, bias, out)
        return out
    M, Kd = x.shape
    if M <= GEMV_MAX_ROWS:
        splits = K.gemv_splits(M, w.shape[0], Kd, target_ctas, allow_split=target_ctas > 0)
        if splits > 1 and parts is not None and bias is None and splits <= MAX_PARTS:
            view = parts.view(-1)[:splits * M * w.shape[0]].view(splits, M, w.shape[0])
            K.gemv(x, w, None, view, K.GEMV_PARTIAL, splits, prefetch=upcoming, prefetch_bytes=UPCOMING_BYTES)
            return view
        if splits >= 1:
            K.gemv(x, w, bias, out, K.GEMV_F32 if out.dtype == torch.float32 else K.GEMV_BF16, splits,
                   prefetch=upcoming, prefetch_bytes=UPCOMING_BYTES)
            return out
    if stream_gemm(M, w.shape[0], Kd):
        K.gemm_stream(x, w, bias, out, status=status)
        return out
    if PROMPT_GEMM == "tcgen05" and K.gemm_tc_supported(M, w.shape[0], Kd):
        K.gemm_tc(x, w, bias, out)
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
