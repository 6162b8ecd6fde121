"""Dense gated feed-forward (SwiGLU)."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import FeedForward, Runtime
from .linear import GEMV_MAX_ROWS, MAX_PARTS, fused_prompt_gemm, matmul, stream_gemm


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """down( silu(gate(x)) * up(x) ), no biases (engine/model.py:213-216 and
    engine/ops.py:201-204 of davidjoyme/flashdecode-cuda).  gate and up are one
    [2I, H] matrix here, so they are one product."""

    offers_parts = True     # forward(..., parts_ok=True) may return float partial sums [parts, T, H]

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int):
        self.prefix, self.hidden_size, self.inter = prefix, hidden_size, intermediate_size

    def tensor_specs(self) -> List[TensorSpec]:
        p, H, I = self.prefix, self.hidden_size, self.inter
        return [TensorSpec(f"{p}.gate_proj.weight", (I, H)),
                TensorSpec(f"{p}.up_proj.weight", (I, H)),
                TensorSpec(f"{p}.down_proj.weight", (H, I))]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p, I = self.prefix, self.inter
        gate, up = tensors.pop(f"{p}.gate_proj.weight"), tensors.pop(f"{p}.up_proj.weight")
        # tiles of 16 rows: 8 gate rows, then the 8 up rows of the same outputs, so the decode
        # kernel's thread that holds gate_i also holds up_i (csrc/gemv_mma.cu)
        self.tiled = I % 8 == 0
        if self.tiled:
            H = gate.shape[1]
            self.w_gate_up = torch.stack([gate.view(I // 8, 8, H), up.view(I // 8, 8, H)], dim=1) \
                .reshape(2 * I, H).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[f"{p}.down_proj.weight"]

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.w_gate_up

    def forward(self, ctx, x: torch.Tensor, parts_ok: bool = False) -> torch.Tensor:
        """delta [T, H]; with ``parts_ok`` (the caller's consumer adds partial sums up) a decode step's down
        projection may come back as float32 [parts, T, H] instead."""
        T, ws = ctx.T, ctx.ws
        act = ws.get("ffn_act", (T, self.inter), x.dtype)
        if (self.tiled and x.dtype == torch.bfloat16 and T <= GEMV_MAX_ROWS
                and K.gemv_splits(T, 2 * self.inter, self.hidden_size, 1, allow_split=False) == 1):
            K.gemv(x, self.w_gate_up, None, act, K.GEMV_GATED)          # product and silu(gate) * up in one kernel
        elif self.tiled and x.dtype == torch.bfloat16 and stream_gemm(T, 2 * self.inter, self.hidden_size):
            K.gemm_stream(x, self.w_gate_up, None, act, gated=True, status=self.rt.status)      # 17 to 128 rows: the same fusion
        elif self.tiled and x.dtype == torch.bfloat16 and fused_prompt_gemm(T, 2 * self.inter, self.hidden_size):
            K.gemm_tc(x, self.w_gate_up, None, act, gated=True, status=self.rt.status)     # prompts: tcgen05, same fusion
        else:
            gu = ws.get("gate_up", (T, 2 * self.inter), x.dtype)
            matmul(x, self.w_gate_up, None, gu, status=self.rt.status)
            K.silu_mul(gu, act, tiled=self.tiled)
        out = ws.get("ffn_out", (T, self.hidden_size), x.dtype)
        parts = None
        if parts_ok and T <= GEMV_MAX_ROWS:
            parts = ws.get("ffn_out_parts", (MAX_PARTS, T, self.hidden_size), torch.float32)
        return matmul(act, self.w_down, None, out, target_ctas=4 * self.rt.sm_count, parts=parts, status=self.rt.status,
                      upcoming=ctx.upcoming)
