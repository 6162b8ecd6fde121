"""Grouped-query attention over the paged cache: the mixer of this architecture."""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import KVRequest, LayerCache, Mixer, Runtime
from .linear import GEMV_MAX_ROWS, UPCOMING_BYTES, fused_prompt_gemm, matmul, stream_gemm


MAX_SPLITS = 32
PREFETCH_BYTES = 16 << 20   # an output projection up to this size is asked for ahead by the decode q/k/v kernel (whole; a 16 MB
                            # beginning of a larger one made the step slower: + 1.4 % at the sizes of Qwen2.5-7B, batch 8)
FP32_SPLIT_LEN = 256      # keys per split of a decode step in float32


def plan_splits(n_rows: int, n_kv: int, kv_len_bound: int, sm_count: int):
    """How a decode step cuts each sequence's keys: (n_splits, split_len).
    Split boundaries are multiples of ``split_len`` in absolute position, so
    they do not move with the batch's contents (only with its size and the
    length bound).  Few (sequence, KV head) pairs: one CTA of eight warps per SM
    (the kernel takes that form from four splits on, when all CTAs fit the GPU
    at one per SM); many: about two CTAs of four warps per SM."""
    ctas = max(1, n_rows * n_kv)
    # at most 32 splits: beyond that the merge of the splits costs more than longer splits do (measured at
    # batch 1: 16k context 1.54 ms per step with 32 splits of 512 keys, 1.72 ms with 128 splits of 128)
    if ctas * 4 <= sm_count:
        want = min(MAX_SPLITS, sm_count // ctas)
    else:
        want = max(1, min(MAX_SPLITS, (2 * sm_count) // ctas))
    split_len = -(-kv_len_bound // want)
    split_len = max(128, -(-split_len // 32) * 32)
    n_splits = max(1, -(-kv_len_bound // split_len))
    return n_splits, split_len


@register_part("mixer", "gqa_attention")
class GQAAttention(Mixer):
    """q/k/v projections (bias optional), rotary encoding of q and k fused with
    the append to the cache, causal attention of each new token over its
    sequence's cached keys, output projection.

    Formulas: engine/model.py:188-208,273-293 and engine/ops.py:153-194 of
    davidjoyme/flashdecode-cuda; query head h reads KV head h // G; scale
    1/sqrt(head_dim).  ``window``: a query sees only the last ``window`` keys.
    ``bias``: True = required, False = refused, None = taken if the checkpoint
    has it (the reference's rule, engine/loader.py:29-33).
    """

    def __init__(self, prefix: str, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: "RotaryHalf", window: Optional[int] = None, bias: Optional[bool] = None):
        if head_dim < 16 or head_dim > 256 or head_dim % 16 != 0:
            raise ValueError(f"{prefix}: head size {head_dim} is not taken: the attention kernels take multiples of 16 "
                             f"from 16 to 256")
        if n_kv_heads < 1 or n_heads % n_kv_heads != 0 or n_heads // n_kv_heads > 64:
            raise ValueError(f"{prefix}: {n_heads} query heads for {n_kv_heads} key/value heads: the kernels take whole "
                             f"groups of up to 64 query heads per key/value head")
        self.prefix = prefix
        self.hidden_size, self.n_q, self.n_kv, self.d = hidden_size, n_heads, n_kv_heads, head_dim
        self.position, self.window, self.bias = position, window, bias
        self.scale = 1.0 / math.sqrt(head_dim)

    # --- what it needs -------------------------------------------------
    def tensor_specs(self) -> List[TensorSpec]:
        p, H, d = self.prefix, self.hidden_size, self.d
        specs = [TensorSpec(f"{p}.q_proj.weight", (self.n_q * d, H)),
                 TensorSpec(f"{p}.k_proj.weight", (self.n_kv * d, H)),
                 TensorSpec(f"{p}.v_proj.weight", (self.n_kv * d, H)),
                 TensorSpec(f"{p}.o_proj.weight", (H, self.n_q * d))]
        if self.bias is not False:
            opt = self.bias is None
            specs += [TensorSpec(f"{p}.q_proj.bias", (self.n_q * d,), "vector", optional=opt, init="bias"),
                      TensorSpec(f"{p}.k_proj.bias", (self.n_kv * d,), "vector", optional=opt, init="bias"),
                      TensorSpec(f"{p}.v_proj.bias", (self.n_kv * d,), "vector", optional=opt, init="bias")]
        return specs

    def kv_request(self) -> KVRequest:
        return KVRequest(self.n_kv, self.d, self.window)

    def _paired_order(self) -> torch.Tensor:
        """Row order of the packed q/k/v matrix: inside every q and k head, tiles
        of 8 dims followed by their 8 rotation partners (dims + d/2), so that the
        decode kernel's thread that holds x_j also holds x_{j + d/2}
        (csrc/gemv_mma.cu, mode 4); v heads stay in natural order."""
        d, half = self.d, self.d // 2
        head = torch.arange(d).view(2, d // 16, 8).permute(1, 0, 2).reshape(d)     # [t][lo|hi][8] -> dims
        rows = [h * d + head for h in range(self.n_q + self.n_kv)]
        rows += [torch.arange((self.n_q + self.n_kv) * d, (self.n_q + 2 * self.n_kv) * d)]
        return torch.cat(rows)

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p = self.prefix
        names = [f"{p}.{x}_proj" for x in "qkv"]
        # one [ (n_q + 2 n_kv) d, H ] matrix: one product instead of three
        w_qkv = torch.cat([tensors.pop(f"{n}.weight") for n in names], dim=0)
        have = [f"{n}.bias" in tensors for n in names]
        if any(have) and not all(have):
            raise ValueError(f"{p}: q/k/v biases must be all present or all absent")
        b_qkv = torch.cat([tensors.pop(f"{n}.bias") for n in names]) if all(have) else None
        self.paired = self.d % 16 == 0
        if self.paired:
            order = self._paired_order().to(w_qkv.device)
            w_qkv = w_qkv[order]
            b_qkv = b_qkv[order] if b_qkv is not None else None
        self.w_qkv = w_qkv.contiguous()
        self.b_qkv = b_qkv.contiguous() if b_qkv is not None else None
        self.w_o = tensors[f"{p}.o_proj.weight"]

    def weight_bytes(self) -> int:
        n = self.w_qkv.numel() * self.w_qkv.element_size() + self.w_o.numel() * self.w_o.element_size()
        if self.b_qkv is not None:
            n += self.b_qkv.numel() * self.b_qkv.element_size()
        return n

    # --- a step ----------------------------------------------------------
    def first_weights(self) -> Optional[torch.Tensor]:
        return self.w_qkv

    def forward(self, ctx, x: torch.Tensor, lc: LayerCache) -> torch.Tensor:
        T, d = ctx.T, self.d
        ws = ctx.ws
        q = ws.get("q_rot", (T, self.n_q * d), x.dtype)
        rope = self.position
        splits = 0
        if self.paired and x.dtype == torch.bfloat16 and T <= GEMV_MAX_ROWS:
            splits = K.gemv_splits(T, self.w_qkv.shape[0], self.hidden_size, 4 * self.rt.sm_count)
        if splits >= 1:
            # decode: projection, bias, rotation and cache append in one kernel
            # (and it asks L2 for the output projection's weights, which are read after the attention)
            K.gemv_qkv_rope(x, self.w_qkv, self.b_qkv, q, rope.cos, rope.sin, ctx.tok_row, ctx.tok_pos, ctx.row_slot,
                            lc.k_pool, lc.v_pool, lc.group.table, self.n_q, self.n_kv, d, lc.writes, self.rt.status,
                            splits, prefetch=self.w_o if self.w_o.numel() * 2 <= PREFETCH_BYTES else None)
        elif self.paired and x.dtype == torch.bfloat16 and stream_gemm(T, self.w_qkv.shape[0], self.hidden_size):
            # larger decode batches and short prompts: the same fusion in the streaming tcgen05 kernel
            K.gemm_stream_qkv_rope(x, self.w_qkv, self.b_qkv, q, rope.cos, rope.sin, ctx.tok_row, ctx.tok_pos,
                                   ctx.row_slot, lc.k_pool, lc.v_pool, lc.group.table, self.n_q, self.n_kv, d,
                                   lc.writes, self.rt.status)
        elif self.paired and x.dtype == torch.bfloat16 and fused_prompt_gemm(T, self.w_qkv.shape[0], self.hidden_size):
            # prompts: the same fusion on the tcgen05 tensor cores
            K.gemm_tc_qkv_rope(x, self.w_qkv, self.b_qkv, q, rope.cos, rope.sin, ctx.tok_row, ctx.tok_pos, ctx.row_slot,
                               lc.k_pool, lc.v_pool, lc.group.table, self.n_q, self.n_kv, d, lc.writes, self.rt.status)
        else:
            qkv = ws.get("qkv", (T, (self.n_q + 2 * self.n_kv) * d), x.dtype)
            matmul(x, self.w_qkv, self.b_qkv, qkv, status=self.rt.status)
            K.rope_append(qkv, q, rope.cos, rope.sin, ctx.tok_row, ctx.tok_pos, ctx.row_slot, lc.k_pool, lc.v_pool,
                          lc.group.table, self.n_q, self.n_kv, d, lc.writes, self.rt.status, paired=self.paired)
        attn = ws.get("attn", (T, self.n_q * d), x.dtype)
        n_splits, split_len, scratch = 1, 0, None
        if ctx.max_q_len == 1 and x.dtype == torch.float32:
            # the 32-bit path: splits of a fixed length, so that where a sequence's partial sums are cut - and with
            # it every bit of its result - depends on nothing but its own length
            split_len = FP32_SPLIT_LEN
            n_splits = max(1, -(-ctx.kv_len_bound // split_len))
            if n_splits > 1:
                scratch = ws.get("attn_scratch", (K.attention_scratch_floats(T, self.n_q, d, n_splits),),
                                 torch.float32)
        elif ctx.max_q_len == 1:
            n_splits, split_len = plan_splits(ctx.n_rows, self.n_kv, ctx.kv_len_bound, self.rt.sm_count)
            if n_splits > 1:
                scratch = ws.get("attn_scratch", (K.attention_scratch_floats(T, self.n_q, d, n_splits),),
                                 torch.float32)
        # a small decode step: when its keys and values are through, the attention kernel asks L2 for the beginning of
        # what the step streams after this part (the output projection's weights are in L2 already, see above)
        ahead = ctx.upcoming if ctx.max_q_len == 1 and T <= GEMV_MAX_ROWS and x.dtype == torch.bfloat16 else None
        K.attention(q, lc.k_pool, lc.v_pool, attn, lc.group.table, ctx.tok_row, ctx.row_slot,
                         ctx.row_q_start, ctx.row_q_len, ctx.row_ctx_len, ctx.n_rows, ctx.max_q_len,
                         self.n_q, self.n_kv, d, self.scale, self.window or 0, n_splits, split_len, scratch,
                         self.rt.status, prefetch=ahead, prefetch_bytes=UPCOMING_BYTES)
        out = ws.get("mixer_out", (T, self.hidden_size), x.dtype)
        return matmul(attn, self.w_o, None, out, target_ctas=4 * self.rt.sm_count, status=self.rt.status)
