"""Consecutive layers of one kind, run by one persistent kernel in decode steps.

A decode step of a small batch is a chain of short kernels whose time is
mostly launch gaps and the start of each kernel's first loads.  Where the
schedule holds a run of layers that are all "pre-norm block of RMSNorm,
grouped-query attention with rotary encoding, RMSNorm, gated SiLU feed-forward"
with the same sizes, ``DecodeStack`` runs the whole run as ONE cooperative
kernel (``csrc/decode_stack.cu``): the CTAs stay resident, phases are separated
by grid barriers, and the next phase's weights are already on their way into L2
while a phase runs.

This is a property of the parts, not of a model: ``find_stacks`` looks at the
parts of each schedule entry, so any architecture assembled from these parts
gets it, and a layer with another mixer, feed-forward or norm simply ends the
run and goes through its own ``forward``.  The result equals calling the
blocks one after another (same formulas, same order of every sum that the
parts' own kernels use within a layer), up to the rounding of the attention's
output projection, which stays in float32 here instead of being rounded to
bfloat16 before the residual add.

Off by default: ``FD_DECODE_STACK=1`` in the environment switches it on.
Measured on B200 (Qwen2.5-1.5B sizes, batch 8, context 3.4k, 8 layers inside a
captured graph) it is correct but slower than the layers' own kernels, 1.07 ms
against 0.54 ms per step.  Leaving phases out one at a time gives, per layer:
the five grid barriers 12.5 us; q/k/v 7 us; attention 22 us; o 4 us; gate/up 26
us (10.5 us as a kernel of its own); down 14.5 us; the two norms, each run by
the one CTA that arrives last, 18 us.  With one CTA of 16 warps per SM (the
attention phase needs 118 registers per thread) the products have too few loads
in flight, and a barrier costs as much as a kernel boundary, so residency alone
gains nothing; what it would take is products fed by TMA through a deep ring of
shared memory, which keep HBM busy at low occupancy.
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels as K
from ..parts.attention import GQAAttention, plan_splits
from ..parts.base import LayerCache
from ..parts.block import PreNormBlock
from ..parts.mlp import SwiGLU
from ..parts.norm import RMSNorm

MAX_ROWS = 16          # rows of a step the kernel takes (two 8-row tensor-core tiles)
MAX_SPLITS = 4         # most ranges of K whose partial sums a norm adds up


def enabled() -> bool:
    return os.environ.get("FD_DECODE_STACK", "0") == "1"


def _signature(block) -> Optional[Tuple]:
    """What two blocks must share to sit in one stack; None if the block is of another kind."""
    if type(block) is not PreNormBlock:
        return None
    n1, mx, n2, ff = block.norm1, block.mixer, block.norm2, block.feed_forward
    if type(n1) is not RMSNorm or type(n2) is not RMSNorm or type(mx) is not GQAAttention or type(ff) is not SwiGLU:
        return None
    if not getattr(mx, "paired", False) or not getattr(ff, "tiled", False):
        return None
    H, I, d, G = mx.hidden_size, ff.inter, mx.d, mx.n_q // mx.n_kv
    if d not in (64, 128) or G > 16 or H % 32 or I % 32 or (mx.n_q * d) % 32 or ff.hidden_size != H:
        return None
    tensors = [mx.w_qkv, mx.w_o, ff.w_gate_up, ff.w_down]
    if any(t.dtype != torch.bfloat16 for t in tensors):
        return None
    norm_dt = n1.weight.dtype
    if n2.weight.dtype != norm_dt or n1.size != H or n2.size != H:
        return None
    bias_dt = mx.b_qkv.dtype if mx.b_qkv is not None else None
    return (H, I, mx.n_q, mx.n_kv, d, id(mx.position), norm_dt, bias_dt, mx.b_qkv is None)


class DecodeStack:
    """Schedule entries ``first .. last`` (inclusive) as one kernel."""

    def __init__(self, model, first: int, last: int):
        self.model, self.first, self.last = model, first, last
        self.blocks = [model.blocks[model.schedule[i].layer] for i in range(first, last + 1)]
        b0 = self.blocks[0]
        mx, ff = b0.mixer, b0.feed_forward
        self.H, self.I, self.n_q, self.n_kv, self.d = mx.hidden_size, ff.inter, mx.n_q, mx.n_kv, mx.d
        self.scale, self.position = mx.scale, mx.position
        self.bias_f32 = int(mx.b_qkv is not None and mx.b_qkv.dtype == torch.float32)
        self.norm_w_f32 = int(b0.norm1.weight.dtype == torch.float32)
        rt = model.rt
        self.ctas = rt.sm_count
        qkv_rows = (self.n_q + 2 * self.n_kv) * self.d
        self.qkv_wk, _ = K.decode_stack_plan(qkv_rows, self.H, self.ctas, 1)
        self.o_wk, self.o_splits = K.decode_stack_plan(self.H, self.n_q * self.d, self.ctas, MAX_SPLITS)
        self.gu_wk, _ = K.decode_stack_plan(2 * self.I, self.H, self.ctas, 1)
        self.down_wk, self.down_splits = K.decode_stack_plan(self.H, self.I, self.ctas, MAX_SPLITS)
        self.barrier = torch.zeros(4, dtype=torch.int32, device=rt.device)
        self._tables: Dict[Tuple, torch.Tensor] = {}
        self.failed = False
        self.skip = 0          # timing studies: phases the kernel leaves out (see kernels.decode_stack)

    def takes(self, ctx) -> bool:
        return (enabled() and not self.failed and ctx.max_q_len == 1 and ctx.T == ctx.n_rows and ctx.T <= MAX_ROWS
                and ctx.rt.dtype == torch.bfloat16 and self.model.trace is None)

    def _layer_table(self, caches: List[LayerCache]) -> torch.Tensor:
        """The device array of per-layer pointers and constants for this cache (built once per cache)."""
        mine = caches[self.first:self.last + 1]
        key = tuple((lc.k_pool.data_ptr(), lc.group.table.data_ptr(), lc.writes) for lc in mine)
        tab = self._tables.get(key)
        if tab is None:
            raw = b""
            for j, (blk, lc) in enumerate(zip(self.blocks, mine)):
                nxt = self.blocks[j + 1].norm1 if j + 1 < len(self.blocks) else None
                mx, ff = blk.mixer, blk.feed_forward
                raw += K.pack_stack_layer(mx.w_qkv, mx.b_qkv, mx.w_o, ff.w_gate_up, ff.w_down, blk.norm2.weight,
                                          nxt.weight if nxt is not None else None, lc.k_pool, lc.v_pool, lc.group.table,
                                          blk.norm2.eps, nxt.eps if nxt is not None else 0.0, mx.window or 0, lc.writes)
            tab = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(self.model.rt.device)
            if len(self._tables) > 8:
                self._tables.clear()
            self._tables[key] = tab
        return tab

    def forward(self, ctx, resid: torch.Tensor, delta: Optional[torch.Tensor], caches: List[LayerCache]) -> torch.Tensor:
        """What the blocks' own ``forward`` calls would do one after another; returns the last
        feed-forward's output as float32 partial sums [parts, T, H], still to be added."""
        M, ws, rt = ctx.T, ctx.ws, ctx.rt
        dt = rt.dtype
        xn = ws.get("normed", (M, self.H), dt)
        self.blocks[0].norm1.forward(ctx, delta, resid, xn)
        layers = self._layer_table(caches)
        qd = self.n_q * self.d
        q = ws.get("q_rot", (M, qd), dt)
        attn = ws.get("attn", (M, qd), dt)
        o_parts = ws.get("stack_o_parts", (self.o_splits, M, self.H), torch.float32)
        act = ws.get("ffn_act", (M, self.I), dt)
        down_parts = ws.get("stack_down_parts", (self.down_splits, M, self.H), torch.float32)
        n_splits, split_len = plan_splits(ctx.n_rows, self.n_kv, ctx.kv_len_bound, rt.sm_count)
        scratch = counters = None
        if n_splits > 1:
            scratch = ws.get("attn_scratch", (K.attention_scratch_floats(M, self.n_q, self.d, n_splits),), torch.float32)
            counters = K._counters(rt.device, M * self.n_kv)
        rope = self.position
        pointers = [layers, ctx.tok_row, ctx.tok_pos, ctx.row_slot, ctx.row_q_start, ctx.row_q_len, ctx.row_ctx_len,
                    rope.cos, rope.sin, resid, xn, q, attn, o_parts, act, down_parts, scratch, counters, self.barrier,
                    rt.status]
        ints = [len(self.blocks), M, self.H, self.I, self.n_q, self.n_kv, self.d, rope.cos.shape[0], n_splits, split_len,
                self.qkv_wk, self.o_wk, self.o_splits, self.gu_wk, self.down_wk, self.down_splits, self.bias_f32,
                self.norm_w_f32]
        K.decode_stack(pointers, ints, self.scale, self.ctas, self.skip)
        return down_parts

    def reset(self) -> None:
        """After a launch that gave up: its barrier words are meaningless."""
        self.barrier.zero_()


def find_stacks(model) -> Dict[int, DecodeStack]:
    """Maximal runs of schedule entries with the same signature, keyed by their first entry."""
    sigs = [_signature(model.blocks[run.layer]) for run in model.schedule]
    out: Dict[int, DecodeStack] = {}
    i, n = 0, len(sigs)
    while i < n:
        j = i
        while sigs[i] is not None and j + 1 < n and sigs[j + 1] == sigs[i]:
            j += 1
        if sigs[i] is not None and j >= i:
            out[i] = DecodeStack(model, i, j)
        i = j + 1
    return out
