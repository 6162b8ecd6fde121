"""Arrangements of two norms, a mixer and a feed-forward in one layer."""

from __future__ import annotations

from typing import Optional

import torch

from ..registry import register_part
from .base import Block, LayerCache


@register_part("block", "prenorm")
class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += feed_forward(norm2(x)).

    Carried across sub-layers as (resid, delta): each norm first adds the
    previous sub-layer's output to the residual stream, so add and norm are one
    kernel (the threading of engine/model.py:173-184,210-212 in
    davidjoyme/flashdecode-cuda).  Returns the feed-forward's output, still to
    be added by whoever norms next.
    """

    def __init__(self, norm1, mixer, norm2, feed_forward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.feed_forward]

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.mixer.first_weights()

    @property
    def accepts_parts(self) -> bool:
        """The incoming delta goes straight to norm1."""
        return bool(getattr(self.norm1, "accepts_parts", False))

    def forward(self, ctx, resid: torch.Tensor, delta: Optional[torch.Tensor], lc: LayerCache) -> torch.Tensor:
        xn = ctx.ws.get("normed", tuple(resid.shape), ctx.rt.dtype)
        after_block = ctx.upcoming                       # what the step streams after this block (set by the model)
        self.norm1.forward(ctx, delta, resid, xn)
        ctx.upcoming = self.feed_forward.first_weights()
        d1 = self.mixer.forward(ctx, xn, lc)
        self.norm2.forward(ctx, d1, resid, xn)
        ctx.upcoming = after_block
        # float partial sums only if whoever adds this block's output has said it takes them
        if ctx.delta_parts_ok and getattr(self.feed_forward, "offers_parts", False):
            return self.feed_forward.forward(ctx, xn, parts_ok=True)
        return self.feed_forward.forward(ctx, xn)
