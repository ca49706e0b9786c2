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
    be added by whoever norms next.  A layer without a feed-forward
    (``feed_forward`` None) is x += mixer(norm1(x)) alone; a ``norm2`` it is
    given all the same declares its tensor and never runs.  ``side``: a
    ``side_input`` part that runs last; it completes the stream with the
    pending output and returns its own, x += side(x, tokens).  Norms that add
    their delta times a constant (``delta_scale``) make every one of these sums
    x += c * (...).
    """

    def __init__(self, norm1, mixer, norm2=None, feed_forward=None, side=None):
        self.norm1, self.mixer, self.norm2, self.feed_forward, self.side = norm1, mixer, norm2, feed_forward, side
        if feed_forward is not None and norm2 is None:
            raise ValueError("a pre-norm layer with a feed-forward needs its second norm")

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward, self.side) if p is not None]

    def stream_state(self, resid: torch.Tensor, delta) -> torch.Tensor:
        scale = float(getattr(self.norm1, "delta_scale", 1.0))
        if delta is None or scale == 1.0:
            return super().stream_state(resid, delta)
        return resid + scale * (delta.float().sum(0) if delta.dim() == 3 else delta.float())

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
        if self.feed_forward is None:
            d = self.mixer.forward(ctx, xn, lc)
            return d if self.side is None else self.side.forward(ctx, resid, d)
        ctx.upcoming = self.feed_forward.first_weights()
        d1 = self.mixer.forward(ctx, xn, lc)
        self.norm2.forward(ctx, d1, resid, xn)
        ctx.upcoming = after_block
        if self.side is not None:
            return self.side.forward(ctx, resid, self.feed_forward.forward(ctx, xn))
        # float partial sums only if whoever adds this block's output has said it takes them
        if ctx.delta_parts_ok and getattr(self.feed_forward, "offers_parts", False):
            return self.feed_forward.forward(ctx, xn, parts_ok=True)
        return self.feed_forward.forward(ctx, xn)
