"""Arrangements of a layer.

Pre-norm: ``x += mixer(norm1(x)); x += ff(norm2(x))`` (src/arch/transformer_block.cpp:199-296).
Parallel: ``h = norm1(x); x += mixer(h) + ff(h)``, one norm whose output both sublayers read; a layer
without a feed-forward adds the mixer's output alone.

Output norm: ``x += norm1(mixer(x)); x += norm2(ff(x))``: the sublayers read the stream itself and the norms sit on
their outputs.

Each residual sum is handed to the norm that follows it, which does both in one pass over the row, in
32-bit; a parallel block hands on its two outputs as a pair, and that norm forms their sum first."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .base import (Block, ChannelScalePart, FeedForward, LayerCache, Mixer, Norm, Normed, Part, Scaled, StepContext,
                   delta_pair)
from .registry import register_block


class PreNormBlock(Block):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm] = None, feed_forward: Optional[FeedForward] = None,
                 scale1: Optional[ChannelScalePart] = None, scale2: Optional[ChannelScalePart] = None):
        if (norm2 is None) != (feed_forward is None):
            raise ValueError("a pre-norm block has a second norm exactly when it has a feed-forward")
        if scale2 is not None and feed_forward is None:
            raise ValueError("a block without a feed-forward has no second channel scale")
        self.norm1, self._mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        self.scale1, self.scale2 = scale1, scale2       # learned vectors on the two sublayers' outputs (layer scale)

    def parts(self) -> Dict[str, Part]:
        p = {"norm1": self.norm1, "mixer": self._mixer}
        if self.feed_forward is not None:
            p.update(norm2=self.norm2, feed_forward=self.feed_forward)
        if self.scale1 is not None:
            p["scale1"] = self.scale1
        if self.scale2 is not None:
            p["scale2"] = self.scale2
        return p

    def mixer(self) -> Mixer:
        return self._mixer

    def forward(self, residual: torch.Tensor, delta, ctx: StepContext, cache: LayerCache):
        if isinstance(delta, (tuple, list, Scaled, Normed)):
            # the block before was a parallel one, or its output waits with a channel scale: the fused first kernels
            # take one plain pending tensor
            h = self.norm1.add_forward(delta, residual, ctx.dtype)
            a = self._mixer.forward(h, ctx, cache)
        # a part may take the residual sum and the norm into its first kernel (decode steps)
        elif self._mixer.fuses_norm(self.norm1, residual, ctx, cache):
            a, residual = self._mixer.forward_with_norm(residual, delta, self.norm1, ctx, cache)
        else:
            h = self.norm1.add_forward(delta, residual, ctx.dtype)
            a = self._mixer.forward(h, ctx, cache)
        if self.scale1 is not None:
            a = self.scale1.apply(a)
        if self.feed_forward is None:
            return residual, a                      # a layer without a feed-forward: the mixer's output stays pending
        if not isinstance(a, Scaled) and self.feed_forward.fuses_norm(self.norm2, residual, ctx):
            d, residual = self.feed_forward.forward_with_norm(residual, a, self.norm2, ctx)
        else:
            h2 = self.norm2.add_forward(a, residual, ctx.dtype)
            d = self.feed_forward.forward(h2, ctx)
        return residual, self.scale2.apply(d) if self.scale2 is not None else d


class ParallelBlock(Block):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm] = None, feed_forward: Optional[FeedForward] = None):
        if norm2 is not None:
            raise ValueError("a parallel block has one norm")
        self.norm1, self._mixer, self.feed_forward = norm1, mixer, feed_forward

    def parts(self) -> Dict[str, Part]:
        p = {"norm1": self.norm1, "mixer": self._mixer}
        if self.feed_forward is not None:
            p["feed_forward"] = self.feed_forward
        return p

    def mixer(self) -> Mixer:
        return self._mixer

    def forward(self, residual: torch.Tensor, delta, ctx: StepContext, cache: LayerCache):
        h = self.norm1.add_forward(delta, residual, ctx.dtype)
        a = self._mixer.forward(h, ctx, cache)
        if self.feed_forward is None:
            return residual, a
        return residual, (a, self.feed_forward.forward(h, ctx))


class OutputNormBlock(Block):
    """Norms on the sublayers' outputs: ``x <- x + norm1(mixer(x)); x <- x + norm2(ff(x))``.  The sublayers read the
    stream itself (rounded to the run type).  Norm, sum and the rounded copy of the new stream for the next sublayer are
    one kernel (``Norm.add_normed``); the last output of the block stays pending with its norm (``Normed``), so that the
    next block's first kernel, or the model's final norm, takes it."""

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm] = None, feed_forward: Optional[FeedForward] = None):
        if (norm2 is None) != (feed_forward is None):
            raise ValueError("a block has a second norm exactly when it has a feed-forward")
        self.norm1, self._mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self) -> Dict[str, Part]:
        p = {"norm1": self.norm1, "mixer": self._mixer}
        if self.feed_forward is not None:
            p.update(norm2=self.norm2, feed_forward=self.feed_forward)
        return p

    def mixer(self) -> Mixer:
        return self._mixer

    def _enter(self, residual: torch.Tensor, delta, ctx: StepContext) -> torch.Tensor:
        """Adds what is pending and returns the stream's rows in the run type."""
        if isinstance(delta, Normed):
            return delta.norm.add_normed(delta.tensor, residual, ctx.dtype, bias=delta.bias)
        d1, d2 = delta_pair(delta)
        if d1 is not None:
            residual.add_(d1.to(residual.dtype) + d2.to(residual.dtype) if d2 is not None else d1.to(residual.dtype))
        return self.norm1.add_normed(None, residual, ctx.dtype)

    def forward(self, residual: torch.Tensor, delta, ctx: StepContext, cache: LayerCache):
        h = self._enter(residual, delta, ctx)
        a, bias = self._mixer.forward_deferred_bias(h, ctx, cache)      # the output product's bias rides in the norm kernel
        if self.feed_forward is None:
            return residual, Normed(a, self.norm1, bias)
        h2 = self.norm1.add_normed(a, residual, ctx.dtype, bias=bias)
        return residual, Normed(self.feed_forward.forward(h2, ctx), self.norm2)


register_block("pre_norm", PreNormBlock)
register_block("parallel", ParallelBlock)
register_block("output_norm", OutputNormBlock)
