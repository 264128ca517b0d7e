"""Arrangements of a layer's parts.

"prenorm_residual": h = h + mixer(norm(h)); h = h + feed_forward(norm(h)), the
order of the reference's attention-plus-dense layer
(crates/braidinfer-runtime/src/megakernel/megakernel_compile.rs:115-236).  The
residual stream h is float32; mixers and feed-forwards add into it.  A layer that has an input of its
own about each token (`LayerSpec.layer_input`) applies it last: h = layer_input(h).

"sublayer_norm_residual": h = h + norm(mixer(h)); h = h + norm(feed_forward(h)): the sublayers read the stream
itself (cast to the run's type) and the norm is applied to what they return, before the residual sum.  The norm
and the sum are one float32 kernel (`Norm.add_into`).
"""
from __future__ import annotations

import torch

from .base import BLOCKS, Block


@BLOCKS.register("prenorm_residual")
class PreNormResidualBlock(Block):
    def forward(self, h, ctx, cache, state):
        # h may still wait for a deferred sum (see StepContext.deferred); a norm that
        # accepts that adds it up in its own kernel, any other part gets h completed first
        x = self._norm(self.mixer_norm, h, ctx, self.mixer)
        h = self.mixer.forward(x, h, ctx, cache, state)
        if self.feed_forward is not None:
            x = self._norm(self.feed_forward_norm, h, ctx, self.feed_forward)
            h = self.feed_forward.forward(x, h, ctx)
        if ctx.row_scales:
            raise RuntimeError("a part left a row scale unapplied (see StepContext.row_scales)")
        if self.layer_input is not None:
            h = self.layer_input.forward(ctx.resolve(h), ctx)
        return h

    @staticmethod
    def _norm(norm, h, ctx, reader):
        if not norm.accepts_deferred:
            return norm.forward(ctx.resolve(h), ctx)
        # a norm that knows deferred sums may also leave its scale to a reader that takes row scales
        return norm.forward(h, ctx, reader_takes_row_scale=bool(reader.takes_row_scale()))


@BLOCKS.register("sublayer_norm_residual")
class SublayerNormResidualBlock(Block):
    """The norms need `add_into` (see parts/norm.py).  A sublayer with `plain_output` returns its result alone;
    any other is handed a stream of zeros to add into, which gives the same."""

    def forward(self, h, ctx, cache, state):
        h = ctx.resolve(h)
        y = self._branch(self.mixer, h, ctx, lambda x, r: self.mixer.forward(x, r, ctx, cache, state))
        h = self.mixer_norm.add_into(y, h, ctx)
        if self.feed_forward is not None:
            y = self._branch(self.feed_forward, h, ctx, lambda x, r: self.feed_forward.forward(x, r, ctx))
            h = self.feed_forward_norm.add_into(y, h, ctx)
        if self.layer_input is not None:
            h = self.layer_input.forward(h, ctx)
        return h

    def _branch(self, part, h, ctx, call):
        rt = part.rt
        if rt.is_f32:
            x = h                                        # the sublayers only read their input
        else:
            x = rt.empty(*h.shape)
            rt.kernels.cast(h, x)
        y = call(x, None if part.plain_output else torch.zeros_like(h))
        return ctx.resolve(y)
