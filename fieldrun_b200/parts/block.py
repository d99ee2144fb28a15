"""The arrangement of a layer: norm -> mixer -> residual, norm -> feed-forward -> residual
(the reference's two-norm pre-norm block, src/minimax.rs:261-284).  Each residual sum is
left to the norm that follows it, which adds in float32 while it reads the stream."""
from __future__ import annotations

from .base import Block, as_tensor, register_part


class PreNormBlock(Block):
    def forward(self, ctx, x, pending, line, writes_cache):
        if not self.mixer_norm.accepts_deferred:
            pending = as_tensor(ctx, pending)
        act, _ = self.mixer_norm.forward(ctx, x, delta=pending)
        update = self.mixer.forward(ctx, act, line, writes_cache)
        if not self.feed_forward_norm.accepts_deferred:
            update = as_tensor(ctx, update)
        act2, act2_32 = self.feed_forward_norm.forward(ctx, x, delta=update,
                                                       want32=self.feed_forward.wants_float32_input)
        return x, self.feed_forward.forward_deferred(ctx, act2, act2_32)


register_part("block", "pre_norm", PreNormBlock, replace=True)
