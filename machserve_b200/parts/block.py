"""Arrangements of a layer's parts around the residual stream."""
from __future__ import annotations

from .base import Block, as_delta, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    """x += mixer(norm(x)); x += feed_forward(norm(x))
    (crates/mach-model/src/batched.rs:3200, :4031, :4050, :4453 of gqf2008/machserve).

    The adds are done by the norm that follows them, in float32: the block hands the
    last delta on as `pending`, and the next norm (the next layer's, or the model's
    final one) adds it.

    A part that said at bind time that it can take its norm into its own kernels
    (`Part.fuse_norm`) is run through `forward_fused` for steps of up to its
    `fused_rows` rows: it reads the residual's rounded copy and row statistics that the
    part before it left (`RowStats`), adds its own delta into the residual and leaves the
    same for the part after it, so that neither the norm nor the add needs a kernel of
    its own.  Each half of the block decides for itself; a part without the protocol is
    given normed rows and returns a delta, as ever.
    """

    graph_safe = True
    accepts_row_stats = True

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.fuse_mixer = bool(self.mixer.fuse_norm(self.mixer_norm))
        self.fuse_feed_forward = bool(self.feed_forward.fuse_norm(self.ff_norm))

    def forward(self, ctx, residual, pending, cache, owns_cache=True):
        rt = ctx.rt
        t, d = residual.shape
        if self.fuse_mixer and t <= self.mixer.fused_rows:
            pending = self.mixer.forward_fused(ctx, residual, pending, self.mixer_norm, cache, owns_cache)
        else:
            xn = rt.workspace.get("block.normed", (t, d), rt.dtype)
            self.mixer_norm.forward(residual, as_delta(pending), xn)
            pending = self.mixer.forward(ctx, xn, cache, owns_cache)
        if self.fuse_feed_forward and t <= self.feed_forward.fused_rows:
            return self.feed_forward.forward_fused(ctx, residual, pending, self.ff_norm)
        xn = rt.workspace.get("block.normed", (t, d), rt.dtype)
        self.ff_norm.forward(residual, as_delta(pending), xn)
        return self.feed_forward.forward(ctx, xn)
