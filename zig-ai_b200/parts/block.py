"""Arrangement of a layer's parts: pre-norm residual block.

    r  = norm_a(h);  h = h + mixer(r);  r2 = norm_b(h);  h = h + feed_forward(r2)

(src/transformer/hybrid_layer.zig:364-365, 370-377, 409-422, 488-491; LFM2 uses `ffn_norm` as the
second norm, :302-305).  Both kinds of LFM2 layer use it; the reference's device path leaves out
the residual on ShortConv layers (:627), which is not followed.  Each addition is carried as a
pending term into the next norm's kernel, which adds it into the 32-bit residual stream.
"""
from __future__ import annotations

from .base import Block, register_part


class PreNormResidual(Block):
    graph_safe = True      # forward launches kernels only; nothing is read back to the host

    def __init__(self, mixer, feed_forward, mixer_norm, ff_norm):
        super().__init__()
        self.mixer_norm = self.sub("mixer_norm", "norm", mixer_norm)
        self.mixer = self.sub("mixer", "mixer", mixer)
        self.ff_norm = self.sub("ff_norm", "norm", ff_norm)
        self.feed_forward = self.sub("feed_forward", "feed_forward", feed_forward)

    def params(self):
        return {}

    def forward(self, h, pending, step, cache, write_cache=True):
        r = self.mixer_norm.forward(h, pending, step, lazy=self.mixer.accepts_lazy_input)
        m = self.mixer.forward(r, step, self.cache_for(self.mixer, cache), write_cache)
        r2 = self.ff_norm.forward(h, m, step, lazy=self.feed_forward.accepts_lazy_input)
        f = self.feed_forward.forward(r2, step)
        return h, f


register_part("block", "prenorm_residual", PreNormResidual)
