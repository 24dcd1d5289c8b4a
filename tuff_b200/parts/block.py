"""Arrangements of a layer's parts.  `prenorm`: x += mixer(norm_a(x)), then
x += ffn(norm_b(x)), the residual stream staying in fp32 throughout
(reference: src/lfm25_engine.c:365-423)."""
from __future__ import annotations

from .base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    def forward(self, ctx, x, layer, cache, reads_only=False, next_norm=None):
        # a part that says `takes_lazy_norm` may get its input as a norm still to run (ops.NormedRows);
        # each norm is told of x before the part that writes x ahead of it runs
        h = layer.mixer_norm.forward(ctx, x, lazy=getattr(layer.mixer, "takes_lazy_norm", False))
        layer.ffn_norm.announce(ctx, x)
        layer.mixer.forward(ctx, cache, h, x, reads_only)
        h = layer.ffn_norm.forward(ctx, x, lazy=getattr(layer.ffn, "takes_lazy_norm", False))
        if next_norm is not None:
            next_norm.announce(ctx, x)
        layer.ffn.forward(ctx, h, x)
