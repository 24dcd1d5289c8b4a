"""SwiGLU feed-forward: act = silu(h W1^T) * (h W3^T), out = act W2^T, added to
the residual (reference: src/lfm25_gpu.cu:583-618, down projection with
accumulation src/lfm25_engine.c:416-419).  W1 (gate) and W3 (up) are stacked
into one [2F, d] matrix when bound (in blocks of 128 rows of each when the
width allows, so that one tile of the product holds matching gate and up
columns), so one product yields both and the activation runs in its epilogue."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, WeightDecl, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    takes_lazy_norm = True

    def __init__(self, d_model: int, ffn_dim: int):
        self.d, self.F = int(d_model), int(ffn_dim)

    def weight_decls(self):
        return {"w1": WeightDecl((self.F, self.d)), "w3": WeightDecl((self.F, self.d)),
                "w2": WeightDecl((self.d, self.F))}

    def bind(self, weights, act_dtype):
        super().bind(weights, act_dtype)
        self.w13, self.w13_block = ops.stack_gate_up(weights["w1"], weights["w3"])
        self.w2 = weights["w2"]
        self.w = {"w2": self.w2}            # the stacked copy replaces w1 and w3

    def forward(self, ctx, h, residual):
        T = h.shape[0]
        act = torch.empty((T, self.F), dtype=self.act_dtype, device=h.device)
        ops.linear_swiglu(h, self.w13, act, self.w13_block)
        ops.linear(act, self.w2, residual, accumulate=True)
