"""Gated short convolution mixer (reference: src/lfm25_gpu.cu:344-415 fused with
the input projection, :287-337 and :1046-1099 stand-alone; output projection
with accumulation src/lfm25_engine.c:380):

    [B | C | x] = h W_in^T          three d-wide thirds, in this order
    u = B * x
    y_t = sum_j taps[:, j] * u_{t-(K-1)+j}     causal, depthwise, K taps
    out = (C * y) W_out^T, added to the residual

Its cache need is a fixed-size state per request: the last K-1 values of u.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, StateNeed, WeightDecl, register_mixer


@register_mixer("gated_short_conv")
class GatedShortConv(Mixer):
    takes_lazy_norm = True

    def __init__(self, d_model: int, kernel_size: int):
        self.d, self.K = int(d_model), int(kernel_size)
        if self.K < 2:
            raise ValueError("gated_short_conv needs kernel_size >= 2")

    def weight_decls(self):
        return {"in_proj": WeightDecl((3 * self.d, self.d)),
                "conv": WeightDecl((self.d, 1, self.K), role="vector"),
                "out_proj": WeightDecl((self.d, self.d))}

    def cache_need(self):
        return StateNeed(shape=(self.K - 1, self.d), dtype="float32")

    def bind(self, weights, act_dtype):
        super().bind(weights, act_dtype)
        self.taps = weights["conv"].reshape(self.d, self.K).contiguous()

    def forward(self, ctx, cache, h, residual, reads_only=False):
        if reads_only:
            raise ValueError("a gated_short_conv layer cannot run on another layer's state")
        T = h.shape[0]
        g = torch.empty((T, self.d), dtype=self.act_dtype, device=h.device)
        if ctx.all_single and ops.linear_shortconv(h, self.w["in_proj"], self.taps, cache.state, ctx.slot_of_row, g):
            ops.linear(g, self.w["out_proj"], residual, accumulate=True)
            return
        bcx = torch.empty((T, 3 * self.d), dtype=self.act_dtype, device=h.device)
        ops.linear(h, self.w["in_proj"], bcx)
        ops.shortconv(bcx, self.taps, cache.state, ctx.slot_of_row, ctx.row_of_token, ctx.cu_q, g,
                      all_single=ctx.all_single)
        ops.linear(g, self.w["out_proj"], residual, accumulate=True)
