"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, statistics in fp32; the weight
multiplies directly, with no "+1" (reference: src/lfm25_gpu.cu:207-262, weight
use at :244; eps from the model file, src/lfm25_model.c:92-93)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm, WeightDecl, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, dim: int, eps: float):
        self.dim, self.eps = int(dim), float(eps)

    def weight_decls(self):
        return {"weight": WeightDecl((self.dim,), role="vector", init="norm")}

    def announce(self, ctx, x):
        # few rows in bf16: the product that adds into x last can prepare this norm
        if x.shape[0] <= ops.CLUSTER_MAX_TOKENS and self.act_dtype == torch.bfloat16:
            ops.announce_norm(x, self.w["weight"], self.eps)

    def forward(self, ctx, x, row_index=None, lazy=False):
        """`lazy`: the caller's next step is a matrix product that can norm its own rows; it gets
        an `ops.NormedRows` (which any other consumer turns into the tensor with `.dense()`)."""
        if lazy and row_index is None and x.shape[0] <= ops.CLUSTER_MAX_TOKENS and self.act_dtype == torch.bfloat16:
            return ops.NormedRows(x, self.w["weight"], self.eps, self.act_dtype)
        n = x.shape[0] if row_index is None else row_index.numel()
        out = torch.empty((n, self.dim), dtype=self.act_dtype, device=x.device)
        ops.rmsnorm(x, self.w["weight"], self.eps, out, row_index)
        return out
