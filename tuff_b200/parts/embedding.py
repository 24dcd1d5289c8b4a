"""Token embedding (a row gather into the fp32 residual stream; no scale and no
positional term: src/lfm25_engine.c:360, src/lfm25_gpu.cu:725-741) and the
output head (final norm of the wanted rows, then the product with the output
matrix, which may be the embedding itself: src/lfm25_gpu.cu:1216-1237,
src/lfm25_model.c:128-131)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Embedding, Head, WeightDecl, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, vocab_size: int, d_model: int):
        self.V, self.d = int(vocab_size), int(d_model)

    def weight_decls(self):
        return {"weight": WeightDecl((self.V, self.d))}

    def forward(self, ctx):
        x = torch.empty((ctx.n_tokens, self.d), dtype=torch.float32, device=ctx.device)
        ops.embed(ctx.tokens, self.w["weight"], x)
        return x


@register_head("lm_head")
class LMHead(Head):
    def __init__(self, vocab_size: int, d_model: int):
        self.V, self.d = int(vocab_size), int(d_model)

    def weight_decls(self):
        return {"weight": WeightDecl((self.V, self.d))}

    def forward(self, ctx, x, norm):
        """Logits (fp32) of the rows that `ctx.want_index` names."""
        n = ctx.n_wanted
        logits = torch.empty((n, self.V), dtype=torch.float32, device=x.device)
        if n == 0:
            return logits
        # every row wanted, in order (a decode step): the product may norm the rows itself
        h = norm.forward(ctx, x, None if ctx.wants_all_rows else ctx.want_index, lazy=ctx.wants_all_rows)
        ops.linear(h, self.w["weight"], logits)
        return logits
