"""Grouped-query attention mixer over the paged cache (reference: projections
src/lfm25_engine.c:386-390; per-head RMSNorm of q and k, NeoX rotation and the
cache write src/lfm25_gpu.cu:420-501; scores, causal bound and online softmax
src/lfm25_gpu.cu:506-558, scale 1/sqrt(hd) at :520, head-to-group map at :518;
output projection with accumulation src/lfm25_engine.c:405).

q, k and v projections are stacked into one [(H+2G)*hd, d] matrix when bound.
Optional, all parameters: the q/k norm (`qk_norm_eps=None` switches it off), the
position encoding (a PartSpec or None), a window of keys, the score scale.
A layer that runs on another layer's cache (`reads_only`) projects q alone.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import POSITION_ENCODINGS, Mixer, PagedKVNeed, PartSpec, WeightDecl, register_mixer


@register_mixer("gqa_attention")
class GQAAttention(Mixer):
    takes_lazy_norm = True

    def __init__(self, d_model: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qk_norm_eps: float | None = None, position_encoding: PartSpec | dict | None = None,
                 window: int | None = None, scale: float | None = None):
        self.d, self.H, self.G, self.hd = int(d_model), int(num_heads), int(num_kv_heads), int(head_dim)
        if self.H % self.G:
            raise ValueError(f"num_heads {self.H} is not a multiple of num_kv_heads {self.G}")
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.window = None if not window else int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        if isinstance(position_encoding, dict):
            position_encoding = PartSpec(**position_encoding)
        self.pos = POSITION_ENCODINGS.build(position_encoding) if position_encoding is not None else None

    def weight_decls(self):
        H, G, hd, d = self.H, self.G, self.hd, self.d
        decls = {"q_proj": WeightDecl((H * hd, d)), "k_proj": WeightDecl((G * hd, d)),
                 "v_proj": WeightDecl((G * hd, d)), "out_proj": WeightDecl((d, H * hd))}
        if self.qk_norm_eps is not None:
            decls["q_layernorm"] = WeightDecl((hd,), role="vector", init="norm")
            decls["k_layernorm"] = WeightDecl((hd,), role="vector", init="norm")
        return decls

    def reserve(self, device, max_rows, max_context):
        if self.act_dtype == torch.bfloat16:
            ops.reserve_attention_workspace(device, max_rows, max_context, self.H, self.G, self.hd)

    def cache_need(self):
        return PagedKVNeed(kv_heads=self.G, head_dim=self.hd, window=self.window)

    def bind(self, weights, act_dtype):
        super().bind(weights, act_dtype)
        self.wqkv = torch.cat([weights["q_proj"], weights["k_proj"], weights["v_proj"]], dim=0).contiguous()
        self.wq = self.wqkv[: self.H * self.hd]
        self.wo = weights["out_proj"]
        self.qn = weights.get("q_layernorm")
        self.kn = weights.get("k_layernorm")
        self.w = {"out_proj": self.wo}

    def forward(self, ctx, cache, h, residual, reads_only=False):
        T = h.shape[0]
        H, G, hd = self.H, self.G, self.hd
        g_here = 0 if reads_only else G
        qkv = torch.empty((T, (H + 2 * g_here) * hd), dtype=self.act_dtype, device=h.device)
        ops.linear(h, self.wq if reads_only else self.wqkv, qkv)
        table = ctx.block_tables[cache.group]
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        fused = self.pos.fused_tables(qkv.device) if (self.pos is not None and hasattr(self.pos, "fused_tables")) else None
        if self.pos is None or fused is not None:
            inv_freq, rot = fused if fused is not None else (None, 0)
            ops.qk_norm_rope_write(qkv, self.qn, self.kn, inv_freq, ctx.positions, ctx.row_of_token, table,
                                   cache.k_pages, cache.v_pages, H, g_here, hd, rot, eps,
                                   write_kv=not reads_only)
        else:
            # norm, then the position encoding's own rotation, then the cache write
            ops.qk_norm_rope_write(qkv, self.qn, self.kn, None, ctx.positions, ctx.row_of_token, None, None, None,
                                   H, g_here, hd, 0, eps, write_kv=False)
            q3 = qkv[:, : H * hd].unflatten(1, (H, hd))
            k3 = None if reads_only else qkv[:, H * hd:(H + G) * hd].unflatten(1, (G, hd))
            self.pos.rotate(ctx, q3, k3)
            if not reads_only:
                ops.qk_norm_rope_write(qkv, None, None, None, ctx.positions, ctx.row_of_token, table,
                                       cache.k_pages, cache.v_pages, H, G, hd, 0, 0.0, write_kv=True)
        att = torch.empty((T, H * hd), dtype=self.act_dtype, device=qkv.device)
        ops.paged_attention(qkv, cache.k_pages, cache.v_pages, table, ctx.positions, ctx.row_of_token, att,
                            H, G, hd, self.scale, self.window or 0, ctx=ctx)
        ops.linear(att, self.wo, residual, accumulate=True)
