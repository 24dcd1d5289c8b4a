"""LFM2 / LFM2.5 dense (`Lfm2ForCausalLM`) as a `ModelSpec`.

Layer i is pre-norm with `operator_norm` before the mixer and `ffn_norm` before
a SwiGLU feed-forward; the mixer is a gated short convolution or grouped-query
attention with per-head q/k RMSNorm and NeoX rotation, as the configuration's
layer kinds say (reference: layer loop src/lfm25_engine.c:365-423; kinds
src/lfm25_model.h:13-16; tensor names src/lfm25_model.c:120-216 in their GGUF
spelling — the names below are the checkpoint's own).  The final norm is
`model.embedding_norm`; the head is `lm_head.weight` or, tied, the embedding
(src/lfm25_model.c:123-131).
"""
from __future__ import annotations

from ..config.lfm2 import ARCHITECTURE, Lfm2Config
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec


def lfm2_spec(cfg: Lfm2Config) -> ModelSpec:
    d, eps = cfg.hidden_size, cfg.norm_eps
    layers = []
    for i, kind in enumerate(cfg.layer_types):
        p = f"model.layers.{i}."
        if kind == "attention":
            mixer = PartSpec(
                "gqa_attention",
                dict(d_model=d, num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
                     head_dim=cfg.head_dim, qk_norm_eps=eps,
                     position_encoding=PartSpec("rope_neox", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta))),
                {n: f"{p}self_attn.{n}.weight" for n in
                 ("q_proj", "k_proj", "v_proj", "out_proj", "q_layernorm", "k_layernorm")})
        else:
            mixer = PartSpec(
                "gated_short_conv", dict(d_model=d, kernel_size=cfg.conv_L_cache),
                {"in_proj": f"{p}conv.in_proj.weight", "conv": f"{p}conv.conv.weight",
                 "out_proj": f"{p}conv.out_proj.weight"})
        ffn = PartSpec("swiglu", dict(d_model=d, ffn_dim=cfg.ffn_dim),
                       {n: f"{p}feed_forward.{n}.weight" for n in ("w1", "w2", "w3")})
        layers.append(LayerSpec(
            mixer=mixer, ffn=ffn,
            mixer_norm=PartSpec("rmsnorm", dict(dim=d, eps=eps), {"weight": f"{p}operator_norm.weight"}),
            ffn_norm=PartSpec("rmsnorm", dict(dim=d, eps=eps), {"weight": f"{p}ffn_norm.weight"})))
    embed_name = "model.embed_tokens.weight"
    return ModelSpec(
        architecture=ARCHITECTURE, d_model=d, vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, d_model=d), {"weight": embed_name}),
        layers=layers,
        final_norm=PartSpec("rmsnorm", dict(dim=d, eps=eps), {"weight": "model.embedding_norm.weight"}),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, d_model=d),
                      {"weight": embed_name if cfg.tie_embedding else "lm_head.weight"}),
        max_context=cfg.max_position_embeddings)
