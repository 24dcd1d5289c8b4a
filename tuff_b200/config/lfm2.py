"""`Lfm2Config`: the hyper-parameters of an LFM2 / LFM2.5 dense decoder.

The reference reads the same quantities from GGUF metadata
(src/lfm25_model.c:75-103: block_count, embedding_length, attention.head_count,
attention.layer_norm_rms_epsilon, shortconv.l_cache, feed_forward_length,
rope.freq_base) and checks them in lfm25_model_validate (src/lfm25_model.c:319-379).
Here they come from config.json; every size is a field, nothing is fixed in code
(the reference accepts only head size 64 and a 3-tap convolution:
src/lfm25_model.c:325,331).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, asdict
from typing import Tuple

from .base import ConfigError, KeyReader

ARCHITECTURE = "Lfm2ForCausalLM"

_KIND_ALIASES = {
    "conv": "conv",
    "short_conv": "conv",
    "full_attention": "attention",
    "attention": "attention",
}


def adjusted_ffn_dim(intermediate_size: int, auto_adjust: bool, multiplier: float | None,
                     multiple_of: int) -> int:
    """Width of the SwiGLU feed-forward from the config's intermediate size.

    With `block_auto_adjust_ff_dim` the width is two thirds of the given size,
    times `ffn_dim_multiplier` if that is set, rounded up to a multiple of
    `block_multiple_of` (8192 -> 5632, 6656 -> 4608, 10752 -> 7168 at 256).
    """
    f = int(intermediate_size)
    if auto_adjust:
        f = int(2 * f / 3)
        if multiplier is not None:
            f = int(multiplier * f)
        f = multiple_of * ((f + multiple_of - 1) // multiple_of)
    return f


@dataclass(frozen=True)
class Lfm2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    block_auto_adjust_ff_dim: bool
    ffn_dim_multiplier: float | None
    block_multiple_of: int
    rope_theta: float
    norm_eps: float
    conv_L_cache: int
    layer_types: Tuple[str, ...]          # "conv" or "attention" for each layer
    tie_embedding: bool
    max_position_embeddings: int
    bos_token_id: int | None = None
    eos_token_id: int | None = None
    pad_token_id: int | None = None
    architectures: Tuple[str, ...] = (ARCHITECTURE,)
    ignored_keys: Tuple[str, ...] = field(default=(), compare=False)

    # ---- derived ---------------------------------------------------------
    @property
    def ffn_dim(self) -> int:
        return adjusted_ffn_dim(self.intermediate_size, self.block_auto_adjust_ff_dim,
                                self.ffn_dim_multiplier, self.block_multiple_of)

    @property
    def full_attn_idxs(self) -> Tuple[int, ...]:
        return tuple(i for i, t in enumerate(self.layer_types) if t == "attention")

    @property
    def conv_idxs(self) -> Tuple[int, ...]:
        return tuple(i for i, t in enumerate(self.layer_types) if t == "conv")

    @property
    def conv_state_len(self) -> int:
        return self.conv_L_cache - 1

    # ---- reading ---------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "Lfm2Config":
        r = KeyReader(raw, where)
        archs = r.string_list("architectures", default=[ARCHITECTURE])
        r.used.update(("model_type", "torch_dtype", "dtype", "transformers_version", "use_cache"))
        d = r.integer("hidden_size", min_value=1)
        L = r.integer("num_hidden_layers", min_value=1)
        H = r.integer("num_attention_heads", "num_heads", min_value=1)
        G = r.integer("num_key_value_heads", default=H, min_value=1)
        hd = r.optional_integer("head_dim", min_value=1)
        if hd is None:
            if d % H != 0:
                raise ConfigError(f"{where}: hidden_size {d} is not divisible by num_attention_heads {H} "
                                  f"and no head_dim is given")
            hd = d // H
        V = r.integer("vocab_size", min_value=1)
        inter = r.integer("intermediate_size", "block_ff_dim", min_value=1)
        if r.has("intermediate_size") and r.has("block_ff_dim") and r.integer("block_ff_dim") != inter:
            # two names of one size; which of them would win is not for this reader to guess
            raise ConfigError(f"{where}: intermediate_size {inter} and block_ff_dim {r.integer('block_ff_dim')} "
                              f"name the same feed-forward width and disagree; keep one of them")
        auto = r.boolean("block_auto_adjust_ff_dim", default=False)
        mult = r.optional_number("ffn_dim_multiplier", "block_ffn_dim_multiplier")
        mof = r.integer("block_multiple_of", default=256, min_value=1)
        theta = r.number("rope_theta", positive=True)
        eps = r.number("norm_eps", "block_norm_eps", positive=True)
        K = r.integer("conv_L_cache", min_value=2)
        if r.has("conv_bias") and r.boolean("conv_bias"):
            raise ConfigError(f"{where}: conv_bias=true is not supported (the architecture's "
                              f"projections and convolution carry no bias)")
        tie = r.boolean("tie_embedding", "tie_word_embeddings", default=True)
        max_pos = r.integer("max_position_embeddings", default=128000, min_value=1)

        types = r.string_list("layer_types", default=None)
        idxs = r.integer_list("full_attn_idxs", default=None)
        if types is None and idxs is None:
            raise ConfigError(f"{where}: needs 'layer_types' or 'full_attn_idxs' to tell the "
                              f"attention layers from the short-convolution layers")
        if types is not None:
            if len(types) != L:
                raise ConfigError(f"{where}: layer_types has {len(types)} entries, num_hidden_layers is {L}")
            kinds = []
            for i, t in enumerate(types):
                if t not in _KIND_ALIASES:
                    raise ConfigError(f"{where}: layer_types[{i}] = {t!r}; known kinds: "
                                      f"{', '.join(sorted(_KIND_ALIASES))}")
                kinds.append(_KIND_ALIASES[t])
        if idxs is not None:
            bad = [i for i in idxs if not 0 <= i < L]
            if bad or len(set(idxs)) != len(idxs):
                raise ConfigError(f"{where}: full_attn_idxs {idxs} must be distinct layer numbers below {L}")
            from_idxs = ["attention" if i in set(idxs) else "conv" for i in range(L)]
            if types is not None and from_idxs != kinds:
                raise ConfigError(f"{where}: layer_types and full_attn_idxs disagree "
                                  f"(attention layers {[i for i, k in enumerate(kinds) if k == 'attention']} "
                                  f"vs {sorted(idxs)})")
            kinds = from_idxs

        cfg = cls(
            vocab_size=V, hidden_size=d, num_hidden_layers=L, num_attention_heads=H,
            num_key_value_heads=G, head_dim=hd, intermediate_size=inter,
            block_auto_adjust_ff_dim=auto, ffn_dim_multiplier=mult, block_multiple_of=mof,
            rope_theta=theta, norm_eps=eps, conv_L_cache=K, layer_types=tuple(kinds),
            tie_embedding=tie, max_position_embeddings=max_pos,
            bos_token_id=r.optional_integer("bos_token_id"),
            eos_token_id=r.optional_integer("eos_token_id"),
            pad_token_id=r.optional_integer("pad_token_id"),
            architectures=tuple(archs), ignored_keys=tuple(r.unused()),
        )
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(f"{where}: num_attention_heads {self.num_attention_heads} is not a multiple "
                              f"of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"{where}: head_dim {self.head_dim} must be even (rotary pairs)")
        if self.ffn_dim < 1:
            raise ConfigError(f"{where}: feed-forward width works out to {self.ffn_dim}")
        if not math.isfinite(self.rope_theta) or not math.isfinite(self.norm_eps):
            raise ConfigError(f"{where}: rope_theta and norm_eps must be finite")

    # ---- writing ---------------------------------------------------------
    def to_dict(self) -> dict:
        """A config.json dictionary that `from_dict` reads back to an equal configuration."""
        out = {
            "architectures": list(self.architectures),
            "model_type": "lfm2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "block_auto_adjust_ff_dim": self.block_auto_adjust_ff_dim,
            "block_multiple_of": self.block_multiple_of,
            "rope_theta": self.rope_theta,
            "norm_eps": self.norm_eps,
            "conv_L_cache": self.conv_L_cache,
            "conv_bias": False,
            "layer_types": ["full_attention" if t == "attention" else "conv" for t in self.layer_types],
            "full_attn_idxs": list(self.full_attn_idxs),
            "tie_embedding": self.tie_embedding,
            "max_position_embeddings": self.max_position_embeddings,
        }
        if self.ffn_dim_multiplier is not None:
            out["ffn_dim_multiplier"] = self.ffn_dim_multiplier
        for k in ("bos_token_id", "eos_token_id", "pad_token_id"):
            if getattr(self, k) is not None:
                out[k] = getattr(self, k)
        return out

    def describe(self) -> dict:
        d = asdict(self)
        d["ffn_dim"] = self.ffn_dim
        d["full_attn_idxs"] = list(self.full_attn_idxs)
        d.pop("ignored_keys", None)
        return d
