"""What a model is put together from: parts, their declarations and registries.

A part is a piece of a layer (a mixer, a feed-forward, a norm, a position
encoding, an embedding, a head) or the arrangement of such pieces (a block).
Every part
  * takes all of its sizes and constants as constructor parameters,
  * declares the weights it needs (`weight_decls`) under local names,
  * receives them on the device through `bind`,
  * and never learns which model it sits in.
A mixer may also declare what it needs from the cache manager (`cache_need`).

A model description (`tuff_b200.models.spec.ModelSpec`) names parts by their
registered kind and maps each local weight name to a checkpoint tensor name, so
a new kind becomes usable by registering a class here; nothing else changes.

Interfaces (ctx is the step's `StepContext`):
  Norm.forward(ctx, x, row_index=None) -> h            x fp32 [T, d] -> activation dtype
  Mixer.forward(ctx, cache, h, residual, reads_only)   residual (fp32 [T, d]) += mixer(h)
  FeedForward.forward(ctx, h, residual)                residual += ffn(h)
  PositionEncoding.rotate(ctx, q, k) or fused_tables() see parts/rope.py
  Block.forward(ctx, x, layer, cache, reads_only, next_norm=None)   runs one layer on the residual x
  Embedding.forward(ctx) -> x                          fp32 [T, d]
  Head.forward(ctx, x, norm) -> logits                 fp32 [n_wanted, vocab]
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Tuple, Type

import torch


@dataclass(frozen=True)
class WeightDecl:
    """One weight a part needs.

    role: "matrix"  kept in the checkpoint's dtype (bf16 stays bf16, fp32 stays fp32;
                    the 32-bit engine raises everything to fp32),
          "vector"  small per-channel parameters, held in fp32 on the device,
          "table"   integer tables, held as int32.
    init: how the random-weights mode draws it: "normal" = N(0, 0.02),
          "norm" = 1 + N(0, 0.05).
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values that grow with the tokens; `window` = how many of the
    latest keys a token may see (None: all of them).  `v_head_dim`: the width of a value where it
    differs from a key's (the pages of V are then `[pages, kv_heads, page_size, v_head_dim]`)."""
    kv_heads: int
    head_dim: int
    window: int | None = None
    v_head_dim: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size, set to `fill` (the state's neutral element; zero for sums)
    when a request gets its slot."""
    shape: Tuple[int, ...]
    dtype: str = "float32"
    fill: float = 0.0


@dataclass
class PartSpec:
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    tensors: Dict[str, str] = field(default_factory=dict)   # local weight name -> checkpoint tensor name


class Part:
    kind: str = ""
    # Whether a step that runs this part can be captured once and replayed as a CUDA graph: its
    # forward then launches the same kernels on the same buffers whatever the step's values are,
    # reads nothing on the host (no `ctx.host`, no `.item()`, no shape that depends on data) and
    # takes everything that changes from step to step from the context's device tensors.  A part
    # that cannot promise this sets it to False, and a model with such a part runs every step as
    # plain launches.
    replayable: bool = True

    def reserve(self, device, max_rows: int, max_context: int) -> None:
        """Called once before the first step: a part whose kernels use scratch memory sizes it here for
        the most rows a step may bring and the longest context, so that it never moves afterwards."""

    def weight_decls(self) -> Dict[str, WeightDecl]:
        return {}

    def bind(self, weights: Dict[str, torch.Tensor], act_dtype: torch.dtype) -> None:
        """Receives the declared weights (device tensors, converted by role)."""
        self.w = weights
        self.act_dtype = act_dtype


class Norm(Part):
    def forward(self, ctx, x, row_index=None):
        raise NotImplementedError

    def announce(self, ctx, x) -> None:
        """Told before the part that writes `x` last runs: this norm will be the next reader of x.
        A norm may use it to have that write prepare its work; the default does nothing."""


class PositionEncoding(Part):
    pass


class Mixer(Part):
    def cache_need(self) -> PagedKVNeed | StateNeed | None:
        return None

    def forward(self, ctx, cache, h, residual, reads_only: bool = False) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h, residual) -> None:
        raise NotImplementedError


class Block(Part):
    def forward(self, ctx, x, layer, cache, reads_only: bool = False, next_norm=None) -> None:
        """`next_norm`: the norm that reads x after this layer (the next layer's first norm, or the
        final norm), if the caller knows it; a block may `announce` x to it before its last write."""
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ctx):
        raise NotImplementedError


class Head(Part):
    def forward(self, ctx, x, norm):
        raise NotImplementedError


class Registry:
    """Kind name -> part class, for one family of parts."""

    def __init__(self, family: str, base: Type[Part]):
        self.family, self.base = family, base
        self._classes: Dict[str, Type[Part]] = {}

    def register(self, kind: str) -> Callable[[Type[Part]], Type[Part]]:
        def deco(cls: Type[Part]) -> Type[Part]:
            if not issubclass(cls, self.base):
                raise TypeError(f"{cls.__name__} is not a {self.base.__name__}")
            if kind in self._classes and self._classes[kind] is not cls:
                raise ValueError(f"{self.family} kind {kind!r} is already registered")
            cls.kind = kind
            self._classes[kind] = cls
            return cls
        return deco

    def unregister(self, kind: str) -> None:
        self._classes.pop(kind, None)

    def build(self, spec: PartSpec) -> Part:
        if spec.kind not in self._classes:
            raise KeyError(f"unknown {self.family} kind {spec.kind!r}; registered: "
                           f"{', '.join(sorted(self._classes)) or '(none)'}")
        return self._classes[spec.kind](**spec.params)

    def kinds(self) -> list[str]:
        return sorted(self._classes)


NORMS = Registry("norm", Norm)
POSITION_ENCODINGS = Registry("position encoding", PositionEncoding)
MIXERS = Registry("mixer", Mixer)
FEED_FORWARDS = Registry("feed-forward", FeedForward)
BLOCKS = Registry("block", Block)
EMBEDDINGS = Registry("embedding", Embedding)
HEADS = Registry("head", Head)

register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_block = BLOCKS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register
