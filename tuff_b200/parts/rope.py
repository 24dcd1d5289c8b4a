"""Rotary position encoding, NeoX pairing: within the rotated span of a head,
element j pairs with j + span/2 and the pair turns by pos * theta^(-2j/span)
(reference: src/lfm25_gpu.cu:459-474; the reference rotates the whole head).

The attention mixer asks a position encoding for `fused_tables`: if it gets a
table of inverse frequencies and a span, the rotation runs inside the fused
q/k-norm kernel.  A position encoding without such tables implements
`rotate(ctx, q, k)` on [T, heads, head_dim] views instead and is applied between
the norm and the cache write.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rope_neox")
class RotaryNeox(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim) if rotary_dim is not None else self.head_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        self._inv_freq = None

    def inv_freq_host(self) -> np.ndarray:
        j = np.arange(self.rotary_dim // 2, dtype=np.float64)
        return (self.theta ** (-2.0 * j / self.rotary_dim)).astype(np.float32)

    def fused_tables(self, device):
        """(inverse frequencies as fp32 [rotary_dim/2], rotary_dim), computed in fp64 then rounded."""
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            self._inv_freq = torch.from_numpy(self.inv_freq_host()).to(device)
        return self._inv_freq, self.rotary_dim
