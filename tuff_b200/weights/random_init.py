"""Random-weights mode: writes a model folder (config.json, model.safetensors)
from a configuration and a seed.

Each tensor is drawn from its own generator, seeded by a hash of (seed, tensor
name), so a tensor's values do not depend on which other tensors the model
has.  Matrices and convolution taps are N(0, 0.02); norm weights are
1 + N(0, 0.05).  Values are drawn in fp32 and stored as bfloat16 unless
`store_dtype` says float32.  The reference has no such mode (it runs published
GGUF files only).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Iterator, Tuple

import torch

from ..config.registry import config_from_dict, get_architecture
from ..models.model import Model
from ..parts.base import WeightDecl
from .safetensors_io import write_safetensors


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{int(seed)}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def draw_tensor(seed: int, name: str, decl: WeightDecl, store_dtype: torch.dtype) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed(tensor_seed(seed, name))
    if decl.role == "table":
        return torch.zeros(decl.shape, dtype=torch.int32)
    t = torch.empty(decl.shape, dtype=torch.float32)
    if decl.init == "norm":
        t.normal_(0.0, 0.05, generator=g).add_(1.0)
    else:
        t.normal_(0.0, 0.02, generator=g)
    return t.to(store_dtype)


def random_tensors(expected: Dict[str, WeightDecl], seed: int,
                   store_dtype: torch.dtype = torch.bfloat16) -> Iterator[Tuple[str, torch.Tensor]]:
    for name in sorted(expected):
        yield name, draw_tensor(seed, name, expected[name], store_dtype)


def random_device_tensors(expected: Dict[str, WeightDecl], seed: int, engine_dtype: torch.dtype,
                          device) -> Dict[str, torch.Tensor]:
    """The random-weights mode without a file: every tensor is drawn on the device (same
    distributions, seeded per tensor name; not the same values as the file mode's CPU draws)
    and rounded to bfloat16 as a checkpoint would store it."""
    out: Dict[str, torch.Tensor] = {}
    for name in sorted(expected):
        decl = expected[name]
        g = torch.Generator(device=device)
        g.manual_seed(tensor_seed(seed, name))
        if decl.role == "table":
            out[name] = torch.zeros(decl.shape, dtype=torch.int32, device=device)
            continue
        t = torch.empty(decl.shape, dtype=torch.float32, device=device)
        if decl.init == "norm":
            t.normal_(0.0, 0.05, generator=g).add_(1.0)
        else:
            t.normal_(0.0, 0.02, generator=g)
        t = t.to(torch.bfloat16)
        if decl.role == "vector" or engine_dtype == torch.float32:
            t = t.to(torch.float32)
        out[name] = t
    return out


def write_random_model(model_dir: str, config: Any, seed: int, store_dtype: torch.dtype = torch.bfloat16) -> str:
    """`config` is a config.json dictionary or a typed configuration of a registered architecture."""
    if isinstance(config, dict):
        arch, cfg = config_from_dict(config, "config")
        raw = dict(config)
    else:
        arch = get_architecture(config.architectures[0])
        cfg, raw = config, None
    if raw is None:
        raw = arch.config_to_dict(cfg)
    model = Model(arch.model_spec(cfg))
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw, f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      random_tensors(model.expected_tensors(), seed, store_dtype),
                      metadata={"format": "pt", "weight_seed": str(seed)})
    return model_dir
