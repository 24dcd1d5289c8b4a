"""Loads a checkpoint's tensors by name for a model's declared weights.

Every expected tensor is looked up by its checkpoint name; the file's tensors
are compared with the declarations as a whole, and one `WeightError` lists
everything that is missing, unexpected or of the wrong shape (the reference
stops at the first missing tensor, naming it: src/lfm25_model.c:35-49, and
checks shapes tensor by tensor: src/lfm25_model.c:296-317).

Element types by role: a matrix stays as stored (bf16 stays bf16, a tensor
stored in 32-bit stays 32-bit); the 32-bit engine raises every matrix to fp32,
which is exact.  Small per-channel vectors are held in fp32 and integer tables
as int32 whatever the engine's dtype.  A tensor that two parts share (a tied
head) is read and placed on the device once.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..parts.base import WeightDecl
from .safetensors_io import ModelFiles


class WeightError(ValueError):
    def __init__(self, model_dir: str, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = [f"{model_dir}: the checkpoint does not match the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} expected {list(want)}, found {list(got)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  wrong element type: {name} is {got}")
        super().__init__("\n".join(lines))


_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)


def convert_for_role(t: torch.Tensor, decl: WeightDecl, engine_dtype: torch.dtype) -> torch.Tensor:
    if decl.role == "table":
        return t.to(torch.int32)
    if decl.role == "vector":
        return t.to(torch.float32)
    if engine_dtype == torch.float32:
        return t.to(torch.float32)
    if t.dtype in (torch.float32, torch.bfloat16):
        return t
    return t.to(torch.bfloat16)


def load_checkpoint(model_dir: str, expected: Dict[str, WeightDecl], engine_dtype: torch.dtype,
                    device: str | torch.device) -> Dict[str, torch.Tensor]:
    files = ModelFiles(model_dir)
    try:
        have = files.entries
        missing = sorted(n for n in expected if n not in have)
        unexpected = sorted(n for n in have if n not in expected)
        wrong_shape, wrong_dtype = [], []
        for n, decl in expected.items():
            if n in have:
                if tuple(have[n].shape) != tuple(decl.shape):
                    wrong_shape.append((n, decl.shape, have[n].shape))
                ok = _INTS if decl.role == "table" else _FLOATS
                if have[n].dtype not in ok:
                    wrong_dtype.append((n, str(have[n].dtype)))
        if missing or unexpected or wrong_shape or wrong_dtype:
            raise WeightError(model_dir, missing, unexpected, wrong_shape, wrong_dtype)
        out: Dict[str, torch.Tensor] = {}
        for n, decl in expected.items():
            host = convert_for_role(files.tensor(n), decl, engine_dtype)
            out[n] = host.to(device)
        return out
    finally:
        files.close()
