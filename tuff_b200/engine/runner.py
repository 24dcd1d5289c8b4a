"""The step function: one batch of (request, its next tokens) through the model,
from the cache, returning the logits at the wanted places.

`ModelRunner` owns the model on the device, the cache manager and nothing else:
no queue and no sampling.  Generation, the scheduler and trace replay all drive
this one `step`.  Reference counterparts: src/lfm25_engine.c:434-475 (one token)
and :496-599 (up to eight tokens of one sequence).
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..cache.manager import CacheManager, RequestCache
from ..cache.pool import OutOfPages
from ..config.registry import load_config
from ..models.model import Model
from ..weights.loader import load_checkpoint
from .batch import BatchError, StepContext, StepEntry, layout_entries, to_device, validate_entries

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine runs in bfloat16 or float32, not {name}")
        return name
    if name not in DTYPES:
        raise ValueError(f"dtype {name!r}: choose bfloat16 or float32")
    return DTYPES[name]


def require_cuda(device) -> torch.device:
    dev = torch.device(device)
    if dev.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("tuff_b200 runs on a CUDA device (NVIDIA B200, sm_100a) only: there is no CPU path. "
                           f"Asked for device {device!r}; torch.cuda.is_available() = {torch.cuda.is_available()}")
    return dev


class ModelRunner:
    def __init__(self, model_dir: str, dtype="bfloat16", device="cuda:0", max_tokens: int = 8192,
                 page_size: int = 16, max_requests: int = 64, max_context: int | None = None):
        self.device = require_cuda(device)
        self.dtype = parse_dtype(dtype)
        self.arch, self.config = load_config(model_dir)
        self.model = Model(self.arch.model_spec(self.config))
        with torch.cuda.device(self.device):
            weights = load_checkpoint(model_dir, self.model.expected_tensors(), self.dtype, self.device)
            self.model.bind_weights(weights, self.dtype)
        del weights
        self.vocab_size = self.model.spec.vocab_size
        limit = self.model.spec.max_context
        self.max_context = min(x for x in (max_context, limit, 1 << 30) if x is not None)
        self.cache = CacheManager(self.model.storage_needs(), page_size, max_tokens, max_requests,
                                  dtype=self.dtype, device=self.device)

    # ---- requests ------------------------------------------------------------
    def open(self, request_id) -> RequestCache:
        return self.cache.open(request_id)

    def close(self, rc: RequestCache) -> None:
        self.cache.close(rc)

    # ---- the step ------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs the entries' tokens as one batch; returns fp32 logits [wanted, vocab] on the
        device, in the order of the entries and of their `want`.  Nothing is cached or
        reserved if validation fails or the pages do not suffice (`OutOfPages`)."""
        validate_entries(entries, self.vocab_size, self.max_context)
        done: List[StepEntry] = []
        try:
            for e in entries:
                self.cache.reserve(e.cache, len(e.tokens))
                done.append(e)
        except OutOfPages:
            for e in done:
                self.cache.cancel(e.cache)
            raise
        with torch.cuda.device(self.device):
            ctx = to_device(layout_entries(entries, self.cache), self.device, self.dtype)
            logits = self.model.forward(ctx, self.cache.storages)
        for e in entries:
            self.cache.commit(e.cache, len(e.tokens))
        return logits
