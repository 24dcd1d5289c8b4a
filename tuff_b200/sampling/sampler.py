"""Chooses the next token of every logits row on the device.

One kernel launch per step: rows with temp <= 0 take the first maximum, the
others go through the reference's chain (src/sampler.c:99-230) inside
`tuff_sample` (csrc/sampling.cu).  The random draw of a row is a function of
(seed, request key, index of the token being drawn) alone, so a request's
tokens do not depend on the batch it was sampled in, nor on being recomputed
after a preemption.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import List, Sequence

import torch

from ..kernels import ops
from .params import SamplingParams

MAX_RECENT = 256


@dataclass
class SampleRow:
    params: SamplingParams
    request_key: int            # stable number of the request
    token_index: int            # index of the token being drawn among the request's outputs
    recent: Sequence[int] = ()  # the request's latest tokens (prompt and outputs), oldest first


class Sampler:
    def __init__(self, vocab_size: int, device):
        self.V, self.device = int(vocab_size), torch.device(device)
        self._work = None
        self._stage: dict = {}

    def _upload(self, name: str, host: torch.Tensor) -> torch.Tensor:
        """Copies a small host tensor to the device through pinned memory without waiting for the
        GPU: two pinned buffers per name take turns, each guarded by an event of its last copy, so
        a step that was launched ahead of the one before it does not stall the host here."""
        n = host.numel()
        ring = self._stage.get(name)
        if ring is None or ring["size"] < n or ring["dtype"] != host.dtype:
            size = max(n, 256)
            pin = torch.cuda.is_available()
            ring = self._stage[name] = dict(size=size, dtype=host.dtype, turn=0, slots=[
                dict(pinned=torch.empty(size, dtype=host.dtype, pin_memory=pin), event=None) for _ in range(2)])
        slot = ring["slots"][ring["turn"]]
        ring["turn"] ^= 1
        if slot["event"] is not None:
            slot["event"].synchronize()
        slot["pinned"][:n].copy_(host.reshape(-1))
        dev = slot["pinned"][:n].to(self.device, non_blocking=True)
        if slot["event"] is None:
            slot["event"] = torch.cuda.Event()
        slot["event"].record()
        return dev.view(host.shape)

    def sample(self, logits: torch.Tensor, rows: Sequence[SampleRow]) -> torch.Tensor:
        """int32 device tensor with one token per logits row."""
        n = logits.shape[0]
        assert n == len(rows) and logits.shape[1] == self.V
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        if n == 0:
            return out
        if all(r.params.greedy for r in rows):
            ops.argmax(logits, out)
            return out
        width = 0
        recents: List[List[int]] = []
        for r in rows:
            p = r.params
            k = min(p.repeat_last_n, MAX_RECENT) if p.repeat_penalty > 1.0 and not p.greedy else 0
            rec = list(r.recent)[-k:] if k else []
            recents.append(rec)
            width = max(width, len(rec))
        blob = bytearray()
        for r, rec in zip(rows, recents):
            p = r.params
            blob += struct.pack(ops.SAMPLE_ROW_FORMAT, float(p.temp), float(p.top_p), float(p.min_p),
                                float(p.repeat_penalty), int(p.top_k), len(rec), int(p.seed) & ((1 << 64) - 1),
                                int(r.request_key) & ((1 << 64) - 1), int(r.token_index))
        rows_dev = self._upload("rows", torch.frombuffer(blob, dtype=torch.uint8))
        recent_dev = None
        if width:
            host = torch.full((n, width), -1, dtype=torch.int32)
            for i, rec in enumerate(recents):
                if rec:
                    host[i, :len(rec)] = torch.tensor(rec, dtype=torch.int32)
            recent_dev = self._upload("recent", host)
        if self._work is None or self._work.numel() < n * self.V:
            self._work = torch.empty(n * self.V, dtype=torch.float32, device=self.device)
        ops.sample(logits, rows_dev, recent_dev, self._work, out)
        return out
