"""The step function: one batch of (request, its next tokens) through the model,
from the cache, returning the logits at the wanted places.

`ModelRunner` owns the model on the device, the cache manager and nothing else:
no queue and no sampling.  Generation, the scheduler and trace replay all drive
this one `step`.  Reference counterparts: src/lfm25_engine.c:434-475 (one token)
and :496-599 (up to eight tokens of one sequence).
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..cache.manager import CacheManager, RequestCache
from ..cache.pool import OutOfPages
from ..config.registry import config_from_dict, load_config
from ..models.model import Model
from ..weights.loader import load_checkpoint
from ..weights.random_init import random_device_tensors
from .batch import StepEntry, layout_entries, to_device, validate_entries

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
    def __init__(self, model_dir: str | None, dtype="bfloat16", device="cuda:0", max_tokens: int = 8192,
                 page_size: int = 64, max_requests: int = 64, max_context: int | None = None,
                 cuda_graphs: bool = True, config: dict | None = None, weight_seed: int = 0):
        """`model_dir`: a folder with config.json and safetensors.  With `model_dir=None`, `config`
        (a config.json dictionary) and `weight_seed` make a random-weights model on the device
        without a file.  `cuda_graphs`: replay pure decode steps from captured CUDA graphs."""
        self.device = require_cuda(device)
        self.dtype = parse_dtype(dtype)
        if model_dir is not None:
            self.arch, self.config = load_config(model_dir)
        else:
            self.arch, self.config = config_from_dict(config, "config")
        self.model = Model(self.arch.model_spec(self.config))
        with torch.cuda.device(self.device):
            if model_dir is not None:
                weights = load_checkpoint(model_dir, self.model.expected_tensors(), self.dtype, self.device)
            else:
                weights = random_device_tensors(self.model.expected_tensors(), weight_seed, self.dtype, self.device)
            self.model.bind_weights(weights, self.dtype)
        del weights
        self.cuda_graphs = bool(cuda_graphs) and self.model.replayable     # every part must allow replay
        self._graphs: Dict[int, dict] = {}
        self._seen_rows: Dict[int, int] = {}
        self.graph_replays = 0
        self.vocab_size = self.model.spec.vocab_size
        limit = self.model.spec.max_context
        self.max_context = min(x for x in (max_context, limit, 1 << 30) if x is not None)
        self.cache = CacheManager(self.model.storage_needs(), page_size, max_tokens, max_requests,
                                  dtype=self.dtype, device=self.device)
        # scratch memory of the kernels at its final size and address before any step can be captured
        self.model.reserve(self.device, max_requests, self.max_context)

    # ---- requests ------------------------------------------------------------
    def open(self, request_id) -> RequestCache:
        return self.cache.open(request_id)

    def synthetic_fill(self, rc: RequestCache, n_tokens: int) -> None:
        """Makes a request hold `n_tokens` cached tokens without running them: their pages are
        taken and keep whatever they hold.  For measurements that need a long context whose
        content does not matter; never used by generation."""
        self.cache.reserve(rc, n_tokens)
        self.cache.commit(rc, n_tokens)

    def randomize_cache(self, seed: int = 0) -> None:
        """Fills every page and state with small random numbers (see `synthetic_fill`)."""
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        for st in self.cache.storages:
            for name in ("k_pages", "v_pages", "state"):
                t = getattr(st, name, None)
                if t is not None:
                    t.copy_(torch.empty(t.shape, dtype=torch.float32, device=self.device).normal_(0, 0.5, generator=g))

    def close(self, rc: RequestCache) -> None:
        self.cache.close(rc)

    # ---- the step ------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], token_source: torch.Tensor | None = None) -> torch.Tensor:
        """Runs the entries' tokens as one batch; returns fp32 logits [wanted, vocab] on the
        device, in the order of the entries and of their `want`.  Nothing is cached or
        reserved if validation fails or the pages do not suffice (`OutOfPages`).
        `token_source`: an int32 device tensor with one id per token of the batch that replaces
        the entries' ids on the device (ids that an earlier step has sampled and the host has not
        read yet); the entries then carry placeholders."""
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
        try:
            with torch.cuda.device(self.device):
                logits = self._run(entries, token_source)
        except BaseException:
            for e in entries:
                self.cache.cancel(e.cache)
            raise
        for e in entries:
            self.cache.commit(e.cache, len(e.tokens))
        return logits

    MAX_GRAPHS = 128

    def _run(self, entries: Sequence[StepEntry], token_source: torch.Tensor | None = None) -> torch.Tensor:
        R = len(entries)
        decode = (self.cuda_graphs and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries))
        if not decode:
            ctx = to_device(layout_entries(entries, self.cache), self.device, self.dtype)
            if token_source is not None:
                ctx.tokens.copy_(token_source)
            return self.model.forward(ctx, self.cache.storages)
        # A pure decode step: the same kernels with the same shapes every time, so it is captured
        # once per number of rows (after one plain run that lets workspaces grow) and replayed.
        width = (self.max_context + self.cache.page_size - 1) // self.cache.page_size
        host = layout_entries(entries, self.cache, table_width=width)
        host["max_seq_len"] = self.max_context            # launch shapes must not depend on the step
        g = self._graphs.get(R)
        if g is None:
            self._seen_rows[R] = self._seen_rows.get(R, 0) + 1
            if self._seen_rows[R] < 2:
                ctx = to_device(host, self.device, self.dtype)
                if token_source is not None:
                    ctx.tokens.copy_(token_source)
                return self.model.forward(ctx, self.cache.storages)
            if len(self._graphs) >= self.MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))
            n_ints = 8 * (R + 4) + len(self.cache.groups) * (R * width + 4)
            static = (torch.empty(n_ints, dtype=torch.int32, pin_memory=True),
                      torch.empty(n_ints, dtype=torch.int32, device=self.device), torch.cuda.Event())
            ctx = to_device(host, self.device, self.dtype, static)
            if token_source is not None:
                ctx.tokens.copy_(token_source)
            torch.cuda.current_stream().synchronize()
            from ..kernels import ops
            before = ops.LAUNCHES["n"]
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx, self.cache.storages)
            g = self._graphs[R] = dict(graph=graph, static=static, logits=logits, ctx=ctx,
                                       launches=ops.LAUNCHES["n"] - before)
            ops.LAUNCHES["n"] = before                   # captured, not run: replays are counted instead
        else:
            ctx = to_device(host, self.device, self.dtype, g["static"])
            if token_source is not None:
                ctx.tokens.copy_(token_source)              # into the buffer that the captured step reads
        g["graph"].replay()
        self.graph_replays += 1
        return g["logits"].clone()        # the graph's own output is overwritten by the next replay
