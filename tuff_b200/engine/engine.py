"""The Python entry point: `Engine(model_dir, ...)`, `engine.generate(prompts, params)`.

Token ids in, token ids out.  `generate` puts the prompts into the scheduler
and loops: plan a step, run it through `ModelRunner.step`, sample on the device,
read the sampled ids back, update the scheduler; until every request is
finished.  The reference's counterpart is the body of its command-line run
(src/main.c:1165-1918): prefill in chunks, then one token per step for `-n`
tokens, greedy on the LFM path.
"""
from __future__ import annotations

import time
from typing import Dict, List, Sequence

import torch

from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, SampleRow
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Request, Scheduler, StepPlan


class Engine:
    def __init__(self, model_dir: str | None, dtype="bfloat16", device="cuda:0", ctx_size: int | None = None,
                 max_tokens: int | None = None, page_size: int = 64, max_batched_tokens: int = 2048,
                 max_running: int = 64, cuda_graphs: bool = True, config: dict | None = None,
                 weight_seed: int = 0):
        """ctx_size: longest request (prompt + new tokens), the command line's -c;
        max_tokens: tokens the cache pool holds over all live requests (default: ctx_size, or
        8192: one full-length request fits).  `model_dir=None` with `config` and `weight_seed`
        builds a random-weights model on the device."""
        ctx = ctx_size or 8192
        self.runner = ModelRunner(model_dir, dtype=dtype, device=device,
                                  max_tokens=max_tokens if max_tokens is not None else ctx,
                                  page_size=page_size, max_requests=max_running, max_context=ctx,
                                  cuda_graphs=cuda_graphs, config=config, weight_seed=weight_seed)
        self.scheduler = Scheduler(self.runner.cache, max_batched_tokens=max_batched_tokens,
                                   max_running=max_running, max_context=self.runner.max_context)
        self.sampler = Sampler(self.runner.vocab_size, self.runner.device)
        self.timing: Dict[str, float] = dict(steps=0, step_seconds=0.0)

    @property
    def config(self):
        return self.runner.config

    # ---- requests ------------------------------------------------------------
    def add_request(self, request_id, prompt: Sequence[int], params: SamplingParams | None = None) -> Request:
        params = params or SamplingParams()
        if params.seed == 0 and not params.greedy:
            params = SamplingParams(**{**params.__dict__, "seed": time.time_ns() & ((1 << 63) - 1) or 1})
        for t in prompt:
            if not 0 <= int(t) < self.runner.vocab_size:
                raise ValueError(f"request {request_id!r}: token {t} is outside the vocabulary "
                                 f"(0..{self.runner.vocab_size - 1})")
        return self.scheduler.add(request_id, prompt, params)

    def step(self) -> List[Request]:
        """Plans and runs one step; returns the requests it finished."""
        plan = self.scheduler.plan()
        if not plan.entries:
            return []
        sampled = self._run(plan)
        return self.scheduler.update(plan, sampled)

    def _run(self, plan: StepPlan) -> List[int]:
        t0 = time.perf_counter()
        entries = [StepEntry(e.request.cache, e.tokens, [len(e.tokens) - 1] if e.samples else [])
                   for e in plan.entries]
        logits = self.runner.step(entries)
        rows = []
        for e in plan.entries:
            if e.samples:
                r = e.request
                p = r.params
                n_all = len(r.prompt) + len(r.output)
                recent = r.token_slice(n_all - p.repeat_last_n) if (p.repeat_penalty > 1.0 and p.repeat_last_n) else ()
                rows.append(SampleRow(p, r.key, len(r.output), recent))
        out: List[int] = []
        if rows:
            out = self.sampler.sample(logits, rows).tolist()
        self.timing["steps"] += 1
        self.timing["step_seconds"] += time.perf_counter() - t0
        return out

    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams] | None = None
                 ) -> List[List[int]]:
        """Generates for every prompt (lists of token ids); returns the new tokens of each."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        base = self.scheduler._next_key
        reqs = [self.add_request(("gen", base + i), p, sp) for i, (p, sp) in enumerate(zip(prompts, params))]
        while self.scheduler.has_work():
            self.step()
        return [list(r.output) for r in reqs]

    def stats(self) -> Dict[str, float]:
        s = dict(self.scheduler.stats)
        s.update(self.timing)
        s["free_pages"] = min([g.pool.n_free for g in self.runner.cache.groups] + [self.runner.cache.num_pages])
        return s
