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

from ..kernels import ops
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, SampleRow
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Request, Scheduler, StepPlan


class _Result:
    """A step's sampled ids: on the device (the next step may take its input from there), and the pinned
    host buffer they are being copied to with the event that says the copy is done."""
    __slots__ = ("ids", "host", "n", "copied")

    def __init__(self, ids, host, n, copied):
        self.ids, self.host, self.n, self.copied = ids, host, n, copied


class Engine:
    def __init__(self, model_dir: str | None, dtype="bfloat16", device="cuda:0", ctx_size: int | None = None,
                 max_tokens: int | None = None, page_size: int = 64, max_batched_tokens: int = 2048,
                 max_running: int = 64, cuda_graphs: bool = True, config: dict | None = None,
                 weight_seed: int = 0, run_ahead: bool = True):
        """ctx_size: longest request (prompt + new tokens), the command line's -c;
        max_tokens: tokens the cache pool holds over all live requests (default: ctx_size, or
        8192: one full-length request fits).  `model_dir=None` with `config` and `weight_seed`
        builds a random-weights model on the device.  `run_ahead`: while all requests decode,
        launch the next step before the current step's tokens have been read (see `step`)."""
        ctx = ctx_size or 8192
        self.runner = ModelRunner(model_dir, dtype=dtype, device=device,
                                  max_tokens=max_tokens if max_tokens is not None else ctx,
                                  page_size=page_size, max_requests=max_running, max_context=ctx,
                                  cuda_graphs=cuda_graphs, config=config, weight_seed=weight_seed)
        self.scheduler = Scheduler(self.runner.cache, max_batched_tokens=max_batched_tokens,
                                   max_running=max_running, max_context=self.runner.max_context)
        self.sampler = Sampler(self.runner.vocab_size, self.runner.device)
        self.timing: Dict[str, float] = dict(steps=0, step_seconds=0.0)
        self.run_ahead = bool(run_ahead)
        self._ahead = None            # (plan, its `_Result`) of a step launched and not yet read
        # Set to a list to have every step bracketed by CUDA events: (start, end, tokens of the step) is
        # appended per step; after a synchronize, start.elapsed_time(end) is the step's time on the device.
        self.step_events: list | None = None
        # Sampled ids come back on a stream of their own: the copy of step N waits for step N's sampling
        # only, so the host reads it while step N+1, already queued on the compute stream, runs.
        self._copy_stream = torch.cuda.Stream(device=self.runner.device)
        self._host_ids = [torch.empty(max_running + 1, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._host_next = 0

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
        """Plans and runs one step; returns the requests it finished.

        While every request decodes, the step after this one is launched before this one's
        sampled ids are read: its input ids are taken on the device from this step's result, and
        everything else about it (positions, pages) is known.  The GPU then never waits for the
        host to plan, lay out and launch.  The host learns the ids one step late; a request that
        turns out to have met a stop token has run one step too many, whose result is dropped."""
        if self._ahead is not None:
            plan, result = self._ahead
            self._ahead = None
        else:
            plan = self.scheduler.plan()
            if not plan.entries:
                return []
            result = self._launch(plan, None)
        nxt = None
        if self.run_ahead and result is not None and self._may_run_ahead(plan):
            nxt_plan = self.scheduler.plan_ahead(plan)
            if nxt_plan is not None:
                nxt = (nxt_plan, self._launch(nxt_plan, result.ids))
        sampled = self._read_ids(result) if result is not None else []
        finished = self.scheduler.update(plan, sampled)
        if nxt is not None and self.scheduler.running:
            self._ahead = nxt
        return finished

    def _send_home(self, ids: torch.Tensor) -> "_Result":
        """Starts the copy of a step's sampled ids, and of the kernels' status word behind them, into pinned
        host memory on the copy stream, which waits for the sampling only: not for what the compute stream is
        given afterwards."""
        n = ids.numel()
        host = self._host_ids[self._host_next]
        self._host_next = (self._host_next + 1) % len(self._host_ids)
        sampled = torch.cuda.Event()
        sampled.record()
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(sampled)
            host[:n].copy_(ids.view(-1), non_blocking=True)
            host[n:n + 1].copy_(ops.status_word(self.runner.device), non_blocking=True)
            copied = torch.cuda.Event()
            copied.record()
        return _Result(ids, host, n, copied)

    def _read_ids(self, result: "_Result") -> List[int]:
        """The sampled ids on the host, read together with the kernels' status word (one wait, on the copy's
        own event): a kernel whose bounded wait ran out has left a code there, and what the step wrote is
        invalid."""
        result.copied.synchronize()
        both = result.host[:result.n + 1].tolist()
        if both[-1]:
            self.reset()
            ops.raise_on_status(both[-1])
        return both[:-1]

    def reset(self) -> None:
        """Aborts every request (their pages and slots are free again) and forgets a step that was
        launched ahead; the engine is then as it was before the first request."""
        self._ahead = None
        for req in list(self.scheduler.running) + list(self.scheduler.waiting):
            self.scheduler.abort(req)

    @staticmethod
    def _may_run_ahead(plan: StepPlan) -> bool:
        # the repetition penalty needs the latest ids on the host before the next draw
        return all(not (e.request.params.repeat_penalty > 1.0 and e.request.params.repeat_last_n
                        and not e.request.params.greedy) for e in plan.entries)

    def _launch(self, plan: StepPlan, token_source) -> "_Result | None":
        """Runs the plan's step and samples; returns the sampled ids, on the device and on their way to
        the host (None if no entry samples).  `token_source`: the ids sampled by the step before, on the
        device, for a plan made ahead of them."""
        t0 = time.perf_counter()
        ahead = token_source is not None
        entries = [StepEntry(e.request.cache, e.tokens, [len(e.tokens) - 1] if e.samples else [])
                   for e in plan.entries]
        if self.step_events is not None:
            ev0 = torch.cuda.Event(enable_timing=True)
            ev0.record()
        logits = self.runner.step(entries, token_source)
        rows = []
        for e in plan.entries:
            if e.samples:
                r = e.request
                p = r.params
                n_all = len(r.prompt) + len(r.output)
                recent = r.token_slice(n_all - p.repeat_last_n) if (p.repeat_penalty > 1.0 and p.repeat_last_n) else ()
                rows.append(SampleRow(p, r.key, len(r.output) + (1 if ahead else 0), recent))
        out = self._send_home(self.sampler.sample(logits, rows)) if rows else None
        if self.step_events is not None:
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            self.step_events.append((ev0, ev1, sum(len(e.tokens) for e in plan.entries)))
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
