"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees.

The reference's LFM path serves one request at a time, feeding the prompt in
chunks of up to eight tokens and then one token per step (src/main.c:260-293,
1801-1849); its server for another model admits from a first-in-first-out queue
while a slot is idle and runs one prompt chunk and one decode launch per loop
(src/qwen35/q35_server.c:892-975).  Here every step is one mixed batch.

Each call of `plan()` builds one step, in this order:
  1. every running request whose prompt is done brings its one new token;
  2. running requests still in their prompt bring a portion, in arrival order,
     as long as the step's token budget lasts;
  3. waiting requests are admitted, first come first served, while a slot is
     free, the budget lasts, and pages for a first portion exist (none in a
     step that preempted someone).
A portion is cut to the budget and to the pages that are free.

When pages run out.  A decode token that has no page left takes one from the
request that was admitted last: that request is preempted — its pages and its
slot go back, it returns to the head of the waiting queue, and it is later
recomputed from its prompt plus the tokens it has produced so far, which are
kept.  The draws of a request depend only on (seed, request, token index), so
its output does not change by being preempted.  If nothing at all can run (every
running request waits for pages) the last admitted one is preempted as well.  A
single request that does not fit into the empty pool is an error.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Sequence
from collections import deque

from ..cache.manager import CacheManager, RequestCache
from ..sampling.params import SamplingParams


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class SchedulerError(RuntimeError):
    pass


@dataclass
class Request:
    request_id: object
    prompt: List[int]
    params: SamplingParams
    key: int = 0                          # stable number, part of the request's random stream
    output: List[int] = field(default_factory=list)
    status: RequestStatus = RequestStatus.WAITING
    cache: RequestCache | None = None
    preemptions: int = 0
    finish_reason: str | None = None

    @property
    def n_cached(self) -> int:
        return self.cache.n_tokens if self.cache is not None else 0

    def all_tokens(self) -> List[int]:
        return self.prompt + self.output

    def token_slice(self, start: int, stop: int | None = None) -> List[int]:
        """Tokens start..stop-1 of prompt followed by output, without building the whole list
        (a decode step asks for one token of a request that may hold thousands)."""
        n_p = len(self.prompt)
        total = n_p + len(self.output)
        stop = total if stop is None else min(stop, total)
        start = max(0, start)
        if start >= n_p:
            return self.output[start - n_p:stop - n_p]
        if stop <= n_p:
            return self.prompt[start:stop]
        return self.prompt[start:] + self.output[:stop - n_p]

    def n_pending(self) -> int:
        return len(self.prompt) + len(self.output) - self.n_cached


@dataclass
class PlannedEntry:
    request: Request
    tokens: List[int]
    samples: bool                          # the portion ends the known tokens: its last logits pick the next one
    start: int = 0                         # position of the portion's first token, as planned


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    admitted: List[Request] = field(default_factory=list)

    @property
    def n_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, max_batched_tokens: int = 2048, max_running: int = 64,
                 max_context: int | None = None):
        if max_batched_tokens < 1 or max_running < 1:
            raise ValueError("max_batched_tokens and max_running must be positive")
        self.cache = cache
        self.max_batched_tokens = int(max_batched_tokens)
        self.max_running = min(int(max_running), cache.max_requests)
        self.max_context = max_context
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []            # in order of admission
        self.finished: List[Request] = []
        self._next_key = 0
        self.stats: Dict[str, int] = dict(steps=0, preemptions=0, prompt_tokens=0, decode_tokens=0, admitted=0)

    # ---- requests ------------------------------------------------------------
    def add(self, request_id, prompt: Sequence[int], params: SamplingParams) -> Request:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise SchedulerError(f"request {request_id!r}: the prompt is empty")
        total = len(prompt) + params.max_new_tokens
        if self.max_context is not None and total > self.max_context:
            raise SchedulerError(f"request {request_id!r}: {len(prompt)} prompt + {params.max_new_tokens} new tokens "
                                 f"exceed the context of {self.max_context}")
        cap = self.cache.num_pages * self.cache.page_size
        if self.cache.groups and total - 1 > cap:
            raise SchedulerError(f"request {request_id!r}: its {total - 1} cached tokens would not fit the whole "
                                 f"cache ({cap} tokens)")
        req = Request(request_id, prompt, params, key=self._next_key)
        self._next_key += 1
        if params.max_new_tokens == 0:
            req.status, req.finish_reason = RequestStatus.FINISHED, "length"
            self.finished.append(req)
        else:
            self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- planning ------------------------------------------------------------
    def _free_pages(self) -> List[int]:
        return [g.pool.n_free for g in self.cache.groups]

    def _fits(self, need: List[int], free: List[int]) -> bool:
        return all(n <= f for n, f in zip(need, free))

    def _take(self, need: List[int], free: List[int]) -> None:
        for i, n in enumerate(need):
            free[i] -= n

    def _tokens_that_fit(self, rc: RequestCache | None, want: int, free: List[int]) -> int:
        """The longest portion <= want whose pages are free."""
        if not self.cache.groups:
            return want
        ps = self.cache.page_size
        held = rc.n_tokens if rc is not None else 0
        room = want
        for gi, f in enumerate(free):
            blocks_held = len(rc.tables[gi]) if rc is not None else 0
            room = min(room, (blocks_held + f) * ps - held)
        return max(0, room)

    def _preempt(self, req: Request, plan: StepPlan) -> None:
        self.cache.close(req.cache)
        req.cache = None
        req.status = RequestStatus.WAITING
        req.preemptions += 1
        self.running.remove(req)
        self.waiting.appendleft(req)
        plan.preempted.append(req)
        self.stats["preemptions"] += 1

    def plan(self) -> StepPlan:
        plan = StepPlan()
        while True:
            self._plan_once(plan)
            if plan.entries or not self.running:
                break
            # every running request waits for pages: make room by preempting the last admitted
            if len(self.running) == 1:
                raise SchedulerError(f"request {self.running[0].request_id!r} cannot get pages in an otherwise "
                                     f"empty cache")
            self._preempt(self.running[-1], plan)
        if not plan.entries and self.waiting and not self.running:
            raise SchedulerError(f"request {self.waiting[0].request_id!r} cannot be admitted into an empty cache")
        self.stats["steps"] += 1 if plan.entries else 0
        return plan

    def _plan_once(self, plan: StepPlan) -> None:
        plan.entries.clear()
        budget = self.max_batched_tokens
        free = self._free_pages()
        planned = set()
        # 1. decode tokens
        for req in list(self.running):
            if req.status is not RequestStatus.RUNNING or req.n_pending() != 1 or budget < 1:
                continue
            need = self.cache.pages_needed(req.cache, 1)
            while not self._fits(need, free):
                victim = self.running[-1]
                if id(victim) in planned:
                    break                                   # cannot happen: victims are admitted later than `req`
                self._preempt(victim, plan)
                free = [f - t for f, t in zip(self._free_pages(), self._taken(plan))]
                if victim is req:
                    break
            if req.status is not RequestStatus.RUNNING or not self._fits(need, free):
                continue
            self._take(need, free)
            plan.entries.append(PlannedEntry(req, req.token_slice(req.n_cached), True, req.n_cached))
            planned.add(id(req))
            budget -= 1
        # 2. portions of running prompts
        for req in self.running:
            if id(req) in planned or budget < 1 or req.n_pending() < 2:
                continue
            n = self._tokens_that_fit(req.cache, min(req.n_pending(), budget), free)
            if n < 1:
                continue
            self._take(self.cache.pages_needed(req.cache, n), free)
            toks = req.token_slice(req.n_cached, req.n_cached + n)
            plan.entries.append(PlannedEntry(req, toks, n == req.n_pending(), req.n_cached))
            planned.add(id(req))
            budget -= n
        # 3. admission (not in a step that had to preempt: the freed pages are for those who run)
        while (not plan.preempted and self.waiting and budget >= 1 and len(self.running) < self.max_running and self.cache.can_open()):
            req = self.waiting[0]
            n = self._tokens_that_fit(None, min(req.n_pending(), budget), free)
            if n < 1:
                break
            self.waiting.popleft()
            req.cache = self.cache.open(req.request_id)
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            plan.admitted.append(req)
            self.stats["admitted"] += 1
            self._take(self.cache.pages_needed(req.cache, n), free)
            plan.entries.append(PlannedEntry(req, req.token_slice(0, n), n == req.n_pending(), 0))
            planned.add(id(req))
            budget -= n

    def plan_ahead(self, prev: StepPlan) -> StepPlan | None:
        """The step after `prev`, planned before `prev`'s sampled tokens are known: the same
        requests, one more token each, the token itself still on the device (the entries carry a
        placeholder).  Only when nothing else could happen in that step: `prev` is pure decoding,
        nobody waits, nobody reaches its length or the context with the token that `prev` samples
        (a stop token cannot be foreseen; `update` skips the entry of a request that met one), and
        every request finds its page.  Otherwise None, and the next step is planned as usual."""
        if self.waiting or not prev.entries or prev.preempted or prev.admitted:
            return None
        if len(prev.entries) != len(self.running):
            return None
        free = self._free_pages()
        plan = StepPlan()
        for e in prev.entries:
            req = e.request
            if not e.samples or len(e.tokens) != 1 or req.status is not RequestStatus.RUNNING or req.n_pending() != 0:
                return None
            n_out = len(req.output) + 1                       # once `prev`'s token has arrived
            if n_out >= req.params.max_new_tokens:
                return None
            if self.max_context is not None and len(req.prompt) + n_out >= self.max_context:
                return None
            need = self.cache.pages_needed(req.cache, 1)
            if not self._fits(need, free):
                return None
            self._take(need, free)
            plan.entries.append(PlannedEntry(req, [0], True, req.n_cached))
        self.stats["steps"] += 1
        return plan

    def _taken(self, plan: StepPlan) -> List[int]:
        """Pages that the entries planned so far will take, per group."""
        out = [0] * len(self.cache.groups)
        for e in plan.entries:
            for i, n in enumerate(self.cache.pages_needed(e.request.cache, len(e.tokens))):
                out[i] += n
        return out

    # ---- after the step ------------------------------------------------------
    def update(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """Takes the tokens sampled for the plan's sampling entries (in their order);
        returns the requests that finished, whose pages and slots are free again."""
        it = iter(sampled)
        done: List[Request] = []
        for e in plan.entries:
            req = e.request
            if req.status is not RequestStatus.RUNNING:
                # planned ahead, and finished by the token before this one: its result is dropped
                if e.samples:
                    next(it)
                continue
            # counted from the position planned for the portion (the cache may already count a step launched after this one)
            self.stats["prompt_tokens"] += max(0, min(len(req.prompt), e.start + len(e.tokens)) - e.start)
            if not e.samples:
                continue
            tok = int(next(it))
            req.output.append(tok)
            self.stats["decode_tokens"] += 1
            reason = None
            if tok in req.params.stop_token_ids:
                reason = "stop"
            elif len(req.output) >= req.params.max_new_tokens:
                reason = "length"
            elif self.max_context is not None and len(req.prompt) + len(req.output) >= self.max_context:
                reason = "context"
            if reason:
                self._finish(req, reason)
                done.append(req)
        return done

    def _finish(self, req: Request, reason: str) -> None:
        if req.cache is not None:
            self.cache.close(req.cache)
            req.cache = None
        if req in self.running:
            self.running.remove(req)
        req.status, req.finish_reason = RequestStatus.FINISHED, reason
        self.finished.append(req)

    def abort(self, req: Request) -> None:
        if req.status is RequestStatus.WAITING:
            self.waiting.remove(req)
        self._finish(req, "aborted")
