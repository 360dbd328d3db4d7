"""Continuous batching above the step function.  The reference has no scheduler
(its caller slices a prompt into tiles and loops over decode tokens:
src/core/engine.cpp:1529-1545, src/apps/main.cpp:428-439); this one is designed
here.  It decides on the host, from the cache manager's bookkeeping alone.

Each step, in this order:

1. Every running request that is decoding gets its one token.  If the pages for
   those tokens do not exist, the most recently admitted running request is
   preempted (all its pages and its slot are given back, it returns to the FRONT
   of the waiting queue and will recompute its prompt plus what it had
   generated) until they do.
2. Running requests that still have prompt left get a portion: what is left,
   capped by the step's token budget, by ``chunk`` if set, and by the free pages
   (a portion may shrink to fit; it is never the cause of a preemption).
3. Waiting requests are admitted in arrival order while a request slot is free,
   fewer than ``max_running`` are running, budget is left and the first portion's
   pages exist.

A request that could not run alone in the pool (prompt + max_new_tokens needs more
pages than the pool has, or more positions than ``max_context``) is refused when
it is submitted.  A request finishes on an end-of-sequence token ("eos"), after
``max_new_tokens`` ("limit"), or at ``max_context`` ("ctx") (the reference's stop
reasons, src/apps/main.cpp:427-439); its pages and slot are freed in that step.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams


class RequestRefused(ValueError):
    pass


@dataclass
class Request:
    rid: int
    prompt: List[int]
    params: SamplingParams
    seed: int
    generated: List[int] = field(default_factory=list)
    num_computed: int = 0          # tokens of prompt + generated that are in the cache
    state: str = "waiting"         # waiting | running | finished
    finish_reason: Optional[str] = None
    preemptions: int = 0
    admitted_at: int = -1          # admission counter: larger = more recent

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.generated) - self.num_computed

    def span(self, start: int, n: int) -> List[int]:
        """tokens[start:start + n] without joining the two lists."""
        p = len(self.prompt)
        if start >= p:
            return self.generated[start - p:start - p + n]
        if start + n <= p:
            return self.prompt[start:start + n]
        return self.prompt[start:] + self.generated[:start + n - p]


@dataclass
class PlannedEntry:
    request: Request
    tokens: List[int]
    samples: bool  # this portion ends at the request's last token: its last logits are wanted


@dataclass
class StepPlan:
    entries: List[PlannedEntry]
    preempted: List[Request]


@dataclass
class SchedulerStats:
    steps: int = 0
    admitted: int = 0
    finished: int = 0
    preemptions: int = 0
    tokens: int = 0


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_tokens: int = 2048, max_running: Optional[int] = None,
                 chunk: Optional[int] = None, max_context: Optional[int] = None,
                 eos_token_ids: Sequence[int] = (), seed: int = 0):
        if max_batch_tokens < 1:
            raise ValueError("max_batch_tokens must be >= 1")
        if chunk is not None and chunk < 1:
            raise ValueError("chunk must be >= 1")
        self.cache = cache
        self.max_batch_tokens = max_batch_tokens
        self.max_running = min(max_running or cache.max_requests, cache.max_requests)
        self.chunk = chunk
        self.max_context = max_context
        self.eos = set(int(e) for e in eos_token_ids)
        self.seed = seed
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: Dict[int, Request] = {}
        self.stats = SchedulerStats()
        self._next_rid = 0
        self._admissions = 0

    # ------------------------------------------------------------------ submission
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> Request:
        params = params or SamplingParams()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise RequestRefused("a request needs at least one prompt token")
        most = len(prompt) + params.max_new_tokens
        if self.max_context is not None and len(prompt) >= self.max_context:
            raise RequestRefused(f"prompt of {len(prompt)} tokens does not fit max_context={self.max_context}")
        if self.max_context is not None:
            most = min(most, self.max_context)
        ps = self.cache.page_size
        # the last sampled token is never fed back, so at most `most - 1` tokens enter the cache
        need = -(-(most - 1) // ps)
        for g in self.cache.groups:
            if need > g.num_pages:
                raise RequestRefused(
                    f"request needs up to {need} pages of {ps} tokens but the pool has {g.num_pages}; "
                    f"shorten the prompt or max_new_tokens")
        rid = self._next_rid
        self._next_rid += 1
        seed = params.seed if params.seed is not None else (self.seed * 1_000_003 + rid)
        req = Request(rid, prompt, params, seed)
        self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning
    def _pages_for(self, req: Request, n: int) -> List[int]:
        if self.cache.has(req.rid):
            return self.cache.pages_needed(req.rid, n)
        return [-(-n // self.cache.page_size)] * len(self.cache.groups)

    def _fit(self, req: Request, n: int, free: List[int]) -> int:
        """Largest m <= n whose pages fit in ``free``."""
        ps = self.cache.page_size
        length = self.cache.length(req.rid) if self.cache.has(req.rid) else 0
        have = [self.cache.num_blocks(req.rid, g) for g in range(len(free))] if self.cache.has(req.rid) \
            else [0] * len(free)
        cap = min((h + f) * ps - length for h, f in zip(have, free)) if free else n
        return max(0, min(n, cap))

    def _preempt(self, req: Request) -> None:
        if self.cache.has(req.rid):
            self.cache.free_request(req.rid)
        self.running.remove(req)
        req.num_computed = 0
        req.state = "waiting"
        req.preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(req)

    def plan(self) -> StepPlan:
        """The next step.  If nothing can run although requests are running (every one of them is
        in its prompt and needs a page, and none is free), the most recently admitted one is
        preempted and the step is planned again: the oldest request always gets to finish."""
        preempted: List[Request] = []
        while True:
            entries = self._plan_once(preempted)
            if entries or not self.running:
                return StepPlan(entries, preempted)
            victim = max(self.running, key=lambda r: r.admitted_at)
            self._preempt(victim)
            preempted.append(victim)

    def _plan_once(self, preempted: List[Request]) -> List[PlannedEntry]:
        n_groups = len(self.cache.groups)
        # 1. decodes, preempting the most recent admissions until their pages exist
        while True:
            decodes = [r for r in self.running if r.remaining == 1 and r.num_computed > 0]
            need = self.cache.pages_needed_many([r.rid for r in decodes], 1) if decodes else [0] * n_groups
            free = self.cache.free_pages()
            if all(n <= f for n, f in zip(need, free)) or not self.running:
                break
            victim = max(self.running, key=lambda r: r.admitted_at)
            self._preempt(victim)
            preempted.append(victim)
        budget = self.max_batch_tokens
        entries: List[PlannedEntry] = []
        free = [f - n for f, n in zip(self.cache.free_pages(), need)]
        for r in decodes[:budget]:
            entries.append(PlannedEntry(r, r.span(r.num_computed, 1), True))
        budget -= len(entries)
        decoding = {r.rid for r in decodes}
        # 2. prompt portions of running requests
        for r in self.running:
            if r.rid in decoding or budget <= 0:
                continue
            n = min(r.remaining, budget, self.chunk or r.remaining)
            n = self._fit(r, n, free)
            if n <= 0:
                continue
            pn = self._pages_for(r, n)
            free = [f - p for f, p in zip(free, pn)]
            entries.append(PlannedEntry(r, r.span(r.num_computed, n), n == r.remaining))
            budget -= n
        # 3. admissions (a request preempted in this step waits for the next one)
        while (self.waiting and budget > 0 and len(self.running) < self.max_running
               and self.cache.slots.num_free > sum(1 for e in entries if not self.cache.has(e.request.rid))
               and self.waiting[0] not in preempted):
            r = self.waiting[0]
            n = min(r.remaining, budget, self.chunk or r.remaining)
            n = self._fit(r, n, free)
            if n <= 0:
                break
            self.waiting.popleft()
            pn = self._pages_for(r, n)
            free = [f - p for f, p in zip(free, pn)]
            r.state = "running"
            r.admitted_at = self._admissions
            self._admissions += 1
            self.stats.admitted += 1
            self.running.append(r)
            entries.append(PlannedEntry(r, r.span(0, n), n == r.remaining))
            budget -= n
        return entries

    # ------------------------------------------------------------------ after the step
    def commit(self, plan: StepPlan, sampled: Dict[int, int]) -> List[Request]:
        """``sampled``: rid -> token for every planned entry that samples.  Returns the
        requests that finished; their cache is freed here."""
        done: List[Request] = []
        self.stats.steps += 1
        for e in plan.entries:
            r = e.request
            r.num_computed += len(e.tokens)
            self.stats.tokens += len(e.tokens)
            if not e.samples:
                continue
            tok = int(sampled[r.rid])
            r.generated.append(tok)
            reason = None
            if not r.params.ignore_eos and (tok in self.eos or tok in r.params.stop_token_ids):
                reason = "eos"
            elif len(r.generated) >= r.params.max_new_tokens:
                reason = "limit"
            elif self.max_context is not None and len(r.prompt) + len(r.generated) >= self.max_context:
                reason = "ctx"
            if reason is not None:
                r.state = "finished"
                r.finish_reason = reason
                self.running.remove(r)
                if self.cache.has(r.rid):
                    self.cache.free_request(r.rid)
                self.finished[r.rid] = r
                self.stats.finished += 1
                done.append(r)
        return done
