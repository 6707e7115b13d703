"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

The reference's scheduler (src/paged_attention/scheduler.zig:35-258) keeps a waiting queue, a
running list and a preempted list (:39-42); admits first-come-first-served while blocks for the
whole prompt plus two are free (:97-107); flips a sequence from prefill to decode in one call
(:141-144); grows a decoding sequence by one token (:236-245); finishes it after `max_new_tokens`
(:242-244) and frees its blocks (:221-234).  When no block is free it preempts the running
sequence of lowest priority, the most recent arrival among equals, copies its blocks to the host
and restores them later (:156-219).  The driver cuts prompts into `--ubatch-size` chunks
(src/main.zig:836-837).

Here one plan per step holds, under `max_batched_tokens`: first one token for every request that
is decoding, then prompt portions of the running requests, oldest first, then newly admitted
requests while a slot and the pages of their first portion are free.  Pages are taken portion by
portion, just before the step that fills them.

When pages run out for a running request, the most recently admitted other running request is
preempted: all it holds is given back, and it returns to the front of the waiting queue to be
recomputed from its prompt and the tokens it has produced (no copy to the host; the recomputed
logits and, through the per-token random numbers, the sampled tokens are the same).  A request
that cannot be served even alone ends with the reason "out_of_pages".  A request whose prompt and
new tokens can never fit the model's positions or the pool is refused when it is added.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple

from ..cache import CacheManager
from ..sampling.sampler import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


class RequestRefused(ValueError):
    pass


@dataclass(eq=False)
class Request:
    request_id: object
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    status: str = WAITING
    computed: int = 0                 # tokens whose keys/values/state are in the cache
    arrival: int = 0
    finish_reason: Optional[str] = None
    preemptions: int = 0

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def last_token(self) -> int:
        return self.output[-1] if self.output else self.prompt[-1]

    def token_range(self, a: int, b: int) -> List[int]:
        """Tokens a..b-1 of prompt followed by output."""
        n = len(self.prompt)
        if b <= n:
            return self.prompt[a:b]
        if a >= n:
            return self.output[a - n:b - n]
        return self.prompt[a:] + self.output[:b - n]

    @property
    def remaining(self) -> int:
        """Tokens known but not yet run through the model."""
        return len(self.prompt) + len(self.output) - self.computed


@dataclass(eq=False)
class PlanEntry:
    request: Request
    tokens: List[int]
    sample: bool                      # the last of `tokens` is the request's last known token


@dataclass
class StepPlan:
    entries: List[PlanEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    failed: List[Request] = field(default_factory=list)

    @property
    def n_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_batched_tokens: int, max_model_len: int,
                 owner=None):
        """`owner` is told when a request enters or leaves the cache (`admit(id)`, `release(id)`);
        by default the cache manager itself."""
        if max_num_seqs < 1 or max_batched_tokens < 1:
            raise ValueError("max_num_seqs and max_batched_tokens should be positive")
        self.cache = cache
        self.owner = owner if owner is not None else cache
        self.max_num_seqs = min(int(max_num_seqs), cache.max_requests)
        self.max_batched_tokens = int(max_batched_tokens)
        self.max_model_len = int(max_model_len)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # in order of admission
        self._arrivals = 0
        self.n_preemptions = 0

    # ------------------------------------------------------------------ adding
    def add(self, request: Request) -> None:
        request.params.validate()
        if not request.prompt:
            raise RequestRefused("a request needs at least one prompt token")
        total = len(request.prompt) + request.params.max_new_tokens
        if total > self.max_model_len:
            raise RequestRefused(f"prompt ({len(request.prompt)}) plus new tokens ({request.params.max_new_tokens}) "
                                 f"exceed the model's length {self.max_model_len}")
        # the last new token is sampled but never run, so the cache holds at most total - 1 positions
        if total - 1 > self.cache.max_tokens_possible():
            raise RequestRefused(f"the request needs {total - 1} cached positions; the pool holds "
                                 f"{self.cache.max_tokens_possible()}")
        request.arrival = self._arrivals
        self._arrivals += 1
        request.status = WAITING
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning
    def _try_reserve(self, req: Request, n: int) -> bool:
        return self.cache.try_reserve(req.request_id, req.computed + n)

    def _preempt(self, victim: Request, plan: StepPlan) -> None:
        self.owner.release(victim.request_id)
        self.running.remove(victim)
        victim.status, victim.computed = WAITING, 0
        victim.preemptions += 1
        self.n_preemptions += 1
        self.waiting.appendleft(victim)
        plan.preempted.append(victim)
        plan.entries = [e for e in plan.entries if e.request is not victim]

    def _fail(self, req: Request, plan: StepPlan) -> None:
        self.owner.release(req.request_id)
        self.running.remove(req)
        req.status, req.finish_reason = FINISHED, "out_of_pages"
        plan.failed.append(req)

    def _reserve_or_preempt(self, req: Request, n: int, plan: StepPlan) -> bool:
        """Reserve pages for `n` more tokens of a running request, preempting the most recently
        admitted other running requests while that is needed.  False if `req` itself had to go."""
        while not self._try_reserve(req, n):
            others = [r for r in self.running if r is not req]
            if not others:
                self._fail(req, plan)
                return False
            self._preempt(others[-1], plan)
        return True

    def schedule(self) -> StepPlan:
        plan = StepPlan()
        budget = self.max_batched_tokens
        # 1. one token for every decoding request, oldest first
        planned = set()
        for req in list(self.running):
            if req.status != RUNNING or req.remaining != 1 or req.computed < len(req.prompt):
                continue
            if budget < 1:
                break
            if self._reserve_or_preempt(req, 1, plan):
                plan.entries.append(PlanEntry(req, [req.last_token], True))
                planned.add(id(req))
                budget -= 1
        # 2. prompt portions of running requests (also recomputation after a preemption)
        for req in list(self.running):
            if req.status != RUNNING or id(req) in planned:
                continue
            if budget < 1:
                break
            n = min(req.remaining, budget)
            if self._reserve_or_preempt(req, n, plan):
                plan.entries.append(PlanEntry(req, req.token_range(req.computed, req.computed + n), n == req.remaining))
                planned.add(id(req))
                budget -= n
        # 3. admissions, first come first served; never right after a preemption in the same plan
        while self.waiting and budget >= 1 and len(self.running) < self.max_num_seqs and not plan.preempted:
            req = self.waiting[0]
            if self.cache.slots.n_free < 1:
                break
            n = min(req.remaining, budget)
            self.owner.admit(req.request_id)
            if not self.cache.can_reserve(req.request_id, n):
                self.owner.release(req.request_id)
                if self.running:
                    break                       # wait until a running request finishes
                # nothing else holds pages, and still the portion does not fit
                self.waiting.popleft()
                req.status, req.finish_reason = FINISHED, "out_of_pages"
                plan.failed.append(req)
                continue
            self.cache.reserve(req.request_id, n)
            self.waiting.popleft()
            req.status, req.computed = RUNNING, 0
            self.running.append(req)
            plan.entries.append(PlanEntry(req, req.token_range(0, n), n == req.remaining))
            budget -= n
        return plan

    # ------------------------------------------------------------------ after the step
    def commit(self, plan: StepPlan, sampled: Dict[object, int]) -> List[Request]:
        """Record that the plan ran; `sampled` maps the requests that wanted a token to it.
        Returns the requests that finished (their pages and slots are already given back)."""
        finished = []
        for e in plan.entries:
            req = e.request
            req.computed += len(e.tokens)
            if not e.sample:
                continue
            tok = int(sampled[req.request_id])
            req.output.append(tok)
            p = req.params
            reason = None
            if p.eos_id is not None and tok == p.eos_id:
                reason = "eos"
            elif len(req.output) >= p.max_new_tokens:
                reason = "length"
            elif len(req.prompt) + len(req.output) >= self.max_model_len:
                reason = "model_length"
            if reason:
                req.status, req.finish_reason = FINISHED, reason
                self.owner.release(req.request_id)
                self.running.remove(req)
                finished.append(req)
        return finished
