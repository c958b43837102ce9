"""Continuous batching: which requests run in the next step, and with how many tokens.

Every live request has tokens that are not in the cache yet: the rest of its prompt, or
the one token sampled last.  A step takes, under a budget of `max_tokens_per_step`
tokens: first the requests with a single pending token (decoding), oldest first; then
the pending prompt portions of running requests, oldest first, cut to the budget; then
new requests from the queue (first come, first served) while a state slot is free, the
budget is not used up and the pool could hold the whole prompt.  The logits of an
entry's last token are asked for only if the entry reaches the end of what is known of
the sequence; the token sampled there is the next pending token.

When pages run out: a prompt portion is cut to the pages that are free (or waits); a
decoding request that needs a page which is not there preempts the youngest running
request - its pages and slot are given back, it returns to the front of the queue, and
it is later run again over its prompt and the tokens it had generated (recomputation;
with prefix reuse most of it is a cache hit).  A request that could never fit
(prompt + max_new_tokens beyond the pool or max_model_len) is refused when it is added.
The reference never gets there: it refuses any pool smaller than the worst case
(jllm/engine/engine.py:85-94); its order of work is admit, prefill, decode
(jllm/engine/engine.py:161-168).
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass

from ..cache import CacheManager
from .request import EngineStats, Request


@dataclass
class Scheduled:
    request: Request
    tokens: list
    wants_logits: bool


class Scheduler:
    def __init__(self, cache: CacheManager, max_tokens_per_step: int, max_model_len: int, prompt_limit: int,
                 stats: EngineStats | None = None):
        self.cache = cache
        self.max_tokens_per_step, self.max_model_len, self.prompt_limit = max_tokens_per_step, max_model_len, prompt_limit
        self.waiting: deque = deque()
        self.running: list = []            # in order of admission
        self.stats = stats or EngineStats()
        self.version = 0                   # changes whenever the set of waiting or running requests does

    # --------------------------------------------------------------------- intake
    def validate(self, prompt_ids, sampling) -> None:
        if len(prompt_ids) < 1:
            raise ValueError("empty prompt")
        if len(prompt_ids) > self.prompt_limit:
            raise ValueError(f"the prompt has {len(prompt_ids)} tokens; the longest accepted (max_prefill_len) is "
                             f"{self.prompt_limit}")
        total = len(prompt_ids) + sampling.max_new_tokens
        if total > self.max_model_len:
            raise ValueError(f"{len(prompt_ids)} prompt tokens and {sampling.max_new_tokens} new ones make {total}; "
                             f"max_model_len is {self.max_model_len}")
        pages = -(-total // self.cache.page_size)
        if self.cache.groups and pages > self.cache.num_pages:
            raise ValueError(f"prompt+max_new needs {pages} pages, the pool has {self.cache.num_pages}")

    def add(self, request: Request) -> None:
        self.validate(request.prompt_ids, request.sampling)
        self.waiting.append(request)
        self.version += 1

    def has_work(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    # ------------------------------------------------------------------- planning
    def _preempt(self, victim: Request) -> None:
        self.version += 1
        self.cache.release(victim.request_id)
        self.running.remove(victim)
        victim.slot = None
        victim.preemptions += 1
        self.waiting.appendleft(victim)
        self.stats.preemptions += 1

    def _pending(self, req: Request) -> int:
        return len(req.prompt_ids) + len(req.output_ids) - self.cache.live[req.request_id].num_tokens

    def schedule(self) -> list:
        """Plans one step and allocates its pages.  Returns the entries, oldest request first
        within each class (decoding, then prompt portions, then new requests)."""
        self.stats.scheduler_loops += 1
        for _ in range(self.cache.max_live + 2):
            plan = self._plan()
            if plan or not self.running:
                return plan
            # nothing can move although requests are running: they hold pages that none of them can
            # complete with.  Free the youngest and plan again.
            if len(self.running) == 1 and not self.waiting:
                raise MemoryError("the only running request cannot get the pages it needs")
            self._preempt(self.running[-1])
        return []

    def _plan(self) -> list:
        budget = self.max_tokens_per_step
        plan: list = []
        cache = self.cache
        # 1. decoding requests
        for req in list(self.running):
            if req not in self.running or budget == 0:
                continue
            if self._pending(req) != 1:
                continue
            rc = cache.live[req.request_id]
            preempted_self = False
            while not cache.can_grow(rc, rc.num_tokens + 1):
                victim = self.running[-1]
                if victim is req and len(self.running) == 1:
                    raise MemoryError("a single request ran out of pages")
                self._preempt(victim)
                if victim is req:
                    preempted_self = True
                    break
            if preempted_self:
                continue
            cache.grow(rc, rc.num_tokens + 1)
            plan.append(Scheduled(req, [req.tokens[-1]], True))
            budget -= 1
        # 2. prompt portions of running requests
        for req in self.running:
            if budget == 0:
                break
            pending = self._pending(req)
            if pending <= 1:
                continue
            budget -= self._take_portion(req, budget, plan)
        # 3. new requests
        while self.waiting and budget > 0 and cache.can_admit():
            req = self.waiting[0]
            toks = req.tokens
            rc = cache.admit(req.request_id, toks)
            if not cache.can_grow(rc, len(toks) + 1 if len(toks) + 1 <= self.max_model_len else len(toks)):
                cache.release(req.request_id)
                break
            self.waiting.popleft()
            self.running.append(req)
            self.version += 1
            req.slot = rc.slot
            self.stats.admissions += 1
            self.stats.cache_hit_blocks += len(rc.hashes)
            self.stats.cache_hit_tokens += rc.num_tokens
            budget -= self._take_portion(req, budget, plan)
        return plan

    def _take_portion(self, req: Request, budget: int, plan: list) -> int:
        cache = self.cache
        rc = cache.live[req.request_id]
        toks = req.tokens
        pending = len(toks) - rc.num_tokens
        n = min(pending, budget, cache.max_len_allocatable(rc) - rc.num_tokens)
        if n <= 0:
            return 0
        cache.grow(rc, rc.num_tokens + n)
        plan.append(Scheduled(req, toks[rc.num_tokens:rc.num_tokens + n], n == pending))
        return n

    # ------------------------------------------------------------------ after a step
    def committed(self, plan: list) -> None:
        """The step that runs `plan` has been issued: its tokens are in the cache."""
        for s in plan:
            self.cache.commit(self.cache.live[s.request.request_id], s.tokens)
            if len(s.tokens) == 1:
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += len(s.tokens)

    def plan_ahead(self, plan: list):
        """While the device runs `plan` (already committed): the plan of the next step if that is sure to be
        one more token for every running request - nobody waits, all of them are decoding and the pages are
        there without taking any from another.  The tokens are not known yet (`tokens` is None); `take_ahead`
        fills them in.  Returns None when the next step has to be planned in the ordinary way."""
        if self.waiting or len(plan) != len(self.running):
            return None
        for s, req in zip(plan, self.running):
            if s.request is not req or not s.wants_logits:
                return None
        cache = self.cache
        for req in self.running:
            rc = cache.live[req.request_id]
            if rc.num_tokens + 1 > self.max_model_len or not cache.can_grow(rc, rc.num_tokens + 1):
                return None                # pages grown so far stay: the ordinary plan would grow them too
            cache.grow(rc, rc.num_tokens + 1)
        return (self.version, [Scheduled(req, None, True) for req in self.running])

    def take_ahead(self, ahead):
        """The plan made by `plan_ahead`, with each request's newest token, if nothing has changed since
        (no request came, finished or was preempted) and every request has exactly that one token pending."""
        if ahead is None or ahead[0] != self.version or self.waiting:
            return None
        plan = ahead[1]
        for s in plan:
            if s.request.finished or self._pending(s.request) != 1:
                return None
            s.tokens = [s.request.output_ids[-1]]        # pending == 1: the token sampled last
        self.stats.scheduler_loops += 1
        return plan

    def finish(self, req: Request) -> None:
        self.version += 1
        req.finished = True
        req.slot = None
        self.cache.release(req.request_id)
        self.running.remove(req)
        self.stats.finished += 1
