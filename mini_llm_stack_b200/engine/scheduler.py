"""The scheduler: admits requests, cuts prompts into portions, decodes, frees.

Reference (serve/engine.py:160-267): FCFS admission of the head of the waiting
list while ``len(running) < max_batch`` and ``can_allocate(len(tokens) + 1)``
(:190-198); every admitted prompt is prefilled whole and alone (:199-206); one
slot per running request is reserved before the decode step and, when the pool
is empty, the newest running request is preempted: its pages are freed, it goes
back to the front of the waiting list and is recomputed from its tokens when
re-admitted (:208-216,236-245); a request finishes at ``max_new_tokens``, at its
eos token or at ``max_seq_len`` (:218-227).

What differs, on purpose: prompts are cut into portions under a token budget,
so one step mixes single decoded tokens with portions of prompts; a request
that finishes its prompt in a step gets its first token from that step and
decodes from the next (the reference also decodes it once in the admitting
step; the token streams are the same).

When pages run out: a running request that cannot get pages for its share of
the step makes the newest running request give up everything (possibly
itself); a request that could not even fit alone is refused at ``submit``.

The scheduler only decides; it touches the cache manager's accounting and no
tensor, so it runs and is tested without a GPU.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field

from .request import FINISHED, RUNNING, WAITING, Request


class SchedulerError(RuntimeError):
    pass


@dataclass
class Planned:
    request: Request
    n_tokens: int
    wants_logits: bool        # the portion ends at the request's last token


@dataclass
class StepPlan:
    entries: list = field(default_factory=list)
    preempted: list = field(default_factory=list)
    admitted: list = field(default_factory=list)

    @property
    def n_tokens(self) -> int:
        return sum(p.n_tokens for p in self.entries)


class Scheduler:
    def __init__(self, cache, max_batch: int, max_tokens_per_step: int, chunk_size: int,
                 max_seq_len: int):
        self.cache = cache
        self.max_batch, self.budget = int(max_batch), int(max_tokens_per_step)
        self.chunk_size, self.max_seq_len = int(chunk_size), int(max_seq_len)
        self.waiting: deque = deque()
        self.running: list = []
        self.finished: list = []
        self.preemptions = 0
        self.steps = 0

    # ------------------------------------------------------------------- submit
    def add(self, req: Request) -> None:
        n = len(req.prompt)
        if n == 0:
            raise SchedulerError("a request needs at least one prompt token")
        if n + 1 > self.max_seq_len:          # serve/engine.py:181
            raise SchedulerError(f"prompt too long: {n} tokens, the model's positions "
                                 f"end at {self.max_seq_len}")
        most = min(n + req.max_new_tokens, self.max_seq_len)
        if not self.cache.fits_at_all(most, self.chunk_size):
            raise SchedulerError(
                f"request of up to {most} tokens can never fit the cache "
                f"({self.cache.num_blocks} pages of {self.cache.block_size})")
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # --------------------------------------------------------------------- plan
    def _preempt(self, victim: Request, plan: StepPlan) -> None:
        """serve/engine.py:208-216: free everything, requeue at the front."""
        self.running.remove(victim)
        self.cache.free(victim.req_id)
        victim.state = WAITING
        victim.num_computed = 0
        victim.preemptions += 1
        self.preemptions += 1
        self.waiting.appendleft(victim)
        plan.entries = [p for p in plan.entries if p.request is not victim]
        plan.preempted.append(victim)

    def _share(self, req: Request, budget_left: int) -> int:
        return min(req.remaining, self.chunk_size, budget_left)

    def plan(self) -> StepPlan:
        """Decide this step: who runs how many tokens, who is preempted or admitted."""
        plan = StepPlan()
        budget = self.budget
        # running requests first: those that decode (one token), then those still
        # in their prompt, each in admission order
        order = ([r for r in self.running if r.remaining == 1]
                 + [r for r in self.running if r.remaining > 1])
        for req in order:
            if req.state != RUNNING:            # preempted while others were served
                continue
            n = self._share(req, budget)
            if n <= 0:
                continue
            while not self.cache.reserve(req.req_id, n):
                victim = self.running[-1]
                if victim is req and len(self.running) == 1:
                    raise SchedulerError(
                        "a single request exceeds the cache's capacity")   # :242-244
                self._preempt(victim, plan)
                if victim is req:
                    break
            if req.state != RUNNING:
                continue
            plan.entries.append(Planned(req, n, n == req.remaining))
            budget -= n
        # then admit from the head of the waiting list (FCFS, no skipping: :190-198)
        while self.waiting and len(self.running) < self.max_batch and budget > 0:
            req = self.waiting[0]
            if req in plan.preempted:
                break                            # not in the step that preempted it
            if not self.cache.can_hold(req.n_tokens + 1, self.chunk_size):
                break
            n = self._share(req, budget)
            if not self.cache.admit(req.req_id):
                break
            if not self.cache.reserve(req.req_id, n):
                self.cache.free(req.req_id)
                break
            self.waiting.popleft()
            req.state = RUNNING
            self.running.append(req)
            plan.admitted.append(req)
            plan.entries.append(Planned(req, n, n == req.remaining))
            budget -= n
        if not plan.entries and self.has_work():
            raise SchedulerError(
                "nothing can run: no waiting request fits the free pages and none "
                "is running")
        return plan

    # ------------------------------------------------------------------- commit
    def complete(self, plan: StepPlan, sampled: dict) -> list:
        """Account for a finished step.  ``sampled`` maps req_id -> token for the
        entries that wanted logits.  Returns the requests that finished."""
        done = []
        now = time.perf_counter()
        for p in plan.entries:
            req = p.request
            req.num_computed += p.n_tokens
            if not p.wants_logits:
                continue
            tok = int(sampled[req.req_id])
            req.generated.append(tok)
            if req.first_token_time is None:
                req.first_token_time = now
            if (len(req.generated) >= req.max_new_tokens                     # :219
                    or (req.eos_token is not None and tok == req.eos_token)  # :220
                    or req.n_tokens >= self.max_seq_len):                    # :221
                req.state = FINISHED
                req.finish_time = now
                self.running.remove(req)
                self.finished.append(req)
                self.cache.free(req.req_id)
                done.append(req)
        self.steps += 1
        return done
