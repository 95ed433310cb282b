"""The engine: scheduler + step function + sampler behind the reference's names.

Reference: ``Engine(model, num_blocks=256, block_size=16, max_batch=16, ...)``,
``submit(prompt, max_new_tokens=32, eos_token=None) -> Request``, ``step() -> bool``,
``run_until_done(max_steps=10_000) -> {"wall_s", "generated_tokens",
"tokens_per_s", "requests"}`` (serve/engine.py:163-185,229-267).
"""

from __future__ import annotations

import time

from ..sampling.sampler import Sampler, uniform_for
from .batch import Entry
from .request import RUNNING, Request
from .runner import ModelRunner
from .scheduler import Planned, Scheduler, StepPlan


class Engine:
    def __init__(self, model, num_blocks: int = 256, block_size: int = 16, max_batch: int = 16,
                 max_tokens_per_step: int = 2048, chunk_size: int = 2048,
                 cuda_graphs: bool = True, launch_ahead: bool = True, seed: int = 0):
        self.model = model
        self.seed = int(seed)                # sampling seed of requests that bring none
        self.runner = ModelRunner(model, num_blocks=num_blocks, block_size=block_size,
                                  max_requests=max_batch, cuda_graphs=cuda_graphs)
        self.cache = self.runner.cache
        self.max_seq_len = model.config.max_seq_len
        self.scheduler = Scheduler(self.cache, max_batch, max_tokens_per_step, chunk_size,
                                   self.max_seq_len)
        self.sampler = Sampler(model.runtime, max_rows=max_batch)
        self._next_id = 0
        self._prepared = None                # (plan, arrays) of a step prepared ahead
        self.launch_ahead = launch_ahead
        self._ahead = None                   # (plan, logits) of a step already on the device
        self.step_tokens: list = []

    @classmethod
    def from_options(cls, model, options) -> "Engine":
        """An engine from an ``EngineOptions`` record (whose ``dtype``, ``kv_dtype`` and
        ``device`` must agree with how ``model`` was loaded)."""
        rt = model.runtime
        options.check_against(str(rt.act_dtype).replace("torch.", ""), rt.device)
        return cls(model, num_blocks=options.num_blocks, block_size=options.block_size,
                   max_batch=options.max_batch, max_tokens_per_step=options.max_tokens_per_step,
                   chunk_size=options.chunk_size, cuda_graphs=options.cuda_graphs,
                   launch_ahead=options.launch_ahead, seed=options.seed)

    # the reference's attribute names
    @property
    def waiting(self):
        return self.scheduler.waiting

    @property
    def running(self):
        return self.scheduler.running

    @property
    def finished(self):
        return self.scheduler.finished

    @property
    def steps(self) -> int:
        return self.scheduler.steps

    def submit(self, prompt, max_new_tokens: int = 32, eos_token=None,
               temperature: float = 0.0, seed: int | None = None) -> Request:
        req = Request(self._next_id, list(prompt), int(max_new_tokens), eos_token,
                      float(temperature), self.seed if seed is None else int(seed))
        self.scheduler.add(req)
        self._next_id += 1
        return req

    def step(self) -> bool:
        """One scheduler iteration; True while work remains (serve/engine.py:229-256).

        While the device computes a step of single decoded tokens, the host lays
        out the next step's arrays (they depend on lengths and pages, not on the
        tokens being sampled).  With ``launch_ahead`` that next step is put on the
        device at once, reading its token ids where the sampler writes them, before
        the host has read them: the device never waits for the host between steps
        of decoding.  A request that turns out to have ended with the token just
        sampled has one row in the step launched ahead, which nobody reads (a row
        does not depend on the rest of its batch).  Without ``launch_ahead`` the
        prepared step waits for the tokens and starts without planning or building
        if nothing changed meanwhile.

        The kernels' status word comes back with the sampled tokens: a kernel that
        refused its input (a token, position or slot outside its table) or gave up a
        bounded wait raises ``KernelError`` in the step that ran it (the reference
        raises inside the step too: serve/engine.py:242-244).  The lengths of that
        step are committed by then and its rows are wrong, so the engine is not to be
        used further after such an error.
        """
        if not self.scheduler.has_work():
            self._ahead = None
            return False
        plan = logits = rows = None
        if self._ahead is not None:
            ahead_plan, ahead_logits = self._ahead
            self._ahead = None
            keep = [i for i, p in enumerate(ahead_plan.entries) if p.request.state == RUNNING]
            if keep:
                plan = StepPlan(entries=[ahead_plan.entries[i] for i in keep])
                logits = ahead_logits
                if len(keep) != len(ahead_plan.entries):
                    rows = keep
        if plan is None:
            ahead = self._take_prepared()
            if ahead is not None:
                plan, prepared = ahead
                logits = self.runner.step_prepared(
                    prepared, [p.request.generated[-1] for p in plan.entries])
            else:
                plan = self.scheduler.plan()
                entries = []
                for p in plan.entries:
                    r = p.request
                    toks = r.token_slice(r.num_computed, p.n_tokens)
                    entries.append(Entry(r.req_id, toks,
                                         [p.n_tokens - 1] if p.wants_logits else []))
                logits = self.runner.step(entries)
        sampled = {}
        nxt = None
        if logits is not None:
            if rows is not None:                     # the rows of the requests still running
                logits = logits[rows].contiguous()
            wanting = [p.request for p in plan.entries if p.wants_logits]
            temps = [r.temperature for r in wanting]
            us = [uniform_for(r.seed, r.req_id, len(r.generated)) if r.temperature > 0 else 0.0
                  for r in wanting]
            n = self.sampler.launch(logits, temps, us)
            nxt = self._prepare_next(plan)          # host work under the device's
            if nxt is not None and self.launch_ahead:
                next_plan, prepared = nxt
                self._ahead = (next_plan, self.runner.step_prepared(
                    prepared, None, device_tokens=self.sampler.device_tokens(n)))
                nxt = None
            toks = self.sampler.finish(n)
            sampled = {r.req_id: t for r, t in zip(wanting, toks)}
        done = self.scheduler.complete(plan, sampled)
        self._prepared = None if done else nxt
        self.step_tokens.append(plan.n_tokens)
        return self.scheduler.has_work()

    def _prepare_next(self, plan):
        """The next step's plan and arrays, if it is bound to be one more token for
        exactly the requests of ``plan`` (none of them ends by count, nobody waits)."""
        sch = self.scheduler
        if sch.waiting or len(plan.entries) != len(sch.running) or plan.preempted:
            return None
        for p in plan.entries:
            r = p.request
            if (not p.wants_logits or len(r.generated) + 1 >= r.max_new_tokens
                    or r.n_tokens + 1 >= self.max_seq_len):
                return None
        for p in plan.entries:
            if not self.cache.reserve(p.request.req_id, 1):
                return None                          # the usual path decides who gives way
        nxt = StepPlan(entries=[Planned(p.request, 1, True) for p in plan.entries])
        prepared = self.runner.builder.prepare(
            [Entry(p.request.req_id, [0], [0]) for p in plan.entries])
        return nxt, prepared

    def _take_prepared(self):
        """The step prepared ahead, if the world is still as it was assumed."""
        ahead, self._prepared = self._prepared, None
        if ahead is None:
            return None
        plan, _ = ahead
        sch = self.scheduler
        if sch.waiting or len(sch.running) != len(plan.entries):
            return None
        for p, r in zip(plan.entries, sch.running):
            if p.request is not r or r.remaining != 1:
                return None
        return ahead

    def run_until_done(self, max_steps: int = 10_000) -> dict:
        t0 = time.perf_counter()
        start = self.scheduler.steps
        while self.step():
            if self.scheduler.steps - start >= max_steps:
                raise RuntimeError("engine exceeded max_steps")
        self.model.runtime.ops.check_status()
        wall = time.perf_counter() - t0
        toks = sum(len(r.generated) for r in self.finished)
        return {"wall_s": wall, "generated_tokens": toks,
                "tokens_per_s": toks / wall if wall > 0 else float("inf"),
                "requests": len(self.finished), "steps": self.scheduler.steps,
                "preemptions": self.scheduler.preemptions,
                "page_high_water": max((g.pool.high_water for g in self.cache.paged),
                                       default=0)}
