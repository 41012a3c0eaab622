"""Continuous batching above the step function.  Each call to schedule() makes ONE planning
pass over the running and the waiting requests and returns a StepPlan: which span of which
request runs, who was admitted, who was evicted, what is left of the token budget.

The decisions are the reference's (engine/core/scheduler.py):
  * requests wait in arrival order and are admitted head of line (:124-129, :158-162) when the
    cache has pages for the whole request plus its watermark (engine/core/kv_cache.py:192-197)
    and a state slot is free;
  * a step spends at most max_batched_tokens.  Requests that already run are served first,
    those with one pending token (decoding) before those with more (unfinished prompts, :138-140),
    then newcomers with what is left (:158-166);
  * chunked_prefill=False is the same pass with an unbounded take per request: everybody runs
    all pending tokens, a newcomer whose prompt exceeds what is left waits unless nothing
    else runs (:123-132);
  * when a request cannot get its pages, the NEWEST running request is evicted: pages and state
    slot freed, tokens kept, back to the FRONT of the queue, recomputed from position 0 later
    (:98-107).  If the evicted one already had a span in this plan, the span is dropped and its
    tokens return to the budget (:148-150).
"""
from __future__ import annotations

from collections import deque
from typing import Iterator, List, NamedTuple, Optional

from .request import Request


class Span(NamedTuple):
    """Tokens start..end-1 of a request (prompt + generated) run in one step."""
    request: Request
    start: int
    end: int

    @property
    def size(self) -> int:
        return self.end - self.start

    @property
    def completes(self) -> bool:
        """The span reaches the request's last token: the step samples its next one."""
        return self.end == self.request.total_len

    @property
    def is_decode(self) -> bool:
        """One token fed behind a non-empty cache."""
        return self.size == 1 and self.start > 0


class StepPlan:
    """The outcome of one planning pass.  Iterates as (request, start, end) in the order the
    step runs them."""

    def __init__(self, budget: int):
        self.budget = budget                     # tokens still unspent
        self.spans: List[Span] = []
        self.admitted: List[Request] = []
        self.evicted: List[Request] = []

    def give(self, req: Request, count: int) -> None:
        self.spans.append(Span(req, req.num_computed, req.num_computed + count))
        self.budget -= count

    def withdraw(self, req: Request) -> None:
        for i, span in enumerate(self.spans):
            if span.request is req:
                self.budget += span.size
                del self.spans[i]
                return

    @property
    def num_tokens(self) -> int:
        return sum(s.size for s in self.spans)

    def pure_decode(self) -> bool:
        return bool(self.spans) and all(s.is_decode for s in self.spans)

    def __iter__(self) -> Iterator[Span]:
        return iter(self.spans)

    def __len__(self) -> int:
        return len(self.spans)

    def __getitem__(self, i):
        return self.spans[i]


class Scheduler:
    def __init__(self, cache, max_num_seqs: int, max_batched_tokens: int, max_model_len: int,
                 chunked_prefill: bool = False):
        self.cache = cache
        self.max_num_seqs, self.max_batched_tokens = max_num_seqs, max_batched_tokens
        self.max_model_len, self.chunked_prefill = max_model_len, chunked_prefill
        self.waiting: deque = deque()            # arrival order; an evicted request re-enters at the left
        self.running: List[Request] = []         # admission order: the last one is the newest
        # cumulative counters under the reference's names (engine/core/scheduler.py:24-33)
        self.steps = self.preemptions = self.prefill_tokens = self.decode_tokens = 0
        self.last_batch_size = self.last_step_tokens = self.max_step_tokens = 0
        self.prefill_chunks = self.mixed_steps = 0

    def add(self, req: Request) -> None:
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---------------------------------------------------------------- planning
    def schedule(self, now: float = 0.0) -> StepPlan:
        plan = StepPlan(self.max_batched_tokens)
        bounded = self.chunked_prefill
        # requests that run already, one-token ones first (a stable sort keeps admission order within each kind)
        for req in sorted(self.running, key=lambda r: r.pending > 1):
            if req.seq is None:                          # evicted earlier in this pass
                continue
            if bounded and plan.budget <= 0:
                continue
            count = min(req.pending, plan.budget) if bounded else req.pending
            if self._grow(req, req.num_computed + count, plan):
                plan.give(req, count)
        # newcomers, head of line
        while self.waiting and len(self.running) < self.max_num_seqs:
            head = self.waiting[0]
            if bounded:
                if plan.budget <= 0:
                    break
                count = min(head.total_len, plan.budget)
            else:
                count = head.total_len
                if count > plan.budget and self.running:     # too long for what is left: it runs once it can run alone
                    break
            if not self._admit(head, count, now):
                break
            plan.admitted.append(head)
            plan.give(head, count)
        self._count(plan)
        return plan

    def _grow(self, req: Request, upto: int, plan: StepPlan) -> bool:
        """Pages for the request's positions < upto, evicting from the newest end while the pool is short.
        False when the request itself had to go."""
        while not self.cache.ensure(req.seq, upto):
            newest = self.running[-1]
            self._evict(newest, plan)
            if newest is req:
                return False
        return True

    def _evict(self, req: Request, plan: StepPlan) -> None:
        self.cache.free(req.seq)
        self.running.remove(req)
        req.evict()
        self.waiting.appendleft(req)
        self.preemptions += 1
        plan.withdraw(req)
        plan.evicted.append(req)

    def _admit(self, req: Request, first_tokens: int, now: float) -> bool:
        """A cache hold for a waiting request (engine/core/scheduler.py:67-96): the whole request must fit
        beside the watermark, and the pages of its first span are taken at once."""
        if req.total_len > self.max_model_len:
            return False
        seq = self.cache.admit(req.id, req.total_len, self.max_batched_tokens if self.chunked_prefill else None)
        if seq is None:
            return False
        if not self.cache.ensure(seq, first_tokens):
            self.cache.free(seq)
            return False
        self.waiting.popleft()
        self.running.append(req)
        req.begin(seq, now)
        return True

    def _count(self, plan: StepPlan) -> None:
        if not plan.spans:
            return
        self.steps += 1
        self.last_batch_size = len(plan.spans)
        self.last_step_tokens = plan.num_tokens
        self.max_step_tokens = max(self.max_step_tokens, self.last_step_tokens)
        decodes = 0
        for span in plan.spans:
            # a generated token being fed for the first time counts as decoding; anything else is prompt work
            if span.size == 1 and span.completes and span.request.output_ids:
                decodes += 1
            else:
                self.prefill_tokens += span.size
                self.prefill_chunks += int(not span.completes)
        self.decode_tokens += decodes
        self.mixed_steps += int(0 < decodes < len(plan.spans))

    def count_decode_step(self, n: int) -> None:
        """A decode step of the n running requests that the engine launched itself, ahead of time."""
        self.steps += 1
        self.decode_tokens += n
        self.last_batch_size = self.last_step_tokens = n
        self.max_step_tokens = max(self.max_step_tokens, n)

    # ---------------------------------------------------------------- leaving
    def finish(self, req: Request) -> None:
        self.running.remove(req)
        self.cache.free(req.seq)
        req.seq = None

    def abort_all(self) -> List[Request]:
        """After a failed step: everything that runs leaves and gives its cache back
        (engine/core/scheduler.py:212-219)."""
        gone, self.running = self.running, []
        for req in gone:
            self.cache.free(req.seq)
            req.seq = None
        return gone

    def stats(self) -> dict:
        return {
            "scheduler": "continuous", "chunked_prefill": self.chunked_prefill,
            "running": len(self.running), "waiting": len(self.waiting),
            "steps": self.steps, "batch_size": self.last_batch_size, "step_tokens": self.last_step_tokens,
            "max_step_tokens": self.max_step_tokens, "prefill_tokens": self.prefill_tokens,
            "decode_tokens": self.decode_tokens, "prefill_chunks": self.prefill_chunks,
            "mixed_steps": self.mixed_steps, "preemptions": self.preemptions,
        }
