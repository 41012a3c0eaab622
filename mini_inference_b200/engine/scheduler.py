"""Continuous batching above the step function: admission, a token budget, prompts cut into
portions, decoding, finishing and freeing.

Behaviour follows the reference's scheduler (engine/core/scheduler.py):
  * waiting requests are admitted oldest first, head of line (:124-129, :158-162), when the
    cache has pages for the whole request plus a watermark (engine/core/kv_cache.py:192-197);
  * without chunked prefill a step runs every running request's new tokens; a prompt larger
    than the budget runs only alone (:123-132);
  * with chunked prefill each step has max_batched_tokens: decoding requests first, then
    unfinished prompts, then new ones, each taking what is left (:134-166);
  * when pages run out, the NEWEST running request is preempted: its pages and state slot are
    freed, it returns to the FRONT of the queue with its tokens kept, and is recomputed from
    position 0 when re-admitted (:98-107); a victim already scheduled in this step gives its
    budget back (:148-150).
"""
from __future__ import annotations

from collections import deque
from typing import List, Tuple

from .request import RUNNING, WAITING, Request


class Scheduler:
    def __init__(self, cache, max_num_seqs: int, max_batched_tokens: int, max_model_len: int,
                 chunked_prefill: bool = False):
        self.cache = cache
        self.max_num_seqs, self.max_batched_tokens = max_num_seqs, max_batched_tokens
        self.max_model_len, self.chunked_prefill = max_model_len, chunked_prefill
        self.waiting: deque = deque()
        self.running: List[Request] = []
        # cumulative counters, names as in engine/core/scheduler.py:24-33
        self.steps = self.preemptions = self.prefill_tokens = self.decode_tokens = 0
        self.last_batch_size = self.last_step_tokens = self.max_step_tokens = 0
        self.prefill_chunks = self.mixed_steps = 0

    def add(self, req: Request) -> None:
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---------------------------------------------------------------- one step's decisions
    def schedule(self, now: float = 0.0) -> List[Tuple[Request, int, int]]:
        """[(request, start, end)]: the tokens all_ids[start:end] of each request run this step."""
        chunks = self._schedule_chunked(now) if self.chunked_prefill else self._schedule_whole(now)
        if chunks:
            self.steps += 1
            self.last_batch_size = len(chunks)
            self.last_step_tokens = sum(e - s for _, s, e in chunks)
            self.max_step_tokens = max(self.max_step_tokens, self.last_step_tokens)
            has_decode = has_prefill = False
            for req, s, e in chunks:
                if e - s == 1 and req.output_ids and e == req.total_len:
                    self.decode_tokens += 1
                    has_decode = True
                else:
                    self.prefill_tokens += e - s
                    has_prefill = True
                    if e < req.total_len:
                        self.prefill_chunks += 1
            self.mixed_steps += int(has_decode and has_prefill)
        return chunks

    def _admit(self, req: Request, now: float, token_limit=None):
        """Cache and a state slot for a waiting request; returns how many of its tokens run this
        step, or None if it does not fit (engine/core/scheduler.py:67-96)."""
        if req.total_len > self.max_model_len:
            return None
        seq = self.cache.admit(req.id, req.total_len)
        if seq is None:
            return None
        take = req.total_len if token_limit is None else min(req.total_len, token_limit)
        if not self.cache.ensure(seq, take):
            self.cache.free(seq)
            return None
        req.seq, req.num_computed = seq, 0
        self.waiting.remove(req)
        req.state = RUNNING
        if req.first_scheduled is None:
            req.first_scheduled = now
        self.running.append(req)
        return take

    def _preempt(self, req: Request) -> None:
        self.cache.free(req.seq)
        req.seq = None
        self.running.remove(req)
        req.state = WAITING
        req.num_computed = 0
        req.preemptions += 1
        self.preemptions += 1
        self.waiting.appendleft(req)

    def _schedule_whole(self, now):
        # 1. room for every running request's next token; preempt the newest if needed
        for req in list(self.running):
            if req not in self.running:
                continue
            while not self.cache.ensure(req.seq, req.total_len):
                victim = self.running[-1]
                self._preempt(victim)
                if victim is req:
                    break
        # 2. admit waiting requests while batch size, token budget and cache allow
        budget = self.max_batched_tokens - len(self.running)
        while self.waiting and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            if req.num_new_tokens() > budget and self.running:     # a long prompt may still run alone
                break
            if not self._admit(req, now):
                break
            budget -= req.num_new_tokens()
        return [(r, r.num_computed, r.total_len) for r in self.running]

    def _schedule_chunked(self, now):
        budget = self.max_batched_tokens
        scheduled = {}
        decoding = [r for r in self.running if r.num_new_tokens() == 1]
        prefilling = [r for r in self.running if r.num_new_tokens() > 1]
        for req in decoding + prefilling:
            if req not in self.running or budget <= 0:
                continue
            take = min(req.num_new_tokens(), budget)
            end = req.num_computed + take
            while not self.cache.ensure(req.seq, end):
                victim = self.running[-1]
                self._preempt(victim)
                if victim.id in scheduled:
                    _, s, e = scheduled.pop(victim.id)
                    budget += e - s
                if victim is req:
                    break
            if req not in self.running:
                continue
            scheduled[req.id] = (req, req.num_computed, end)
            budget -= take
        while self.waiting and len(self.running) < self.max_num_seqs and budget > 0:
            req = self.waiting[0]
            take = self._admit(req, now, token_limit=budget)
            if take is None:
                break
            scheduled[req.id] = (req, 0, take)
            budget -= take
        return list(scheduled.values())

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
        """Drop every running request (after a failed step) and free what they hold
        (engine/core/scheduler.py:212-219)."""
        dropped = list(self.running)
        for r in dropped:
            self.cache.free(r.seq)
            r.seq = None
        self.running = []
        return dropped

    def stats(self) -> dict:
        return {
            "scheduler": "continuous", "running": len(self.running), "waiting": len(self.waiting),
            "batch_size": self.last_batch_size, "step_tokens": self.last_step_tokens, "steps": self.steps,
            "preemptions": self.preemptions, "prefill_tokens": self.prefill_tokens,
            "decode_tokens": self.decode_tokens, "chunked_prefill": self.chunked_prefill,
            "prefill_chunks": self.prefill_chunks, "mixed_steps": self.mixed_steps,
            "max_step_tokens": self.max_step_tokens,
        }
