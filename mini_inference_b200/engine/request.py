"""A generation request as the engine sees it: its tokens, where it stands, its hold on the
cache and the wall-clock marks of its life.

The reference keeps the same facts in one dataclass (engine/core/request.py:10-56); the
field names that callers and result files share with it are kept (prompt_ids, output_ids,
num_computed, preemptions, finish_reason).  Here the request also answers the questions the
scheduler and the step builder ask of it (how many tokens wait to be fed, which tokens a span
covers) and owns its timing figures (time to first token, time per output token, gaps)."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence


class Phase(str, enum.Enum):
    WAITING = "waiting"          # in the queue: no cache held (new, or preempted with its tokens kept)
    RUNNING = "running"          # holds pages and a state slot
    FINISHED = "finished"


WAITING, RUNNING, FINISHED = Phase.WAITING, Phase.RUNNING, Phase.FINISHED


@dataclass
class SamplingParams:
    max_new_tokens: int = 100         # engine/core/request.py:12
    temperature: float = 0.0          # 0 = greedy (engine/core/request.py:13)
    seed: Optional[int] = None        # None: derived from the engine's seed and the request id
    ignore_eos: bool = False


@dataclass
class Timeline:
    """time.perf_counter() marks; None until the event happened."""
    arrived: float = field(default_factory=time.perf_counter)
    first_scheduled: Optional[float] = None
    finished: Optional[float] = None
    tokens: List[float] = field(default_factory=list)      # one mark per delivered token

    def ttft_s(self) -> Optional[float]:
        return self.tokens[0] - self.arrived if self.tokens else None

    def tpot_ms(self) -> Optional[float]:
        n = len(self.tokens)
        return (self.tokens[-1] - self.tokens[0]) / (n - 1) * 1e3 if n > 1 else None

    def gaps_ms(self) -> List[float]:
        return [(b - a) * 1e3 for a, b in zip(self.tokens, self.tokens[1:])]

    def latency_s(self) -> Optional[float]:
        return None if self.finished is None else self.finished - self.arrived


class Request:
    _issued = 0                        # ids are handed out in arrival order

    def __init__(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None):
        self.id = Request._issued
        Request._issued += 1
        self.prompt_ids: List[int] = list(prompt_ids)
        self.output_ids: List[int] = []
        self.params = params or SamplingParams()
        self.state = Phase.WAITING
        self.num_computed = 0          # tokens whose keys/values (or state) the cache holds
        self.seq = None                # cache.SeqCache while running
        self.preemptions = 0
        self.finish_reason: Optional[str] = None
        self.error: Optional[str] = None
        self.times = Timeline()

    # ---------------------------------------------------------------- tokens
    @property
    def total_len(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def pending(self) -> int:
        """Tokens the model has not seen yet: 1 while decoding, the whole sequence after a
        preemption (what was generated is fed again behind the prompt)."""
        return self.total_len - self.num_computed

    def token_at(self, i: int) -> int:
        n = len(self.prompt_ids)
        return self.prompt_ids[i] if i < n else self.output_ids[i - n]

    def span(self, start: int, end: int) -> List[int]:
        """Tokens start..end-1 of prompt + generated, without joining the two lists."""
        n = len(self.prompt_ids)
        if end <= n:
            return self.prompt_ids[start:end]
        if start >= n:
            return self.output_ids[start - n:end - n]
        return self.prompt_ids[start:] + self.output_ids[:end - n]

    # ---------------------------------------------------------------- transitions
    def begin(self, seq, now: float) -> None:
        self.seq, self.num_computed, self.state = seq, 0, Phase.RUNNING
        if self.times.first_scheduled is None:
            self.times.first_scheduled = now

    def evict(self) -> None:
        """Loses its cache; keeps its tokens and starts again from position 0 when re-admitted."""
        self.seq, self.num_computed, self.state = None, 0, Phase.WAITING
        self.preemptions += 1

    def deliver(self, token: int, now: float) -> None:
        self.output_ids.append(token)
        self.times.tokens.append(now)

    def close(self, reason: str, error: Optional[str] = None) -> None:
        self.state, self.finish_reason, self.error = Phase.FINISHED, reason, error
        self.times.finished = time.perf_counter()

    def __repr__(self):
        return (f"Request(id={self.id}, {self.state.value}, prompt={len(self.prompt_ids)}, "
                f"generated={len(self.output_ids)}, computed={self.num_computed})")
