"""Per-request state (engine/core/request.py:10-56 in the reference)."""
from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field
from typing import List, Optional

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
_ids = itertools.count()


@dataclass
class SamplingParams:
    max_new_tokens: int = 100         # engine/core/request.py:12
    temperature: float = 0.0          # 0 = greedy (engine/core/request.py:13)
    seed: Optional[int] = None        # None: derived from the engine's seed and the request id
    ignore_eos: bool = False


@dataclass
class Request:
    prompt_ids: List[int]
    params: SamplingParams
    id: int = field(default_factory=lambda: next(_ids))
    state: str = WAITING
    output_ids: List[int] = field(default_factory=list)
    num_computed: int = 0             # tokens whose keys/values are in the cache
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    seq: object = None                # the request's hold on the cache while it runs
    arrived: float = field(default_factory=time.perf_counter)
    first_scheduled: Optional[float] = None
    first_token_at: Optional[float] = None
    finished_at: Optional[float] = None
    token_times: List[float] = field(default_factory=list)
    preemptions: int = 0

    @property
    def all_ids(self):
        """Prompt plus everything generated so far: what the model has to see."""
        return self.prompt_ids + self.output_ids

    def token_at(self, i: int) -> int:
        """all_ids[i] without building the list."""
        n = len(self.prompt_ids)
        return self.prompt_ids[i] if i < n else self.output_ids[i - n]

    @property
    def total_len(self):
        return len(self.prompt_ids) + len(self.output_ids)

    def num_new_tokens(self):
        """Tokens to feed next: the whole (re)prompt on prefill, 1 when decoding."""
        return self.total_len - self.num_computed
