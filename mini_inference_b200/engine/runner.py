"""The step function: a batch of (request, its next tokens) in, logits at the wanted places
out.  It runs only the tokens it is given, as one flat batch, against the cache that earlier
steps left (engine/core/model_runner.py:90-103 is the reference's forward(chunks))."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.manager import CacheManager
from ..parts.base import StepContext
from ..parts.model import DecoderModel
from .batch import BatchBuilder, StepBatch, StepEntry


class CacheFull(RuntimeError):
    pass


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, ops=None):
        if model.embedding is None:
            raise RuntimeError("the model has no weights loaded")
        if ops is None:
            from ..ops import get_ops          # fails loudly without a GPU or the extension
            ops = get_ops(model.device)
        self.model, self.cache, self.ops = model, cache, ops
        self.device, self.dtype = model.device, model.dtype
        self.vocab_size = model.spec.vocab_size
        self.builder = BatchBuilder(cache, self.device, model.step_array_hooks(), tile=getattr(ops, "prefill_tile", 64),
                                    vocab_size=self.vocab_size)
        self.builder.ops = ops
        self.last_batch: Optional[StepBatch] = None

    @torch.inference_mode()
    def step(self, entries: List[StepEntry], ensure: bool = True):
        """Returns float32 logits [wanted rows, vocab] in the order of the entries and of each
        entry's want list, or None when nothing is wanted.  With ensure=False the caller (the
        scheduler) has already secured the pages."""
        seen = set()
        for e in entries:
            if id(e.seq) in seen:
                raise ValueError(f"request {e.seq.seq_id!r} appears twice in one step")
            seen.add(id(e.seq))
            if not e.seq.alive:
                raise ValueError(f"request {e.seq.seq_id!r} holds no cache any more")
        if ensure:
            for e in entries:
                end = e.seq.num_tokens + len(e.tokens)
                if not self.cache.ensure(e.seq, end):
                    raise CacheFull(f"no pages left for request {e.seq.seq_id!r} to reach {end} tokens")
        batch = self.builder.build(entries)
        self.last_batch = batch
        logits = self.forward(batch)
        for e in entries:
            self.cache.commit(e.seq, e.seq.num_tokens + len(e.tokens))
        return logits

    def forward(self, batch: StepBatch):
        """The device work of a step whose batch is built: block-table changes first, then the model."""
        batch.apply_table_updates(self.ops)
        ctx = StepContext(self.ops, batch, self.dtype, self.device)
        return self.model.forward(ctx, self.cache.layer_caches)
