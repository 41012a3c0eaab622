"""The flat, unpadded batch of one step.

The reference builds a BatchMetadata per step (engine/core/model_runner.py:11-57): token
ids, positions and cache write positions of every fed token, a list of prompt portions and
a list of decode rows with their page tables.  The same facts are laid out here as int32
arrays in ONE host buffer that reaches the device in one copy:

  per token    token_ids, positions, token_seg (which entry it belongs to),
               per cache group: slots (page * page_size + offset it is written to)
  per entry    seg_q_start (S+1 prefix sums), seg_pos0 (position of its first fed token),
               seg_kv_len (keys it sees at its last token), seg_slot (state slot),
               per cache group: block_table [S, pages] by page index (0 = no page)
  work lists   decode_segs (entries that feed one token), prefill_tiles (entry, first row)
               for every tile of `tile` rows of the longer entries (prefill_tiles2: 2 * tile rows)
  logit_rows   flat rows whose logits are wanted

Only wanted rows reach the final norm and the head; the reference computes a row per chunk
and drops those of unfinished prompts (engine/custom_engine.py:139,155-157)."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch


class StepEntry:
    """A request's next tokens.  want: indices among these tokens whose logits are wanted."""
    __slots__ = ("seq", "tokens", "want")

    def __init__(self, seq, tokens: Sequence[int], want: Sequence[int] = ()):
        self.seq, self.tokens, self.want = seq, list(tokens), list(want)
        if not self.tokens:
            raise ValueError("a step entry needs at least one token")
        for w in self.want:
            if not 0 <= w < len(self.tokens):
                raise ValueError(f"want index {w} outside the entry's {len(self.tokens)} tokens")


class GroupMeta:
    """Attention's view of the step for one cache group (shared arrays plus the group's own)."""
    def __init__(self, batch, page_size, slots, block_table, max_pages):
        self.batch, self.page_size = batch, page_size
        self.slots, self.block_table, self.max_pages = slots, block_table, max_pages

    def __getattr__(self, name):              # shared per-step arrays live on the batch
        return getattr(self.batch, name)


class StepBatch:
    def __init__(self, entries: List[StepEntry], cache, device, tile: int = 64, vocab_size: int = None):
        self.entries = entries
        self.device = torch.device(device)
        S = len(entries)
        lens = [len(e.tokens) for e in entries]
        pos0 = [e.seq.num_tokens for e in entries]
        T = sum(lens)
        self.num_tokens, self.num_segs, self.tile = T, S, tile
        q_start = np.zeros(S + 1, dtype=np.int32)
        np.cumsum(lens, out=q_start[1:])
        kv_len = [p + n for p, n in zip(pos0, lens)]
        self.max_kv_len = max(kv_len)
        self.max_q_len = max(lens)

        ids = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=T)
        if vocab_size is not None and T and (ids.min() < 0 or ids.max() >= vocab_size):
            raise ValueError(f"token id outside [0, {vocab_size})")
        positions = np.concatenate([np.arange(p, p + n, dtype=np.int32) for p, n in zip(pos0, lens)])
        token_seg = np.repeat(np.arange(S, dtype=np.int32), lens)
        decode = [i for i, n in enumerate(lens) if n == 1]
        tiles = [(i, r) for i, n in enumerate(lens) if n > 1 for r in range(0, n, tile)]
        tiles2 = [(i, r) for i, n in enumerate(lens) if n > 1 for r in range(0, n, 2 * tile)]
        rows = [int(q_start[i]) + w for i, e in enumerate(entries) for w in e.want]
        self.num_decode, self.num_prefill_tiles, self.num_logit_rows = len(decode), len(tiles), len(rows)
        self.host = {"seg_q_start": q_start, "seg_pos0": np.asarray(pos0, dtype=np.int32),
                     "seg_kv_len": np.asarray(kv_len, dtype=np.int32), "decode_segs": decode,
                     "prefill_tiles": tiles, "positions": positions,
                     "seg_slot": [e.seq.slot for e in entries]}

        parts = {
            "token_ids": ids.astype(np.int32), "positions": positions, "token_seg": token_seg,
            "seg_q_start": q_start, "seg_pos0": self.host["seg_pos0"], "seg_kv_len": self.host["seg_kv_len"],
            "seg_slot": np.asarray([e.seq.slot for e in entries], dtype=np.int32),
            "decode_segs": np.asarray(decode, dtype=np.int32),
            "prefill_tiles": np.asarray(tiles, dtype=np.int32).reshape(-1),
            "prefill_tiles2": np.asarray(tiles2, dtype=np.int32).reshape(-1),
            "logit_rows": np.asarray(rows, dtype=np.int32),
        }
        seqs = [e.seq for e in entries]
        max_pages = max(1, cache.pages_for(self.max_kv_len))
        for gi in range(len(cache.kv_groups)):
            parts[f"slots{gi}"] = np.concatenate(
                [cache.slots_for(gi, e.seq, p, p + n) for e, p, n in zip(entries, pos0, lens)])
            parts[f"table{gi}"] = np.ascontiguousarray(cache.table_rows(gi, seqs, max_pages)).reshape(-1)

        # one buffer, every array starting on a 16-byte boundary, one copy to the device
        offsets, total = {}, 0
        for k, a in parts.items():
            offsets[k] = total
            total += (a.size + 3) // 4 * 4
        buf = np.zeros(max(total, 4), dtype=np.int32)
        for k, a in parts.items():
            buf[offsets[k]:offsets[k] + a.size] = a
        host = torch.from_numpy(buf)
        if self.device.type == "cuda":
            host = host.pin_memory()
        dev = host.to(self.device, non_blocking=True)
        self._host_buffer = host                     # keeps the pinned memory alive until the copy ran
        self.h2d_bytes = buf.nbytes

        def view(k):
            return dev[offsets[k]:offsets[k] + parts[k].size]
        for k in ("token_ids", "positions", "token_seg", "seg_q_start", "seg_pos0", "seg_kv_len",
                  "seg_slot", "decode_segs", "logit_rows"):
            setattr(self, k, view(k))
        self.prefill_tiles = view("prefill_tiles").view(-1, 2)
        self.prefill_tiles2 = view("prefill_tiles2").view(-1, 2)          # the same rows in tiles twice as tall
        self.num_prefill_tiles2 = len(tiles2)
        self.groups = [GroupMeta(self, cache.page_size, view(f"slots{gi}"),
                                 view(f"table{gi}").view(S, max_pages), max_pages)
                       for gi in range(len(cache.kv_groups))]
