"""Trace replay: drive the step function with given tokens, sample nothing.

A ``TraceSession`` owns a model, a cache pool made for a stated number of
tokens, and a map from request ids to cache slots.  ``run_step`` takes the
entries of one step (request id, its next tokens, the places whose logits are
wanted) and the ids that end after it.  It has no forward pass, cache or
loader of its own: it calls ``ModelRunner.step``.

The reference has nothing comparable; its dummy weights are seeded "so that it
is possible to check whether the results are correct"
(src/csrc/model/gpt/gpt_weight.cc:337-340) but nothing consumes them.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..models.registry import load_model
from .step import ModelRunner, StepEntry, StepError


class TraceSession:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16,
                 max_requests: int = 8, device: str = "cuda", max_batch_tokens: Optional[int] = None):
        self.model = load_model(model_dir, dtype, device)
        max_len = self.model.max_positions or max_tokens
        # every live request's count is rounded up to a multiple of 64 by the
        # caller; a page never straddles such a boundary when 64 % page_size == 0,
        # otherwise one spare page per request covers the rounding.
        pages = (max_tokens + page_size - 1) // page_size
        if 64 % page_size:
            pages += max_requests
        self.cache = CacheManager(self.model.definition.cache_specs(), self.model.dtype, device,
                                  page_size=page_size, num_pages=max(pages, 1), max_seqs=max_requests,
                                  max_seq_len=max_len)
        self.runner = ModelRunner(self.model, self.cache,
                                  max_batch_tokens=max_batch_tokens or max(max_tokens, 64))
        self.slots: Dict[Any, int] = {}

    def run_step(self, entries: Sequence[dict], end: Sequence[Any] = ()) -> Optional[torch.Tensor]:
        batch: List[StepEntry] = []
        for e in entries:
            rid = e["id"]
            if rid not in self.slots:
                slot = self.cache.alloc_slot()
                if slot is None:
                    raise StepError(f"more than {self.cache.max_seqs} requests are live")
                self.slots[rid] = slot
            slot = self.slots[rid]
            batch.append(StepEntry(slot, list(e["tokens"]), self.cache.lengths[slot], list(e.get("want", []))))
        logits = self.runner.step(batch) if batch else None
        for rid in end:
            if rid in self.slots:
                self.cache.free_slot(self.slots.pop(rid))
        return logits

    def check(self) -> None:
        self.runner.check_status()
        self.cache.check()
