"""Choosing the next token from float32 logits.

The reference picks greedily only (src/csrc/model/gpt/gpt.cc:205-210, kernel
src/csrc/kernel/findmax.cu:15-39, with a TODO for anything else at gpt.cc:628-629).
Here: greedy (temperature 0; ties -> lowest id), temperature, and top-k.  The
random number of a draw depends on (seed of the request, index of the output
token) only, so a request's tokens do not depend on what else is scheduled
with it, and a request that is preempted and recomputed continues its stream.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence

import torch

from .. import ops


@dataclasses.dataclass
class SamplingParams:
    temperature: float = 0.0          # 0: greedy
    top_k: int = 0                    # 0: all ids
    seed: int = 0
    max_new_tokens: int = 128         # the reference's MAX_DECODING_STEP (src/examples/run_gpt.cc:24)
    eos_id: Optional[int] = None      # the reference's END_TOKEN (src/examples/run_gpt.cc:23)
    ignore_eos: bool = False

    def validate(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")


class Sampler:
    """Batches the per-request sampling parameters and calls the kernels."""

    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int]) -> List[int]:
        """One token per row of ``logits``; ``counters[r]`` is the index of the output token being drawn."""
        return self.sample_on_device(logits, params, counters).tolist()

    def sample_on_device(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                         counters: Sequence[int]) -> torch.Tensor:
        """The same, left on the device as int32 [rows]: nothing waits for the GPU."""
        if logits.shape[0] != len(params):
            raise ValueError("one set of sampling parameters per row of logits")
        if all(p.temperature <= 0 for p in params):
            return ops.argmax(logits)
        temps = torch.tensor([p.temperature for p in params], dtype=torch.float32, device=self.device)
        topk = torch.tensor([p.top_k for p in params], dtype=torch.int32, device=self.device)
        seeds = torch.tensor([p.seed for p in params], dtype=torch.int64, device=self.device)
        ctrs = torch.tensor(list(counters), dtype=torch.int64, device=self.device)
        return ops.sample(logits, temps, topk, seeds, ctrs)
