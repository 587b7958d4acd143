"""Random weights from a configuration and a seed.

Matrices, tables and vectors are N(0, std); norm gains are 1 + N(0, 0.1).
Values are rounded to bfloat16 before they are used or written, so the 32-bit
and the bfloat16 engine (and an independent implementation that reads the
written folder) work on identical numbers.  Each tensor has its own generator
seeded from (seed, index in the spec list): the values do not depend on the
order in which tensors are produced.  (A CPU and a CUDA generator give
different streams; a written folder is always generated on the CPU.)

The reference's dummy weights are uniform in +-1e-3 for every tensor
(src/csrc/model/gpt/gpt_weight.cc:329-408), which makes all logits ~0; a
normal distribution with a real scale is used here instead.
"""
from __future__ import annotations

import os
from typing import Dict, Iterable, Iterator, Tuple

import torch

from .safetensors_io import write_safetensors
from .spec import GAIN, INT_TABLE, ParamSpec

GAIN_STD = 0.1


def _one(spec: ParamSpec, index: int, seed: int, std: float, device) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed((int(seed) * 1000003 + index * 7919 + 12345) % (2 ** 63 - 1))
    if spec.role == INT_TABLE:
        return torch.randint(0, 2 ** 15, spec.shape, generator=gen, device=device, dtype=torch.int32)
    t = torch.randn(spec.shape, generator=gen, device=device, dtype=torch.float32)
    if spec.role == GAIN:
        t.mul_(GAIN_STD).add_(1.0)
    else:
        t.mul_(std)
    return t.to(torch.bfloat16)


def random_tensors(specs: Iterable[ParamSpec], seed: int, std: float = 0.02,
                   device="cpu") -> Iterator[Tuple[ParamSpec, torch.Tensor]]:
    """Yield (spec, bfloat16 or int32 tensor) for every spec that is not tied."""
    for i, s in enumerate(specs):
        if s.tied_to is not None:
            continue
        yield s, _one(s, i, seed, std, device)


def random_named_tensors(specs: Iterable[ParamSpec], seed: int, compute_dtype: torch.dtype,
                         device, std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Random parameters generated directly on ``device`` in their storage types."""
    specs = list(specs)
    out: Dict[str, torch.Tensor] = {}
    for s, t in random_tensors(specs, seed, std, device):
        out[s.name] = t.to(s.storage_dtype(compute_dtype)).contiguous()
    for s in specs:
        if s.tied_to is not None:
            out[s.name] = out[s.tied_to]
    return out


def write_random_checkpoint(model_dir: str, specs: Iterable[ParamSpec], seed: int, std: float = 0.02) -> str:
    """Write ``model.safetensors`` (bfloat16 values, int32 tables) into ``model_dir``."""
    os.makedirs(model_dir, exist_ok=True)
    path = os.path.join(model_dir, "model.safetensors")
    write_safetensors(path, ((s.name, t) for s, t in random_tensors(list(specs), seed, std, "cpu")),
                      metadata={"format": "pt", "seed": seed, "std": std})
    return path
