"""Position encodings.

``LearnedPositions`` is OPT's: a table row per position, added to the token
embedding, stored with ``offset`` unused leading rows (the reference strips
them offline, scripts/lib/converter_lib.py:271, and adds the row in the
embedding kernel, src/csrc/kernel/embedding.cu:25-33).

An encoding that acts on queries and keys instead (rotary and the like) would
implement ``apply_qk``; the attention mixer calls it, when present, before the
keys go to the cache.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..weights.spec import TABLE, ParamSpec
from .base import POSITION_ENCODINGS, Part


class PositionEncoding(Part):
    def hidden_table(self) -> Optional[Tuple[torch.Tensor, int]]:
        """(table, offset) if this encoding is a row added to the hidden state, else None."""
        return None

    def max_positions(self) -> Optional[int]:
        return None

    # encodings of queries / keys override this: apply_qk(q, k, ctx) changes q [N, heads, head_dim] and
    # k [N, kv_heads, head_dim] in place (ctx.positions holds each token's position; -1 marks padding rows)
    apply_qk = None


@POSITION_ENCODINGS.register("none")
class NoPositions(PositionEncoding):
    def __init__(self, **_):
        pass


@POSITION_ENCODINGS.register("learned")
class LearnedPositions(PositionEncoding):
    def __init__(self, max_positions: int, width: int, offset: int, name: str):
        self._max, self.width, self.offset, self.name = max_positions, width, offset, name
        self.table: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.name, (self._max + self.offset, self.width), TABLE)]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.name]

    def hidden_table(self):
        return self.table, self.offset

    def max_positions(self) -> int:
        return self._max

    def add_to(self, x: torch.Tensor, positions: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        return ops.add_positions(x, positions, self.table, self.offset, out)
