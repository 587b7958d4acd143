"""Token embedding (with optional input projection) and the output head.

Reference: lookup + position add src/csrc/kernel/embedding.cu:16-35 called from
src/csrc/model/gpt/gpt.cc:112-145; last-token gather, output product and
argmax src/csrc/model/gpt/gpt.cc:175-221.  The input / output projections
(embedding width != hidden width) have no counterpart there: the embedding row
goes through ``project_in`` before the position row is added, and the hidden
state through ``project_out`` before the product with the (tied) table.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..weights.spec import MATRIX, TABLE, ParamSpec
from .base import Part
from .position import PositionEncoding


class Embedding(Part):
    def __init__(self, vocab: int, embed_width: int, hidden: int, table_name: str,
                 project_in_name: Optional[str] = None):
        self.vocab, self.embed_width, self.hidden = vocab, embed_width, hidden
        self.table_name, self.project_in_name = table_name, project_in_name
        self.table: Optional[torch.Tensor] = None
        self.project_in: Optional[torch.Tensor] = None
        if (embed_width != hidden) != (project_in_name is not None):
            raise ValueError("an input projection is needed exactly when the embedding width differs from the hidden width")

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(self.table_name, (self.vocab, self.embed_width), TABLE)]
        if self.project_in_name:
            specs.append(ParamSpec(self.project_in_name, (self.hidden, self.embed_width), MATRIX))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.table_name]
        if self.project_in_name:
            self.project_in = tensors[self.project_in_name]

    def forward(self, ids: torch.Tensor, positions: torch.Tensor, position: PositionEncoding) -> torch.Tensor:
        """The float32 residual stream [N, hidden] for the step's tokens."""
        n = ids.numel()
        dev = self.table.device
        x = torch.empty((n, self.hidden), dtype=torch.float32, device=dev)
        tab = position.hidden_table()
        if self.project_in is None:
            if tab is not None:
                ops.embed(ids, self.table, x, positions, tab[0], tab[1])
            else:
                ops.embed(ids, self.table, x)
            return x
        e = torch.empty((n, self.embed_width), dtype=self.table.dtype, device=dev)
        ops.embed(ids, self.table, e)
        h = ops.linear(e, self.project_in)
        if tab is not None:
            ops.add_positions(h, positions, tab[0], tab[1], x)
        else:
            x.copy_(h)
        return x

    def param_bytes(self) -> int:
        return self.project_in.numel() * self.project_in.element_size() if self.project_in is not None else 0


class OutputHead(Part):
    """logits = (project_out . h) . table^T as float32."""

    def __init__(self, vocab: int, embed_width: int, hidden: int, weight_name: str,
                 tied_to: Optional[str] = None, project_out_name: Optional[str] = None):
        self.vocab, self.embed_width, self.hidden = vocab, embed_width, hidden
        self.weight_name, self.tied_to, self.project_out_name = weight_name, tied_to, project_out_name
        self.weight: Optional[torch.Tensor] = None
        self.project_out: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(self.weight_name, (self.vocab, self.embed_width), MATRIX, tied_to=self.tied_to)]
        if self.project_out_name:
            specs.append(ParamSpec(self.project_out_name, (self.embed_width, self.hidden), MATRIX))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name]
        if self.project_out_name:
            self.project_out = tensors[self.project_out_name]

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        if self.project_out is not None:
            h = ops.linear(h, self.project_out)
        return ops.linear(h, self.weight, out_dtype=torch.float32)

    def param_bytes(self) -> int:
        b = self.weight.numel() * self.weight.element_size()
        if self.project_out is not None:
            b += self.project_out.numel() * self.project_out.element_size()
        return b
