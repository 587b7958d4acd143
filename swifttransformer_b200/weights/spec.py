"""What a part asks of a checkpoint: tensor names, shapes and roles."""
from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

import torch

# roles decide the storage type and the random initialisation
MATRIX = "matrix"        # [out, in] weight of a matrix product: compute dtype
TABLE = "table"          # rows looked up by an integer id: compute dtype
VECTOR = "vector"        # bias / shift: always 32-bit
GAIN = "gain"            # multiplicative norm weight: always 32-bit, initialised near one
INT_TABLE = "int_table"  # integer lookup table: int32


@dataclasses.dataclass(frozen=True)
class ParamSpec:
    name: str                     # tensor name in the checkpoint
    shape: Tuple[int, ...]
    role: str = MATRIX
    # an optional tensor may be absent from the checkpoint (e.g. an output
    # matrix that is tied to the embedding table); `tied_to` names the tensor
    # whose values it then takes.
    tied_to: Optional[str] = None

    def storage_dtype(self, compute_dtype: torch.dtype, stored: Optional[torch.dtype] = None) -> torch.dtype:
        if self.role in (VECTOR, GAIN):
            return torch.float32
        if self.role == INT_TABLE:
            return torch.int32
        return compute_dtype
