"""Normalisation parts.  One kernel (``ops.add_norm``) serves LayerNorm, RMS
norm and the plain residual add; statistics are float for every storage type.

LayerNorm in the reference: src/csrc/kernel/layernorm.cu:16-98 (with the fused
residual add of src/csrc/model/gpt/gpt.cc:423-436); its eps is the constant
1e-5 (src/csrc/model/gpt/gpt_weight.h:63), here a constructor argument.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..weights.spec import GAIN, VECTOR, ParamSpec
from .base import NORMS, Delta, Part


class Norm(Part):
    """y = norm(x + delta).  ``kind`` is one of ops.NORM_CODES."""

    kind = "none"

    def __init__(self, width: int, eps: float = 1e-5, affine: bool = True, prefix: str = ""):
        self.width, self.eps, self.affine, self.prefix = width, float(eps), affine, prefix
        self.gamma: Optional[torch.Tensor] = None
        self.beta: Optional[torch.Tensor] = None

    def apply(self, x: torch.Tensor, delta: Optional[Delta], *, act_dtype: torch.dtype,
              update_residual: bool = True, normalise_residual: bool = False,
              rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Return norm(x + delta) in the activation dtype.

        update_residual:    x <- x + delta            (pre-norm use)
        normalise_residual: x <- norm(x + delta)      (post-norm use; overrides the former)
        rows:               only these rows are read and produced (no residual write)
        """
        n = rows.numel() if rows is not None else x.shape[0]
        out = torch.empty((n, self.width), dtype=act_dtype, device=x.device)
        ops.add_norm(
            x,
            delta=delta.value if delta is not None else None,
            delta_bias=delta.bias if delta is not None else None,
            parts=delta.parts if delta is not None else None,
            resid_out=x if (update_residual and not normalise_residual and rows is None and delta is not None) else None,
            gamma=self.gamma, beta=self.beta, eps=self.eps, kind=self.kind, rows=rows,
            out_act=out, out_f32=x if (normalise_residual and rows is None) else None)
        return out


@NORMS.register("layernorm")
class LayerNorm(Norm):
    kind = "layernorm"

    def param_specs(self) -> List[ParamSpec]:
        if not self.affine:
            return []
        return [ParamSpec(self.prefix + ".weight", (self.width,), GAIN),
                ParamSpec(self.prefix + ".bias", (self.width,), VECTOR)]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if self.affine:
            self.gamma = tensors[self.prefix + ".weight"]
            self.beta = tensors[self.prefix + ".bias"]

    def param_bytes(self) -> int:
        return 8 * self.width if self.affine else 0


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    kind = "rmsnorm"

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.prefix + ".weight", (self.width,), GAIN)] if self.affine else []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if self.affine:
            self.gamma = tensors[self.prefix + ".weight"]

    def param_bytes(self) -> int:
        return 4 * self.width if self.affine else 0


@NORMS.register("none")
class NoNorm(Norm):
    """Residual add and cast only."""
    kind = "none"
