"""The dense feed-forward: z = act(h fc1^T + b1) fc2^T + b2.

Reference: ``st::layer::ffn`` (src/csrc/layer/ffn.cc:49-126): fc1 product (71-80),
fused bias + activation (85-92), fc2 product (96-105), bias (124).  The second
bias travels with the result so the next norm kernel adds it with the residual.
"""
from __future__ import annotations

from typing import Any, Dict, List

import torch

from .. import ops
from ..weights.spec import MATRIX, VECTOR, ParamSpec
from .base import FEED_FORWARDS, Delta, FeedForward


@FEED_FORWARDS.register("dense")
class DenseFFN(FeedForward):
    def __init__(self, hidden: int, inner: int, activation: str, fc1_name: str, fc2_name: str, bias: bool = True):
        if activation not in ops.ACT_CODES:
            raise ValueError(f"activation '{activation}' is not supported ({', '.join(ops.ACT_CODES)})")
        self.hidden, self.inner, self.activation, self.bias = hidden, inner, activation, bias
        self.fc1_name, self.fc2_name = fc1_name, fc2_name
        self.w1 = self.b1 = self.w2 = self.b2 = self.b1_bf16 = None

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(self.fc1_name + ".weight", (self.inner, self.hidden), MATRIX),
                 ParamSpec(self.fc2_name + ".weight", (self.hidden, self.inner), MATRIX)]
        if self.bias:
            specs += [ParamSpec(self.fc1_name + ".bias", (self.inner,), VECTOR),
                      ParamSpec(self.fc2_name + ".bias", (self.hidden,), VECTOR)]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w1, self.w2 = tensors[self.fc1_name + ".weight"], tensors[self.fc2_name + ".weight"]
        if self.bias:
            self.b1, self.b2 = tensors[self.fc1_name + ".bias"], tensors[self.fc2_name + ".bias"]
            if self.w1.dtype == torch.bfloat16:
                # lets the library product add the bias (and apply ReLU) in its epilogue
                self.b1_bf16 = ops.lossless_bf16(self.b1)

    def forward(self, h: torch.Tensor, ctx: Any) -> Delta:
        u = ops.linear(h, self.w1, self.b1, self.activation, bias_bf16=self.b1_bf16)
        if u.shape[0] > ops.SKINNY_MAX_ROWS and ops.linear_parts_slices(u.shape[0], self.w2) > 1:
            # fc2 for this many tokens is cut over k: its slices' sums are left for the next norm kernel
            return Delta(None, self.b2, ops.linear_parts(u, self.w2))
        return Delta(ops.linear(u, self.w2), self.b2)

    def forward_into_residual(self, x: torch.Tensor, norm: Any, ctx: Any, pending: Optional[Delta] = None) -> Any:
        """x <- (x + pending) + ffn(norm(x + pending)) for a step of a few tokens: norm (which adds what is pending)
        and fc1 + bias + activation; then fc2 + bias + residual sum in one kernel, or, where that kernel would cut
        fc2 over k, the slices' sums left as a Delta for the next norm kernel to add."""
        if norm.kind not in ops.NORM_CODES or not ops.fused_norm_applies(x.shape[0], self.hidden, self.w1):
            return False
        if self.inner % 8 or (pending is not None and ops.FUSE_NORM):
            return False
        u = ops.norm_linear(x, norm.kind, norm.gamma, norm.beta, norm.eps, self.w1, self.b1, self.activation,
                            delta=pending.value if pending else None, delta_bias=pending.bias if pending else None,
                            parts=pending.parts if pending else None)
        if not ops.FUSE_NORM and ops.linear_parts_slices(x.shape[0], self.w2) > 1 and self.inner > ops.UNCUT_MAX_INNER:
            return Delta(None, self.b2, ops.linear_parts(u, self.w2))
        ops.linear_add(u, self.w2, self.b2, x)
        return True

    def param_bytes(self) -> int:
        return (self.w1.numel() + self.w2.numel()) * self.w1.element_size()
