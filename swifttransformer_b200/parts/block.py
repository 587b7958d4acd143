"""Blocks: how a mixer, a feed-forward and norms are arranged around the
residual stream.

pre_norm  (OPT with do_layer_norm_before; src/csrc/model/gpt/gpt.cc:304-503):
    r = x + mixer(norm1(x));  x' = r + ffn(norm2(r))
post_norm (do_layer_norm_before false; the reference refuses it, gpt.cc:238-240):
    r = norm1(x + mixer(x));  x' = norm2(r + ffn(r))

The residual stream is float32 for every storage type.  A block leaves the
feed-forward's result as ``pending``: the next norm kernel (of the next block
or the model's final norm) adds it, so every residual sum is one fused pass.
"""
from __future__ import annotations

import dataclasses
from typing import Any, List, Optional

import torch

from .. import ops
from .base import BLOCKS, Delta, FeedForward, Mixer, Part
from .norm import Norm


@dataclasses.dataclass
class ResidualStream:
    x: torch.Tensor                        # [N, width] float32
    act_dtype: torch.dtype
    pending: Optional[Delta] = None        # still to be added to x
    act: Optional[torch.Tensor] = None     # x in the activation dtype, when current

    def materialise(self, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x + pending in the activation dtype (all rows, folding pending into x; or only ``rows``)."""
        if rows is None and self.pending is None and self.act is not None:
            return self.act
        n = rows.numel() if rows is not None else self.x.shape[0]
        out = torch.empty((n, self.x.shape[1]), dtype=self.act_dtype, device=self.x.device)
        p = self.pending
        ops.add_norm(self.x, delta=p.value if p else None, delta_bias=p.bias if p else None,
                     parts=p.parts if p else None,
                     resid_out=self.x if (p is not None and rows is None) else None,
                     kind="none", rows=rows, out_act=out)
        if rows is None:
            self.pending, self.act = None, out
        return out


class Block(Part):
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norm1: Norm, norm2: Norm):
        self.mixer, self.feed_forward, self.norm1, self.norm2 = mixer, feed_forward, norm1, norm2

    def children(self) -> List[Part]:
        return [self.norm1, self.mixer, self.norm2, self.feed_forward]

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        raise NotImplementedError


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        # A sub-layer that can take its norm and its residual sum into its own kernels does so (steps of a
        # few tokens, where every kernel less shortens the chain); otherwise norm kernel, sub-layer, and the
        # result left pending for the next norm kernel to add.
        x, pending = stream.x, stream.pending
        low = stream.act_dtype != torch.float32
        done = self.mixer.forward_into_residual(x, self.norm1, ctx, cache, pending) if low else False
        if done is False:
            h = self.norm1.apply(x, pending, act_dtype=stream.act_dtype)
            pending = self.mixer.forward(h, ctx, cache)
        else:
            pending = None if done is True else done
        done = self.feed_forward.forward_into_residual(x, self.norm2, ctx, pending) if low else False
        if done is False:
            h = self.norm2.apply(x, pending, act_dtype=stream.act_dtype)
            pending = self.feed_forward.forward(h, ctx)
        else:
            pending = None if done is True else done
        stream.pending = pending
        stream.act = None


@BLOCKS.register("post_norm")
class PostNormBlock(Block):
    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        h = stream.materialise()
        a = self.mixer.forward(h, ctx, cache)
        h = self.norm1.apply(stream.x, a, act_dtype=stream.act_dtype, normalise_residual=True)
        f = self.feed_forward.forward(h, ctx)
        stream.act = self.norm2.apply(stream.x, f, act_dtype=stream.act_dtype, normalise_residual=True)
        stream.pending = None
