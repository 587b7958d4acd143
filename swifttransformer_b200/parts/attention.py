"""The attention mixer: fused q|k|v projection, keys and values into the paged
cache, causal attention over the cache, output projection.

Order of operations as in the reference's ``st::layer::attention``
(src/csrc/layer/attention.cc:35-290): qkv product (102-111), bias (122-130),
K/V of the step into pages (158-177), attention (179-246), output product and
bias (255-288).  Differences: one attention formulation for every kind of
token (queries at positions start..start+n-1 read keys 0..own position from the
pages), so a prompt may arrive in portions; the scale 1/sqrt(head_dim)
(attention.cc:91) and an optional window are constructor arguments; the output
bias is handed on with the result so the next norm kernel adds it.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

from .. import ops
from ..weights.spec import MATRIX, VECTOR, ParamSpec
from .base import MIXERS, Delta, Mixer, PagedKVSpec

# requests that bring fewer new tokens than this are served token by token by
# the bandwidth-bound kernel, the others in tiles of 64 queries on tensor cores
SHORT_PORTION = 16


def paged_attention(q: torch.Tensor, cache: Any, ctx: Any, nh: int, scale: float, window: int) -> torch.Tensor:
    """Attention of the step's queries q [N, nh*d] over a paged cache view; returns [N, nh*d]."""
    out = torch.empty_like(q)
    d = cache.pool.shape[-1]
    fast = q.dtype == torch.bfloat16 and d % 16 == 0 and d <= 256
    if not fast:
        ops.attention_plain(q, cache.pool, cache.layer, out, ctx.positions, ctx.seq_of_token, ctx.slots,
                            cache.block_table, nh, scale, window)
        return out
    plan = ctx.attention_plan()
    if plan.n_tiles:
        ops.attention_prefill(q, cache.pool, cache.layer, out, plan.tiles, plan.n_tiles, ctx.q_start,
                              ctx.start_pos, ctx.slots, cache.block_table, nh, scale, window, status=ctx.status)
    if plan.n_items:
        n_splits = plan.splits(nh, d)
        nkv = cache.pool.shape[3]
        ops.attention_decode(q, cache.pool, cache.layer, out, plan.items, plan.n_items, ctx.positions,
                             ctx.seq_of_token, ctx.slots, cache.block_table, nh, scale, window,
                             n_splits, ctx.scratch_f32(ops.attention_decode_scratch(plan.n_items, nh, d, n_splits))
                             if n_splits > 1 else None,
                             warps=ops.decode_warps(plan.n_items, nkv, d, n_splits, plan.max_item_kv))
    return out


@MIXERS.register("attention")
class Attention(Mixer):
    """Multi-head / grouped-query attention over a paged cache.

    names: checkpoint prefixes of the four projections, e.g.
           {"q": "...self_attn.q_proj", "k": ..., "v": ..., "o": "...self_attn.out_proj"};
           each has ``.weight`` [out, in] and, with ``bias``, ``.bias``.
    qk_position: a position encoding that acts on queries and keys (``apply_qk(q, k, ctx)``, in place on
           [tokens, heads, head_dim] views, device operations only so that decode steps can still be recorded),
           or None.
    """

    def __init__(self, hidden: int, num_heads: int, head_dim: int, names: Dict[str, str],
                 num_kv_heads: Optional[int] = None, bias: bool = True, window: Optional[int] = None,
                 scale: Optional[float] = None, qk_position: Any = None):
        self.hidden, self.nh, self.d = hidden, num_heads, head_dim
        self.nkv = num_kv_heads or num_heads
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads cannot share {self.nkv} key/value heads")
        self.bias, self.window, self.names = bias, window, dict(names)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.qk_position = qk_position
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    def param_specs(self) -> List[ParamSpec]:
        qw, kw = self.nh * self.d, self.nkv * self.d
        specs = []
        for key, rows, cols in (("q", qw, self.hidden), ("k", kw, self.hidden), ("v", kw, self.hidden),
                                ("o", self.hidden, qw)):
            specs.append(ParamSpec(self.names[key] + ".weight", (rows, cols), MATRIX))
            if self.bias:
                specs.append(ParamSpec(self.names[key] + ".bias", (rows,), VECTOR))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_qkv = torch.cat([tensors.pop(n[k] + ".weight") for k in "qkv"], dim=0).contiguous()
        self.w_o = tensors.pop(n["o"] + ".weight")
        if self.bias:
            self.b_qkv = torch.cat([tensors.pop(n[k] + ".bias") for k in "qkv"], dim=0).contiguous()
            self.b_o = tensors.pop(n["o"] + ".bias")

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.nkv, self.d, self.window)

    def forward(self, h: torch.Tensor, ctx: Any, cache: Any) -> Delta:
        q = torch.empty((h.shape[0], self.nh * self.d), dtype=h.dtype, device=h.device)
        encode = getattr(self.qk_position, "apply_qk", None)
        if encode is not None:
            # a position encoding of queries and keys: it sees them with their bias, as [tokens, heads,
            # head_dim] views of the fused projection, changes them in place, and the keys go to the cache after
            n, qw, kw = h.shape[0], self.nh * self.d, self.nkv * self.d
            qkv = ops.linear(h, self.w_qkv, self.b_qkv)
            encode(qkv[:, :qw].view(n, self.nh, self.d), qkv[:, qw:qw + kw].view(n, self.nkv, self.d), ctx)
            ops.qkv_to_cache(qkv, None, q, cache.pool, cache.layer, ctx.positions, ctx.seq_of_token,
                             ctx.slots, cache.block_table, self.nh, self.nkv, self.d, ctx.status,
                             write_kv=cache.writable)
        elif h.dtype == torch.bfloat16 and h.shape[0] <= ops.SKINNY_MAX_ROWS and self.hidden % 8 == 0:
            # a few tokens: one weight-streaming kernel does the product, the bias and the cache write
            ops.qkv_linear_to_cache(h, self.w_qkv, self.b_qkv, q, cache.pool, cache.layer, ctx.positions,
                                    ctx.seq_of_token, ctx.slots, cache.block_table, self.nh, self.nkv, self.d,
                                    ctx.status, write_kv=cache.writable)
        else:
            qkv = ops.linear(h, self.w_qkv)
            ops.qkv_to_cache(qkv, self.b_qkv, q, cache.pool, cache.layer, ctx.positions, ctx.seq_of_token,
                             ctx.slots, cache.block_table, self.nh, self.nkv, self.d, ctx.status,
                             write_kv=cache.writable)
        o = paged_attention(q, cache, ctx, self.nh, self.scale, self.window or 0)
        return Delta(ops.linear(o, self.w_o), self.b_o)

    def param_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()
