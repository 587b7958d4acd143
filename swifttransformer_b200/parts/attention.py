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
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

from .. import ops
from ..weights.spec import MATRIX, VECTOR, ParamSpec
from .base import MIXERS, Delta, Mixer, PagedKVSpec, StepPlan

# requests that bring fewer new tokens than this are served token by token by
# the bandwidth-bound kernel, the others in tiles of queries on tensor cores
SHORT_PORTION = 16

# Keys one block of the single-token attention walks alone before the key range is cut into parts (for head
# sizes up to 64, where a block has eight warps; half of it beyond).  Recorded steps are keyed by the number
# of such spans the longest single-token request needs, so the cut follows the real lengths, not the
# longest possible one.
KEYS_PER_BLOCK = 768
# (token, head) pairs from which a launch of the single-token attention fills the device by itself: the key
# ranges are then never cut (for head size 64; in proportion for others)
FULL_LAUNCH_PAIRS = 250


def choose_splits(n_items: int, nh: int, max_kv: int, sms: int, head_dim: int = 64) -> int:
    """Parts the key range of a single-token query is cut into: one while the launch fills the device or the
    range is short (cutting costs a merge through global memory), else about KEYS_PER_BLOCK keys per part
    for head sizes up to 64 and at least 128 keys per part beyond, within two blocks per SM (measured on
    OPT-1.3B and OPT-6.7B decode steps: one part is best whenever the launch fills the device)."""
    blocks = max(1, n_items * nh)
    if blocks * 64 >= FULL_LAUNCH_PAIRS * head_dim:
        return 1
    room = max(1, (2 * sms + blocks - 1) // blocks)
    if head_dim <= 64:
        want = (max_kv + KEYS_PER_BLOCK - 1) // KEYS_PER_BLOCK
    else:
        want = max(1, max_kv // 128)
    return max(1, min(want, room, 32))


class AttentionStepView:
    """Which of the step's tokens go to which attention kernel (bfloat16 path): ``items`` lists the tokens
    served one by one (-1: none), ``tiles`` pairs of (request, offset of a tile of query rows among its new
    tokens); ``max_item_kv`` bounds the keys a single token reads."""

    def __init__(self, items, n_items, tiles, n_tiles, max_item_kv):
        self.items, self.n_items, self.tiles, self.n_tiles = items, n_items, tiles, n_tiles
        self.max_item_kv = max_item_kv

    def splits(self, nh: int, head_dim: int = 64) -> int:
        dev = self.items.device if self.items is not None else None
        return choose_splits(self.n_items, nh, self.max_item_kv, ops.sm_count(dev), head_dim)


class PagedAttentionPlan(StepPlan):
    """The step's tokens sorted for the paged attention kernels: short portions token by token, long ones in
    tiles of ``tile_rows`` queries, the tile with the longest key range first."""

    name = "paged_attention"
    PAD_TILE_OFFSET = 1 << 24          # a tile offset past any request's tokens: its block leaves at once

    def __init__(self):
        self.tile_rows = ops.attention_prefill_tile_rows()
        self.token_multiple = self.tile_rows

    def _tile_cap(self, n_cap: int, b_cap: int) -> int:
        return (n_cap + self.tile_rows - 1) // self.tile_rows + b_cap

    def words(self, n_cap: int, b_cap: int) -> int:
        return n_cap + 2 * self._tile_cap(n_cap, b_cap)

    def shape_key(self, lens, start, n_cap: int, b_cap: int) -> Tuple:
        short = lens < SHORT_PORTION
        n_items = int(lens[short].sum())
        item_kv = int((start + lens)[short].max()) if n_items else 0
        i_pad = min(-(-n_items // 16) * 16, n_cap)
        t_pad = 0 if bool(short.all()) else self._tile_cap(n_cap, b_cap)
        return (i_pad, t_pad, max(-(-item_kv // KEYS_PER_BLOCK), 1) * KEYS_PER_BLOCK)

    def fill(self, lens, q_start, start, out, n_cap: int, b_cap: int) -> Tuple:
        short = lens < SHORT_PORTION
        tiles: List[tuple] = []
        if bool(short.all()):
            n_items = int(q_start[-1])
            out[:n_items] = np.arange(n_items, dtype=np.int32)
        else:
            items: List[int] = []
            tr = self.tile_rows
            for i in range(len(lens)):
                n, s = int(lens[i]), int(start[i])
                if short[i]:
                    items.extend(range(int(q_start[i]), int(q_start[i + 1])))
                else:
                    tiles.extend((s + min(off + tr, n), i, off) for off in range(0, n, tr))
            tiles.sort(reverse=True)
            n_items = len(items)
            out[:n_items] = items
        out[n_items:n_cap] = -1
        t = out[n_cap:]
        k = 2 * len(tiles)
        t[0:k:2] = [x[1] for x in tiles]
        t[1:k:2] = [x[2] for x in tiles]
        t[k::2] = 0
        t[k + 1::2] = self.PAD_TILE_OFFSET
        item_kv = int((start + lens)[short].max()) if n_items else 0
        return (n_items, len(tiles), max(item_kv, 1))

    def view(self, dev: torch.Tensor, key: Tuple, n_cap: int, b_cap: int) -> AttentionStepView:
        n_items, n_tiles, max_kv = key
        return AttentionStepView(dev[:n_items], n_items, dev[n_cap:], n_tiles, max_kv)


def paged_attention(q: torch.Tensor, cache: Any, ctx: Any, nh: int, scale: float, window: int) -> torch.Tensor:
    """Attention of the step's queries q [N, nh*d] over a paged cache view; returns [N, nh*d]."""
    out = torch.empty_like(q)
    d = cache.pool.shape[-1]
    fast = q.dtype == torch.bfloat16 and d % 16 == 0 and d <= 256
    if not fast:
        ops.attention_plain(q, cache.pool, cache.layer, out, ctx.positions, ctx.seq_of_token, ctx.slots,
                            cache.block_table, nh, scale, window, status=ctx.status)
        return out
    plan = ctx.plan(PagedAttentionPlan.name)
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
                             warps=ops.decode_warps(plan.n_items, nkv, d, n_splits, plan.max_item_kv),
                             status=ctx.status, start_pos=ctx.start_pos)
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
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.b_qkv_bf16 = None

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
            if self.w_qkv.dtype == torch.bfloat16:
                # lets the library product add the bias in its epilogue when that is exact
                self.b_qkv_bf16 = ops.lossless_bf16(self.b_qkv)

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.nkv, self.d, self.window)

    def step_plan(self) -> StepPlan:
        return PagedAttentionPlan()

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
        elif self._queries_in_place(h, ctx):
            # a step of tiles only (prompt portions): the library product adds the bias in its epilogue, keys
            # and values are scattered into their pages, and the tile kernel reads the queries where the
            # product left them, with the row's stride: no pass that copies the queries, none that adds the bias
            qkv = ops.linear(h, self.w_qkv, self.b_qkv, bias_bf16=self.b_qkv_bf16)
            ops.qkv_to_cache(qkv, None, None, cache.pool, cache.layer, ctx.positions, ctx.seq_of_token,
                             ctx.slots, cache.block_table, self.nh, self.nkv, self.d, ctx.status,
                             write_kv=cache.writable)
            plan = ctx.plan(PagedAttentionPlan.name)
            o = torch.empty((h.shape[0], self.nh * self.d), dtype=h.dtype, device=h.device)
            ops.attention_prefill(qkv, cache.pool, cache.layer, o, plan.tiles, plan.n_tiles, ctx.q_start,
                                  ctx.start_pos, ctx.slots, cache.block_table, self.nh, self.scale, self.window or 0,
                                  status=ctx.status, q_stride=qkv.shape[1])
            return self._project(o)
        elif self._decode_from_projection(h, ctx, cache):
            # single tokens only, more of them than the weight-streaming product serves: the library product adds
            # the bias in its epilogue, and the attention kernel takes the product as it is, writes each token's
            # key and value into its page and attends: no cache-write kernel
            qkv = ops.linear(h, self.w_qkv, self.b_qkv, bias_bf16=self.b_qkv_bf16)
            plan = ctx.plan(PagedAttentionPlan.name)
            n_splits = plan.splits(self.nh, self.d)
            o = torch.empty((h.shape[0], self.nh * self.d), dtype=h.dtype, device=h.device)
            ops.attention_decode_qkv(qkv, cache.pool, cache.layer, o, plan.items,
                                     plan.n_items, ctx.positions, ctx.seq_of_token, ctx.slots, ctx.start_pos,
                                     cache.block_table, self.nh, self.scale, self.window or 0, n_splits,
                                     ctx.scratch_f32(ops.attention_decode_scratch(plan.n_items, self.nh, self.d, n_splits))
                                     if n_splits > 1 else None,
                                     warps=ops.decode_warps(plan.n_items, self.nkv, self.d, n_splits, plan.max_item_kv),
                                     status=ctx.status)
            return self._project(o)
        else:
            qkv = ops.linear(h, self.w_qkv)
            ops.qkv_to_cache(qkv, self.b_qkv, q, cache.pool, cache.layer, ctx.positions, ctx.seq_of_token,
                             ctx.slots, cache.block_table, self.nh, self.nkv, self.d, ctx.status,
                             write_kv=cache.writable)
        o = paged_attention(q, cache, ctx, self.nh, self.scale, self.window or 0)
        return self._project(o)

    def _project(self, o: torch.Tensor) -> Delta:
        """The output projection, left for the next norm kernel to add: as one matrix, or, where the product for
        this many tokens is cut over k, as its slices' sums."""
        if o.shape[0] > ops.SKINNY_MAX_ROWS and ops.linear_parts_slices(o.shape[0], self.w_o) > 1:
            return Delta(None, self.b_o, ops.linear_parts(o, self.w_o))
        return Delta(ops.linear(o, self.w_o), self.b_o)

    def _decode_from_projection(self, h: torch.Tensor, ctx: Any, cache: Any) -> bool:
        """Whether this step's attention can work from the fused projection itself: every token of the step stands
        alone (no prompt tiles, whose kernel reads this step's keys from the cache), the layer writes its own cache,
        the product's epilogue adds the bias exactly (or there is none), and the kernel takes the sizes."""
        if not (ops.DECODE_FROM_PROJECTION and cache.writable) or (self.bias and self.b_qkv_bf16 is None):
            return False
        plan = ctx.plan(PagedAttentionPlan.name)
        if plan.n_tiles or not plan.n_items:
            return False
        return ops.attention_decode_qkv_applies(h, cache.pool, plan.n_items, self.nh, plan.splits(self.nh, self.d))

    def _queries_in_place(self, h: torch.Tensor, ctx: Any) -> bool:
        """Whether this step can leave the queries in the fused product: bfloat16, a head size the tile kernels
        take, every token of the step in a tile, and a bias the product's epilogue adds exactly (or none)."""
        if h.dtype != torch.bfloat16 or self.d % 16 or self.d > 256:
            return False
        if self.bias and self.b_qkv_bf16 is None:
            return False
        plan = ctx.plan(PagedAttentionPlan.name)
        return plan.n_items == 0 and plan.n_tiles > 0

    def forward_into_residual(self, x: torch.Tensor, norm: Any, ctx: Any, cache: Any,
                              pending: Optional[Delta] = None) -> Any:
        """x <- (x + pending) + attention(norm(x + pending)) for a step of a few tokens in three or four kernels: norm
        (which adds what is pending) and q|k|v product + bias + cache write; attention; output product + bias +
        residual sum."""
        if getattr(self.qk_position, "apply_qk", None) is not None or norm.kind not in ops.NORM_CODES:
            return False
        if not ops.fused_norm_applies(x.shape[0], self.hidden, self.w_qkv) or (pending is not None and ops.FUSE_NORM):
            return False
        q = torch.empty((x.shape[0], self.nh * self.d), dtype=self.w_qkv.dtype, device=x.device)
        ops.norm_qkv_linear_to_cache(x, norm.kind, norm.gamma, norm.beta, norm.eps, self.w_qkv, self.b_qkv, q,
                                     cache.pool, cache.layer, ctx.positions, ctx.seq_of_token, ctx.slots,
                                     cache.block_table, self.nh, self.nkv, self.d, ctx.status,
                                     write_kv=cache.writable,
                                     delta=pending.value if pending else None,
                                     delta_bias=pending.bias if pending else None,
                                     parts=pending.parts if pending else None)
        o = paged_attention(q, cache, ctx, self.nh, self.scale, self.window or 0)
        if (not ops.FUSE_NORM and ops.linear_parts_slices(x.shape[0], self.w_o) > 1
                and self.w_o.shape[1] > ops.UNCUT_MAX_INNER):
            # the output product would be cut over k: its slices' sums are left for the next norm kernel
            return Delta(None, self.b_o, ops.linear_parts(o, self.w_o))
        ops.linear_add(o, self.w_o, self.b_o, x)
        return True

    def param_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()
