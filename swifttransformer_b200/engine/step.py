"""The step function: one batch of (request, its next tokens) through the model.

A step holds, for each request in it, the tokens that come next (a portion of a
prompt, cut anywhere, or a single decoded token), the number of tokens the
request already has in the cache, and the places among the new tokens whose
logits are wanted.  All entries run as one batch over the flattened tokens;
only the new tokens are computed, everything earlier is read from the cache.

Reference: ``Gpt<T>::forward`` (src/csrc/model/gpt/gpt.cc:507-657) takes whole
prompts (first_token_index == 0) beside single decode tokens and returns one
greedy token per request; its per-step host work is eight blocking copies
(gpt.cc:92-103,118-144,269-300,536-539).  Here every index array of the step
is packed into one pinned buffer and reaches the device in one asynchronous
copy; block-table changes ride along and are applied by a small kernel.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager
from ..models.base import CausalLM
from ..parts.attention import SHORT_PORTION


class OutOfPages(RuntimeError):
    """The page pool cannot hold the tokens of this step."""


class StepError(ValueError):
    """A step that cannot be run as given (bad token id, position beyond the model's limit, ...)."""


@dataclasses.dataclass
class StepEntry:
    slot: int                       # the request's cache slot
    tokens: Sequence[int]           # its next tokens (at least one)
    start_pos: int                  # tokens it already has in the cache
    want: Sequence[int] = ()        # places among `tokens` whose logits are wanted


class AttentionPlan:
    """Which of the step's tokens go to which attention kernel (bfloat16 path)."""

    def __init__(self, items, n_items, tiles, n_tiles, max_item_kv):
        self.items, self.n_items, self.tiles, self.n_tiles = items, n_items, tiles, n_tiles
        self.max_item_kv = max_item_kv
        self.fixed_splits: Optional[int] = None

    def splits(self, nh: int) -> int:
        """Parts the key range of a single-token query is cut into, so that the launch fills the GPU."""
        if self.fixed_splits is not None:
            return self.fixed_splits
        return choose_splits(self.n_items, nh, self.max_item_kv)


def choose_splits(n_items: int, nh: int, max_kv: int, sms: int = 148) -> int:
    blocks = max(1, n_items * nh)
    s = max(1, (2 * sms + blocks - 1) // blocks)
    s = min(s, max(1, max_kv // 128), 32)
    return s


class StepContext:
    """Everything a part may ask about the running step.

    Device tensors (int32): token_ids[N], positions[N], seq_of_token[N], q_start[B+1],
    start_pos[B], kv_len[B] (length after the step), slots[B], want_rows[n_want].
    Host lists of the same names with an ``h_`` prefix.
    """

    def __init__(self):
        self.n_tokens = self.n_seqs = self.n_want = 0
        self.token_ids = self.positions = self.seq_of_token = None
        self.q_start = self.start_pos = self.kv_len = self.slots = self.want_rows = None
        self.h_q_start: List[int] = []
        self.h_start_pos: List[int] = []
        self.h_kv_len: List[int] = []
        self.h_slots: List[int] = []
        self.status: Optional[torch.Tensor] = None
        self.act_dtype: torch.dtype = torch.float32
        self.device: Optional[torch.device] = None
        self._plan: Optional[AttentionPlan] = None
        self._runner: Any = None

    def attention_plan(self) -> AttentionPlan:
        return self._plan

    def scratch_f32(self, n: int) -> torch.Tensor:
        return self._runner._scratch(n)


class ModelRunner:
    """Owns the model, its cache and the staging buffers; runs steps."""

    def __init__(self, model: CausalLM, cache: CacheManager, max_batch_tokens: int = 8192,
                 use_cuda_graphs: bool = False):
        self.model, self.cache = model, cache
        self.device = model.device
        self.max_batch_tokens = max_batch_tokens
        self.use_cuda_graphs = use_cuda_graphs and self.device.type == "cuda" and model.graph_safe()
        self.max_seqs = cache.max_seqs
        self.tile_rows = 64
        cap = self._layout(max_batch_tokens, self.max_seqs, max_batch_tokens,
                           [self.max_seqs * cache.max_pages_per_seq + 16] * len(cache.groups))["total"]
        pin = self.device.type == "cuda"
        # two pinned staging buffers used in turn: a buffer is rewritten only after
        # the copy that last read it has finished (the host may run ahead of the GPU)
        self._hosts = [torch.zeros(cap, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._host_events = [torch.cuda.Event() if pin else None for _ in range(2)]
        self._host_turn = 0
        self._dev = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._scratch_buf: Optional[torch.Tensor] = None
        self._entries = cache.entries()
        self.steps_run = 0

    # ------------------------------------------------------------ buffers
    def _scratch(self, n: int) -> torch.Tensor:
        if self._scratch_buf is None or self._scratch_buf.numel() < n:
            self._scratch_buf = torch.empty(max(n, 1 << 20), dtype=torch.float32, device=self.device)
        return self._scratch_buf

    def _layout(self, n_cap: int, b_cap: int, w_cap: int, upd_caps: Sequence[int]) -> Dict[str, Any]:
        off = 0
        lay: Dict[str, Any] = {}

        def take(name, n):
            nonlocal off
            lay[name] = (off, n)
            off += n
        g = len(upd_caps)
        take("upd_count", max(g, 1))
        for name in ("token_ids", "positions", "seq_of_token"):
            take(name, n_cap)
        take("q_start", b_cap + 1)
        for name in ("start_pos", "kv_len", "slots"):
            take(name, b_cap)
        take("want_rows", w_cap)
        take("items", n_cap)
        take("tiles", 2 * ((n_cap + self.tile_rows - 1) // self.tile_rows + b_cap))
        for i, c in enumerate(upd_caps):
            take(f"upd_idx{i}", c)
            take(f"upd_val{i}", c)
        lay["total"] = off
        return lay

    # --------------------------------------------------------------- step
    def validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        vocab, maxpos = self.model.vocab_size, self.model.max_positions
        seen = set()
        total = 0
        for e in entries:
            n = len(e.tokens)
            if n < 1:
                raise StepError("an entry needs at least one token")
            if e.slot in seen:
                raise StepError(f"slot {e.slot} occurs twice in one step")
            seen.add(e.slot)
            if e.start_pos != self.cache.lengths[e.slot]:
                raise StepError(f"slot {e.slot} holds {self.cache.lengths[e.slot]} tokens, the step says {e.start_pos}")
            if maxpos is not None and e.start_pos + n > maxpos:
                raise StepError(f"a request would reach {e.start_pos + n} tokens; the model's positions end at {maxpos}")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= vocab:
                raise StepError(f"token id {lo if lo < 0 else hi} is outside the vocabulary of {vocab}")
            for w in e.want:
                if w < 0 or w >= n:
                    raise StepError(f"wanted place {w} is outside the entry's {n} tokens")
            total += n
        if total > self.max_batch_tokens:
            raise StepError(f"{total} tokens in one step exceed the limit of {self.max_batch_tokens}")
        if len(entries) > self.max_seqs:
            raise StepError(f"{len(entries)} requests in one step exceed the limit of {self.max_seqs}")

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one step; returns float32 logits [number of wanted places, vocab] (None if none wanted)."""
        self.validate(entries)
        for e in entries:
            if not self.cache.can_reserve(e.slot, e.start_pos, e.start_pos + len(e.tokens)):
                raise OutOfPages(f"no pages left for {len(e.tokens)} tokens of slot {e.slot}")
        # pages for all entries together, or none
        need = [sum(len(g.missing(e.slot, e.start_pos, e.start_pos + len(e.tokens))) for e in entries)
                for g in self.cache.groups]
        for g, n in zip(self.cache.groups, need):
            if n > g.pool.num_free:
                raise OutOfPages(f"the step needs {n} pages, {g.pool.num_free} are free")
        for e in entries:
            ok = self.cache.reserve(e.slot, e.start_pos, e.start_pos + len(e.tokens))
            assert ok
        ctx = self._build_context(entries)
        logits = self.model.forward(ctx, self._entries)
        for e in entries:
            self.cache.commit(e.slot, e.start_pos + len(e.tokens))
        self.steps_run += 1
        return logits

    def check_status(self) -> None:
        """Raise if a kernel recorded a fault (a hole in a block table).  Synchronises."""
        if int(self.status.item()) != 0:
            self.status.zero_()
            raise RuntimeError("a kernel found a token whose position has no page in its block table")

    def _build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        B = len(entries)
        lens = [len(e.tokens) for e in entries]
        N = sum(lens)
        W = sum(len(e.want) for e in entries)
        updates = [g.take_updates() for g in self.cache.groups]
        lay = self._layout(N, B, W, [len(u) for u in updates])
        turn = self._host_turn
        self._host_turn ^= 1
        host = self._hosts[turn]
        if lay["total"] > host.numel():
            raise StepError("the step's index arrays exceed the staging buffer")
        if self._host_events[turn] is not None:
            self._host_events[turn].synchronize()
        h = host.numpy()

        def put(name, values):
            o, n = lay[name]
            h[o:o + len(values)] = values

        q_start = np.zeros(B + 1, dtype=np.int32)
        np.cumsum(lens, out=q_start[1:])
        start = np.fromiter((e.start_pos for e in entries), dtype=np.int32, count=B)
        tok = np.empty(N, dtype=np.int32)
        pos = np.empty(N, dtype=np.int32)
        seq = np.empty(N, dtype=np.int32)
        want_rows: List[int] = []
        for i, e in enumerate(entries):
            a, b = q_start[i], q_start[i + 1]
            tok[a:b] = e.tokens
            pos[a:b] = np.arange(e.start_pos, e.start_pos + lens[i], dtype=np.int32)
            seq[a:b] = i
            want_rows.extend(int(a) + w for w in e.want)
        put("upd_count", [len(u) for u in updates] or [0])
        put("token_ids", tok)
        put("positions", pos)
        put("seq_of_token", seq)
        put("q_start", q_start)
        put("start_pos", start)
        put("kv_len", start + np.asarray(lens, dtype=np.int32))
        put("slots", [e.slot for e in entries])
        put("want_rows", want_rows)
        # attention plan: short portions token by token, long ones in tiles (longest key range first)
        items: List[int] = []
        tiles: List[tuple] = []
        max_item_kv = 0
        for i, e in enumerate(entries):
            if lens[i] < SHORT_PORTION:
                items.extend(range(int(q_start[i]), int(q_start[i + 1])))
                max_item_kv = max(max_item_kv, e.start_pos + lens[i])
            else:
                for off in range(0, lens[i], self.tile_rows):
                    tiles.append((e.start_pos + min(off + self.tile_rows, lens[i]), i, off))
        tiles.sort(reverse=True)
        put("items", items)
        put("tiles", [v for t in tiles for v in (t[1], t[2])])
        for gi, u in enumerate(updates):
            put(f"upd_idx{gi}", [x[0] for x in u])
            put(f"upd_val{gi}", [x[1] for x in u])
        total = lay["total"]
        self._dev[:total].copy_(host[:total], non_blocking=True)
        if self._host_events[turn] is not None:
            self._host_events[turn].record()

        def view(name):
            o, n = lay[name]
            return self._dev[o:o + n]

        for gi, (g, u) in enumerate(zip(self.cache.groups, updates)):
            if u:
                ops.scatter_i32(g.block_table, view(f"upd_idx{gi}"), view(f"upd_val{gi}"),
                                self._dev[lay["upd_count"][0] + gi:lay["upd_count"][0] + gi + 1], len(u))
        ctx = StepContext()
        ctx.n_tokens, ctx.n_seqs, ctx.n_want = N, B, W
        ctx.token_ids, ctx.positions, ctx.seq_of_token = view("token_ids"), view("positions"), view("seq_of_token")
        ctx.q_start, ctx.start_pos, ctx.kv_len, ctx.slots = (view("q_start"), view("start_pos"), view("kv_len"),
                                                             view("slots"))
        ctx.want_rows = view("want_rows") if W else None
        ctx.h_q_start, ctx.h_start_pos = q_start.tolist(), start.tolist()
        ctx.h_kv_len = [s + n for s, n in zip(ctx.h_start_pos, lens)]
        ctx.h_slots = [e.slot for e in entries]
        ctx.status, ctx.act_dtype, ctx.device = self.status, self.model.dtype, self.device
        ctx._plan = AttentionPlan(view("items"), len(items), view("tiles"), len(tiles), max_item_kv)
        ctx._runner = self
        return ctx
