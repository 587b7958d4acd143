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

Steps that hold only single tokens whose logits are all wanted (decoding) are
recorded once per batch-size bucket into a CUDA graph and replayed: the step's
index arrays live at fixed addresses, the batch is padded to the bucket with
entries at position -1, which every kernel skips.
"""
from __future__ import annotations

import dataclasses
import gc
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


# Keys one block of the decode attention walks alone before the key range is cut into parts (for head sizes
# up to 64, where a block has eight warps; half of it beyond).  Recorded decode steps are keyed by the number
# of such spans the longest request needs, so the cut follows the real lengths, not the longest possible one.
KEYS_PER_BLOCK = 768


def choose_splits(n_items: int, nh: int, max_kv: int, sms: int = 148, head_dim: int = 64) -> int:
    """Parts the key range of a single-token query is cut into.

    Measured on one B200 at context ~550 with 32 heads.  Head size 64 (OPT-1.3B, tensor-core kernel with
    eight warps per block): cutting costs a merge (a trip through global memory and an atomic) and one part
    is best at every batch (ms per step, one part against two blocks per SM: batch 1: 1.043 / 1.084,
    4: 1.116 / 1.167, 8: 1.299 / 1.323); longer ranges are cut so that a block walks about KEYS_PER_BLOCK
    keys, as long as the launch stays within two blocks per SM.  Head size 128 (OPT-6.7B, lanes kernel, whose
    blocks walk their keys more slowly): two blocks per SM, parts of at least 128 keys (batch 1: 3.20 with
    ten parts against 3.28 with two; batch 8: 3.78 with two against 3.86 with one)."""
    blocks = max(1, n_items * nh)
    if blocks * 64 >= 250 * head_dim:
        return 1
    room = max(1, (2 * sms + blocks - 1) // blocks)
    if head_dim <= 64:
        want = (max_kv + KEYS_PER_BLOCK - 1) // KEYS_PER_BLOCK
    else:
        want = max(1, max_kv // 128)
    return max(1, min(want, room, 32))


class AttentionPlan:
    """Which of the step's tokens go to which attention kernel (bfloat16 path)."""

    def __init__(self, items, n_items, tiles, n_tiles, max_item_kv):
        self.items, self.n_items, self.tiles, self.n_tiles = items, n_items, tiles, n_tiles
        self.max_item_kv = max_item_kv

    def splits(self, nh: int, head_dim: int = 64) -> int:
        return choose_splits(self.n_items, nh, self.max_item_kv, head_dim=head_dim)


class StepContext:
    """Everything a part may ask about the running step.

    Device tensors (int32): token_ids[N], positions[N], seq_of_token[N], q_start[B+1],
    start_pos[B], kv_len[B] (length after the step), slots[B], want_rows[n_want].
    Host lists of the same names with an ``h_`` prefix (None while a graph is recorded
    or replayed: a part that needs them is not ``graph_safe``).
    """

    def __init__(self):
        self.n_tokens = self.n_seqs = self.n_want = 0
        self.token_ids = self.positions = self.seq_of_token = None
        self.q_start = self.start_pos = self.kv_len = self.slots = self.want_rows = None
        self.h_q_start: Optional[List[int]] = None
        self.h_start_pos: Optional[List[int]] = None
        self.h_kv_len: Optional[List[int]] = None
        self.h_slots: Optional[List[int]] = None
        self.status: Optional[torch.Tensor] = None
        self.act_dtype: torch.dtype = torch.float32
        self.device: Optional[torch.device] = None
        self._plan: Optional[AttentionPlan] = None
        self._scratch_owner: Any = None

    def attention_plan(self) -> AttentionPlan:
        return self._plan

    def scratch_f32(self, n: int) -> torch.Tensor:
        return self._scratch_owner._scratch(n)


class _Staging:
    """Pinned host buffers used in turn, and the device buffer they are copied to.  A host buffer is
    rewritten only after the copy that last read it has finished (the host may run ahead of the GPU)."""

    def __init__(self, words: int, device: torch.device, turns: int = 2):
        pin = device.type == "cuda"
        self.hosts = [torch.zeros(words, dtype=torch.int32, pin_memory=pin) for _ in range(turns)]
        self.events = [torch.cuda.Event() if pin else None for _ in range(turns)]
        self.dev = torch.zeros(words, dtype=torch.int32, device=device)
        self.turn = 0
        self.bytes_copied = 0

    def begin(self) -> np.ndarray:
        self.turn = (self.turn + 1) % len(self.hosts)
        if self.events[self.turn] is not None:
            self.events[self.turn].synchronize()
        return self.hosts[self.turn].numpy()

    def commit(self, words: int) -> None:
        self.dev[:words].copy_(self.hosts[self.turn][:words], non_blocking=True)
        if self.events[self.turn] is not None:
            self.events[self.turn].record()
        self.bytes_copied += 4 * words


GRAPH_BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512)


class _RecordedStep:
    """A step of fixed shape recorded as a CUDA graph: its context, its scratch memory, the recording."""

    def _init_recording(self, runner: "ModelRunner") -> None:
        self.runner = runner
        self._scratch_buf: Optional[torch.Tensor] = None
        self._frozen = False
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.kernels = 0
        self.last_used = 0               # the runner's step count when this recording last ran

    def _scratch(self, n: int) -> torch.Tensor:
        if self._scratch_buf is None or self._scratch_buf.numel() < n:
            if self._frozen:
                raise RuntimeError("a recorded step asked for more scratch memory than when it was recorded")
            self._scratch_buf = torch.empty(max(n, 1), dtype=torch.float32, device=self.runner.device)
        return self._scratch_buf

    def record(self) -> None:
        r = self.runner
        # once without recording: sizes the scratch memory and lets libraries set themselves up
        r.model.forward(self.ctx, r._entries)
        torch.cuda.synchronize()
        self._frozen = True
        before = ops.launch_count()
        g = torch.cuda.CUDAGraph()
        # Nothing may destroy a CUDA object while the stream records: collect dead objects (an
        # engine that went out of scope owns graphs of its own) now, and keep the collector off
        # until the recording has ended.
        gc.collect()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(g, pool=r._graph_pool):
                self.logits = r.model.forward(self.ctx, r._entries)
        finally:
            if gc_was_on:
                gc.enable()
        self.kernels = ops.launch_count() - before
        self.graph = g


class _DecodeGraph(_RecordedStep):
    """One recorded decode step for up to ``cap`` requests."""

    FIELDS = ("token_ids", "positions", "start_pos", "kv_len", "slots")

    def __init__(self, runner: "ModelRunner", cap: int, max_kv: int):
        self._init_recording(runner)
        self.cap = cap
        self.staging = _Staging(6 * cap, runner.device)
        dev = runner.device
        ar = torch.arange(cap + 1, dtype=torch.int32, device=dev)
        d = self.staging.dev
        ctx = StepContext()
        ctx.n_tokens = ctx.n_seqs = ctx.n_want = cap
        ctx.token_ids, ctx.positions = d[0:cap], d[cap:2 * cap]
        ctx.start_pos, ctx.kv_len, ctx.slots = d[2 * cap:3 * cap], d[3 * cap:4 * cap], d[4 * cap:5 * cap]
        self.token_from = d[5 * cap:6 * cap]     # per token: index into the previous step's sampled tokens, or -1
        ctx.seq_of_token, ctx.q_start, ctx.want_rows = ar[:cap], ar, ar[:cap]
        ctx.status, ctx.act_dtype, ctx.device = runner.status, runner.model.dtype, dev
        ctx._plan = AttentionPlan(None, cap, None, 0, max_kv)
        ctx._scratch_owner = self
        self.ctx = ctx
        self._keep = ar

    def fill(self, entries: Sequence[StepEntry], token_from: Optional[Sequence[int]] = None) -> None:
        cap, b = self.cap, len(entries)
        h = self.staging.begin()
        h[0:cap] = 0
        h[cap:2 * cap] = -1                      # padding entries: position -1, skipped by every kernel
        h[2 * cap:5 * cap] = 0
        for i, e in enumerate(entries):
            h[i] = e.tokens[0]
            h[cap + i] = e.start_pos
            h[2 * cap + i] = e.start_pos
            h[3 * cap + i] = e.start_pos + 1
            h[4 * cap + i] = e.slot
        if token_from is not None:
            h[5 * cap:6 * cap] = -1
            h[5 * cap:5 * cap + b] = token_from
            self.staging.commit(6 * cap)
        else:
            self.staging.commit(5 * cap)

    def run(self, entries: Sequence[StepEntry], feedback=None) -> torch.Tensor:
        self.fill(entries, feedback[1] if feedback else None)
        if self.graph is None:
            self.record()
        if feedback:
            ops.gather_where_i32(self.ctx.token_ids, self.token_from, feedback[0])
        self.graph.replay()
        return self.logits[:len(entries)]


class _StepGraph(_RecordedStep):
    """One recorded step of a padded shape, for steps that are not decode-only: ``n_pad`` tokens (a multiple
    of the attention tile), ``b_pad`` requests, ``i_pad`` single-token attention entries, ``w_pad`` wanted
    rows.  What a step does not fill is padding that every kernel skips (see ModelRunner._pack)."""

    def __init__(self, runner: "ModelRunner", n_pad: int, b_pad: int, i_pad: int, w_pad: int, max_kv: int):
        self._init_recording(runner)
        self.n_pad = n_pad
        self.lay = lay = runner._layout(n_pad, b_pad, w_pad)
        self.staging = _Staging(lay["total"], runner.device)
        d = self.staging.dev

        def view(name):
            o, n = lay[name]
            return d[o:o + n]

        t_pad = lay["tiles"][1] // 2
        ctx = StepContext()
        ctx.n_tokens, ctx.n_seqs, ctx.n_want = n_pad, b_pad, w_pad
        ctx.token_ids, ctx.positions, ctx.seq_of_token = view("token_ids"), view("positions"), view("seq_of_token")
        ctx.q_start, ctx.start_pos, ctx.kv_len, ctx.slots = (view("q_start"), view("start_pos"), view("kv_len"),
                                                             view("slots"))
        ctx.want_rows = view("want_rows") if w_pad else None
        ctx.status, ctx.act_dtype, ctx.device = runner.status, runner.model.dtype, runner.device
        ctx._plan = AttentionPlan(view("items")[:i_pad], i_pad, view("tiles"), t_pad, max_kv)
        ctx._scratch_owner = self
        self.ctx = ctx
        self.token_from = view("token_from")

    def run(self, entries: Sequence[StepEntry], feedback=None) -> Optional[torch.Tensor]:
        r = self.runner
        h = self.staging.begin()
        info = r._pack(entries, self.lay, h, feedback)
        self.staging.commit(self.lay["total"])
        if self.graph is None:
            self.record()
        if feedback is not None:
            ops.gather_where_i32(self.ctx.token_ids, self.token_from, feedback[0])
        self.graph.replay()
        return self.logits[:info["W"]] if info["W"] else None


class ModelRunner:
    """Owns the model, its cache and the staging buffers; runs steps."""

    def __init__(self, model: CausalLM, cache: CacheManager, max_batch_tokens: int = 8192,
                 use_cuda_graphs: bool = True):
        self.model, self.cache = model, cache
        self.device = model.device
        self.max_batch_tokens = max_batch_tokens
        self.use_cuda_graphs = use_cuda_graphs and self.device.type == "cuda" and model.graph_safe()
        self.max_seqs = cache.max_seqs
        self.tile_rows = ops.attention_prefill_tile_rows()   # query rows one attention tile covers
        self._upd_cap = self.max_seqs * cache.max_pages_per_seq + 16
        words = self._layout(max_batch_tokens, self.max_seqs, max_batch_tokens)["total"]
        self._staging = _Staging(words, self.device)
        self._upd_staging = _Staging(1 + 2 * self._upd_cap, self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._scratch_buf: Optional[torch.Tensor] = None
        self._entries = cache.entries()
        self._graphs: Dict[Any, _DecodeGraph] = {}      # (rows, spans of KEYS_PER_BLOCK keys) -> recorded step
        # recorded steps of padded shapes for everything else (prompt portions, mixed steps); bounded in number:
        # a shape beyond the bound takes the place of the recording that has not been used for the longest
        # time if that is more than `evict_idle_steps` steps ago, and runs eagerly otherwise (a working set
        # larger than the bound must not be recorded over and over: recording costs ~15 eager steps)
        self._step_graphs: Dict[Any, _StepGraph] = {}
        self.max_step_graphs = 48
        self.evict_idle_steps = 512
        self._retired_h2d_bytes = 0
        self.padded_graph_steps = 0
        self._graph_pool = torch.cuda.graph_pool_handle() if self.use_cuda_graphs else None
        self.steps_run = 0
        self.graph_steps = 0
        self.kernels_last_step = 0

    # ------------------------------------------------------------ buffers
    def _scratch(self, n: int) -> torch.Tensor:
        if self._scratch_buf is None or self._scratch_buf.numel() < n:
            self._scratch_buf = torch.empty(max(n, 1 << 20), dtype=torch.float32, device=self.device)
        return self._scratch_buf

    def _layout(self, n_cap: int, b_cap: int, w_cap: int) -> Dict[str, Any]:
        off = 0
        lay: Dict[str, Any] = {}
        for name, n in (("token_ids", n_cap), ("positions", n_cap), ("seq_of_token", n_cap),
                        ("q_start", b_cap + 1), ("start_pos", b_cap), ("kv_len", b_cap), ("slots", b_cap),
                        ("want_rows", w_cap), ("items", n_cap), ("token_from", n_cap),
                        ("tiles", 2 * ((n_cap + self.tile_rows - 1) // self.tile_rows + b_cap))):
            lay[name] = (off, n)
            off += n
        lay["total"] = off
        return lay

    @property
    def h2d_bytes(self) -> int:
        """Bytes of step metadata copied host -> device so far."""
        return (self._staging.bytes_copied + self._upd_staging.bytes_copied + self._retired_h2d_bytes
                + sum(g.staging.bytes_copied for g in self._graphs.values())
                + sum(g.staging.bytes_copied for g in self._step_graphs.values()))

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

    def step(self, entries: Sequence[StepEntry], feedback=None) -> Optional[torch.Tensor]:
        """Run one step; returns float32 logits [number of wanted places, vocab] (None if none wanted).

        The returned tensor may be overwritten by the next step: use it (sample from it, copy it) first.

        ``feedback`` = (int32 device tensor of tokens an earlier step sampled, one index into it per token
        of this step or -1): those tokens are taken from the device, whatever the entries say in their
        place, so that a step can be launched before the host has seen the tokens it continues from.
        """
        self.validate(entries)
        if feedback is not None and len(feedback[1]) != sum(len(e.tokens) for e in entries):
            raise StepError("feedback needs one source index per token of the step")
        # pages for all entries together, or none
        for g in self.cache.groups:
            need = sum(len(g.missing(e.slot, e.start_pos, e.start_pos + len(e.tokens))) for e in entries)
            if need > g.pool.num_free:
                raise OutOfPages(f"the step needs {need} pages, {g.pool.num_free} are free")
        for e in entries:
            ok = self.cache.reserve(e.slot, e.start_pos, e.start_pos + len(e.tokens))
            assert ok
        self._flush_block_tables()
        before = ops.launch_count()
        bucket = self._graph_bucket(entries)
        if bucket:
            spans = max(-(-(e.start_pos + 1) // KEYS_PER_BLOCK) for e in entries)
            key = (bucket, spans)
            if key not in self._graphs:
                self._graphs[key] = _DecodeGraph(self, bucket, min(spans * KEYS_PER_BLOCK, self.cache.max_seq_len))
            dg = self._graphs[key]
            logits = dg.run(entries, feedback)
            self.graph_steps += 1
            self.kernels_last_step = dg.kernels
        else:
            sg = self._padded_graph(entries)
            if sg is not None:
                logits = sg.run(entries, feedback)
                self.padded_graph_steps += 1
                self.kernels_last_step = sg.kernels
            else:
                ctx = self._build_context(entries, feedback)
                logits = self.model.forward(ctx, self._entries)
                self.kernels_last_step = ops.launch_count() - before
        for e in entries:
            self.cache.commit(e.slot, e.start_pos + len(e.tokens))
        self.steps_run += 1
        return logits

    def _graph_bucket(self, entries: Sequence[StepEntry]) -> int:
        if not self.use_cuda_graphs:
            return 0
        for e in entries:
            if len(e.tokens) != 1 or len(e.want) != 1:
                return 0
        b = len(entries)
        for cap in GRAPH_BUCKETS:
            if cap >= b:
                return cap
        return 0

    def _padded_graph(self, entries: Sequence[StepEntry]) -> Optional[_StepGraph]:
        """The recorded step whose padded shape takes these entries, made if need be; None: run eagerly.
        Launching a step's ~190 kernels and library calls one by one costs the host ~2.8 ms whatever the step's
        size; replaying a recording costs a few tens of microseconds."""
        if not self.use_cuda_graphs:
            return None
        lens = [len(e.tokens) for e in entries]
        n, b = sum(lens), len(entries)
        w = sum(len(e.want) for e in entries)
        n_items = sum(x for x in lens if x < SHORT_PORTION)
        item_kv = max((e.start_pos + x for e, x in zip(entries, lens) if x < SHORT_PORTION), default=0)
        n_pad = -(-n // self.tile_rows) * self.tile_rows
        b_pad = next((c for c in GRAPH_BUCKETS if c >= b), None)
        if b_pad is None:
            return None
        i_pad = -(-n_items // 16) * 16
        w_pad = 0 if w == 0 else (b_pad if w <= b_pad else n_pad)
        spans = -(-item_kv // KEYS_PER_BLOCK)
        key = (n_pad, b_pad, i_pad, w_pad, spans)
        sg = self._step_graphs.get(key)
        if sg is None:
            if len(self._step_graphs) >= self.max_step_graphs:
                oldest = min(self._step_graphs, key=lambda k: self._step_graphs[k].last_used, default=None)
                if oldest is None or self.steps_run - self._step_graphs[oldest].last_used <= self.evict_idle_steps:
                    return None
                self._retired_h2d_bytes += self._step_graphs.pop(oldest).staging.bytes_copied
            sg = self._step_graphs[key] = _StepGraph(self, n_pad, b_pad, i_pad, w_pad,
                                                     min(max(spans, 1) * KEYS_PER_BLOCK, self.cache.max_seq_len))
        sg.last_used = self.steps_run
        return sg

    def check_status(self) -> None:
        """Raise if a kernel recorded a fault (a hole in a block table).  Synchronises."""
        code = int(self.status.item()) or ops.kernel_status(self.device)
        if code != 0:
            self.status.zero_()
            if code == 5:
                raise RuntimeError("the tcgen05 matrix product gave up waiting for its copies or products; "
                                   "the step's result is invalid")
            if code in (3, 4):
                raise RuntimeError("the tcgen05 attention kernel gave up waiting for the tensor cores; "
                                   "the step's result is invalid")
            raise RuntimeError("a kernel found a token whose position has no page in its block table")

    def _flush_block_tables(self) -> None:
        """Apply the cache manager's queued block-table changes on the device."""
        for g in self.cache.groups:
            u = g.take_updates()
            while u:
                part, u = u[:self._upd_cap], u[self._upd_cap:]
                n = len(part)
                h = self._upd_staging.begin()
                h[0] = n
                h[1:1 + n] = [x[0] for x in part]
                h[1 + n:1 + 2 * n] = [x[1] for x in part]
                self._upd_staging.commit(1 + 2 * n)
                d = self._upd_staging.dev
                ops.scatter_i32(g.block_table, d[1:1 + n], d[1 + n:1 + 2 * n], d[0:1], n)

    def _pack(self, entries: Sequence[StepEntry], lay: Dict[str, Any], h: np.ndarray, feedback=None):
        """Write the step's index arrays into the staging buffer ``h`` laid out by ``lay``.  Where the layout
        has room for more than the step brings (a recorded step of padded shape), the rest is filled with
        entries every kernel skips: tokens at position -1, requests without tokens, tiles without rows,
        single-token entries -1.  Returns what describes the step to the host."""
        B = len(entries)
        lens = [len(e.tokens) for e in entries]
        N = sum(lens)

        def put(name, values, fill):
            o, n = lay[name]
            k = len(values)
            h[o:o + k] = values
            if k < n:
                h[o + k:o + n] = fill

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
        put("token_ids", tok, 0)
        put("positions", pos, -1)
        put("seq_of_token", seq, 0)
        put("q_start", q_start, N)
        put("start_pos", start, 0)
        put("kv_len", start + np.asarray(lens, dtype=np.int32), 0)
        put("slots", [e.slot for e in entries], 0)
        put("want_rows", want_rows, 0)
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
        put("items", items, -1)
        put("tiles", [v for t in tiles for v in (t[1], t[2])], 0)
        o, n = lay["tiles"]
        h[o + 2 * len(tiles) + 1:o + n:2] = 1 << 24      # padding tiles: an offset past any request's tokens
        put("token_from", list(feedback[1]) if feedback is not None else [], -1)
        return dict(N=N, B=B, W=len(want_rows), lens=lens, q_start=q_start, start=start, n_items=len(items),
                    n_tiles=len(tiles), max_item_kv=max_item_kv)

    def _build_context(self, entries: Sequence[StepEntry], feedback=None) -> StepContext:
        B = len(entries)
        N = sum(len(e.tokens) for e in entries)
        W = sum(len(e.want) for e in entries)
        lay = self._layout(N, B, W)
        h = self._staging.begin()
        info = self._pack(entries, lay, h, feedback)
        lens, q_start, start = info["lens"], info["q_start"], info["start"]
        self._staging.commit(lay["total"])
        dev = self._staging.dev
        if feedback is not None:
            o, _ = lay["token_from"]
            t0, _ = lay["token_ids"]
            ops.gather_where_i32(dev[t0:t0 + N], dev[o:o + N], feedback[0])

        def view(name):
            o, n = lay[name]
            return dev[o:o + n]

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
        ctx._plan = AttentionPlan(view("items"), info["n_items"], view("tiles"), info["n_tiles"],
                                  max(info["max_item_kv"], max(ctx.h_kv_len)))
        ctx._scratch_owner = self
        return ctx
