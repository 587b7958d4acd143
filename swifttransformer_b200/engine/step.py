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
import weakref
from math import gcd
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager
from ..models.base import CausalLM
from ..parts.base import StepPlan


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


class StepContext:
    """Everything a part may ask about the running step.

    Device tensors (int32): token_ids[N], positions[N], seq_of_token[N], q_start[B+1],
    start_pos[B], kv_len[B] (length after the step), slots[B], want_rows[n_want].
    Host lists of the same names with an ``h_`` prefix (None while a graph is recorded
    or replayed: a part that needs them is not ``graph_safe``).
    ``plan(name)``: what the step plan of that name (parts.base.StepPlan) made of this step.
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
        self.nvtx = False                # the model wraps every layer in an NVTX range
        self._plans: Dict[str, Any] = {}
        self._scratch_owner: Any = None

    def plan(self, name: str) -> Any:
        return self._plans[name]

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

# tokens of a recorded step that is not decode-only are padded to a multiple of this (and of what the
# model's step plans ask for), so that prompts of any length share a few recordings
PADDED_TOKEN_STEP = 64


class _RecordedStep:
    """A step of fixed shape recorded as a CUDA graph and replayed: ``n_cap`` tokens, ``b_cap`` requests,
    ``w_cap`` wanted rows, and for every step plan of the model the key it gave.  What a step does not fill
    is padding that every kernel skips: tokens at position -1, requests without tokens (see
    ModelRunner._pack).  ``decode``: every request brings one token and wants its logits; the arrays that
    are then the same in every step are written once."""

    def __init__(self, runner: "ModelRunner", n_cap: int, b_cap: int, w_cap: int, plan_keys: Dict[str, Tuple],
                 decode: bool = False):
        # weak references both ways (the runner holds its recordings, a context its scratch owner): a runner
        # that goes out of scope is freed at once, pool and graphs with it, without waiting for the collector
        self.runner = weakref.proxy(runner)
        self.n_cap, self.b_cap, self.w_cap, self.decode = n_cap, b_cap, w_cap, decode
        self._scratch_buf: Optional[torch.Tensor] = None
        self._frozen = False
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.kernels = 0
        self.last_used = 0               # the runner's step count when this recording last ran
        self.lay = lay = runner._layout(n_cap, b_cap, w_cap)
        self.staging = _Staging(lay["total"], runner.device)
        self.ctx = runner._context_over(self.staging.dev, lay, n_cap, b_cap, w_cap, plan_keys, weakref.proxy(self))
        self.token_from = self._view("token_from")
        if decode:
            assert n_cap == b_cap == w_cap
            ar = np.arange(n_cap + 1, dtype=np.int32)
            self._ones = np.ones(n_cap, dtype=np.int32)
            self._arange = ar
            for host in self.staging.hosts:
                h = host.numpy()
                for name, values in (("seq_of_token", ar[:-1]), ("q_start", ar), ("want_rows", ar[:-1])):
                    o, n = lay[name]
                    h[o:o + n] = values

    def _view(self, name: str) -> torch.Tensor:
        o, n = self.lay[name]
        return self.staging.dev[o:o + n]

    def _scratch(self, n: int) -> torch.Tensor:
        if self._scratch_buf is None or self._scratch_buf.numel() < n:
            if self._frozen:
                raise RuntimeError("a recorded step asked for more scratch memory than when it was recorded")
            self._scratch_buf = torch.empty(max(n, 1), dtype=torch.float32, device=self.runner.device)
        return self._scratch_buf

    def fill(self, entries: Sequence[StepEntry], feedback=None) -> int:
        """Stage the step's index arrays and start their copy; returns the number of wanted rows."""
        r = self.runner
        h = self.staging.begin()
        if not self.decode:
            info = r._pack(entries, self.lay, h, self.n_cap, self.b_cap, feedback)
            self.staging.commit(self.lay["total"])
            return info["W"]
        cap, b, lay = self.n_cap, len(entries), self.lay
        start = np.fromiter((e.start_pos for e in entries), dtype=np.int32, count=b)
        for name, values, pad in (("token_ids", [e.tokens[0] for e in entries], 0), ("positions", start, -1),
                                  ("start_pos", start, 0), ("kv_len", start + 1, 0),
                                  ("slots", [e.slot for e in entries], 0),
                                  ("token_from", feedback[1] if feedback is not None else (), -1)):
            o = lay[name][0]
            k = len(values)
            h[o:o + k] = values
            h[o + k:o + cap] = pad
        for p in r.plans:
            o, n = lay["plan:" + p.name]
            p.fill(self._ones[:b], self._arange[:b + 1], start, h[o:o + n], cap, cap)
        self.staging.commit(lay["total"])
        return b

    def run(self, entries: Sequence[StepEntry], feedback=None) -> Optional[torch.Tensor]:
        if self.graph is None:
            self.record()
        w = self.fill(entries, feedback)
        if feedback is not None:
            ops.gather_where_i32(self.ctx.token_ids, self.token_from, feedback[0])
        self.graph.replay()
        return self.logits[:w] if w else None

    def record(self) -> None:
        r = self.runner
        # Once without recording, on a step that is all padding: it sizes the scratch memory and lets
        # libraries set themselves up, and it writes nothing - neither pages nor per-request state - so a
        # shape's first use runs the real step once, like every later use.
        self.fill([])
        r.model.forward(self.ctx, r._entries)
        torch.cuda.synchronize()
        self._frozen = True
        before = ops.launch_count()
        g = torch.cuda.CUDAGraph()
        # Nothing may destroy a CUDA object while the stream records (what torch keeps of an older graph may
        # lie in a reference cycle and wait for the collector): the collector is kept off until the recording
        # has ended.  A full collection beforehand is not needed for that and costs more than the recording
        # itself (25 ms of the 35 a new shape took).
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


class ModelRunner:
    """Owns the model, its cache and the staging buffers; runs steps."""

    BASE_ARRAYS = ("token_ids", "positions", "seq_of_token", "q_start", "start_pos", "kv_len", "slots",
                   "want_rows", "token_from")

    def __init__(self, model: CausalLM, cache: CacheManager, max_batch_tokens: int = 8192,
                 use_cuda_graphs: bool = True):
        self.model, self.cache = model, cache
        self.device = model.device
        self.max_batch_tokens = max_batch_tokens
        self.use_cuda_graphs = use_cuda_graphs and self.device.type == "cuda" and model.graph_safe()
        self.max_seqs = cache.max_seqs
        # the step plans of the model's mixers, one per name
        self.plans: List[StepPlan] = model.step_plans()
        self.token_multiple = PADDED_TOKEN_STEP
        for p in self.plans:
            self.token_multiple = self.token_multiple * p.token_multiple // gcd(self.token_multiple, p.token_multiple)
        self._upd_cap = min(self.max_seqs * cache.max_pages_per_seq, 1 << 16) + 16
        words = self._layout(max_batch_tokens, self.max_seqs, max_batch_tokens)["total"]
        self._staging = _Staging(words, self.device)
        self._upd_staging = _Staging(1 + 2 * self._upd_cap, self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._scratch_buf: Optional[torch.Tensor] = None
        self._entries = cache.entries()
        # Recorded steps by shape.  Decode-only steps: (bucket of requests, the plans' keys).  Everything else
        # (prompt portions, mixed steps): (padded tokens, requests, wanted rows, the plans' keys); those are
        # bounded in number: a shape beyond the bound takes the place of the recording that has not been
        # used for the longest time if that is more than `evict_idle_steps` steps ago, and runs eagerly
        # otherwise (a working set larger than the bound must not be recorded over and over).
        self._graphs: Dict[Any, _RecordedStep] = {}
        self._step_graphs: Dict[Any, _RecordedStep] = {}
        self.max_step_graphs = 48
        self.evict_idle_steps = 512
        self._retired_h2d_bytes = 0
        self.padded_graph_steps = 0
        self._graph_pool = torch.cuda.graph_pool_handle() if self.use_cuda_graphs else None
        self.steps_run = 0
        self.graph_steps = 0
        self.kernels_last_step = 0
        self.nvtx = False                # NVTX ranges around the layers of steps that are launched kernel by kernel

    # ------------------------------------------------------------ buffers
    def _scratch(self, n: int) -> torch.Tensor:
        if self._scratch_buf is None or self._scratch_buf.numel() < n:
            self._scratch_buf = torch.empty(max(n, 1 << 20), dtype=torch.float32, device=self.device)
        return self._scratch_buf

    def _layout(self, n_cap: int, b_cap: int, w_cap: int) -> Dict[str, Any]:
        """Where each index array of a step of at most n_cap tokens, b_cap requests and w_cap wanted rows
        lies in the staging buffer: name -> (offset, words); the step plans' arrays follow the step's own."""
        off = 0
        lay: Dict[str, Any] = {}
        sizes = dict(token_ids=n_cap, positions=n_cap, seq_of_token=n_cap, q_start=b_cap + 1, start_pos=b_cap,
                     kv_len=b_cap, slots=b_cap, want_rows=w_cap, token_from=n_cap)
        for name in self.BASE_ARRAYS:
            lay[name] = (off, sizes[name])
            off += sizes[name]
        for p in self.plans:
            n = p.words(n_cap, b_cap)
            lay["plan:" + p.name] = (off, n)
            off += n
        lay["total"] = off
        return lay

    def _context_over(self, dev: torch.Tensor, lay: Dict[str, Any], n: int, b: int, w: int,
                      plan_keys: Dict[str, Tuple], scratch_owner: Any) -> StepContext:
        """A step context whose arrays are views of ``dev`` laid out by ``lay``."""
        def view(name):
            o, k = lay[name]
            return dev[o:o + k]

        ctx = StepContext()
        ctx.n_tokens, ctx.n_seqs, ctx.n_want = n, b, w
        ctx.token_ids, ctx.positions, ctx.seq_of_token = view("token_ids"), view("positions"), view("seq_of_token")
        ctx.q_start, ctx.start_pos, ctx.kv_len, ctx.slots = (view("q_start"), view("start_pos"), view("kv_len"),
                                                             view("slots"))
        ctx.want_rows = view("want_rows") if w else None
        ctx.status, ctx.act_dtype, ctx.device = self.status, self.model.dtype, self.device
        ctx.nvtx = self.nvtx
        for p in self.plans:
            ctx._plans[p.name] = p.view(view("plan:" + p.name), plan_keys[p.name], n, b)
        ctx._scratch_owner = scratch_owner
        return ctx

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
            if e.start_pos + n > self.cache.max_seq_len:
                raise StepError(f"a request would reach {e.start_pos + n} tokens; the cache holds "
                                f"{self.cache.max_seq_len} per request")
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
        rec = self._recording_for(entries)
        if rec is not None:
            logits = rec.run(entries, feedback)
            if rec.decode:
                self.graph_steps += 1
            else:
                self.padded_graph_steps += 1
            self.kernels_last_step = rec.kernels
        else:
            ctx = self._build_context(entries, feedback)
            logits = self.model.forward(ctx, self._entries)
            self.kernels_last_step = ops.launch_count() - before
        for e in entries:
            self.cache.commit(e.slot, e.start_pos + len(e.tokens))
        self.steps_run += 1
        return logits

    def _recording_for(self, entries: Sequence[StepEntry]) -> Optional[_RecordedStep]:
        """The recorded step whose shape takes these entries, made if need be; None: run eagerly.
        Launching a step's kernels and library calls one by one costs the host milliseconds whatever the
        step's size; replaying a recording costs a few tens of microseconds."""
        if not self.use_cuda_graphs:
            return None
        b = len(entries)
        b_cap = next((c for c in GRAPH_BUCKETS if c >= b), None)
        if b_cap is None:
            return None
        lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=b)
        start = np.fromiter((e.start_pos for e in entries), dtype=np.int32, count=b)
        n = int(lens.sum())
        decode = n == b and all(len(e.want) == 1 for e in entries)
        if decode:
            n_cap = w_cap = b_cap
        else:
            w = sum(len(e.want) for e in entries)
            n_cap = -(-n // self.token_multiple) * self.token_multiple
            w_cap = 0 if w == 0 else (b_cap if w <= b_cap else n_cap)
        plan_keys = {p.name: p.shape_key(lens, start, n_cap, b_cap) for p in self.plans}
        key = (n_cap, b_cap, w_cap) + tuple(plan_keys[p.name] for p in self.plans)
        held = self._graphs if decode else self._step_graphs
        rec = held.get(key)
        if rec is None:
            if not decode and len(held) >= self.max_step_graphs:
                oldest = min(held, key=lambda k: held[k].last_used, default=None)
                if oldest is None or self.steps_run - held[oldest].last_used <= self.evict_idle_steps:
                    return None
                self._retired_h2d_bytes += held.pop(oldest).staging.bytes_copied
            rec = held[key] = _RecordedStep(self, n_cap, b_cap, w_cap, plan_keys, decode=decode)
        rec.last_used = self.steps_run
        return rec

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

    def _pack(self, entries: Sequence[StepEntry], lay: Dict[str, Any], h: np.ndarray, n_cap: int, b_cap: int,
              feedback=None):
        """Write the step's index arrays into the staging buffer ``h`` laid out by ``lay``.  Where the layout
        has room for more than the step brings (a recorded step of padded shape), the rest is filled with
        entries every kernel skips: tokens at position -1, requests without tokens; the step plans pad
        their own arrays.  Returns what describes the step to the host."""
        B = len(entries)
        lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=B)
        N = int(lens.sum())

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
        put("kv_len", start + lens, 0)
        put("slots", [e.slot for e in entries], 0)
        put("want_rows", want_rows, 0)
        put("token_from", list(feedback[1]) if feedback is not None else [], -1)
        plan_keys = {}
        for p in self.plans:
            o, n = lay["plan:" + p.name]
            plan_keys[p.name] = p.fill(lens, q_start, start, h[o:o + n], n_cap, b_cap)
        return dict(N=N, B=B, W=len(want_rows), lens=lens, q_start=q_start, start=start, plan_keys=plan_keys)

    def _build_context(self, entries: Sequence[StepEntry], feedback=None) -> StepContext:
        """The context of a step that runs eagerly: arrays of exactly the step's sizes."""
        B = len(entries)
        N = sum(len(e.tokens) for e in entries)
        W = sum(len(e.want) for e in entries)
        lay = self._layout(N, B, W)
        h = self._staging.begin()
        info = self._pack(entries, lay, h, N, B, feedback)
        self._staging.commit(lay["total"])
        dev = self._staging.dev
        if feedback is not None:
            o, _ = lay["token_from"]
            t0, _ = lay["token_ids"]
            ops.gather_where_i32(dev[t0:t0 + N], dev[o:o + N], feedback[0])
        ctx = self._context_over(dev, lay, N, B, W, info["plan_keys"], self)
        ctx.h_q_start, ctx.h_start_pos = info["q_start"].tolist(), info["start"].tolist()
        ctx.h_kv_len = [s + int(n) for s, n in zip(ctx.h_start_pos, info["lens"])]
        ctx.h_slots = [e.slot for e in entries]
        return ctx
