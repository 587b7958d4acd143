"""The scheduler: which requests run in the next step, and with how many tokens.

Continuous batching under a token budget.  Each step first takes one token
from every running request that is decoding, then fills what is left of the
budget with portions of prompts (of running requests first, then of newly
admitted ones, first come first served), each portion at most ``chunk_size``
tokens and cut to the budget, down to one token.

When pages run out: a decoding request that cannot get the page its next token
needs makes the scheduler preempt the request admitted last (its pages and
slot are given back, its tokens are kept, it returns to the head of the
waiting queue and is later recomputed as one long prompt).  A prompt portion
that finds no pages is shortened to the pages that are free or waits for a
later step.  A request that cannot fit into the empty pool at all is finished
with reason ``cache_full``; nothing ever aborts the process.

The reference has no scheduler: its only driver runs one static batch, all
prompts in the first step and one token per request afterwards, with a block
counter that never frees and ``exit(1)`` when it runs out
(src/examples/lib/inference_batch.cc:58-66,110-118,163-218).
"""
from __future__ import annotations

import collections
import dataclasses
from typing import Any, Deque, Dict, List, Optional, Sequence, Tuple

from ..sampling.sampler import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
PENDING = -1      # stands in a request's output for a token that has been drawn on the GPU but not read yet


@dataclasses.dataclass
class Request:
    id: Any
    prompt: List[int]
    params: SamplingParams
    output: List[int] = dataclasses.field(default_factory=list)
    state: str = WAITING
    slot: Optional[int] = None
    n_computed: int = 0              # tokens of prompt+output whose keys/values are in the cache
    admitted_at: int = -1
    finish_reason: Optional[str] = None
    preemptions: int = 0

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def n_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def remaining(self) -> int:
        return self.n_tokens - self.n_computed


@dataclasses.dataclass
class Scheduled:
    request: Request
    n: int                           # tokens of the request that run in this step
    # whether this portion reaches the request's last token, so that a token is drawn after it
    samples: bool = False

    def __post_init__(self):
        self.samples = self.request.n_computed + self.n == self.request.n_tokens


class Scheduler:
    def __init__(self, cache, max_batch_tokens: int, chunk_size: int, max_num_seqs: int,
                 max_positions: Optional[int]):
        if max_batch_tokens < 1 or chunk_size < 1 or max_num_seqs < 1:
            raise ValueError("max_batch_tokens, chunk_size and max_num_seqs must be positive")
        self.cache = cache
        self.max_batch_tokens, self.chunk_size = max_batch_tokens, chunk_size
        self.max_num_seqs = min(max_num_seqs, cache.max_seqs)
        self.max_positions = max_positions
        self.waiting: Deque[Request] = collections.deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self._clock = 0
        self.num_preemptions = 0

    # ----------------------------------------------------------- requests
    def add(self, req: Request) -> None:
        req.params.validate()
        if not req.prompt:
            raise ValueError("a request needs at least one prompt token")
        limit = self.max_positions
        if limit is not None and len(req.prompt) > limit:
            raise ValueError(f"a prompt of {len(req.prompt)} tokens exceeds the limit of {limit} positions per request")
        req.state = WAITING
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def take_finished(self) -> List[Request]:
        """The requests that finished since the last call (the scheduler keeps none of them)."""
        done, self.finished = self.finished, []
        return done

    def abort(self, req: Request) -> None:
        """Take a request out of the queues now; its slot and pages are free when this returns.  Tokens a
        step in flight draws for it are dropped (``update`` and ``resolve`` skip it)."""
        if req.state == FINISHED:
            return
        if req.state == WAITING:
            self.waiting.remove(req)
        req.output = [t for t in req.output if t != PENDING]
        self._finish(req, "aborted")

    # ----------------------------------------------------------- one step
    def schedule(self) -> List[Scheduled]:
        """Decide the next step and reserve its pages.  May preempt; may return [] only when idle."""
        while True:
            plan = self._try_schedule()
            if plan or not self.has_work():
                return plan
            # nothing could be scheduled although there is work: no running request can move and
            # none can be admitted.  Free the pages of the request admitted last; or give up on a
            # request that cannot move although it is the only one that holds pages (preempted, it
            # would start again and come to the same place for ever), or that cannot even start in
            # an empty pool.
            if len(self.running) > 1:
                self._preempt(max(self.running, key=lambda r: r.admitted_at))
            elif self.running:
                self._finish(self.running[0], "cache_full")
            else:
                req = self.waiting.popleft()
                self._finish(req, "cache_full")

    def _try_schedule(self) -> List[Scheduled]:
        budget = self.max_batch_tokens
        plan: List[Scheduled] = []
        preemptions_before = self.num_preemptions
        # 1. one token for every decoding request (oldest first); preempt the youngest when a page is missing
        for req in sorted(self.running, key=lambda r: r.admitted_at):
            if req.state != RUNNING or req.remaining != 1 or budget < 1:
                continue
            while not self.cache.reserve(req.slot, req.n_computed, req.n_computed + 1):
                victims = [r for r in self.running if r is not req and r.state == RUNNING
                           and not any(s.request is r for s in plan)]
                if not victims:
                    break
                self._preempt(max(victims, key=lambda r: r.admitted_at))
            else:
                plan.append(Scheduled(req, 1))
                budget -= 1
                continue
            # no page even after preempting everyone that is not already in the plan
            if len(self.running) == 1 and not plan:
                self._finish(req, "cache_full")
        # 2. prompt portions of running requests
        for req in sorted(self.running, key=lambda r: r.admitted_at):
            if req.state != RUNNING or req.remaining <= 1 or budget < 1:
                continue
            n = self._fit_portion(req, min(req.remaining, self.chunk_size, budget))
            if n > 0:
                plan.append(Scheduled(req, n))
                budget -= n
        # 3. admit waiting requests, first come first served; not in a step that had to preempt
        #    (the pages just freed are for the requests that stayed).  A newcomer is admitted only if
        #    the free pages cover all the tokens it holds, after what the running requests will still
        #    ask for to get through theirs: admitted on the strength of one portion it would run into
        #    the others half-way, be preempted and start again (simulated with pools a fifth of the
        #    load: 3-5 times the useful tokens computed, against 1.1-1.3 times this way).
        portion = min(self.chunk_size, self.max_batch_tokens)
        groups = self.cache.groups
        promised = None
        while (self.waiting and budget >= 1 and len(self.running) < self.max_num_seqs
               and self.num_preemptions == preemptions_before):
            req = self.waiting[0]
            need = self.cache.pages_to_come(None, len(req.tokens), portion)
            if any(n > g.pool.num_pages for n, g in zip(need, groups)):
                self.waiting.popleft()                 # its tokens alone exceed the pool
                self._finish(req, "cache_full")
                continue
            if promised is None:
                promised = [0] * len(groups)
                for r in self.running:
                    if r.state == RUNNING:
                        for k, v in enumerate(self.cache.pages_to_come(r.slot, len(r.tokens), portion)):
                            promised[k] += v
            if any(n > g.pool.num_free - p for n, g, p in zip(need, groups, promised)):
                break
            slot = self.cache.alloc_slot()
            if slot is None:
                break
            req.slot = slot
            n = min(req.remaining, self.chunk_size, budget)
            if not self.cache.reserve(slot, req.n_computed, req.n_computed + n):
                self.cache.free_slot(slot)
                req.slot = None
                break
            for k, v in enumerate(self.cache.pages_to_come(slot, len(req.tokens), portion)):
                promised[k] += v
            self.waiting.popleft()
            req.state = RUNNING
            req.admitted_at = self._clock
            self._clock += 1
            self.running.append(req)
            plan.append(Scheduled(req, n))
            budget -= n
        return plan

    def _fit_portion(self, req: Request, n: int) -> int:
        """Reserve pages for up to n further tokens of req; returns how many got pages (page-granular)."""
        start = req.n_computed
        while n > 0:
            if self.cache.reserve(req.slot, start, start + n):
                return n
            # shorten to the last page boundary that is still inside the portion
            ps = self.cache.page_size
            cut = ((start + n - 1) // ps) * ps - start
            n = cut if cut < n else n - 1
        return 0

    def _preempt(self, req: Request) -> None:
        self.cache.free_slot(req.slot)
        req.slot, req.n_computed, req.state = None, 0, WAITING
        req.preemptions += 1
        self.num_preemptions += 1
        self.running.remove(req)
        self.waiting.appendleft(req)

    def _finish(self, req: Request, reason: str) -> None:
        if req.slot is not None:
            self.cache.free_slot(req.slot)
            req.slot = None
        if req in self.running:
            self.running.remove(req)
        req.state, req.finish_reason = FINISHED, reason
        self.finished.append(req)

    # ------------------------------------------------------ after the step
    def update(self, plan: Sequence[Scheduled], sampled: Sequence[int]) -> List[Request]:
        """Account for a step that ran: ``sampled`` has one token for every entry whose ``samples`` is true,
        in plan order.  Returns the requests that finished."""
        done: List[Request] = []
        k = 0
        for s in plan:
            req = s.request
            draws = s.samples
            if req.state == FINISHED:
                # it ended (on a token read later than this step was launched) while the step ran:
                # what the step computed for it is dropped
                k += 1 if draws else 0
                continue
            req.n_computed += s.n
            if not draws:
                continue
            tok = int(sampled[k])
            k += 1
            req.output.append(tok)
            p = req.params
            reason = None
            if tok != PENDING and p.eos_id is not None and tok == p.eos_id and not p.ignore_eos:
                reason = "eos"
            elif len(req.output) >= p.max_new_tokens:
                reason = "length"
            elif self.max_positions is not None and req.n_tokens >= self.max_positions:
                reason = "positions"      # the next token would have no position left
            if reason:
                self._finish(req, reason)
                done.append(req)
        if k != len(sampled):
            raise ValueError("the number of sampled tokens does not match the plan")
        return done

    # ------------------------------------- the same in two halves, for steps launched ahead of their tokens
    def update_pending(self, plan: Sequence[Scheduled]) -> Tuple[List[Request], List[Optional[Tuple[Request, int]]]]:
        """Account for a step whose sampled tokens are still on the GPU: every drawing request gets a
        PENDING token (so the next step can be decided and launched) and may finish by length.  Returns
        the finished requests and, per drawn token in plan order, (request, index of the token in its
        output), or None where the step's result is dropped; ``resolve`` takes that list."""
        handles: List[Optional[Tuple[Request, int]]] = []
        n = 0
        for s in plan:
            if s.samples:
                n += 1
                handles.append(None if s.request.state == FINISHED else (s.request, len(s.request.output)))
        return self.update(plan, [PENDING] * n), handles

    def resolve(self, handles: Sequence[Optional[Tuple[Request, int]]], sampled: Sequence[int]) -> List[Request]:
        """Put the tokens of a step accounted for by ``update_pending`` in their places; a request whose
        token is its end-of-sequence token finishes now, and what a later step computed for it is
        dropped.  Returns the requests that finished here."""
        if len(handles) != len(sampled):
            raise ValueError("the number of sampled tokens does not match the plan")
        done: List[Request] = []
        for h, tok in zip(handles, sampled):
            if h is None:
                continue
            req, idx = h
            if req.finish_reason == "aborted":
                continue
            tok = int(tok)
            req.output[idx] = tok
            p = req.params
            if p.eos_id is None or tok != p.eos_id or p.ignore_eos:
                continue
            if req.state == FINISHED:
                req.finish_reason = "eos"        # it also was its last token by length
                continue
            del req.output[idx + 1:]
            if req.state == WAITING:             # preempted meanwhile
                self.waiting.remove(req)
            req.n_computed = min(req.n_computed, req.n_tokens)
            self._finish(req, "eos")
            done.append(req)
        return done
