"""The Python entry point: requests in, tokens out.

``LLMEngine`` ties the model, the cache manager, the step function, the
scheduler and the sampler together.  ``generate`` is the call a user makes;
``step`` runs one scheduler decision through the GPU.

The reference's counterpart is the static-batch loop ``run_batched_inference``
(src/examples/lib/inference_batch.cc:15-232) and, from Python,
``torch.classes.gpt_ops.OptOp.forward`` (src/csrc/pybinding.cc:53-62), which
leaves batching, block allocation and stopping to its caller.
"""
from __future__ import annotations

import dataclasses
import itertools
from typing import Any, Dict, Iterable, List, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager
from ..models.base import CausalLM
from ..models.registry import load_model
from ..sampling.sampler import Sampler, SamplingParams
from .scheduler import PENDING, Request, Scheduled, Scheduler
from .step import ModelRunner, StepEntry


@dataclasses.dataclass
class EngineConfig:
    page_size: int = 16                 # the reference's block_size (src/examples/run_gpt.cc:93-96)
    num_pages: Optional[int] = None     # None: sized from free device memory
    memory_fraction: float = 0.85       # share of the free device memory the cache may take
    max_batch_tokens: int = 2048        # token budget of one step
    # longest prompt portion: as long as the budget (a 2048-token prompt takes 5.9 ms whole, 8.7 ms in portions
    # of 512: every step reads all weights once)
    chunk_size: int = 2048
    max_num_seqs: int = 256             # most requests running at a time
    # most tokens one request may hold (prompt and output): block tables have room for this many.  None: the
    # model's own limit (its context length or what its position encoding can encode), and for a model
    # that sets none, DEFAULT_MAX_SEQ_LEN
    max_seq_len: Optional[int] = None
    use_cuda_graphs: bool = True        # record decode-only steps once per batch size and replay them
    # launch the next step before the tokens of this one have been read: they reach it on the device, and
    # the host's work for a step (scheduling, staging, the read itself) overlaps the GPU's
    pipeline: bool = True
    # NVTX ranges around every step and, in steps that are launched kernel by kernel, around every layer
    # (a profiler's timeline then shows them; recorded steps replay as one graph launch)
    nvtx: bool = False


DEFAULT_MAX_SEQ_LEN = 4096


class _Launched:
    """A step that is on the GPU: its plan and where its sampled tokens are."""

    def __init__(self, plan: List[Scheduled]):
        self.plan = plan
        self.n_samples = 0
        self.sampled: Optional[torch.Tensor] = None      # int32 on the device
        self.host: Optional[torch.Tensor] = None         # its copy in pinned memory, valid after `event`
        self.event = None
        self.sample_index: Dict[int, int] = {}           # id(request) -> row of `sampled`

    def fetch(self) -> List[int]:
        if self.n_samples == 0:
            return []
        if self.event is not None:
            self.event.synchronize()
            return self.host[:self.n_samples].tolist()
        return self.sampled.tolist()


class LLMEngine:
    def __init__(self, model: Union[str, CausalLM], dtype="bfloat16", device="cuda",
                 config: Optional[EngineConfig] = None, **overrides):
        cfg = dataclasses.replace(config or EngineConfig(), **overrides)
        self.config = cfg
        self.model = load_model(model, dtype, device) if isinstance(model, str) else model
        self.device = self.model.device
        specs = self.model.definition.cache_specs()
        limits = [n for n in (self.model.max_positions, cfg.max_seq_len) if n is not None]
        max_len = min(limits) if limits else DEFAULT_MAX_SEQ_LEN
        if max_len < 1:
            raise ValueError("max_seq_len must be positive")
        self.max_seq_len = max_len
        num_pages = cfg.num_pages
        if num_pages is None:
            num_pages = self._pages_that_fit(specs, cfg, max_len)
        self.cache = CacheManager(specs, self.model.dtype, self.device, cfg.page_size, num_pages,
                                  cfg.max_num_seqs, max_len)
        self.runner = ModelRunner(self.model, self.cache, cfg.max_batch_tokens,
                                  use_cuda_graphs=cfg.use_cuda_graphs)
        self.runner.nvtx = cfg.nvtx
        self.scheduler = Scheduler(self.cache, cfg.max_batch_tokens, cfg.chunk_size, cfg.max_num_seqs, max_len)
        self.sampler = Sampler(self.device)
        self._ids = itertools.count()
        self.requests: Dict[Any, Request] = {}
        self._stats = dict(steps=0, prompt_tokens=0, decode_tokens=0)
        self._inflight: Optional[_Launched] = None
        # sampled tokens come back through pinned buffers used in turn (a step's buffer is read before
        # the step after next is launched)
        pin = self.device.type == "cuda"
        self._token_bufs = [torch.zeros(cfg.max_num_seqs, dtype=torch.int32, pin_memory=pin) for _ in range(3)]
        self._token_turn = 0

    def _pages_that_fit(self, specs, cfg: EngineConfig, max_len: int) -> int:
        """Pages per group so that the cache (every group's pages, and the fixed-size state of every
        request slot) takes ``memory_fraction`` of the free device memory, and no more than all slots
        filled to the length limit would need."""
        from ..parts.base import PagedKVSpec, StateSpec
        esize = torch.empty((), dtype=self.model.dtype).element_size()
        per_page = sum(2 * s.num_kv_heads * s.head_dim * cfg.page_size * esize
                       for s in specs if isinstance(s, PagedKVSpec))
        if per_page == 0:
            return 1
        state_bytes = 0
        for s in specs:
            if isinstance(s, StateSpec):
                n = cfg.max_num_seqs * torch.empty((), dtype=s.dtype).element_size()
                for k in s.shape:
                    n *= k
                state_bytes += n
        if self.device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(self.device)
        else:
            free = 1 << 30
        want = cfg.max_num_seqs * ((max_len + cfg.page_size - 1) // cfg.page_size)
        return max(1, min(want, (int(free * cfg.memory_fraction) - state_bytes) // per_page))

    @property
    def stats(self) -> Dict[str, int]:
        """Counters since the engine was made: steps, prompt and decode tokens run, requests preempted;
        and the page pool now (pages free and in all; the smallest group's where there are several)."""
        return dict(self._stats, preemptions=self.scheduler.num_preemptions, pages_free=self.cache.free_pages,
                    pages_total=self.cache.total_pages, running=len(self.scheduler.running),
                    waiting=len(self.scheduler.waiting))

    # ------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, request_id=None):
        rid = request_id if request_id is not None else next(self._ids)
        if rid in self.requests:
            raise ValueError(f"request id {rid!r} is already in use")
        prompt = [int(t) for t in prompt]
        vocab = self.model.vocab_size
        for t in prompt:
            if t < 0 or t >= vocab:
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        req = Request(rid, prompt, params or SamplingParams())
        self.scheduler.add(req)
        self.requests[rid] = req
        return rid

    def pop_request(self, request_id) -> Request:
        """Hand a finished request over (tokens in ``output``, why it ended in ``finish_reason``) and forget it;
        ``generate`` does this itself, a caller of ``add_request`` and ``step`` does it when ``step`` has
        returned the request."""
        req = self.requests[request_id]
        if req.finish_reason is None:
            raise ValueError(f"request {request_id!r} has not finished")
        return self.requests.pop(request_id)

    def abort_request(self, request_id) -> Request:
        """Take a request out, wherever it is: waiting, running, or with a token still on its way from a
        step that has been launched ahead.  Its pages and slot are free when this returns (a step in
        flight may still write the pages; whoever gets them next writes them after it, in stream
        order, and reads only what it wrote itself), what steps in flight compute for it is dropped, and
        no later ``step`` reports it.  Returns the request with the tokens it had got (``finish_reason``
        "aborted", or what it finished with if it already had).  The reference's nearest thing is the
        removal of finished requests from its static batch (src/examples/lib/inference_batch.cc:196-218)."""
        req = self.requests.pop(request_id)
        if req.finish_reason is None:
            self.scheduler.abort(req)
        return req

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    # ---------------------------------------------------------------- step
    def _launch(self, plan: List[Scheduled], prev: Optional[_Launched]) -> _Launched:
        """Put one scheduler decision on the GPU (step and sampling); nothing here waits for the GPU.
        Tokens that are still PENDING are taken on the device from ``prev``, the step that drew them."""
        out = _Launched(plan)
        entries, samplers, counters = [], [], []
        token_from: List[int] = []
        for s in plan:
            r = s.request
            toks = r.tokens[r.n_computed:r.n_computed + s.n]
            for j, t in enumerate(toks):
                if t == PENDING:
                    if prev is None or id(r) not in prev.sample_index:
                        raise RuntimeError("a token that was never drawn is waited for")
                    token_from.append(prev.sample_index[id(r)])
                    toks[j] = 0
                else:
                    token_from.append(-1)
            entries.append(StepEntry(r.slot, toks, r.n_computed, [s.n - 1] if s.samples else []))
            if s.samples:
                out.sample_index[id(r)] = len(samplers)
                samplers.append(r.params)
                counters.append(len(r.output))
            if s.n == 1 and r.n_computed >= len(r.prompt):
                self._stats["decode_tokens"] += 1
            else:
                self._stats["prompt_tokens"] += s.n
        feedback = (prev.sampled, token_from) if prev is not None and any(f >= 0 for f in token_from) else None
        if self.config.nvtx and self.device.type == "cuda":
            torch.cuda.nvtx.range_push(f"step {self._stats['steps']}: {len(entries)} requests, "
                                       f"{sum(len(e.tokens) for e in entries)} tokens")
            try:
                logits = self.runner.step(entries, feedback)
            finally:
                torch.cuda.nvtx.range_pop()
        else:
            logits = self.runner.step(entries, feedback)
        self._stats["steps"] += 1
        if samplers:
            out.n_samples = len(samplers)
            out.sampled = self.sampler.sample_on_device(logits, samplers, counters)
            if self.device.type == "cuda":
                self._token_turn = (self._token_turn + 1) % len(self._token_bufs)
                out.host = self._token_bufs[self._token_turn]
                out.host[:out.n_samples].copy_(out.sampled, non_blocking=True)
                out.event = torch.cuda.Event()
                out.event.record()
        return out

    def step(self) -> List[Request]:
        """One scheduler decision through the GPU; returns the requests that finished in it.

        With ``pipeline`` the step after this one is decided and launched before this one's tokens are
        read (requests continue from PENDING tokens that the GPU fills in): a request that ends on an
        end-of-sequence token is then reported one call later than it was computed, and the token the
        step ahead computed for it is dropped."""
        cur, self._inflight = self._inflight, None
        if cur is None:
            plan = self.scheduler.schedule()
            if not plan:
                return self._drain_finished([])
            cur = self._launch(plan, None)
        if cur.n_samples == 0:
            return self._drain_finished(self.scheduler.update(cur.plan, []))
        if not self.config.pipeline:
            return self._drain_finished(self.scheduler.update(cur.plan, cur.fetch()))
        done, handles = self.scheduler.update_pending(cur.plan)
        if self.scheduler.has_work():
            ahead = self.scheduler.schedule()
            if ahead:
                self._inflight = self._launch(ahead, cur)
        done += self.scheduler.resolve(handles, cur.fetch())
        return self._drain_finished(done)

    def _drain_finished(self, done: List[Request]) -> List[Request]:
        """``done`` and whatever else the scheduler finished since the last call (requests it gave up on
        with cache_full finish without a step of their own); aborted requests are not reported."""
        seen = {id(r) for r in done}
        for r in self.scheduler.take_finished():
            if id(r) not in seen and self.requests.get(r.id) is r:
                seen.add(id(r))
                done.append(r)
        return [r for r in done if self.requests.get(r.id) is r]

    # ------------------------------------------------------------- warm-up
    def warm_up(self, prompt_lengths: Sequence[int] = (), batch_sizes: Sequence[int] = (1,)) -> int:
        """Run throw-away requests so that the recorded steps they need exist before real ones arrive
        (recording a step costs tens of milliseconds, replaying it tens of microseconds): one prompt of each
        given length, and for each batch size that many one-token prompts decoding together.  Needs an idle
        engine; leaves cache and statistics as they were.  Returns how many recorded steps were added."""
        if self.has_work():
            raise RuntimeError("warm_up needs an engine without requests")
        r = self.runner
        before = len(r._graphs) + len(r._step_graphs)
        stats = dict(self._stats)
        limit = self.max_seq_len
        for n in prompt_lengths:
            n = max(1, min(int(n), limit - 2 if limit else int(n)))
            self.generate([[0] * n], SamplingParams(max_new_tokens=2, ignore_eos=True))
        for b in batch_sizes:
            b = max(1, min(int(b), self.config.max_num_seqs))
            self.generate([[0]] * b, SamplingParams(max_new_tokens=3, ignore_eos=True))
        self._stats = stats
        return len(r._graphs) + len(r._step_graphs) - before

    # ------------------------------------------------------------ generate
    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[None, SamplingParams, Sequence[SamplingParams]] = None) -> List[List[int]]:
        """Generate for every prompt (token ids in, token ids out), batching them continuously."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        ids = [self.add_request(p, dataclasses.replace(sp)) for p, sp in zip(prompts, params)]
        while self.has_work():
            self.step()
        out = [self.requests[i].output for i in ids]
        for i in ids:
            del self.requests[i]
        return out
