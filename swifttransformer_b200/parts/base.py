"""Interfaces of the parts a model is put together from.

A model is: an embedding, a position encoding, a list of blocks, an order in
which the blocks run, a final norm and an output head.  A block is put
together from a mixer (attention here), a feed-forward and norms.  Every part
takes its sizes and constants as constructor arguments, declares the tensors
it wants from the checkpoint (``param_specs``) and receives them in ``bind``.
No part knows which model it is in; which parts a layer has is decided by the
architecture's builder, layer by layer, from the configuration.

The reference's counterpart is procedural: ``st::layer::attention`` and
``st::layer::ffn`` take raw pointers and their sizes as parameters
(src/csrc/layer/attention.h:8-53, src/csrc/layer/ffn.h:11-31) and the block
order is written out in src/csrc/model/gpt/gpt.cc:304-503.

Interfaces
----------
Mixer.cache_spec()        -> PagedKVSpec | StateSpec | None
Mixer.step_plan()         -> StepPlan | None  (host work once per step, see StepPlan)
Mixer.forward(h, ctx, cache) -> Delta         h: [N, width] activations
FeedForward.forward(h, ctx)  -> Delta
Mixer.forward_into_residual(x, norm, ctx, cache, pending), FeedForward.forward_into_residual(x, norm, ctx, pending)
                          optional: the whole sub-layer with its norm and residual sum fused in, in place
Norm.apply(x, delta, ...)    -> see parts.norm
PositionEncoding.table()     -> (table, offset) for encodings added to the hidden state
Block.forward(stream, ctx, cache) -> None (updates the residual stream)

``Delta`` is what a sub-layer hands back: ``value + bias`` (bias broadcast over
rows) is to be added to the residual stream.  Leaving the sum to the consumer
lets the next norm kernel do residual add, bias add and normalisation in one
pass over the row.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..weights.spec import ParamSpec


@dataclasses.dataclass
class Delta:
    """What a sub-layer leaves to be added to the residual stream: a tensor in the activation dtype, a bias,
    and/or float32 parts [n, N, width] to be added in order (the slices of k of a product that did not meet
    in the product's own kernel)."""
    value: Optional[torch.Tensor]        # [N, width], activation dtype, or None
    bias: Optional[torch.Tensor] = None  # [width] float32
    parts: Optional[torch.Tensor] = None  # [n, N, width] float32


@dataclasses.dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values per token, kept in pages.  ``window`` None: all keys stay."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size (``shape`` per request), zero when a request starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base of all parts."""

    def param_specs(self) -> List[ParamSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take this part's tensors out of ``tensors`` (name -> device tensor)."""

    def children(self) -> List["Part"]:
        return []

    # bytes of parameters this part reads in one step (for roofline accounting)
    def param_bytes(self) -> int:
        return 0


class StepPlan:
    """Host work that a kind of mixer needs done once per step, before any layer runs.

    The step function knows tokens, requests and wanted rows; how a mixer's kernels cut a step's work
    (which tokens go to which kernel, in tiles of how many rows, over how many keys) is the mixer's
    business.  A mixer that needs index arrays of its own returns a StepPlan from ``step_plan()``.
    The step function gives every plan of the model room in the step's staging buffer (one pinned buffer,
    one copy per step), lets it fill that room on the host, and hands what ``view`` returns to the mixers
    through ``ctx.plan(name)``.  Plans are shared by name: all mixers that return a plan called
    "paged_attention" read the same arrays.

    A step is described to a plan by three int arrays (numpy, one element per request of the step):
    ``lens`` (new tokens), ``q_start`` (offset of its first token among the step's tokens, one element more
    than requests) and ``start`` (tokens it already has in the cache).

    Steps are recorded as CUDA graphs of fixed shape and replayed; a recording made for ``n_cap`` tokens and
    ``b_cap`` requests serves every step that fits and whose ``shape_key`` is equal.  ``fill`` must pad what
    the step does not use with entries the mixer's kernels skip.
    """

    name = ""
    # tokens of a recorded step are padded to a multiple of this (the row count of the mixer's tiles)
    token_multiple = 1

    def words(self, n_cap: int, b_cap: int) -> int:
        """int32 words this plan wants for a step of at most n_cap tokens in b_cap requests."""
        return 0

    def shape_key(self, lens, start, n_cap: int, b_cap: int) -> Tuple:
        """What a recorded step must agree in, beside n_cap and b_cap, to serve this step (padded counts,
        never exact ones: every new key is a new recording)."""
        return ()

    def fill(self, lens, q_start, start, out, n_cap: int, b_cap: int) -> Tuple:
        """Write the plan's arrays for this step into ``out`` (numpy int32, ``words(n_cap, b_cap)`` long);
        returns the key that describes the step exactly, in the form ``shape_key`` returns."""
        return ()

    def view(self, dev: torch.Tensor, key: Tuple, n_cap: int, b_cap: int) -> Any:
        """What the mixers get from ``ctx.plan(name)``: built over ``dev`` (the device copy of the words)
        for a step described by ``key`` (an exact key, or a padded one when the step is recorded)."""
        return None


class Mixer(Part):
    # False for mixers whose forward does host-side work that cannot be
    # recorded into a CUDA graph (the engine then runs them eagerly).
    graph_safe = True

    def cache_spec(self):
        return None

    def step_plan(self) -> Optional[StepPlan]:
        return None

    def forward(self, h: torch.Tensor, ctx: Any, cache: Any) -> Delta:
        raise NotImplementedError

    def forward_into_residual(self, x: torch.Tensor, norm: Any, ctx: Any, cache: Any,
                              pending: Optional[Delta] = None) -> Any:
        """Optional fast path of a pre-norm block: x <- (x + pending) + mixer(norm(x + pending)) in place on the
        float32 residual rows x, with the norm (a parts.norm.Norm: its kind, gain, shift and eps) and the sum with
        ``pending`` (what the sub-layer before left to be added) in the mixer's first kernel and the residual sum
        in its last.  Returns False, having changed nothing, when it does not apply to this step (the block then
        calls ``norm.apply`` and ``forward``); True when x is complete; or a Delta that is still to be added to x."""
        return False


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx: Any) -> Delta:
        raise NotImplementedError

    def forward_into_residual(self, x: torch.Tensor, norm: Any, ctx: Any, pending: Optional[Delta] = None) -> Any:
        """Optional fast path of a pre-norm block: x <- (x + pending) + feed_forward(norm(x + pending)) in place
        (see Mixer: False, True, or a Delta still to be added)."""
        return False


class Registry:
    """Name -> constructor for one kind of part."""

    def __init__(self, kind: str):
        self.kind = kind
        self._items: Dict[str, Callable[..., Any]] = {}

    def register(self, name: str, ctor: Optional[Callable[..., Any]] = None):
        def deco(c):
            self._items[name] = c
            return c
        return deco(ctor) if ctor is not None else deco

    def build(self, kind_name: str, /, **kwargs):
        if kind_name not in self._items:
            raise KeyError(f"unknown {self.kind} '{kind_name}'; registered: "
                           f"{', '.join(sorted(self._items)) or '(none)'}")
        return self._items[kind_name](**kwargs)

    def names(self) -> List[str]:
        return sorted(self._items)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")
