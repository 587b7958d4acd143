"""A causal language model as data: parts, and the order in which layers run.

``ModelDef`` is what an architecture's builder returns; ``CausalLM`` binds it
to weights and runs one step's tokens through it.  The order of execution is a
list of ``LayerStep`` entries: which block runs, and which cache entry it uses.
A block may appear more than once (its weights are then shared), and a step may
point at a cache entry that an earlier step owns (``writes_cache=False``: it
reads that layer's keys and values and writes none).

The reference's model loop is src/csrc/model/gpt/gpt.cc:226-504 (layers) and
:507-657 (embedding, layers, final norm, gather, output product, argmax).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, List, Optional

import torch

from ..config.base import ModelConfig
from ..parts.base import Part
from ..parts.block import Block, ResidualStream
from ..parts.embedding import Embedding, OutputHead
from ..parts.norm import Norm
from ..parts.position import PositionEncoding
from ..weights.spec import ParamSpec


@dataclasses.dataclass(frozen=True)
class LayerStep:
    block: int                  # index into ModelDef.blocks
    cache: int                  # index of the cache entry this step uses
    writes_cache: bool = True   # False: reads the entry another step fills


@dataclasses.dataclass
class ModelDef:
    config: ModelConfig
    embedding: Embedding
    position: PositionEncoding
    blocks: List[Block]
    layer_order: List[LayerStep]
    final_norm: Optional[Norm]
    head: OutputHead
    # maps a tensor name found in a checkpoint to the name the parts use
    # (None: ignore the tensor)
    canonical_name: Optional[Callable[[str], Optional[str]]] = None
    # the most tokens a request may hold (the architecture's context length, from its configuration);
    # None: whatever the position encoding allows, and where that has no limit, the engine's own setting
    max_seq_len: Optional[int] = None

    def parts(self) -> List[Part]:
        out: List[Part] = [self.embedding, self.position]
        for b in self.blocks:
            out.append(b)
        if self.final_norm is not None:
            out.append(self.final_norm)
        out.append(self.head)
        return out

    def all_parts(self) -> List[Part]:
        flat: List[Part] = []

        def walk(p: Part):
            flat.append(p)
            for c in p.children():
                walk(c)
        for p in self.parts():
            walk(p)
        return flat

    def param_specs(self) -> List[ParamSpec]:
        specs: List[ParamSpec] = []
        seen = set()
        for p in self.all_parts():
            for s in p.param_specs():
                if s.name in seen:
                    raise ValueError(f"two parts ask for the tensor '{s.name}'")
                seen.add(s.name)
                specs.append(s)
        return specs

    def num_cache_entries(self) -> int:
        return 1 + max((s.cache for s in self.layer_order), default=-1)

    def cache_specs(self) -> List[Any]:
        """The cache need of every cache entry (PagedKVSpec, StateSpec or None), by entry index."""
        specs: List[Any] = [None] * self.num_cache_entries()
        owner = [False] * len(specs)
        for st in self.layer_order:
            spec = self.blocks[st.block].mixer.cache_spec()
            if st.writes_cache:
                if owner[st.cache]:
                    raise ValueError(f"cache entry {st.cache} is written by two layer steps")
                owner[st.cache] = True
                specs[st.cache] = spec
        for st in self.layer_order:
            if not st.writes_cache:
                spec = self.blocks[st.block].mixer.cache_spec()
                if not owner[st.cache]:
                    raise ValueError(f"cache entry {st.cache} is read but no layer step writes it")
                if spec != specs[st.cache]:
                    raise ValueError(f"layer step reads cache entry {st.cache} whose shape differs from its own")
        return specs


class CausalLM:
    """A ModelDef bound to weights on a device, in one compute dtype."""

    def __init__(self, model_def: ModelDef, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device):
        self.definition = model_def
        self.config = model_def.config
        self.dtype, self.device = dtype, device
        tensors = dict(tensors)
        for p in model_def.all_parts():
            p.bind(tensors)
        self.embedding, self.position = model_def.embedding, model_def.position
        self.blocks, self.layer_order = model_def.blocks, model_def.layer_order
        self.final_norm, self.head = model_def.final_norm, model_def.head

    @property
    def vocab_size(self) -> int:
        return self.head.vocab

    @property
    def max_positions(self) -> Optional[int]:
        """The most tokens a request may hold: the smaller of the architecture's context length and what
        the position encoding can encode (None: neither sets a limit)."""
        limits = [n for n in (self.definition.max_seq_len, self.position.max_positions()) if n is not None]
        return min(limits) if limits else None

    def graph_safe(self) -> bool:
        return all(b.mixer.graph_safe for b in self.blocks)

    def step_plans(self) -> List[Any]:
        """The step plans (parts.base.StepPlan) of the model's mixers, one per name, in layer order."""
        plans: Dict[str, Any] = {}
        for st in self.layer_order:
            p = self.blocks[st.block].mixer.step_plan()
            if p is not None and p.name not in plans:
                plans[p.name] = p
        return list(plans.values())

    def forward(self, ctx: Any, caches: List[Any]) -> Optional[torch.Tensor]:
        """Run the step described by ``ctx``; float32 logits [len(want), vocab] or None if nothing is wanted."""
        x = self.embedding.forward(ctx.token_ids, ctx.positions, self.position)
        stream = ResidualStream(x, self.dtype)
        nvtx = getattr(ctx, "nvtx", False)
        for i, st in enumerate(self.layer_order):
            if nvtx:
                torch.cuda.nvtx.range_push(f"layer {i} (block {st.block})")
            self.blocks[st.block].forward(stream, ctx, caches[st.cache].view(st.writes_cache))
            if nvtx:
                torch.cuda.nvtx.range_pop()
        if ctx.n_want == 0:
            return None
        if self.final_norm is not None:
            h = self.final_norm.apply(stream.x, stream.pending, act_dtype=self.dtype, rows=ctx.want_rows)
        else:
            h = stream.materialise(rows=ctx.want_rows)
        return self.head.forward(h)

    def step_param_bytes(self) -> int:
        """Bytes of parameters one step reads (each layer step counts its block once)."""
        total = self.embedding.param_bytes() + self.head.param_bytes()
        if self.final_norm is not None:
            total += self.final_norm.param_bytes()
        for st in self.layer_order:
            b = self.blocks[st.block]
            total += sum(c.param_bytes() for c in b.children())
        return total
