"""Per-operation device times without a profiler.

``start()`` wraps every public operation of ``swifttransformer_b200.ops`` in a pair of CUDA events on the
current stream; ``stop()`` removes the wrappers and returns, per operation name, how often it ran and how many
milliseconds it took on the device.  Meant for steps that are launched kernel by kernel
(``LLMEngine(..., use_cuda_graphs=False)`` or ``ModelRunner(..., use_cuda_graphs=False)``): inside a recorded
step the events are not part of the recording and the times are meaningless.  Times of back-to-back launches
include the gaps between them; compare shares, not absolutes.

The reference times whole phases with a wall clock around a device synchronisation
(src/examples/lib/inference_batch.cc:102-105,126,161,222-231) and has no per-kernel timing.
"""
from __future__ import annotations

import functools
from typing import Dict, List, Tuple

import torch

TIMED = ("embed", "add_positions", "add_norm", "bias_act", "scatter_i32", "gather_where_i32", "linear", "gemm_plain",
         "gemm_skinny", "gemm_stream_tc", "norm_linear", "linear_add", "norm_qkv_linear_to_cache", "qkv_linear_to_cache",
         "qkv_to_cache", "attention_plain", "attention_decode", "attention_decode_qkv", "attention_prefill",
         "linear_parts", "argmax", "sample")

_originals: Dict[str, object] = {}
_events: List[Tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
_depth = 0


def start() -> None:
    """Begin timing: every operation in TIMED is wrapped (an operation that calls another one, as ``linear`` calls
    ``gemm_skinny``, is timed as a whole; the inner call is not counted again)."""
    from .. import ops
    if _originals:
        raise RuntimeError("timing is already on")
    _events.clear()
    for name in TIMED:
        fn = getattr(ops, name)
        _originals[name] = fn
        setattr(ops, name, _wrap(name, fn))


def _wrap(name, fn):
    @functools.wraps(fn)
    def timed(*args, **kwargs):
        global _depth
        if _depth:
            return fn(*args, **kwargs)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        _depth += 1
        e0.record()
        try:
            return fn(*args, **kwargs)
        finally:
            e1.record()
            _depth -= 1
            _events.append((name, e0, e1))
    return timed


def stop() -> Dict[str, Dict[str, float]]:
    """End timing; returns {operation: {"calls": n, "ms": total device milliseconds}}, largest total first."""
    from .. import ops
    for name, fn in _originals.items():
        setattr(ops, name, fn)
    _originals.clear()
    torch.cuda.synchronize()
    out: Dict[str, Dict[str, float]] = {}
    for name, e0, e1 in _events:
        rec = out.setdefault(name, {"calls": 0, "ms": 0.0})
        rec["calls"] += 1
        rec["ms"] += e0.elapsed_time(e1)
    _events.clear()
    return dict(sorted(out.items(), key=lambda kv: -kv[1]["ms"]))
