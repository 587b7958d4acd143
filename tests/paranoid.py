"""A checking mode for the engine: after every device operation, compare what the kernel wrote with what the
plain CPU reference of the same operation (tests/cpu_ops.py) makes of the same inputs.

``with paranoid.watch() as log:`` wraps the operations of ``swifttransformer_b200.ops``; inside, every call
copies its tensor arguments to the CPU, runs the kernel, runs the CPU reference on the copies, and compares the
outputs (tensors the operation returns or writes in place) within a bound that depends on the storage type.  A
difference raises ``ParanoidError`` naming the operation, its place in the step and the worst element.  It is
slow by design (a device synchronisation and a CPU computation per kernel) and meant for tiny models launched
kernel by kernel; it stands in for the memory checkers that cannot run on this kind of machine.  The reference
has nothing comparable (its debug build synchronises after every kernel and checks the error code only,
src/csrc/util/cuda_utils.h:19-31).
"""
from __future__ import annotations

import contextlib
import functools

import torch

import cpu_ops
from swifttransformer_b200 import ops

# operations that compute (the ones that only report or plan are left alone)
WATCHED = ("embed", "add_positions", "add_norm", "bias_act", "linear", "gemm_plain", "gemm_skinny", "norm_linear",
           "linear_add", "norm_qkv_linear_to_cache", "qkv_linear_to_cache", "qkv_to_cache", "attention_plain",
           "attention_decode", "attention_prefill", "argmax")
TOL = {torch.float32: 3e-5, torch.bfloat16: 1.6e-2}


class ParanoidError(AssertionError):
    pass


def _to_cpu(x, memo):
    """A CPU copy of every tensor; a tensor passed twice (x and resid_out of a pre-norm add_norm are the same
    tensor) gets one copy, so that what the reference writes through one name shows through the other."""
    if isinstance(x, torch.Tensor):
        key = (x.data_ptr(), x.dtype, tuple(x.shape), tuple(x.stride()))
        if key not in memo:
            memo[key] = x.detach().cpu().clone()
        return memo[key]
    if isinstance(x, (list, tuple)):
        return type(x)(_to_cpu(v, memo) for v in x)
    return x


def _compare(name, index, what, got, ref):
    if got.dtype in (torch.int32, torch.int64):
        if not torch.equal(got.cpu(), ref):
            raise ParanoidError(f"{name} (call {index}): {what} differs from the CPU reference")
        return
    g, r = got.detach().float().cpu(), ref.float()
    finite = torch.isfinite(r)
    if not bool(torch.isfinite(g[finite]).all()):
        raise ParanoidError(f"{name} (call {index}): {what} holds a non-finite value where the reference is finite")
    scale = max(float(r[finite].abs().max()) if finite.any() else 0.0, 1e-6)
    err = (g - r)[finite].abs()
    tol = TOL.get(got.dtype, 3e-5) * scale
    if err.numel() and float(err.max()) > tol:
        worst = int(err.argmax())
        raise ParanoidError(f"{name} (call {index}): {what} differs from the CPU reference by {float(err.max()):.3e} "
                            f"(bound {tol:.3e}) at flat element {worst} of the finite ones")


def _wrap(name, fn, log):
    ref_fn = getattr(cpu_ops, name)

    @functools.wraps(fn)
    def checked(*args, **kwargs):
        if log["depth"]:
            return fn(*args, **kwargs)
        memo = {}
        cpu_args, cpu_kwargs = _to_cpu(args, memo), {k: _to_cpu(v, memo) for k, v in kwargs.items()}
        log["depth"] += 1
        try:
            out = fn(*args, **kwargs)
        finally:
            log["depth"] -= 1
        ref_out = ref_fn(*cpu_args, **cpu_kwargs)
        index = log["calls"]
        log["calls"] += 1
        log["by_name"][name] = log["by_name"].get(name, 0) + 1
        # whatever the operation wrote in place: compare every tensor argument after the call
        pairs = list(zip(args, cpu_args)) + [(kwargs[k], cpu_kwargs[k]) for k in kwargs]
        for i, (dev, host) in enumerate(pairs):
            if isinstance(dev, torch.Tensor) and dev.is_cuda and dev.numel():
                _compare(name, index, f"argument {i} after the call", dev, host)
        if isinstance(out, torch.Tensor) and out.is_cuda and not any(out is a for a in args):
            _compare(name, index, "the result", out, ref_out)
        return out
    return checked


@contextlib.contextmanager
def watch():
    log = {"calls": 0, "depth": 0, "by_name": {}}
    saved = {}
    for name in WATCHED:
        saved[name] = getattr(ops, name)
        setattr(ops, name, _wrap(name, saved[name], log))
    try:
        yield log
    finally:
        for name, fn in saved.items():
            setattr(ops, name, fn)
