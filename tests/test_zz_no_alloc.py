"""The allocation-free decode attention entry point, called through its exported C symbol.

Some hosts of this library may not allocate device memory once they run: a server that gives its whole
memory budget to its own pool at start-up, code between the begin and end of a stream capture, a
real-time loop that cannot afford cudaMalloc's device-wide synchronisation, or a plain C caller that has
no allocator to lend.  For them ``st_attention_decode_noalloc`` keeps the scratch of the split decode
attention inside the library.  This test calls it with ctypes, as such a caller would, twice in a row
(the second call reuses the built-in scratch that the first one left dirty), and compares with the
regular entry point that takes its scratch from the caller.  It also checks that too large a request is
refused with a message.  Collected last on purpose: a failure here stops nothing else.
"""
import ctypes
import math

import pytest
import torch

import cpu_ops
from swifttransformer_b200 import ops
from test_kernels_gpu import attention_case

pytestmark = pytest.mark.gpu
DEV = "cuda"


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def call_noalloc(q, pool, out, positions, seq, slots, bt, nh, scale, window, n_splits, n_items=None, items=None):
    lib = ops.lib()
    fn = lib.st_attention_decode_noalloc
    fn.restype = ctypes.c_int
    _, n_layers, _, nkv, page_size, d = pool.shape
    err = ctypes.create_string_buffer(256)
    rc = fn(ptr(q), ptr(pool), ptr(out), ptr(items), q.shape[0] if n_items is None else n_items, ptr(positions), ptr(seq),
            ptr(slots), ptr(bt), bt.shape[1], n_layers, 1, nh, nkv, d, page_size, ctypes.c_float(scale), window,
            n_splits, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), err, 256)
    return rc, err.value.decode()


@pytest.mark.parametrize("shape", [(4, 4, 64, 16), (6, 2, 128, 8)])
def test_no_alloc_entry_point_matches_the_regular_one(shape):
    nh, nkv, d, ps = shape
    outs = []
    # (request lengths, splits, seed, window, the tokens served: None = all, in order)
    calls = [([300, 41, 700], 4, 11, 0, None), ([90, 650, 7, 128, 33], 7, 12, 0, None),
             ([500, 60, 222, 41], 5, 13, 37, [3, 0, 2])]
    for call, (lens, n_splits, seed, window, served) in enumerate(calls):
        new = [1] * len(lens)
        pool, bt, slots, t, q, scale, ref = attention_case(torch.bfloat16, nh, nkv, d, ps, lens, new, seed, window)
        dq, dpool, dpos, dseq, dslots, dbt = (x.to(DEV) for x in (q, pool, t["pos"], t["seq"], slots, bt))
        n = q.shape[0]
        items = torch.tensor(served, dtype=torch.int32, device=DEV) if served is not None else None
        n_items = len(served) if served is not None else n
        # the regular entry point: scratch from the caller
        want = torch.zeros(n, nh * d, dtype=torch.bfloat16, device=DEV)
        partial = torch.empty(ops.attention_decode_scratch(n_items, nh, d, n_splits), device=DEV)
        ops.attention_decode(dq, dpool, 1, want, items, n_items, dpos, dseq, dslots, dbt, nh, scale, window, n_splits,
                             partial, kernel="lanes")
        got = torch.zeros_like(want)
        torch.cuda.synchronize()
        # Free device memory as the driver counts it (cudaMemGetInfo), not torch's allocator: a cudaMalloc
        # inside the library would show here.  The first call on a device may only look up an address.
        free_before, _ = torch.cuda.mem_get_info()
        rc, msg = call_noalloc(dq, dpool, got, dpos, dseq, dslots, dbt, nh, scale, window, n_splits,
                               n_items=n_items, items=items)
        torch.cuda.synchronize()
        assert rc == 0, msg
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before, f"the call took {free_before - free_after} bytes of device memory"
        if served is not None:       # tokens that were not served are untouched by both
            rest = [i for i in range(n) if i not in served]
            assert torch.all(got[rest] == 0) and torch.all(want[rest] == 0)
            ref = ref.clone()
            ref[rest] = 0
        # same kernels, same order of summation: the two must agree far inside the tests' tolerance
        tol = 1e-2 * ref.float().abs().max().item()
        assert (got.float() - want.float()).abs().max().item() <= tol
        assert (got.float().cpu() - ref.float()).abs().max().item() <= tol
        assert torch.equal(got, want)
        outs.append(got)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    nh, nkv, d, ps = 4, 4, 64, 16
    pool, bt, slots, t, q, scale, _ = attention_case(torch.bfloat16, nh, nkv, d, ps, [50, 60], [1, 1], 13)
    dq, dpool, dpos, dseq, dslots, dbt = (x.to(DEV) for x in (q, pool, t["pos"], t["seq"], slots, bt))
    out = torch.zeros(2, nh * d, dtype=torch.bfloat16, device=DEV)
    # as if 5,000 tokens were passed: more (token, head) pairs than the built-in scratch has counters for
    rc, msg = call_noalloc(dq, dpool, out, dpos, dseq, dslots, dbt, nh, scale, 0, 2, n_items=5000)
    assert rc == -3 and "pairs" in msg and "16384" in msg
    rc, msg = call_noalloc(dq, dpool, out, dpos, dseq, dslots, dbt, nh, scale, 0, 4000, n_items=2)
    assert rc == -3 and "floats of scratch" in msg
    torch.cuda.synchronize()
    assert torch.all(out == 0), "a refused call launches nothing"
