"""The plain implementation's attention held to the reference's own attention oracle.

tests/golden/attention_ref_tiny.npz holds inputs and outputs of ``st::reference::kernel::attentionKernelRef``
(src/unittest/kernel/attention_ref.cc:13-141), the LibTorch restatement the reference tests its kernels with,
compiled unchanged for the host by tests/golden/make_attention_ref_golden.py: whole prompts (53-88) beside
single decode tokens that read a paged cache through a block table and append their own key and value
(89-141), multi-head and grouped.  ``plain_opt.causal_attention`` must give the same numbers for every
request.  The oracle computes in float32 with an additive -10000 mask; the plain implementation in float64
with masked keys left out: they agree to float32 rounding.  With SWIFTTRANSFORMER_REFERENCE pointing at a
checkout of the reference the oracle is also compiled and run afresh.
"""
import json
import os
import sys

import numpy as np
import pytest

import plain_opt

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_attention_ref_golden as golden  # noqa: E402


def stored():
    z = np.load(os.path.join(HERE, "golden", "attention_ref_tiny.npz"))
    meta = json.loads(bytes(z["meta"]))
    assert meta["seed"] == golden.SEED and meta["cases"] == [[c[0], c[1], c[2], c[3], c[4]] for c in golden.CASES]
    return z


def plain_result(case, nq, nkv, d, bs, reqs):
    """What the plain implementation's attention gives for the oracle's inputs, request by request."""
    qkvs = case["qkvs"].astype(np.float64)
    group = nq // nkv
    out = np.zeros((qkvs.shape[0], nq * d))
    t0 = 0
    for r, (is_prompt, n) in enumerate(reqs):
        if is_prompt:
            rows = qkvs[t0:t0 + n]
            q = rows[:, :nq].reshape(n, nq * d)
            k = np.repeat(rows[:, nq:nq + nkv], group, axis=1).reshape(n, nq * d)
            v = np.repeat(rows[:, nq + nkv:], group, axis=1).reshape(n, nq * d)
            out[t0:t0 + n] = plain_opt.causal_attention(q, k, v, nq)
            t0 += n
            continue
        # a decode token: keys and values 0..n-1 from the request's pages, its own at position n
        ks = np.zeros((n + 1, nkv, d))
        vs = np.zeros((n + 1, nkv, d))
        for p in range(n):
            page = case["block_table"][r, p // bs]
            ks[p] = case["k_cache"][page, 0, :, p % bs]
            vs[p] = case["v_cache"][page, 0, :, p % bs]
        ks[n], vs[n] = qkvs[t0, nq:nq + nkv], qkvs[t0, nq + nkv:]
        q = np.zeros((n + 1, nq * d))
        q[n] = qkvs[t0, :nq].reshape(-1)
        k = np.repeat(ks, group, axis=1).reshape(n + 1, nq * d)
        v = np.repeat(vs, group, axis=1).reshape(n + 1, nq * d)
        out[t0] = plain_opt.causal_attention(q, k, v, nq)[n]
        t0 += 1
    return out


@pytest.mark.parametrize("spec", golden.CASES, ids=[c[0] for c in golden.CASES])
def test_plain_attention_equals_the_reference_oracle(spec):
    name, nq, nkv, d, bs, reqs = spec
    z = stored()
    case = {k.split(".", 1)[1]: z[k] for k in z.files if k.startswith(name + ".")}
    ref = case["result"]
    got = plain_result(case, nq, nkv, d, bs, reqs)
    assert got.shape == ref.shape
    assert np.abs(ref).max() > 0.1
    assert np.abs(got - ref).max() <= 2e-6 * np.abs(ref).max()


@pytest.mark.skipif(not os.environ.get("SWIFTTRANSFORMER_REFERENCE"),
                    reason="SWIFTTRANSFORMER_REFERENCE does not name a checkout of the reference")
def test_a_fresh_run_of_the_oracle_gives_the_stored_numbers():
    oracle = golden.build_oracle(os.environ["SWIFTTRANSFORMER_REFERENCE"])
    z = stored()
    rng = np.random.default_rng(golden.SEED)
    for name, nq, nkv, d, bs, reqs in golden.CASES:
        case = golden.make_case(nq, nkv, d, bs, reqs, rng)
        for k, v in case.items():
            assert np.array_equal(v, z[f"{name}.{k}"]), (name, k)
        assert np.allclose(golden.run_oracle(oracle, case, d), z[f"{name}.result"], rtol=0, atol=1e-6)
