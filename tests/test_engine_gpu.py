"""The engine on the GPU against the plain implementation: the same requests whole, with the tail decoded
token by token, in portions of changing size, and mixed with page reuse; in float32 and bfloat16."""
import numpy as np
import pytest
import torch

import helpers
from helpers import TINY, TOL

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def requests_for(name):
    cfg = TINY[name]["cfg"]
    maxpos, vocab = cfg["max_position_embeddings"], cfg["vocab_size"]
    lens = {"a": [5, 17, 33, 128, 64, 90], "b": [1, 7, 64, 100, 129, 256], "c": [2, 33, 500, 700, 65, 300]}[name]
    return {f"r{i}": helpers.random_tokens(vocab, n, 100 + i) for i, n in enumerate(lens) if n <= maxpos}


def session(model_dir, name, dtype, max_tokens, **kw):
    from swifttransformer_b200.engine.replay import TraceSession
    return TraceSession(model_dir, dtype, max_tokens, page_size=TINY[name]["page_size"], **kw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(TINY))
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_replay_matches_plain(model_dirs, name, dtype, mode):
    reqs = requests_for(name)
    steps = {"whole": helpers.trace_whole, "decode_tail": helpers.trace_decode_tail,
             "portions": helpers.trace_portions, "mixed": helpers.trace_mixed}[mode](reqs)
    # the pool holds exactly what the live requests need, so pages are used again
    need = helpers.live_token_need(steps)
    s = session(model_dirs[name], name, dtype, need, max_requests=4)
    got = helpers.replay(s, steps)
    helpers.check_against_plain(model_dirs[name], reqs, got, dtype, f"{name}/{mode}")
    assert s.cache.free_pages == s.cache.total_pages, "every page must be back in the pool"
    assert s.runner.padded_graph_steps > 0, "steps that are not decode-only are recorded in padded shapes and replayed"


@pytest.mark.parametrize("dtype", DTYPES)
def test_cut_does_not_change_float32_logits_beyond_rounding(model_dirs, dtype):
    """The engine against itself: whole vs portions vs token by token."""
    name = "c"
    toks = helpers.random_tokens(TINY[name]["cfg"]["vocab_size"], 200, 7)
    reqs = {"x": toks}
    outs = []
    for build in (helpers.trace_whole, helpers.trace_portions, lambda r: helpers.trace_decode_tail(r, tail=200)):
        s = session(model_dirs[name], name, dtype, 256)
        outs.append(helpers.replay(s, build(reqs))["x"])
    scale = np.abs(outs[0]).max()
    tol = (1e-5 if dtype == "float32" else 3e-2) * scale
    for o in outs[1:]:
        bad = helpers.first_bad(o, outs[0], tol)
        assert bad is None, f"first differing position {bad}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_recorded_padded_steps_and_eager_steps_agree(model_dirs, dtype):
    """The same mixed trace with every step launched eagerly, with recorded steps of padded shapes, with
    room for only two recordings (the other shapes fall back to eager launches), and with two recordings of
    which the one unused for more than three steps gives way to a new shape: float32 logits are equal bit for
    bit (a token's result does not depend on the padding beside it), bfloat16 within rounding."""
    name = "c"
    reqs = requests_for(name)
    steps = helpers.trace_mixed(reqs)
    outs = []
    for cap, idle in ((0, 512), (48, 512), (2, 512), (2, 3)):
        s = session(model_dirs[name], name, dtype, helpers.live_token_need(steps), max_requests=4)
        s.runner.max_step_graphs, s.runner.evict_idle_steps = cap, idle
        seen = set()
        outs.append({})
        for st in steps:                       # helpers.replay, watching which shapes are held
            for k, v in helpers.replay(s, [st]).items():
                outs[-1][k] = np.concatenate([outs[-1][k], v]) if k in outs[-1] else v
            seen |= set(s.runner._step_graphs)
            assert len(s.runner._step_graphs) <= cap
        assert (s.runner.padded_graph_steps > 0) == (cap > 0)
        if idle == 3:
            assert len(seen) > cap, "recordings that lay idle were replaced"
        elif cap == 2:
            assert len(seen) == cap
        s.runner.check_status()
    for k in reqs:
        for o in outs[1:]:
            if dtype == "float32":
                assert np.array_equal(o[k], outs[0][k]), k
            else:
                assert helpers.first_bad(o[k], outs[0][k], 3e-2 * np.abs(outs[0][k]).max()) is None, k


@pytest.mark.parametrize("name", ["a", "c"])
def test_decoding_with_the_key_range_cut_into_parts(model_dirs, name, monkeypatch):
    """Long key ranges are cut into parts that separate blocks walk and the last one merges.  With the span a
    block walks alone set to 32 keys, decode steps of a few hundred positions run with up to nine parts, are
    recorded once per number of spans, and must still match the plain implementation."""
    import swifttransformer_b200.parts.attention as attention
    monkeypatch.setattr(attention, "KEYS_PER_BLOCK", 32)
    reqs = {k: v for k, v in requests_for(name).items() if len(v) >= 60}
    steps = helpers.trace_decode_tail(reqs, tail=48)
    s = session(model_dirs[name], name, "bfloat16", helpers.live_token_need(steps), max_requests=4)
    got = helpers.replay(s, steps)
    helpers.check_against_plain(model_dirs[name], reqs, got, "bfloat16", f"{name}/parts")
    assert s.runner.graph_steps > 0 and len(s.runner._graphs) >= 3, "one recorded step per number of spans"
    assert max(g.ctx.plan("paged_attention").splits(TINY[name]["cfg"]["num_attention_heads"])
               for g in s.runner._graphs.values()) > 2
    s.runner.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_long_decoding(model_dirs, dtype):
    """A one-token prompt, then token-by-token decoding up to the model's last position."""
    name = "c"
    maxpos = TINY[name]["cfg"]["max_position_embeddings"]
    toks = helpers.random_tokens(TINY[name]["cfg"]["vocab_size"], maxpos, 8)
    reqs = {"x": toks}
    s = session(model_dirs[name], name, dtype, helpers.live_token_need(helpers.trace_whole(reqs)))
    got = helpers.replay(s, helpers.trace_decode_tail(reqs, tail=maxpos))
    helpers.check_against_plain(model_dirs[name], reqs, got, dtype, "long decode")
    # one more token would pass the last position: refused, not computed wrongly
    from swifttransformer_b200.engine import StepError
    s2 = session(model_dirs[name], name, dtype, 1024)
    s2.run_step([dict(id="y", tokens=toks, want=[])])
    with pytest.raises(StepError):
        s2.run_step([dict(id="y", tokens=[5], want=[0])])


@pytest.mark.parametrize("dtype", DTYPES)
def test_out_of_pages_is_an_error_and_leaves_the_cache_whole(model_dirs, dtype):
    from swifttransformer_b200.engine import OutOfPages
    name = "a"
    s = session(model_dirs[name], name, dtype, 64)
    toks = helpers.random_tokens(512, 100, 9)
    s.run_step([dict(id="p", tokens=toks[:60], want=[59])])
    with pytest.raises(OutOfPages):
        s.run_step([dict(id="q", tokens=toks[:30], want=[29])])
    s.cache.check()
    s.run_step([], end=["p", "q"])
    assert s.cache.free_pages == s.cache.total_pages
