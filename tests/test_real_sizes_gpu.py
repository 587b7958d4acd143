"""Logits at real layer sizes: a few layers of the widths the benchmark runs (OPT-1.3B: 2048 wide, 32 heads of
64, feed-forward 8192; OPT-6.7B: 4096 wide, 32 heads of 128, feed-forward 16384; vocabulary 50272, pages of 16)
with random weights, against the plain implementation.  These are the paths the tiny configurations never
reach together: the TMA-fed prompt attention over a 2048-token prompt, the weight-streaming product with its
longest inner dimension, the decode attention with long key ranges and with more requests than the
weight-streaming product serves (library products, the separate cache write), norms with the row in registers.

Fewer layers than the real models have (the oracle is numpy on the CPU), never narrower ones.  Logits are
compared at every 64th position and at the last 32 of a prompt, and at every decoded position."""
import numpy as np
import pytest

import helpers
import plain_opt

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]

SIZES = {
    "opt_1.3b": dict(vocab_size=50272, hidden_size=2048, num_hidden_layers=2, ffn_dim=8192, num_attention_heads=32,
                     max_position_embeddings=2048, do_layer_norm_before=True, word_embed_proj_dim=2048,
                     enable_bias=True, layer_norm_elementwise_affine=True, activation_function="relu"),
    "opt_6.7b": dict(vocab_size=50272, hidden_size=4096, num_hidden_layers=1, ffn_dim=16384, num_attention_heads=32,
                     max_position_embeddings=2048, do_layer_norm_before=True, word_embed_proj_dim=4096,
                     enable_bias=True, layer_norm_elementwise_affine=True, activation_function="relu"),
}
PAGE = 16
_REFS = {}       # (what, size name) -> the plain implementation's logits, computed once per run


def plain_rows(key, cfg, w, toks, rows):
    if key not in _REFS:
        _REFS[key] = plain_opt.forward(cfg, w, toks, rows=rows)
    return _REFS[key]


@pytest.fixture(scope="module")
def big_models(tmp_path_factory):
    """name -> (model folder, plain config, plain weights), each made when first asked for."""
    made = {}

    def get(name):
        if name not in made:
            from swifttransformer_b200.config import OptConfig
            from swifttransformer_b200.models import write_random_model
            d = str(tmp_path_factory.mktemp(name))
            write_random_model(d, OptConfig.from_dict(dict(SIZES[name])), seed=31, std=0.02)
            made[name] = (d,) + tuple(plain_opt.load_model(d))
        return made[name]
    return get


def session(model_dir, dtype, max_tokens, **kw):
    from swifttransformer_b200.engine.replay import TraceSession
    return TraceSession(model_dir, dtype, max_tokens, page_size=PAGE, **kw)


def compare(got, ref, dtype, what):
    scale = np.abs(ref).max()
    bad = helpers.first_bad(got, ref, helpers.TOL[dtype] * scale)
    assert bad is None, f"{what}/{dtype}: wanted row {bad[0]} of {len(ref)} differs by {bad[1]:.3e} " \
                        f"(tolerance {helpers.TOL[dtype] * scale:.3e})"
    if dtype == "bfloat16":
        assert np.abs(got - ref).mean() < 6e-3 * scale, what


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SIZES))
def test_a_long_prompt_whole_in_portions_and_with_a_decoded_tail(big_models, name, dtype):
    model_dir, cfg, w = big_models(name)
    n = 2048
    toks = helpers.random_tokens(cfg["vocab_size"], n, 77)
    rows = sorted(set(range(63, n, 64)) | set(range(n - 32, n)))
    ref = plain_rows(("prompt", name), cfg, w, toks, rows)

    def want(a, b):
        return [r - a for r in rows if a <= r < b]

    traces = {
        "whole": [dict(entries=[dict(id="x", tokens=toks, want=want(0, n))], end=["x"])],
        "portions of 512": [dict(entries=[dict(id="x", tokens=toks[a:a + 512], want=want(a, a + 512))],
                                 end=["x"] if a + 512 == n else []) for a in range(0, n, 512)],
        "decoded tail": [dict(entries=[dict(id="x", tokens=toks[:n - 32], want=want(0, n - 32))], end=[])] +
                        [dict(entries=[dict(id="x", tokens=[toks[i]], want=[0])], end=["x"] if i == n - 1 else [])
                         for i in range(n - 32, n)],
    }
    for what, steps in traces.items():
        s = session(model_dir, dtype, n, max_requests=2, max_batch_tokens=n)
        got = helpers.replay(s, steps)["x"]
        compare(got, ref, dtype, f"{name}/{what}")
        assert s.cache.free_pages == s.cache.total_pages


@pytest.mark.parametrize("dtype,n_requests", [("float32", 16), ("bfloat16", 16), ("bfloat16", 64), ("bfloat16", 5),
                                              ("bfloat16", 8), ("bfloat16", 2)])
@pytest.mark.parametrize("name", list(SIZES))
def test_many_requests_decoding_together(big_models, name, dtype, n_requests):
    """2 to 64 requests of 300 to 520 tokens: prompts several to a step, then the last 8 tokens of all of
    them together, one by one.  Eight different token sequences (neighbouring requests never share one); every
    request has pages of its own.  Up to 8 requests the decode steps take the weight-streaming products (weights on
    chip before their wait, a product cut over k leaving its parts to the next norm; 5 requests run in a step
    recorded for 8), beyond that the library products."""
    model_dir, cfg, w = big_models(name)
    tail = 8
    lens = [300, 517, 411, 352, 520, 333, 478, 401]
    seqs = [helpers.random_tokens(cfg["vocab_size"], m, 500 + i) for i, m in enumerate(lens)]
    refs = [plain_rows(("together", name, i), cfg, w, t, range(len(t) - tail, len(t))) for i, t in enumerate(seqs)]
    reqs = {f"r{i}": seqs[i % len(seqs)] for i in range(n_requests)}
    steps, batch, held = [], [], 0
    for rid, t in reqs.items():                       # prompts, as many to a step as 2048 tokens take
        if held + len(t) - tail > 2048:
            steps.append(dict(entries=batch, end=[]))
            batch, held = [], 0
        batch.append(dict(id=rid, tokens=t[:-tail], want=[]))
        held += len(t) - tail
    steps.append(dict(entries=batch, end=[]))
    for j in range(tail):                             # then every request's next token, all in one step
        steps.append(dict(entries=[dict(id=rid, tokens=[t[len(t) - tail + j]], want=[0]) for rid, t in reqs.items()],
                          end=list(reqs) if j == tail - 1 else []))
    s = session(model_dir, dtype, helpers.live_token_need(steps), max_requests=n_requests, max_batch_tokens=2048)
    got = helpers.replay(s, steps)
    for i, rid in enumerate(reqs):
        compare(got[rid], refs[i % len(seqs)], dtype, f"{name}/{n_requests} together/{rid}")
    assert s.cache.free_pages == s.cache.total_pages
    assert s.runner.graph_steps >= tail - 1


# The widths of OPT-30B: 56 heads of 128 (a head count that is no multiple of 8), 7168 wide, feed-forward 28672.
# One layer and a small vocabulary that is no power of two keep the oracle on the CPU short; the widths are real.
WIDE = dict(vocab_size=5003, hidden_size=7168, num_hidden_layers=1, ffn_dim=28672, num_attention_heads=56,
            max_position_embeddings=2048, do_layer_norm_before=True, word_embed_proj_dim=7168, enable_bias=True,
            layer_norm_elementwise_affine=True, activation_function="relu")


@pytest.fixture(scope="module")
def wide_model(tmp_path_factory):
    from swifttransformer_b200.config import OptConfig
    from swifttransformer_b200.models import write_random_model
    d = str(tmp_path_factory.mktemp("opt_30b_widths"))
    write_random_model(d, OptConfig.from_dict(dict(WIDE)), seed=47, std=0.02)
    return (d,) + tuple(plain_opt.load_model(d))


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_widest_layers_prompts_and_decoding(wide_model, dtype):
    """Three requests of 97 to 203 tokens at OPT-30B widths: the prompts in portions of 64 beside one another,
    then the last 6 tokens of all three together, one by one."""
    model_dir, cfg, w = wide_model
    tail = 6
    reqs = {f"w{i}": helpers.random_tokens(cfg["vocab_size"], n, 700 + i) for i, n in enumerate([97, 150, 203])}
    rows = {rid: sorted(set(range(31, len(t) - tail, 32)) | set(range(len(t) - tail, len(t)))) for rid, t in reqs.items()}
    refs = {rid: plain_rows(("wide", rid), cfg, w, t, rows[rid]) for rid, t in reqs.items()}
    steps, longest = [], max(len(t) for t in reqs.values()) - tail
    for a in range(0, longest, 64):
        entries = []
        for rid, t in reqs.items():
            b = min(a + 64, len(t) - tail)
            if a < b:
                entries.append(dict(id=rid, tokens=t[a:b], want=[r - a for r in rows[rid] if a <= r < b]))
        steps.append(dict(entries=entries, end=[]))
    for j in range(tail):
        steps.append(dict(entries=[dict(id=rid, tokens=[t[len(t) - tail + j]], want=[0]) for rid, t in reqs.items()],
                          end=list(reqs) if j == tail - 1 else []))
    s = session(model_dir, dtype, helpers.live_token_need(steps), max_requests=3, max_batch_tokens=512)
    got = helpers.replay(s, steps)
    for rid in reqs:
        compare(got[rid], refs[rid], dtype, f"30b widths/{rid}")
    assert s.cache.free_pages == s.cache.total_pages
