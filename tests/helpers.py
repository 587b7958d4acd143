"""Shared test helpers: the tiny configurations, model folders, trace building and comparison."""
from __future__ import annotations

import json
import os

import numpy as np

# Three tiny OPT configurations that differ in every size and option.
TINY = {
    # pre-LN, biases, affine norms, embedding width == hidden
    "a": dict(cfg=dict(vocab_size=512, hidden_size=64, num_hidden_layers=2, ffn_dim=256, num_attention_heads=4,
                       max_position_embeddings=128, do_layer_norm_before=True, word_embed_proj_dim=64,
                       enable_bias=True, layer_norm_elementwise_affine=True, activation_function="relu"),
              seed=0, std=0.08, page_size=8),
    # post-LN, no biases, no affine, project_in/out, odd head count
    "b": dict(cfg=dict(vocab_size=1000, hidden_size=96, num_hidden_layers=3, ffn_dim=320, num_attention_heads=3,
                       max_position_embeddings=256, do_layer_norm_before=False, word_embed_proj_dim=48,
                       enable_bias=False, layer_norm_elementwise_affine=False, activation_function="relu"),
              seed=1, std=0.1, page_size=16),
    # long positions, head size 48, sizes that are no power of two, other eps, gelu
    "c": dict(cfg=dict(vocab_size=777, hidden_size=240, num_hidden_layers=1, ffn_dim=520, num_attention_heads=5,
                       max_position_embeddings=700, do_layer_norm_before=True, word_embed_proj_dim=240,
                       enable_bias=True, layer_norm_elementwise_affine=True, activation_function="gelu",
                       layer_norm_eps=3e-4),
              seed=2, std=0.06, page_size=32),
}


def tiny_config(name):
    from swifttransformer_b200.config import OptConfig
    return OptConfig.from_dict(dict(TINY[name]["cfg"]))


def make_model_dir(path, name):
    from swifttransformer_b200.models import write_random_model
    write_random_model(path, tiny_config(name), seed=TINY[name]["seed"], std=TINY[name]["std"])
    return path


def random_tokens(vocab, n, seed):
    return np.random.default_rng(seed).integers(3, vocab, n).tolist()


_PLAIN_CACHE = {}


def plain_logits(model_dir, tokens):
    """Logits [T, vocab] of the plain implementation for one whole sequence (cached)."""
    import plain_opt
    key = (model_dir, tuple(tokens))
    if key not in _PLAIN_CACHE:
        if model_dir not in _PLAIN_CACHE:
            _PLAIN_CACHE[model_dir] = plain_opt.load_model(model_dir)
        cfg, w = _PLAIN_CACHE[model_dir]
        _PLAIN_CACHE[key] = plain_opt.forward(cfg, w, tokens)
    return _PLAIN_CACHE[key]


# ---------------------------------------------------------------- trace building
def trace_whole(reqs):
    """Each request alone and whole: one step per request, every position wanted."""
    steps = []
    for rid, toks in reqs.items():
        steps.append(dict(entries=[dict(id=rid, tokens=toks, want=list(range(len(toks))))], end=[rid]))
    return steps


def trace_decode_tail(reqs, tail=32):
    """Most of a request in one step, the last `tail` tokens one by one."""
    steps = []
    for rid, toks in reqs.items():
        head = max(len(toks) - tail, 0)
        if head:
            steps.append(dict(entries=[dict(id=rid, tokens=toks[:head], want=list(range(head)))], end=[]))
        for i in range(head, len(toks)):
            steps.append(dict(entries=[dict(id=rid, tokens=[toks[i]], want=[0])],
                              end=[rid] if i == len(toks) - 1 else []))
    return steps


def trace_portions(reqs, sizes=(7, 2, 13, 3, 2, 29, 64, 5, 2, 17)):
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in reqs.items():
        pos, k = 0, 0
        while pos < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - pos)
            k += 1
            steps.append(dict(entries=[dict(id=rid, tokens=toks[pos:pos + n], want=list(range(n)))],
                              end=[rid] if pos + n == len(toks) else []))
            pos += n
    return steps


def trace_mixed(reqs, seed=0, max_live=4, chunk=24, prompt_frac=0.6):
    """Up to `max_live` requests at a time: prompt portions of some beside single tokens of others;
    a request that ends frees its pages for those that start later."""
    rng = np.random.default_rng(seed)
    waiting = list(reqs.items())
    live = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = dict(toks=toks, pos=0, prompt=max(1, int(len(toks) * prompt_frac)))
        entries, end = [], []
        for rid, st in list(live.items()):
            if rng.random() < 0.2 and len(live) > 1:
                continue                                  # left out of this step, goes on later
            if st["pos"] < st["prompt"]:
                n = int(min(st["prompt"] - st["pos"], rng.integers(2, chunk + 1)))
                if st["prompt"] - st["pos"] - n == 1:     # never leave a 1-token prompt portion behind
                    n += 1
            else:
                n = 1
            toks = st["toks"][st["pos"]:st["pos"] + n]
            entries.append(dict(id=rid, tokens=toks, want=list(range(len(toks)))))
            st["pos"] += len(toks)
            if st["pos"] == len(st["toks"]):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append(dict(entries=entries, end=end))
    return steps


def live_token_need(steps, round_to=64):
    """The most tokens live requests hold at any time, each rounded up to a multiple of `round_to`."""
    held, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((v + round_to - 1) // round_to * round_to for v in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def replay(session, steps):
    """Run steps through a TraceSession; returns {request id: array [T, vocab]} in position order."""
    rows = {}
    for st in steps:
        logits = session.run_step(st["entries"], st["end"])
        session.check()
        if logits is None:
            continue
        arr = logits.detach().float().cpu().numpy()
        k = 0
        for e in st["entries"]:
            for _ in e.get("want", []):
                rows.setdefault(e["id"], []).append(arr[k])
                k += 1
        assert k == arr.shape[0]
    return {rid: np.stack(v) for rid, v in rows.items()}


def first_bad(got, ref, tol):
    """Index of the first position whose logits differ by more than tol, or None."""
    err = np.abs(got - ref).max(axis=1)
    bad = np.nonzero(err > tol)[0]
    return (int(bad[0]), float(err[bad[0]])) if len(bad) else None


TOL = {"float32": 2e-5, "bfloat16": 4e-2}   # fraction of the largest reference logit


def check_against_plain(model_dir, reqs, got, dtype, what):
    for rid, toks in reqs.items():
        ref = plain_logits(model_dir, toks)
        assert got[rid].shape == ref.shape, (what, rid, got[rid].shape, ref.shape)
        scale = np.abs(ref).max()
        bad = first_bad(got[rid], ref, TOL[dtype] * scale)
        assert bad is None, (f"{what}/{dtype}: request {rid} first differs at position {bad[0]} of {len(toks)} "
                             f"by {bad[1]:.3e} (tolerance {TOL[dtype] * scale:.3e})")
        if dtype == "bfloat16":
            # the typical error is far below the bound
            assert np.abs(got[rid] - ref).mean() < 6e-3 * scale
