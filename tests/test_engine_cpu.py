"""The engine's host logic without a GPU: the device operations are replaced by their plain CPU references
(tests/cpu_ops.py), everything else - parts, blocks, step building, cache manager, scheduler, sampler - is
the product's."""
import dataclasses

import numpy as np
import pytest
import torch

import helpers
import plain_opt
from helpers import TINY


def session(model_dir, name, max_tokens, **kw):
    from swifttransformer_b200.engine.replay import TraceSession
    return TraceSession(model_dir, "float32", max_tokens, page_size=TINY[name]["page_size"], device="cpu", **kw)


@pytest.mark.parametrize("name", ["a", "b"])
@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_step_function_matches_plain(model_dirs, cpu_ops_installed, name, mode):
    vocab = TINY[name]["cfg"]["vocab_size"]
    reqs = {f"r{i}": helpers.random_tokens(vocab, n, 50 + i) for i, n in enumerate([5, 33, 1, 40, 18])}
    steps = {"whole": helpers.trace_whole, "portions": helpers.trace_portions,
             "mixed": helpers.trace_mixed}[mode](reqs)
    s = session(model_dirs[name], name, helpers.live_token_need(steps), max_requests=4)
    got = helpers.replay(s, steps)
    helpers.check_against_plain(model_dirs[name], reqs, got, "float32", f"cpu/{name}/{mode}")
    assert s.cache.free_pages == s.cache.total_pages


def test_step_validation(model_dirs, cpu_ops_installed):
    from swifttransformer_b200.engine import OutOfPages, StepEntry, StepError
    s = session(model_dirs["a"], "a", 64, max_batch_tokens=256)
    slot = s.cache.alloc_slot()
    r = s.runner
    with pytest.raises(StepError, match="vocabulary"):
        r.step([StepEntry(slot, [5, 512], 0, [])])
    with pytest.raises(StepError, match="at least one token"):
        r.step([StepEntry(slot, [], 0, [])])
    with pytest.raises(StepError, match="wanted place"):
        r.step([StepEntry(slot, [5], 0, [1])])
    with pytest.raises(StepError, match="twice"):
        r.step([StepEntry(slot, [5], 0, []), StepEntry(slot, [6], 1, [])])
    with pytest.raises(StepError, match="holds 0 tokens"):
        r.step([StepEntry(slot, [5], 3, [])])
    with pytest.raises(StepError, match="positions end at 128"):
        r.step([StepEntry(slot, [5] * 129, 0, [])])
    with pytest.raises(OutOfPages):
        r.step([StepEntry(slot, [5] * 100, 0, [])])
    assert s.cache.free_pages == s.cache.total_pages
    assert r.step([StepEntry(slot, [5, 6], 0, [])]) is None


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_generation_matches_plain(model_dirs, cpu_ops_installed, name):
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.models import load_model
    from swifttransformer_b200.sampling import SamplingParams
    model = load_model(model_dirs[name], "float32", "cpu")
    eng = LLMEngine(model, page_size=TINY[name]["page_size"], num_pages=40, max_batch_tokens=24, chunk_size=16,
                    max_num_seqs=3)
    vocab = TINY[name]["cfg"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 70 + i) for i, n in enumerate([5, 17, 33, 1])]
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=6))
    cfg, w = plain_opt.load_model(model_dirs[name])
    for p, o in zip(prompts, outs):
        assert o == plain_opt.greedy_generate(cfg, w, p, 6)
    assert eng.cache.free_pages == eng.cache.total_pages


def test_preempted_requests_generate_the_same_tokens(model_dirs, cpu_ops_installed):
    """So few pages that requests are preempted and recomputed: the tokens must not change, for greedy
    and for seeded temperature sampling alike."""
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.models import load_model
    from swifttransformer_b200.sampling import SamplingParams
    model = load_model(model_dirs["a"], "float32", "cpu")
    prompts = [helpers.random_tokens(512, n, 90 + i) for i, n in enumerate([9, 14, 11])]
    params = [SamplingParams(max_new_tokens=10), SamplingParams(temperature=0.8, seed=3, max_new_tokens=10),
              SamplingParams(temperature=1.2, top_k=20, seed=4, max_new_tokens=10)]
    roomy = LLMEngine(model, page_size=8, num_pages=64, max_batch_tokens=64, chunk_size=32, max_num_seqs=4)
    tight = LLMEngine(model, page_size=8, num_pages=6, max_batch_tokens=64, chunk_size=32, max_num_seqs=4)
    a = roomy.generate(prompts, params)
    b = tight.generate(prompts, params)
    assert tight.scheduler.num_preemptions > 0 and roomy.scheduler.num_preemptions == 0
    assert a == b
    assert a[1] != a[0][:0] and len(a[1]) == 10


@pytest.mark.parametrize("pages", [64, 5])
def test_steps_launched_ahead_change_nothing(model_dirs, cpu_ops_installed, pages):
    """The engine launches a step before it has read the tokens of the one before.  Tokens, finish reasons
    and the order of finishing must be what the engine that waits for every step produces: requests that
    end on their end-of-sequence token (after a step ahead already ran for them), by length, and with so
    few pages that some are preempted while a token of theirs is still on its way."""
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.models import load_model
    from swifttransformer_b200.sampling import SamplingParams
    model = load_model(model_dirs["a"], "float32", "cpu")
    prompts = [helpers.random_tokens(512, n, 120 + i) for i, n in enumerate([9, 14, 11, 3, 20])]

    preempted = []

    def run(pipeline, params):
        eng = LLMEngine(model, page_size=8, num_pages=pages, max_batch_tokens=48, chunk_size=16, max_num_seqs=3,
                        pipeline=pipeline)
        ids = [eng.add_request(p, dataclasses.replace(sp)) for p, sp in zip(prompts, params)]
        order = []
        while eng.has_work():
            order += [r.id for r in eng.step()]
        assert eng.cache.free_pages == eng.cache.total_pages
        assert sorted(order) == sorted(ids), "every request is reported exactly once"
        preempted.append(eng.scheduler.num_preemptions)
        return [(eng.requests[i].output, eng.requests[i].finish_reason) for i in ids], order

    free = [SamplingParams(max_new_tokens=12), SamplingParams(temperature=0.9, seed=5, max_new_tokens=12),
            SamplingParams(temperature=1.3, top_k=30, seed=6, max_new_tokens=9), SamplingParams(max_new_tokens=1),
            SamplingParams(temperature=0.7, seed=8, max_new_tokens=12)]
    base, _ = run(False, free)
    # end-of-sequence ids taken from what the requests really generate, at different depths
    eos = [base[0][0][4], base[1][0][0], base[2][0][8], base[3][0][0], None]      # the last one ends by length
    params = [dataclasses.replace(sp, eos_id=e) for sp, e in zip(free, eos)]
    want, want_order = run(False, params)
    got, got_order = run(True, params)
    assert got == want
    assert any(reason == "eos" for _, reason in want) and any(reason == "length" for _, reason in want)
    for (out, reason), e in zip(want, eos):
        assert reason != "eos" or (out[-1] == e and e not in out[:-1])
    assert sorted(got_order) == sorted(want_order)
    assert all(n > 0 for n in preempted) == (pages < 64), preempted


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_steps_launched_ahead_with_requests_arriving_at_random(model_dirs, cpu_ops_installed, seed):
    """Random prompts, limits, end-of-sequence ids and arrival times, a pool that overflows now and then:
    launching steps ahead never changes what a request generates or why it ends."""
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.models import load_model
    from swifttransformer_b200.sampling import SamplingParams
    model = load_model(model_dirs["a"], "float32", "cpu")
    rng = np.random.default_rng(1000 + seed)
    n_req = 9
    prompts = [helpers.random_tokens(512, int(rng.integers(1, 40)), 700 + 10 * seed + i) for i in range(n_req)]
    arrive = sorted(int(rng.integers(0, 25)) for _ in range(n_req))
    # a small set of end-of-sequence ids makes some requests stop early and leaves others to their limit
    params = [SamplingParams(temperature=float(rng.choice([0.0, 0.8, 1.5])), top_k=int(rng.choice([0, 5, 50])),
                             seed=int(rng.integers(0, 1 << 30)), max_new_tokens=int(rng.integers(1, 14)),
                             eos_id=int(rng.integers(0, 512)) if rng.random() < 0.5 else None) for _ in range(n_req)]

    def run(pipeline):
        eng = LLMEngine(model, page_size=8, num_pages=int(rng_pages), max_batch_tokens=40, chunk_size=16,
                        max_num_seqs=4, pipeline=pipeline)
        ids, step, nxt = [], 0, 0
        while nxt < n_req or eng.has_work():
            while nxt < n_req and arrive[nxt] <= step:
                ids.append(eng.add_request(prompts[nxt], dataclasses.replace(params[nxt])))
                nxt += 1
            eng.step()
            step += 1
            assert step < 2000
        assert eng.cache.free_pages == eng.cache.total_pages and eng.cache.num_free_slots == 4
        return [(eng.requests[i].output, eng.requests[i].finish_reason) for i in ids]

    for rng_pages in (64, 9):
        want, got = run(False), run(True)
        assert got == want
        assert all(len(o) >= 1 for o, _ in got)


def test_warm_up_leaves_the_engine_as_it_was(model_dirs, cpu_ops_installed):
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.models import load_model
    from swifttransformer_b200.sampling import SamplingParams
    model = load_model(model_dirs["a"], "float32", "cpu")
    eng = LLMEngine(model, page_size=8, num_pages=40, max_batch_tokens=48, chunk_size=32, max_num_seqs=4)
    assert eng.warm_up(prompt_lengths=[5, 70, 1000], batch_sizes=[1, 4, 100]) == 0     # nothing is recorded on the CPU
    assert eng.cache.free_pages == eng.cache.total_pages and eng.stats["steps"] == 0 and not eng.requests
    prompt = helpers.random_tokens(512, 9, 77)
    cfg, w = plain_opt.load_model(model_dirs["a"])
    assert eng.generate([prompt], SamplingParams(max_new_tokens=5)) == [plain_opt.greedy_generate(cfg, w, prompt, 5)]
    rid = eng.add_request(prompt, SamplingParams(max_new_tokens=3))
    with pytest.raises(RuntimeError, match="without requests"):
        eng.warm_up(batch_sizes=[1])
    with pytest.raises(ValueError, match="has not finished"):
        eng.pop_request(rid)
    done = []
    while eng.has_work():
        done += eng.step()
    assert [r.id for r in done] == [rid]
    r = eng.pop_request(rid)
    assert r.output == plain_opt.greedy_generate(cfg, w, prompt, 3) and r.finish_reason == "length" and not eng.requests


def test_a_step_packed_into_a_padded_shape_is_padded_with_what_kernels_skip(model_dirs, cpu_ops_installed):
    """The index arrays of a step written into a layout with room to spare: the step's own part is what an exact
    layout gets, the rest are tokens at position -1, requests without tokens, single-token entries -1 and tiles
    whose offset lies past every request."""
    from swifttransformer_b200.engine.step import StepEntry
    s = session(model_dirs["c"], "c", 1024, max_requests=8, max_batch_tokens=1024)
    r = s.runner
    slots = [s.cache.alloc_slot() for _ in range(3)]
    entries = [StepEntry(slots[0], list(range(3, 203)), 0, [199]),      # a portion of 200 tokens: two tiles
               StepEntry(slots[1], [7], 0, [0]),                        # single tokens: attention entries
               StepEntry(slots[2], [8, 9, 10], 0, [])]
    exact, padded = r._layout(204, 3, 2), r._layout(256, 4, 4)
    he, hp = np.zeros(exact["total"], np.int32), np.full(padded["total"], -77, np.int32)
    ie, ip = r._pack(entries, exact, he, 204, 3), r._pack(entries, padded, hp, 256, 4)
    # the attention's step plan describes the step as (single-token entries, tiles, longest key range of an entry)
    assert ie["N"] == ip["N"] == 204 and ip["plan_keys"]["paged_attention"] == (4, 2, 3)

    def part(h, lay, name):
        o, n = lay[name]
        return h[o:o + n]
    for name in r.BASE_ARRAYS:
        k = exact[name][1]
        assert np.array_equal(part(hp, padded, name)[:k], part(he, exact, name)), name
    assert np.all(part(hp, padded, "positions")[204:] == -1)
    assert np.all(part(hp, padded, "q_start")[4:] == 204), "a padding request has no tokens"
    # the plan's own arrays: the tokens served one by one, then (request, offset) of every tile of query rows
    plan_e, plan_p = part(he, exact, "plan:paged_attention"), part(hp, padded, "plan:paged_attention")
    assert list(plan_p[:4]) == [200, 201, 202, 203] == list(plan_e[:4]) and np.all(plan_p[4:256] == -1)
    tiles = plan_p[256:].reshape(-1, 2)
    assert [tuple(t) for t in tiles[:2]] == [(0, 128), (0, 0)], "the tile with the longest key range first"
    assert [tuple(t) for t in plan_e[204:].reshape(-1, 2)[:2]] == [(0, 128), (0, 0)]
    assert np.all(tiles[2:, 1] >= 1 << 24) and np.all(part(hp, padded, "token_from") == -1)
    assert -77 not in hp, "every word of the padded layout is written"
    # a recorded shape is keyed by padded counts: entries in sixteens, all tiles the shape has room for, spans of keys
    lens, start = np.array([200, 1, 3], np.int32), np.zeros(3, np.int32)
    from swifttransformer_b200.parts.attention import KEYS_PER_BLOCK
    assert r.plans[0].shape_key(lens, start, 256, 4) == (16, 2 + 4, KEYS_PER_BLOCK)
    assert r.plans[0].shape_key(np.ones(5, np.int32), np.full(5, 800, np.int32), 8, 8) == (8, 0, 2 * KEYS_PER_BLOCK)


def test_sampler_follows_the_plain_sampler(cpu_ops_installed):
    from swifttransformer_b200 import ops
    from swifttransformer_b200.sampling import Sampler, SamplingParams
    rng = np.random.default_rng(0)
    logits = torch.tensor(rng.normal(size=(6, 300)) * 2, dtype=torch.float32)
    params = [SamplingParams(temperature=t, top_k=k, seed=s) for t, k, s in
              [(0.0, 0, 1), (0.8, 0, 2), (1.0, 10, 3), (0.5, 1, 4), (2.0, 0, 5), (0.8, 299, 6)]]
    got = Sampler("cpu").sample(logits, params, [0, 1, 2, 3, 4, 5])
    for r, p in enumerate(params):
        if p.temperature == 0:
            assert got[r] == int(np.argmax(logits[r].numpy()))
        else:
            u = ops.uniform(p.seed, r)
            assert got[r] == plain_opt.softmax_sample(logits[r].numpy(), p.temperature, u, p.top_k)


@pytest.mark.parametrize("pipeline", [False, True])
def test_aborting_requests_changes_nothing_for_the_others(model_dirs, cpu_ops_installed, pipeline):
    """Requests are taken out while waiting, while their prompt is half computed, while decoding (with steps
    launched ahead: with a token still on its way) and after they finished: pages and slot are back in the same
    call, no later step reports them, and the others generate what they generate alone."""
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.models import load_model
    from swifttransformer_b200.sampling import SamplingParams
    model = load_model(model_dirs["a"], "float32", "cpu")
    cfg, w = plain_opt.load_model(model_dirs["a"])
    prompts = [helpers.random_tokens(512, n, 900 + i) for i, n in enumerate([30, 7, 44, 12, 21, 5])]
    sp = SamplingParams(max_new_tokens=10)
    eng = LLMEngine(model, page_size=8, num_pages=64, max_batch_tokens=24, chunk_size=16, max_num_seqs=3,
                    pipeline=pipeline)
    ids = [eng.add_request(p, dataclasses.replace(sp)) for p in prompts]
    reported = []
    # 5 is still waiting (three slots)
    gone = {ids[5]: eng.abort_request(ids[5])}
    assert gone[ids[5]].finish_reason == "aborted" and gone[ids[5]].output == []
    reported += eng.step()
    # 0 has had one portion of its prompt
    r0 = eng.requests[ids[0]]
    assert 0 < r0.n_computed < len(r0.prompt)
    held = eng.cache.free_pages
    gone[ids[0]] = eng.abort_request(ids[0])
    assert eng.cache.free_pages > held and gone[ids[0]].slot is None
    while not eng.requests[ids[1]].output:
        reported += eng.step()
    reported += eng.step()
    # 1 is decoding; with steps launched ahead its next token is on its way
    gone[ids[1]] = eng.abort_request(ids[1])
    assert -1 not in gone[ids[1]].output and len(gone[ids[1]].output) >= 1
    with pytest.raises(KeyError):
        eng.abort_request(ids[1])
    while eng.has_work():
        reported += eng.step()
    assert sorted(r.id for r in reported) == sorted([ids[2], ids[3], ids[4]])
    assert eng.cache.free_pages == eng.cache.total_pages and eng.cache.num_free_slots == 3
    eng.cache.check()
    for i in (2, 3, 4):
        assert eng.requests[ids[i]].output == plain_opt.greedy_generate(cfg, w, prompts[i], 10), i
    # what 1 had got before it was taken out is the beginning of what it generates alone
    alone = plain_opt.greedy_generate(cfg, w, prompts[1], 10)
    assert gone[ids[1]].output == alone[:len(gone[ids[1]].output)]
    # a finished request can be taken out as well: it keeps its reason
    assert eng.abort_request(ids[2]).finish_reason == "length"
    assert not eng.scheduler.finished, "the scheduler keeps no finished request once a step has reported it"


def test_stats_show_the_pool_and_preemptions(model_dirs, cpu_ops_installed):
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.models import load_model
    from swifttransformer_b200.sampling import SamplingParams
    model = load_model(model_dirs["a"], "float32", "cpu")
    eng = LLMEngine(model, page_size=8, num_pages=9, max_batch_tokens=40, chunk_size=16, max_num_seqs=4)
    assert eng.stats["pages_free"] == eng.stats["pages_total"] == 9 and eng.stats["preemptions"] == 0
    for i in range(4):
        eng.add_request(helpers.random_tokens(512, 14, 40 + i), SamplingParams(max_new_tokens=12, ignore_eos=True))
    low = 9
    while eng.has_work():
        eng.step()
        low = min(low, eng.stats["pages_free"])
    st = eng.stats
    assert low == 0 and st["preemptions"] > 0 and st["pages_free"] == 9 and st["running"] == st["waiting"] == 0
    assert st["decode_tokens"] > 0 and st["prompt_tokens"] >= 4 * 14 and st["steps"] > 12


def test_the_length_limit_comes_from_the_configuration(model_dirs, cpu_ops_installed):
    """Block tables are sized by the per-request limit: the model's, or a smaller one the engine is given."""
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.models import load_model
    from swifttransformer_b200.sampling import SamplingParams
    model = load_model(model_dirs["a"], "float32", "cpu")
    assert model.max_positions == 128
    eng = LLMEngine(model, page_size=8, num_pages=32, max_num_seqs=2)
    assert eng.max_seq_len == 128 and eng.cache.groups[0].block_table.shape == (2, 16)
    eng = LLMEngine(model, page_size=8, num_pages=32, max_num_seqs=2, max_seq_len=40)
    assert eng.max_seq_len == 40 and eng.cache.groups[0].block_table.shape == (2, 5)
    with pytest.raises(ValueError, match="exceeds"):
        eng.add_request([5] * 41)
    out = eng.generate([[5] * 30], SamplingParams(max_new_tokens=50, ignore_eos=True))
    assert len(out[0]) == 10, "a request ends when it holds as many tokens as the limit allows"
