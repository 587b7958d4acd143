"""Generation through the Python entry point and the command line on the GPU."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_opt
from helpers import TINY

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def engine(model_dir, name, dtype, **kw):
    from swifttransformer_b200.engine.engine import LLMEngine
    args = dict(page_size=TINY[name]["page_size"], num_pages=64, max_batch_tokens=48, chunk_size=32, max_num_seqs=4)
    args.update(kw)
    return LLMEngine(model_dir, dtype=dtype, device="cuda", **args)


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_generation_float32_matches_plain(model_dirs, name):
    from swifttransformer_b200.sampling import SamplingParams
    vocab = TINY[name]["cfg"]["vocab_size"]
    lens = [5, 17, 33] if name == "a" else [1, 7, 64, 100, 129]
    prompts = [helpers.random_tokens(vocab, n, 200 + i) for i, n in enumerate(lens)]
    eng = engine(model_dirs[name], name, "float32")
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=16))
    eng.runner.check_status()
    cfg, w = plain_opt.load_model(model_dirs[name])
    for p, o in zip(prompts, outs):
        assert o == plain_opt.greedy_generate(cfg, w, p, 16)
    assert eng.runner.graph_steps > 0, "decode steps are replayed from recorded graphs"
    assert eng.cache.free_pages == eng.cache.total_pages


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_generation_bfloat16_follows_plain_unless_nearly_tied(model_dirs, name):
    from swifttransformer_b200.sampling import SamplingParams
    vocab = TINY[name]["cfg"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 300 + i) for i, n in enumerate([9, 30, 60])]
    eng = engine(model_dirs[name], name, "bfloat16")
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12))
    cfg, w = plain_opt.load_model(model_dirs[name])
    for p, o in zip(prompts, outs):
        ids = list(p)
        for tok in o:
            logits = plain_opt.forward(cfg, w, ids)[-1]
            best = int(np.argmax(logits))
            if tok != best:
                # only allowed where the plain implementation's top two are within bfloat16 error
                assert logits[best] - logits[tok] < 4e-2 * np.abs(logits).max(), (tok, best)
            ids.append(tok)


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_many_requests_decoding_together_bfloat16(model_dirs, name):
    """More requests than the weight-streaming product serves: library products, the separate cache-write
    kernel and the decode attention, recorded and replayed as graphs of 16 rows."""
    from swifttransformer_b200.sampling import SamplingParams
    vocab = TINY[name]["cfg"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 900 + i) for i, n in enumerate([9, 30, 60, 1, 17, 33, 5, 12, 47, 2, 21, 8, 14])]
    eng = engine(model_dirs[name], name, "bfloat16", num_pages=200, max_batch_tokens=256, chunk_size=64, max_num_seqs=16)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=10))
    eng.runner.check_status()
    assert eng.runner.graph_steps > 0 and eng.cache.free_pages == eng.cache.total_pages
    cfg, w = plain_opt.load_model(model_dirs[name])
    for p, o in zip(prompts, outs):
        ids = list(p)
        for tok in o:
            logits = plain_opt.forward(cfg, w, ids)[-1]
            best = int(np.argmax(logits))
            if tok != best:
                assert logits[best] - logits[tok] < 4e-2 * np.abs(logits).max(), (tok, best)
            ids.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_change_nothing_on_the_gpu(model_dirs, dtype):
    """Launching a step before the tokens of the one before have been read (they reach it on the device)
    gives the tokens, finish reasons and free pages of the engine that waits after every step; requests
    end on end-of-sequence tokens at different depths, by length, and some are preempted."""
    import dataclasses
    from swifttransformer_b200.sampling import SamplingParams
    name = "b"
    # lengths just under a page's edge: with few pages the requests outgrow the pool while they decode
    prompts = [helpers.random_tokens(1000, n, 520 + i) for i, n in enumerate([15, 31, 47, 14, 17, 1])]
    free = [SamplingParams(max_new_tokens=14), SamplingParams(temperature=0.9, seed=5, max_new_tokens=14),
            SamplingParams(temperature=1.3, top_k=30, seed=6, max_new_tokens=9), SamplingParams(max_new_tokens=1),
            SamplingParams(temperature=0.7, seed=8, max_new_tokens=14), SamplingParams(max_new_tokens=14)]

    def run(pipeline, params, num_pages):
        eng = engine(model_dirs[name], name, dtype, num_pages=num_pages, max_batch_tokens=128, chunk_size=48,
                     pipeline=pipeline)
        ids = [eng.add_request(p, dataclasses.replace(sp)) for p, sp in zip(prompts, params)]
        reported = []
        while eng.has_work():
            reported += [r.id for r in eng.step()]
        eng.runner.check_status()
        assert sorted(reported) == sorted(ids) and eng.cache.free_pages == eng.cache.total_pages
        return [(eng.requests[i].output, eng.requests[i].finish_reason) for i in ids], eng

    base, _ = run(False, free, 64)
    eos = [base[0][0][5], base[1][0][0], base[2][0][8], base[3][0][0], None, base[5][0][13]]
    params = [dataclasses.replace(sp, eos_id=e) for sp, e in zip(free, eos)]
    # An end-of-sequence token changes which requests share the steps after it (the step ahead still has
    # the request, admissions come a step later): exact equality is asked for in float32, whose results do
    # not depend on the batch; in bfloat16 a sampled token may flip with the batch's rounding.
    for num_pages in (64, 7) if dtype == "float32" else ():
        want, e0 = run(False, params, num_pages)
        got, e1 = run(True, params, num_pages)
        assert got == want
        assert e1.runner.graph_steps > 0
        assert {r for _, r in want} == {"eos", "length"}
    # without end-of-sequence tokens the small pool overflows in both engines: a request is preempted while
    # a token of its is still on its way
    want, e0 = run(False, free, 7)
    got, e1 = run(True, free, 7)
    assert got == want and (got == base or dtype != "float32")
    assert e0.scheduler.num_preemptions > 0 and e1.scheduler.num_preemptions > 0


def test_warm_up_records_the_steps_that_requests_then_replay(model_dirs):
    from swifttransformer_b200.sampling import SamplingParams
    vocab = TINY["a"]["cfg"]["vocab_size"]
    eng = engine(model_dirs["a"], "a", "bfloat16")
    added = eng.warm_up(prompt_lengths=[20], batch_sizes=[1, 3])
    assert added >= 3
    assert eng.cache.free_pages == eng.cache.total_pages and eng.stats["steps"] == 0 and not eng.requests
    r = eng.runner
    known = len(r._graphs) + len(r._step_graphs)
    prompts = [helpers.random_tokens(vocab, 20, 900)]
    first = eng.generate(prompts, SamplingParams(max_new_tokens=3))
    assert len(r._graphs) + len(r._step_graphs) == known, "a warmed-up shape is replayed, not recorded again"
    fresh = engine(model_dirs["a"], "a", "bfloat16")
    assert fresh.generate(prompts, SamplingParams(max_new_tokens=3)) == first
    eng.runner.check_status()


def test_seeded_sampling_is_reproducible_and_batch_independent(model_dirs):
    from swifttransformer_b200.sampling import SamplingParams
    name = "b"
    prompts = [helpers.random_tokens(1000, n, 400 + i) for i, n in enumerate([1, 7, 64, 100, 129])]
    params = [SamplingParams(temperature=0.8, seed=50 + i, max_new_tokens=10) for i in range(5)]
    together = engine(model_dirs[name], name, "float32", chunk_size=32).generate(prompts, params)
    again = engine(model_dirs[name], name, "float32", chunk_size=32).generate(prompts, params)
    assert together == again
    alone = [engine(model_dirs[name], name, "float32", max_batch_tokens=16, chunk_size=7).generate([p], [sp])[0]
             for p, sp in zip(prompts, params)]
    assert alone == together, "a request's tokens do not depend on what else is scheduled or how it is cut"
    assert len({tuple(o) for o in together}) > 1
    # preemption by recompute leaves the tokens unchanged
    # three requests whose prompts fill the pool: when they grow, the youngest is preempted and recomputed
    prompts3 = [helpers.random_tokens(1000, 62, 450 + i) for i in range(3)]
    roomy = engine(model_dirs[name], name, "float32", max_batch_tokens=256, chunk_size=64)
    tight = engine(model_dirs[name], name, "float32", num_pages=12, max_batch_tokens=256, chunk_size=64)
    want = roomy.generate(prompts3, params[:3])
    assert tight.generate(prompts3, params[:3]) == want
    assert tight.scheduler.num_preemptions > 0 and roomy.scheduler.num_preemptions == 0


def test_benchmark_all_input_same_command_line(model_dirs):
    """The reference's benchmark program: same arguments, one line of stage times per experiment."""
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "benchmark_all_input_same"), "tiny", "bf16",
                        "20,3,8,5;7,2,16,3", "-m", model_dirs["a"]], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l.split() for l in r.stdout.strip().splitlines()]
    assert lines[0][:4] == ["input_len", "batch", "block", "steps"]
    assert [l[:4] for l in lines[1:]] == [["20", "3", "8", "5"], ["7", "2", "16", "3"]]
    assert all(float(v) > 0 for l in lines[1:] for v in l[4:])
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "benchmark_all_input_same"), "tiny", "int4",
                          "20,3,8,5"], capture_output=True, text=True, timeout=120)
    assert bad.returncode != 0 and "Invalid precision" in bad.stdout


def test_run_gpt_command_line(model_dirs, tmp_path):
    inp = tmp_path / "in.txt"
    prompts = [helpers.random_tokens(512, n, 500 + i) for i, n in enumerate([5, 17])]
    inp.write_text("\n".join(" ".join(map(str, p)) for p in prompts) + "\n\n")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "run_gpt"), model_dirs["a"], "tiny", "fp32",
                        str(inp), "--max_decoding_step", "6", "--block_size", "8", "--num_total_blocks", "32"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    cfg, w = plain_opt.load_model(model_dirs["a"])
    lines = [l for l in r.stdout.splitlines() if l.startswith("[")]
    assert len(lines) == 2
    for line, p in zip(lines, prompts):
        want = plain_opt.greedy_generate(cfg, w, p, 6)
        assert line.split(")")[1].split("(")[0].split() == [str(t) for t in want]
        assert "(6 tokens generated)" in line
    assert "Context stage" in r.stdout and "Regression stage" in r.stdout and r.stdout.rstrip().endswith("Done!")
    # with a vocabulary the same tokens are printed as text
    vocab = tmp_path / "vocab.json"
    vocab.write_text(json.dumps({f"Ġt{i}": i for i in range(512)}))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "run_gpt"), model_dirs["a"], "tiny", "fp32",
                        str(inp), "--max_decoding_step", "3", "--block_size", "8", "--num_total_blocks", "32",
                        "-v", str(vocab), "-d"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    first = [l for l in r.stdout.splitlines() if l.startswith("[")][0]
    want = plain_opt.greedy_generate(cfg, w, prompts[0], 3)
    assert first.split(")")[1].split("(")[0].strip() == " ".join(f"t{t}" for t in want) and "step 1:" in r.stdout
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "run_gpt"), model_dirs["a"], "tiny", "int8",
                          str(inp)], capture_output=True, text=True, timeout=600)
    assert bad.returncode == 1 and "Invalid precision" in bad.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_dirs, tmp_path, dtype):
    """bin/trace_run over standard input: `done <step>` after every step, <step>.f32 where logits are wanted."""
    name = "a"
    reqs = {f"r{i}": helpers.random_tokens(512, n, 600 + i) for i, n in enumerate([40, 70, 33, 90, 64])}
    steps = helpers.trace_mixed(reqs, seed=5)
    for i, st in enumerate(steps):
        st["step"] = i
        if i % 5 == 3:                      # some steps want nothing
            for e in st["entries"]:
                e["want"] = []
    out = tmp_path / "out"
    p = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs[name],
                          "--dtype", dtype, "--out", str(out), "--max-tokens", str(helpers.live_token_need(steps)),
                          "--page-size", "8"],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    rows = {}
    for st in steps:
        p.stdin.write(json.dumps(st) + "\n")
        p.stdin.flush()
        assert p.stdout.readline().strip() == f"done {st['step']}", p.stderr.read()[-2000:]
        n_want = sum(len(e["want"]) for e in st["entries"])
        path = out / f"{st['step']}.f32"
        if not n_want:
            assert not path.exists()
            continue
        arr = np.fromfile(path, dtype="<f4").reshape(n_want, 512)
        k = 0
        for e in st["entries"]:
            done = rows.setdefault(e["id"], {})
            base = sum(len(x) for x in done.get("_toks", []))
            for wi in e["want"]:
                done[base + wi] = arr[k]
                k += 1
        # remember how many tokens each request has been fed
    p.stdin.close()
    assert p.wait(timeout=120) == 0
    # rebuild positions: replay the bookkeeping
    fed = {}
    got = {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        arr = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(n_want, 512) if n_want else None
        k = 0
        for e in st["entries"]:
            base = fed.get(e["id"], 0)
            for wi in e["want"]:
                got.setdefault(e["id"], {})[base + wi] = arr[k]
                k += 1
            fed[e["id"]] = base + len(e["tokens"])
    for rid, toks in reqs.items():
        ref = helpers.plain_logits(model_dirs[name], toks)
        scale = np.abs(ref).max()
        for pos, row in got[rid].items():
            assert np.abs(row - ref[pos]).max() <= helpers.TOL[dtype] * scale, (rid, pos)
