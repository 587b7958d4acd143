"""Schedules and settings beyond the four replay modes of the tiny configurations: sixteen live requests at
head sizes 64 and 128 (replayed and generated), pages of 1, 2 and 4 positions (the reference's benchmark grids
use them, src/examples/benchmark_all_input_same.cc:41-93), a page pool sized from the free device memory, and
the bfloat16 engine against the CPU reference operations run with bfloat16 storage at the same places."""
import numpy as np
import pytest
import torch

import helpers
import plain_opt
from helpers import TINY

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]

# narrow models with the head sizes of OPT-1.3B and OPT-6.7B
HEADS = {
    "d64": dict(cfg=dict(vocab_size=600, hidden_size=256, num_hidden_layers=2, ffn_dim=384, num_attention_heads=4,
                         max_position_embeddings=320, do_layer_norm_before=True, word_embed_proj_dim=256,
                         enable_bias=True, layer_norm_elementwise_affine=True, activation_function="relu"),
                seed=41, std=0.06),
    "d128": dict(cfg=dict(vocab_size=500, hidden_size=384, num_hidden_layers=2, ffn_dim=520, num_attention_heads=3,
                          max_position_embeddings=300, do_layer_norm_before=False, word_embed_proj_dim=384,
                          enable_bias=True, layer_norm_elementwise_affine=True, activation_function="relu"),
                 seed=42, std=0.05),
}


@pytest.fixture(scope="module")
def head_models(tmp_path_factory):
    from swifttransformer_b200.config import OptConfig
    from swifttransformer_b200.models import write_random_model
    out = {}
    for name, spec in HEADS.items():
        d = str(tmp_path_factory.mktemp(name))
        write_random_model(d, OptConfig.from_dict(dict(spec["cfg"])), seed=spec["seed"], std=spec["std"])
        out[name] = d
    return out


def trace_session(model_dir, dtype, max_tokens, page_size, **kw):
    from swifttransformer_b200.engine.replay import TraceSession
    return TraceSession(model_dir, dtype, max_tokens, page_size=page_size, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(HEADS))
def test_sixteen_live_requests_replayed(head_models, name, dtype):
    """Portions of some requests beside decoded tokens of others, up to sixteen at a time, in a pool that holds
    exactly what the live requests need: more single tokens in a step than the weight-streaming product takes,
    so library products, the separate cache write and the tensor-core decode attention run together."""
    cfg = HEADS[name]["cfg"]
    rng = np.random.default_rng(3)
    lens = [int(x) for x in rng.integers(20, cfg["max_position_embeddings"], 28)]
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], n, 600 + i) for i, n in enumerate(lens)}
    steps = helpers.trace_mixed(reqs, seed=4, max_live=16, chunk=40, prompt_frac=0.4)
    assert max(sum(1 for e in st["entries"] if len(e["tokens"]) == 1) for st in steps) > 8
    s = trace_session(head_models[name], dtype, helpers.live_token_need(steps), 16, max_requests=16,
                      max_batch_tokens=1024)
    got = helpers.replay(s, steps)
    helpers.check_against_plain(head_models[name], reqs, got, dtype, f"{name}/16 live")
    assert s.cache.free_pages == s.cache.total_pages
    s.runner.check_status()


@pytest.mark.parametrize("name", list(HEADS))
def test_steps_of_single_tokens_and_short_portions_attend_from_the_projection(head_models, name, monkeypatch):
    """Twelve requests: prompts in long portions (tiles, the separate cache write), then steps in which every
    request brings one token or a portion of 2 to 15 (all of them single queries to the attention): more tokens
    than the weight-streaming product serves, no tiles, so the attention kernel works from the q|k|v product and
    writes the cache itself.  Keys of the same step, page edges inside a portion, and later steps that read what
    these wrote all show in the logits."""
    from swifttransformer_b200 import ops
    cfg = HEADS[name]["cfg"]
    calls = []
    real = ops.attention_decode_qkv
    monkeypatch.setattr(ops, "attention_decode_qkv", lambda *a, **k: (calls.append(a[0].shape[0]), real(*a, **k))[1])
    rng = np.random.default_rng(11)
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], int(rng.integers(120, 250)), 700 + i) for i in range(12)}
    pos = {rid: int(rng.integers(40, 90)) for rid in reqs}
    steps = [dict(entries=[dict(id=rid, tokens=reqs[rid][:pos[rid]], want=[pos[rid] - 1]) for rid in list(reqs)[a:a + 4]],
                  end=[]) for a in (0, 4, 8)]
    live = set(reqs)
    while live:
        entries, end = [], []
        for rid in sorted(live):
            left = len(reqs[rid]) - pos[rid]
            n = min(left, int(rng.choice([1, 1, 1, 2, 3, 5, 15])))
            entries.append(dict(id=rid, tokens=reqs[rid][pos[rid]:pos[rid] + n], want=list(range(n))))
            pos[rid] += n
            if pos[rid] == len(reqs[rid]):
                end.append(rid)
        live -= set(end)
        steps.append(dict(entries=entries, end=end))
    s = trace_session(head_models[name], "bfloat16", helpers.live_token_need(steps), 16, max_requests=12,
                      max_batch_tokens=1024)
    got = helpers.replay(s, steps)
    layers = cfg["num_hidden_layers"]
    assert len(calls) >= layers * 20 and max(calls) > 8, "the steps of single queries took the kernel under test"
    # the first wanted row of a request is the last of its prompt; the rest follow position by position
    for rid, toks in reqs.items():
        first = len(toks) - got[rid].shape[0]
        ref = helpers.plain_logits(head_models[name], toks)[first:]
        bad = helpers.first_bad(got[rid], ref, helpers.TOL["bfloat16"] * np.abs(ref).max())
        assert bad is None, f"{name}/{rid}: position {first + bad[0]} differs by {bad[1]:.3e}"
    assert s.cache.free_pages == s.cache.total_pages
    s.runner.check_status()


@pytest.mark.parametrize("name", list(HEADS))
def test_sixteen_live_requests_generated_bfloat16(head_models, name):
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.sampling import SamplingParams
    cfg, w = plain_opt.load_model(head_models[name])
    rng = np.random.default_rng(5)
    prompts = [helpers.random_tokens(cfg["vocab_size"], int(n), 700 + i) for i, n in enumerate(rng.integers(1, 90, 20))]
    eng = LLMEngine(head_models[name], dtype="bfloat16", page_size=16, num_pages=200, max_batch_tokens=256,
                    chunk_size=64, max_num_seqs=16)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12))
    eng.runner.check_status()
    assert eng.runner.graph_steps > 0 and eng.cache.free_pages == eng.cache.total_pages
    assert max(b for (_, b, _, *_) in eng.runner._graphs) >= 16, "sixteen requests decoded in one recorded step"
    for p, o in zip(prompts, outs):
        ids = list(p)
        for tok in o:
            logits = plain_opt.forward(cfg, w, ids, rows=[len(ids) - 1])[0]
            best = int(np.argmax(logits))
            if tok != best:       # only where the plain implementation's top two are within bfloat16 error
                assert logits[best] - logits[tok] < 4e-2 * np.abs(logits).max(), (tok, best)
            ids.append(tok)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page_size", [1, 2, 4])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_small_pages(model_dirs, head_models, mode, page_size, dtype):
    """The four ways of cutting the same requests with pages of 1, 2 and 4 positions, on tiny A (head size 16)
    and on the narrow model with head size 64."""
    build = {"whole": helpers.trace_whole, "decode_tail": helpers.trace_decode_tail,
             "portions": helpers.trace_portions, "mixed": helpers.trace_mixed}[mode]
    for model_dir, vocab, lens in ((model_dirs["a"], 512, [5, 33, 128, 64]), (head_models["d64"], 600, [150, 41, 3])):
        reqs = {f"r{i}": helpers.random_tokens(vocab, n, 800 + i) for i, n in enumerate(lens)}
        steps = build(reqs)
        s = trace_session(model_dir, dtype, helpers.live_token_need(steps), page_size, max_requests=4)
        got = helpers.replay(s, steps)
        helpers.check_against_plain(model_dir, reqs, got, dtype, f"page {page_size}/{mode}")
        assert s.cache.free_pages == s.cache.total_pages
        s.runner.check_status()


def test_the_pool_is_sized_from_free_memory_when_no_page_count_is_given(model_dirs):
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.sampling import SamplingParams
    free, _ = torch.cuda.mem_get_info()
    eng = LLMEngine(model_dirs["a"], dtype="bfloat16", page_size=8, max_num_seqs=8, memory_fraction=0.01)
    per_page = eng.cache.bytes_per_token() * 8
    # every slot filled to the model's 128 positions needs 8 * 16 pages; one hundredth of the free memory holds more
    assert eng.cache.total_pages == 8 * 16 and eng.cache.total_pages * per_page < 0.011 * free
    cfg, w = plain_opt.load_model(model_dirs["a"])
    prompt = helpers.random_tokens(512, 20, 6)
    out = eng.generate([prompt], SamplingParams(max_new_tokens=4))[0]
    ids = list(prompt)
    for tok in out:
        logits = plain_opt.forward(cfg, w, ids)[-1]
        assert tok == int(np.argmax(logits)) or logits.max() - logits[tok] < 4e-2 * np.abs(logits).max()
        ids.append(tok)
    # a fraction that holds fewer pages than that bounds the pool
    small = LLMEngine(model_dirs["a"], dtype="bfloat16", page_size=8, max_num_seqs=8,
                      memory_fraction=40 * per_page / free)
    assert 30 <= small.cache.total_pages <= 40


@pytest.mark.parametrize("name", ["a", "b", "c", "d64", "d128"])
def test_bfloat16_engine_against_reference_operations_with_bfloat16_storage(model_dirs, head_models, name, monkeypatch):
    """The bfloat16 engine differs from the float64 plain implementation by a few per cent of the largest
    logit, nearly all of it the rounding of weights' products and activations to bfloat16 where they are
    stored.  Run through the CPU reference operations (tests/cpu_ops.py: float64 arithmetic) with the same
    bfloat16 storage at the same places, the same model must come far closer: what is left is the order of
    float32 sums, probabilities rounded for the tensor cores, and a rounding that flips here and there.  A
    kernel that drops a key or a tile would not hide in this bound."""
    import cpu_ops
    from swifttransformer_b200.engine.replay import TraceSession
    model_dir = model_dirs[name] if name in model_dirs else head_models[name]
    spec = TINY[name] if name in TINY else HEADS[name]
    cfg = spec["cfg"]
    page = spec.get("page_size", 16)
    lens = [n for n in (200, 65, 33, 290) if n <= cfg["max_position_embeddings"]]
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], n, 950 + i) for i, n in enumerate(lens)}
    steps = helpers.trace_mixed(reqs, seed=9, max_live=3, chunk=48)
    need = helpers.live_token_need(steps)
    gpu = TraceSession(model_dir, "bfloat16", need, page_size=page, max_requests=4)
    got = helpers.replay(gpu, steps)
    cpu_ops.install(monkeypatch)
    cpu = TraceSession(model_dir, "bfloat16", need, page_size=page, max_requests=4, device="cpu")
    ref = helpers.replay(cpu, steps)
    monkeypatch.undo()
    for rid in reqs:
        scale = np.abs(ref[rid]).max()
        err = np.abs(got[rid] - ref[rid])
        assert err.max() < 1.5e-2 * scale, (rid, int(err.max(axis=1).argmax()), float(err.max() / scale))
        assert err.mean() < 1.5e-3 * scale, (rid, float(err.mean() / scale))


def test_an_engine_that_goes_out_of_scope_gives_its_memory_back_at_once(model_dirs):
    """Recorded steps and their runner refer to one another weakly: dropping the last reference to an engine frees
    its pool and its graphs without a run of the garbage collector."""
    import gc
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.sampling import SamplingParams

    def use_one():
        eng = LLMEngine(model_dirs["c"], dtype="bfloat16", page_size=32, num_pages=4000, max_num_seqs=4)
        eng.generate([helpers.random_tokens(777, 40, 1), helpers.random_tokens(777, 9, 2)], SamplingParams(max_new_tokens=5))
        assert eng.runner.graph_steps > 0
        torch.cuda.synchronize()
        return torch.cuda.memory_allocated()          # the engine dies with this frame

    use_one()                 # what libraries allocate once and keep (workspaces) is there after this
    gc.collect()
    gc.disable()
    try:
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        during = use_one()
        torch.cuda.synchronize()
        assert during > before + 50e6
        # the pool, the weights and the recorded steps' memory are back; a megabyte or two that torch's graph
        # objects hold in cycles of their own waits for the collector
        assert torch.cuda.memory_allocated() < before + 0.05 * (during - before)
    finally:
        gc.enable()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b"])
def test_every_kernel_of_a_mixed_trace_against_its_reference(model_dirs, name, dtype):
    """The checking mode (tests/paranoid.py): a mixed trace launched kernel by kernel, every operation's outputs
    compared with the CPU reference of that operation on the same inputs."""
    import paranoid
    from swifttransformer_b200.engine.replay import TraceSession
    cfg = TINY[name]["cfg"]
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], n, 70 + i) for i, n in enumerate([40, 9, 64, 23])}
    steps = helpers.trace_mixed(reqs, seed=11, max_live=3, chunk=20)
    s = TraceSession(model_dirs[name], dtype, helpers.live_token_need(steps), page_size=TINY[name]["page_size"],
                     max_requests=4)
    s.runner.use_cuda_graphs = False
    with paranoid.watch() as log:
        got = helpers.replay(s, steps)
    helpers.check_against_plain(model_dirs[name], reqs, got, dtype, f"paranoid/{name}")
    assert log["calls"] > 10 * len(steps)
    assert {"embed", "add_norm", "linear", "attention_plain" if dtype == "float32" else "attention_decode"} <= set(log["by_name"])


def test_the_checking_mode_notices_a_wrong_kernel(model_dirs, monkeypatch):
    import paranoid
    from swifttransformer_b200 import ops
    from swifttransformer_b200.engine.replay import TraceSession
    real = ops.bias_act

    def off_by_a_little(y, bias, act):
        real(y, bias, act)
        y[0, 0] += 0.5
        return y
    monkeypatch.setattr(ops, "bias_act", off_by_a_little)
    s = TraceSession(model_dirs["c"], "bfloat16", 128, page_size=32, max_requests=2)     # gelu: bias_act runs
    s.runner.use_cuda_graphs = False
    with paranoid.watch():
        # the outermost operation is the one compared: the library product whose bias and activation kernel is off
        with pytest.raises(paranoid.ParanoidError, match="linear .* the result differs"):
            s.run_step([dict(id="x", tokens=helpers.random_tokens(777, 30, 3), want=[29])])


def test_operation_times_without_a_profiler(model_dirs):
    from swifttransformer_b200.engine.replay import TraceSession
    from swifttransformer_b200.ops import timing
    s = TraceSession(model_dirs["a"], "bfloat16", 128, page_size=8, max_requests=2)
    s.runner.use_cuda_graphs = False
    toks = helpers.random_tokens(512, 40, 5)
    s.run_step([dict(id="x", tokens=toks[:39], want=[])])
    timing.start()
    with pytest.raises(RuntimeError):
        timing.start()
    s.run_step([dict(id="x", tokens=toks[39:], want=[0])])
    report = timing.stop()
    layers = TINY["a"]["cfg"]["num_hidden_layers"]
    # a single-token step: per layer the norm + q|k|v + cache write (one operation for the engine), the attention,
    # two products with the residual sum behind and the norm + fc1; then the final norm and the output head
    assert report["norm_qkv_linear_to_cache"]["calls"] == layers and report["attention_decode"]["calls"] == layers
    assert report["linear_add"]["calls"] == 2 * layers and report["norm_linear"]["calls"] == layers
    assert report["add_norm"]["calls"] == 1
    assert all(r["ms"] > 0 for r in report.values()) and list(report) == sorted(report, key=lambda k: -report[k]["ms"])
    from swifttransformer_b200 import ops
    assert ops.add_norm.__name__ == "add_norm" and not hasattr(ops.add_norm, "__wrapped__")
