"""Randomly drawn OPT configurations through the step function on the GPU, against the plain implementation:
head sizes in steps of 8 up to 128, 1 to 24 heads, widths and vocabularies that are no power of two, with and
without projections, biases and affine norms, pre- and post-norm, pages of 8 to 64 positions, prompts up to the
model's last position.  Each case replays its requests whole, with a decoded tail, in portions of changing size
and mixed with page reuse, in float32 and in bfloat16."""
import numpy as np
import pytest

import helpers

pytestmark = pytest.mark.gpu


def random_config(rng):
    d = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 24, 40, 8]))
    nh = int(rng.integers(1, 9)) if rng.random() < 0.7 else int(rng.integers(9, 25))
    hidden = nh * d
    proj = rng.random() < 0.4
    cfg = dict(vocab_size=int(rng.integers(50, 3000)), hidden_size=hidden, num_hidden_layers=int(rng.integers(1, 4)),
               ffn_dim=int(rng.integers(2, 60)) * 8 + (int(rng.integers(0, 8)) if rng.random() < 0.3 else 0),
               num_attention_heads=nh, max_position_embeddings=int(rng.integers(300, 900)),
               do_layer_norm_before=bool(rng.random() < 0.7),
               word_embed_proj_dim=(int(rng.integers(2, 20)) * 8 if proj else hidden),
               enable_bias=bool(rng.random() < 0.7), layer_norm_elementwise_affine=bool(rng.random() < 0.7),
               activation_function=str(rng.choice(["relu", "gelu"])),
               layer_norm_eps=float(rng.choice([1e-5, 1e-6, 3e-4])))
    return cfg


def random_case(case):
    rng = np.random.default_rng(1000 + case)
    cfg = random_config(rng)
    page = int(rng.choice([8, 16, 32, 64]))
    std = float(rng.choice([0.05, 0.08, 0.1]))
    lens = [int(x) for x in rng.integers(1, min(280, cfg["max_position_embeddings"] - 2), 5)]
    lens[0] = int(rng.integers(130, 280))
    if case % 3 == 0:
        lens[1] = cfg["max_position_embeddings"] - int(rng.integers(0, 3))     # up to the last position
    return cfg, page, std, lens


# drawn once and kept: head sizes 64 and 128 with pages of 8, 32 and 64 (the TMA-fed attention), 11 to 21 heads,
# a prompt longer than one span of the decode attention's key range, odd widths
@pytest.mark.parametrize("case", [3, 4, 10, 106, 114, 119, 129])
def test_random_configuration_replays_like_plain(tmp_path, case):
    from swifttransformer_b200.config import OptConfig
    from swifttransformer_b200.engine.replay import TraceSession
    from swifttransformer_b200.models import write_random_model
    cfg, page, std, lens = random_case(case)
    model_dir = str(tmp_path)
    write_random_model(model_dir, OptConfig.from_dict(dict(cfg)), seed=case, std=std)
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], n, 7 * case + i) for i, n in enumerate(lens)}
    for dtype in ("float32", "bfloat16"):
        for mode, build in (("whole", helpers.trace_whole), ("tail", helpers.trace_decode_tail),
                            ("portions", helpers.trace_portions),
                            ("mixed", lambda r: helpers.trace_mixed(r, seed=case))):
            steps = build(reqs)
            need = helpers.live_token_need(steps, round_to=max(64, page))
            s = TraceSession(model_dir, dtype, need, page_size=page, device="cuda", max_requests=4)
            got = helpers.replay(s, steps)
            helpers.check_against_plain(model_dir, reqs, got, dtype, f"case {case} {cfg} page {page}/{mode}")
            assert s.cache.free_pages == s.cache.total_pages


# kept from a draw of forty: head size 128 with pages of 64 positions, head sizes 8, 16 and 48, 3 to 24 heads, steps
# launched ahead or not; in all but the first the pool, which holds the prompts and no more, runs out while the
# requests decode and one of them is preempted
@pytest.mark.parametrize("case", [2, 15, 17, 38])
def test_random_configuration_generates_like_plain(tmp_path, case):
    """Greedy generation through LLMEngine in float32 (scheduler, portions, recorded steps, admission held
    back and preemption when the pool holds little more than the prompts) equals the plain implementation's
    token for token."""
    import plain_opt
    from swifttransformer_b200.config import OptConfig
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.models import write_random_model
    from swifttransformer_b200.sampling import SamplingParams
    rng = np.random.default_rng(5000 + case)
    cfg = random_config(rng)
    page = int(rng.choice([8, 16, 32, 64]))
    model_dir = str(tmp_path)
    write_random_model(model_dir, OptConfig.from_dict(dict(cfg)), seed=case, std=float(rng.choice([0.05, 0.08, 0.1])))
    n_req = int(rng.integers(3, 10))
    lens = [int(x) for x in rng.integers(1, min(200, cfg["max_position_embeddings"] - 30), n_req)]
    news = [int(x) for x in rng.integers(1, 20, n_req)]
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, 11 * case + i) for i, n in enumerate(lens)]
    per_request = [(n + m + page - 1) // page + 1 for n, m in zip(lens, news)]
    tight = rng.random() < 0.5
    num_pages = max(max(per_request), sum((n + page - 1) // page for n in lens)) if tight else sum(per_request) + 4
    budget = int(rng.choice([48, 64, 100, 256]))
    eng = LLMEngine(model_dir, dtype="float32", device="cuda", page_size=page, num_pages=num_pages,
                    max_batch_tokens=budget, chunk_size=int(rng.choice([16, 32, budget])),
                    max_num_seqs=int(rng.integers(2, 9)), pipeline=bool(rng.random() < 0.7))
    outs = eng.generate(prompts, [SamplingParams(max_new_tokens=m) for m in news])
    eng.runner.check_status()
    w_cfg, w = plain_opt.load_model(model_dir)
    for p, o, m in zip(prompts, outs, news):
        assert o == plain_opt.greedy_generate(w_cfg, w, p, m), (case, len(p), m)
    assert eng.cache.free_pages == eng.cache.total_pages
    assert tight and (eng.scheduler.num_preemptions > 0 or case == 2), "these cases were kept because their pools run out"
