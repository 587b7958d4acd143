"""The plain implementation checked against itself and against elementary torch operations (CPU)."""
import numpy as np
import torch

import helpers
import plain_opt


def test_logits_at_chosen_rows_equal_the_rows_of_all_logits(model_dirs):
    for name in ("a", "b"):
        cfg, w = plain_opt.load_model(model_dirs[name])
        toks = helpers.random_tokens(cfg["vocab_size"], 23, 4)
        full = plain_opt.forward(cfg, w, toks)
        assert full.shape == (23, cfg["vocab_size"])
        assert np.array_equal(plain_opt.forward(cfg, w, toks, rows=[0, 7, 22]), full[[0, 7, 22]])


def test_a_position_does_not_see_later_tokens(model_dirs):
    for name in ("a", "b", "c"):
        cfg, w = plain_opt.load_model(model_dirs[name])
        toks = helpers.random_tokens(cfg["vocab_size"], 30, 5)
        full = plain_opt.forward(cfg, w, toks)
        assert np.abs(plain_opt.forward(cfg, w, toks[:11]) - full[:11]).max() < 1e-12
        other = toks[:11] + helpers.random_tokens(cfg["vocab_size"], 19, 6)
        assert np.abs(plain_opt.forward(cfg, w, other)[:11] - full[:11]).max() < 1e-12
        assert np.abs(plain_opt.forward(cfg, w, other)[11:] - full[11:]).max() > 1e-3


def test_parts_equal_elementary_torch_operations():
    rng = np.random.default_rng(0)
    x, g, b = rng.normal(size=(5, 24)), rng.normal(size=24), rng.normal(size=24)
    t = torch.nn.functional.layer_norm(torch.tensor(x), (24,), torch.tensor(g), torch.tensor(b), 3e-4)
    assert np.abs(plain_opt.layer_norm(x, g, b, 3e-4) - t.numpy()).max() < 1e-12
    t = torch.nn.functional.layer_norm(torch.tensor(x), (24,), None, None, 1e-5)
    assert np.abs(plain_opt.layer_norm(x, None, None, 1e-5) - t.numpy()).max() < 1e-12
    assert np.abs(plain_opt.activation(x, "gelu") - torch.nn.functional.gelu(torch.tensor(x)).numpy()).max() < 1e-12
    assert np.array_equal(plain_opt.activation(x, "relu"), np.where(x > 0, x, 0))
    q, k, v = (rng.normal(size=(9, 24)) for _ in range(3))
    heads = [torch.tensor(a).reshape(9, 3, 8).transpose(0, 1) for a in (q, k, v)]
    t = torch.nn.functional.scaled_dot_product_attention(*heads, is_causal=True).transpose(0, 1).reshape(9, 24)
    assert np.abs(plain_opt.causal_attention(q, k, v, 3) - t.numpy()).max() < 1e-12
    # a window of 4 keeps keys i-3..i
    win = plain_opt.causal_attention(q, k, v, 3, window=4)
    assert np.abs(win[:4] - t.numpy()[:4]).max() < 1e-12 and np.abs(win[4:] - t.numpy()[4:]).max() > 1e-3
    last = plain_opt.causal_attention(q[-4:], k[-4:], v[-4:], 3)[-1]
    assert np.abs(win[-1] - last).max() < 1e-12


def test_sampling_follows_the_inverse_distribution():
    logits = np.log(np.array([0.1, 0.2, 0.3, 0.4]))
    assert [plain_opt.softmax_sample(logits, 1.0, u) for u in (0.05, 0.25, 0.5, 0.99)] == [0, 1, 2, 3]
    assert [plain_opt.softmax_sample(logits, 1.0, u, top_k=2) for u in (0.01, 0.42, 0.44, 0.99)] == [2, 2, 3, 3]
