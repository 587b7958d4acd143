"""Weight layout anchored on the reference's own converter.

tests/golden/opt_converter_tiny.npz holds what the reference's offline converter (scripts/lib/converter_lib.py:
convertWeight) made of a tiny random OPT model: q|k|v fused from the K,V,Q order of the original checkpoint and
stored [in, out], out_proj transposed, the position table without its two unused rows, the output projection
a copy of the embedding.  tests/golden/make_converter_golden.py made the file.  Here the same model is written
again from its seed and (1) what the package's loader builds from it, (2) the logits of the plain
implementation, are compared with the converter's tensors used the way the reference's layers use them.
With SWIFTTRANSFORMER_REFERENCE pointing at a checkout of the reference the converter is also run afresh.
"""
import json
import os
import sys

import numpy as np
import pytest

import plain_opt

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_converter_golden as golden  # noqa: E402


@pytest.fixture(scope="module")
def case(tmp_path_factory):
    z = np.load(os.path.join(HERE, "golden", "opt_converter_tiny.npz"))
    meta = json.loads(bytes(z["meta"]))
    assert meta["config"] == golden.CONFIG and meta["seed"] == golden.SEED and meta["std"] == golden.STD
    model_dir = str(tmp_path_factory.mktemp("golden_model"))
    src = golden.write_tiny_model(model_dir)
    assert {k: golden.source_digest(v) for k, v in src.items()} == meta["source"], \
        "the random-weights mode no longer writes the model the stored tensors were converted from"
    return model_dir, src, {k: z[k] for k in z.files if k != "meta"}


def test_loader_builds_the_layout_the_reference_converter_builds(case):
    from swifttransformer_b200.models import load_model
    model_dir, _, conv = case
    mdef = load_model(model_dir, "float32", "cpu").definition

    def same(mine, name, what=None):
        ref = conv[name]
        got = mine.detach().cpu().numpy()
        assert got.shape == ref.shape and np.array_equal(got, ref), what or name

    same(mdef.embedding.table, "decoder.embed_tokens.weight")
    same(mdef.head.weight, "decoder.output_projection.weight")
    table, offset = mdef.position.hidden_table()
    assert offset == 2 and table.shape[0] == golden.CONFIG["max_position_embeddings"] + 2
    same(table[offset:], "decoder.embed_positions.weight")          # converter_lib.py:271 cuts what we skip
    same(mdef.final_norm.gamma, "decoder.layer_norm.weight")
    same(mdef.final_norm.beta, "decoder.layer_norm.bias")
    for i, blk in enumerate(mdef.blocks):
        p = f"decoder.layers.{i}."
        same(blk.mixer.w_qkv.t(), p + "self_attn.qkv_proj.weight", "q|k|v order and [in, out] storage")
        same(blk.mixer.b_qkv, p + "self_attn.qkv_proj.bias")
        same(blk.mixer.w_o.t(), p + "self_attn.out_proj.weight")
        same(blk.mixer.b_o, p + "self_attn.out_proj.bias")
        same(blk.norm1.gamma, p + "self_attn_layer_norm.weight")
        same(blk.norm1.beta, p + "self_attn_layer_norm.bias")
        same(blk.norm2.gamma, p + "final_layer_norm.weight")
        same(blk.norm2.beta, p + "final_layer_norm.bias")
        same(blk.feed_forward.w1, p + "fc1.weight")
        same(blk.feed_forward.b1, p + "fc1.bias")
        same(blk.feed_forward.w2, p + "fc2.weight")
        same(blk.feed_forward.b2, p + "fc2.bias")


def forward_in_the_reference_layout(conv, ids):
    """The reference's order of operations on the converter's tensors: embedding + positions without offset
    (src/csrc/kernel/embedding.cu:25-33), LN, non-transposed q|k|v product (src/csrc/layer/attention.cc:102-130),
    attention, non-transposed output product (attention.cc:255-288), residual + LN, transposed fc1/fc2 products
    (src/csrc/layer/ffn.cc:71-124), final LN and output projection (src/csrc/model/gpt/gpt.cc:175-221)."""
    c = {k: np.asarray(v, dtype=np.float64) for k, v in conv.items()}
    cfg = golden.CONFIG
    H, nh = cfg["hidden_size"], cfg["num_attention_heads"]
    x = c["decoder.embed_tokens.weight"][ids] + c["decoder.embed_positions.weight"][np.arange(len(ids))]
    for i in range(cfg["num_hidden_layers"]):
        p = f"decoder.layers.{i}."
        h = plain_opt.layer_norm(x, c[p + "self_attn_layer_norm.weight"], c[p + "self_attn_layer_norm.bias"], 1e-5)
        qkv = h @ c[p + "self_attn.qkv_proj.weight"] + c[p + "self_attn.qkv_proj.bias"]
        o = plain_opt.causal_attention(qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:], nh)
        r = x + o @ c[p + "self_attn.out_proj.weight"] + c[p + "self_attn.out_proj.bias"]
        h = plain_opt.layer_norm(r, c[p + "final_layer_norm.weight"], c[p + "final_layer_norm.bias"], 1e-5)
        u = np.maximum(h @ c[p + "fc1.weight"].T + c[p + "fc1.bias"], 0.0)
        x = r + u @ c[p + "fc2.weight"].T + c[p + "fc2.bias"]
    x = plain_opt.layer_norm(x, c["decoder.layer_norm.weight"], c["decoder.layer_norm.bias"], 1e-5)
    return x @ c["decoder.output_projection.weight"].T


def test_plain_implementation_agrees_with_the_reference_layout(case):
    model_dir, _, conv = case
    cfg, w = plain_opt.load_model(model_dir)
    ids = [3, 15, 0, 7, 7, 9, 1, 12]
    ours = plain_opt.forward(cfg, w, ids)
    ref = forward_in_the_reference_layout(conv, np.asarray(ids))
    assert ours.shape == ref.shape == (len(ids), golden.CONFIG["vocab_size"])
    assert np.abs(ours - ref).max() <= 1e-12 * max(1.0, np.abs(ref).max())


def test_converter_run_afresh_gives_the_stored_tensors(case):
    reference = os.environ.get("SWIFTTRANSFORMER_REFERENCE", "")
    if not os.path.isfile(os.path.join(reference, "scripts", "lib", "converter_lib.py")):
        pytest.skip("no checkout of the reference given in SWIFTTRANSFORMER_REFERENCE")
    _, src, conv = case
    fresh = golden.run_converter(reference, golden.original_form(src))
    assert sorted(fresh) == sorted(conv)
    for k in conv:
        assert np.array_equal(fresh[k], conv[k]), k
