"""Configuration, registry, safetensors reading and the weight loader's errors (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import helpers
from swifttransformer_b200.config import ConfigError, OptConfig, config_from_dict, load_config, opt_preset
from swifttransformer_b200.models import build_model_def, load_model, write_random_model
from swifttransformer_b200.weights import (ParamSpec, SafetensorsError, SafetensorsFile, WeightError,
                                           write_safetensors)


def test_config_reads_its_own_keys(tmp_path):
    raw = dict(helpers.TINY["b"]["cfg"], architectures=["OPTForCausalLM"], dropout=0.1, some_unknown_key=3)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    cfg = load_config(str(tmp_path))
    assert isinstance(cfg, OptConfig)
    assert (cfg.hidden_size, cfg.num_attention_heads, cfg.head_dim, cfg.ffn_dim) == (96, 3, 32, 320)
    assert cfg.has_projections and not cfg.do_layer_norm_before and not cfg.has_final_layer_norm
    assert cfg.layer_norm_eps == 1e-5 and cfg.position_offset == 2
    back = config_from_dict(cfg.to_dict())
    assert back == cfg


def test_config_errors_name_the_key(tmp_path):
    base = dict(helpers.TINY["a"]["cfg"], architectures=["OPTForCausalLM"])
    for key in ("hidden_size", "vocab_size", "ffn_dim", "num_attention_heads", "num_hidden_layers",
                "max_position_embeddings"):
        raw = dict(base)
        del raw[key]
        with pytest.raises(ConfigError, match=key):
            config_from_dict(raw)
    with pytest.raises(ConfigError, match="num_attention_heads"):
        config_from_dict(dict(base, num_attention_heads=5))
    with pytest.raises(ConfigError, match="activation_function"):
        config_from_dict(dict(base, activation_function="swish"))
    with pytest.raises(ConfigError, match="hidden_size"):
        config_from_dict(dict(base, hidden_size="64"))
    with pytest.raises(ConfigError, match="enable_bias"):
        config_from_dict(dict(base, enable_bias=1))
    with pytest.raises(ConfigError, match="unknown architecture.*OPTForCausalLM"):
        config_from_dict(dict(base, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in base.items() if k != "architectures"})
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))


def test_presets_and_remove_final_layer_norm():
    cfg = opt_preset("opt_1.3b")
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.head_dim, cfg.ffn_dim,
            cfg.vocab_size) == (24, 2048, 32, 64, 8192, 50272)
    assert opt_preset("OPT-30B").hidden_size == 7168
    with pytest.raises(ConfigError, match="opt_6.7b"):
        opt_preset("opt_7b")
    raw = dict(helpers.TINY["a"]["cfg"], architectures=["OPTForCausalLM"], _remove_final_layer_norm=True)
    cfg = config_from_dict(raw)
    assert not cfg.has_final_layer_norm
    assert build_model_def(cfg).final_norm is None


def test_model_definition_follows_the_configuration():
    a, b = build_model_def(helpers.tiny_config("a")), build_model_def(helpers.tiny_config("b"))
    names_a = {s.name for s in a.param_specs()}
    names_b = {s.name for s in b.param_specs()}
    assert "model.decoder.layers.1.self_attn.q_proj.bias" in names_a
    assert "model.decoder.final_layer_norm.weight" in names_a
    assert "model.decoder.project_in.weight" not in names_a
    assert not any(n.endswith(".bias") for n in names_b), "no biases and no affine norms in configuration b"
    assert {"model.decoder.project_in.weight", "model.decoder.project_out.weight"} <= names_b
    assert "model.decoder.final_layer_norm.weight" not in names_b
    shapes = {s.name: s.shape for s in b.param_specs()}
    assert shapes["model.decoder.embed_tokens.weight"] == (1000, 48)
    assert shapes["model.decoder.embed_positions.weight"] == (258, 96)
    assert shapes["model.decoder.project_in.weight"] == (96, 48)
    assert shapes["model.decoder.layers.2.fc1.weight"] == (320, 96)
    assert len(a.cache_specs()) == 2 and len(b.cache_specs()) == 3
    assert a.cache_specs()[0].head_dim == 16 and b.cache_specs()[0].num_kv_heads == 3


def test_random_folder_round_trip_and_determinism(tmp_path):
    d1 = write_random_model(str(tmp_path / "m1"), helpers.tiny_config("a"), seed=5)
    d2 = write_random_model(str(tmp_path / "m2"), helpers.tiny_config("a"), seed=5)
    d3 = write_random_model(str(tmp_path / "m3"), helpers.tiny_config("a"), seed=6)
    f1, f2, f3 = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (d1, d2, d3))
    assert "lm_head.weight" not in f1.names(), "the tied output matrix is not stored twice"
    for n in f1.names():
        assert torch.equal(f1.get(n), f2.get(n))
    assert not torch.equal(f1.get("model.decoder.embed_tokens.weight"), f3.get("model.decoder.embed_tokens.weight"))
    assert f1.get("model.decoder.embed_tokens.weight").dtype == torch.bfloat16
    m16 = load_model(d1, "bfloat16", "cpu")
    m32 = load_model(d1, "float32", "cpu")
    assert m16.embedding.table.dtype == torch.bfloat16 and m32.embedding.table.dtype == torch.float32
    assert torch.equal(m16.embedding.table.float(), m32.embedding.table), "both dtypes see the same numbers"
    assert m16.final_norm.gamma.dtype == torch.float32, "vectors are kept in 32-bit"
    assert m16.head.weight.data_ptr() == m16.embedding.table.data_ptr(), "tied: one tensor, not a copy"
    blk = m32.blocks[0]
    assert blk.mixer.w_qkv.shape == (3 * 64, 64) and blk.mixer.b_qkv.shape == (3 * 64,)
    q = f1.get("model.decoder.layers.0.self_attn.q_proj.weight").float()
    v = f1.get("model.decoder.layers.0.self_attn.v_proj.weight").float()
    assert torch.equal(blk.mixer.w_qkv[:64], q) and torch.equal(blk.mixer.w_qkv[128:], v)
    # the plain implementation reads the same folder
    import plain_opt
    cfg, w = plain_opt.load_model(d1)
    assert np.array_equal(w["model.decoder.embed_tokens.weight"], m32.embedding.table.double().numpy())


def _rewrite(src_dir, dst_dir, edit):
    os.makedirs(dst_dir, exist_ok=True)
    with open(os.path.join(src_dir, "config.json")) as f:
        open(os.path.join(dst_dir, "config.json"), "w").write(f.read())
    sf = SafetensorsFile(os.path.join(src_dir, "model.safetensors"))
    tensors = {n: sf.get(n).clone() for n in sf.names()}
    edit(tensors)
    write_safetensors(os.path.join(dst_dir, "model.safetensors"), tensors.items())
    return dst_dir


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    src = write_random_model(str(tmp_path / "ok"), helpers.tiny_config("a"), seed=1)

    def edit(t):
        del t["model.decoder.layers.0.fc1.bias"]
        del t["model.decoder.layers.1.self_attn.k_proj.weight"]
        t["model.decoder.layers.7.fc1.weight"] = torch.zeros(2, 2)
        t["model.decoder.embed_positions.weight"] = torch.zeros(128, 64, dtype=torch.bfloat16)   # offset rows cut
        t["model.decoder.final_layer_norm.weight"] = torch.zeros(64, dtype=torch.int32)
    bad = _rewrite(src, str(tmp_path / "bad"), edit)
    with pytest.raises(WeightError) as ei:
        load_model(bad, "float32", "cpu")
    e = ei.value
    assert sorted(e.missing) == ["model.decoder.layers.0.fc1.bias", "model.decoder.layers.1.self_attn.k_proj.weight"]
    assert e.unexpected == ["model.decoder.layers.7.fc1.weight"]
    assert len(e.wrong_shape) == 2
    msg = str(e)
    for needle in ("missing", "unexpected", "wrong shape", "[128, 64]", "[130, 64]", "layers.7.fc1.weight"):
        assert needle in msg


def test_checkpoint_variants(tmp_path):
    src = write_random_model(str(tmp_path / "ok"), helpers.tiny_config("a"), seed=2)
    # names without the leading "model.", a version marker, a repeated (identical) tied output matrix, float32 storage
    def edit(t):
        for n in list(t):
            t[n[len("model."):]] = t.pop(n).float()
        t["decoder.version"] = torch.zeros(1)
        t["lm_head.weight"] = t["decoder.embed_tokens.weight"].clone()
    alt = _rewrite(src, str(tmp_path / "alt"), edit)
    m, ref = load_model(alt, "float32", "cpu"), load_model(src, "float32", "cpu")
    assert torch.equal(m.blocks[1].feed_forward.w1, ref.blocks[1].feed_forward.w1)
    # a tied output matrix that differs from the embedding is an error
    def edit2(t):
        t["lm_head.weight"] = t["model.decoder.embed_tokens.weight"].clone() + 1
    with pytest.raises(WeightError, match="ties"):
        load_model(_rewrite(src, str(tmp_path / "untied"), edit2), "float32", "cpu")
    # an untied configuration wants the tensor
    cfg = OptConfig.from_dict(dict(helpers.TINY["a"]["cfg"], tie_word_embeddings=False))
    d = write_random_model(str(tmp_path / "untied_ok"), cfg, seed=3)
    assert "lm_head.weight" in SafetensorsFile(os.path.join(d, "model.safetensors")).names()
    m = load_model(d, "float32", "cpu")
    assert m.head.weight.data_ptr() != m.embedding.table.data_ptr()


def test_damaged_files(tmp_path):
    src = write_random_model(str(tmp_path / "ok"), helpers.tiny_config("a"), seed=4)
    blob = open(os.path.join(src, "model.safetensors"), "rb").read()
    cases = {"short": blob[:5], "truncated": blob[:len(blob) // 2],
             "bad_header_len": struct.pack("<Q", 1 << 40) + blob[8:],
             "not_json": blob[:8] + b"x" * 20 + blob[28:]}
    for name, data in cases.items():
        d = tmp_path / name
        d.mkdir()
        (d / "config.json").write_text(open(os.path.join(src, "config.json")).read())
        (d / "model.safetensors").write_bytes(data)
        with pytest.raises(SafetensorsError):
            load_model(str(d), "float32", "cpu")
    empty = tmp_path / "empty"
    empty.mkdir()
    (empty / "config.json").write_text(open(os.path.join(src, "config.json")).read())
    with pytest.raises(SafetensorsError, match="no .safetensors"):
        load_model(str(empty), "float32", "cpu")
    with pytest.raises(ValueError, match="dtype"):
        load_model(src, "float16", "cpu")


def test_run_gpt_reads_its_input_and_decodes_with_a_vocabulary(tmp_path):
    """The command line's host-side helpers: one line of ids per request (blank lines skipped), and the id ->
    token table of a vocab.json with the byte-level markers for space and newline turned back."""
    import json
    from swifttransformer_b200.cli.run_gpt import PRECISIONS, VocabDecoder, build_parser, read_input
    inp = tmp_path / "in.txt"
    inp.write_text("5 17 3\n\n  9 \n100 2 2 2\n")
    assert read_input(str(inp)) == [[5, 17, 3], [9], [100, 2, 2, 2]]
    vocab = tmp_path / "vocab.json"
    vocab.write_text(json.dumps({"One": 5, ",": 17, "Ġtwo": 3, "Ċ": 9}))
    dec = VocabDecoder(str(vocab))
    assert "".join(dec.decode(t) for t in [5, 17, 3, 9, 44]) == "One, two\n<44>"
    args = build_parser().parse_args(["dummy", "opt_125m", "fp16", str(inp), "-v", str(vocab), "-d"])
    assert args.vocab_json_path == str(vocab) and args.debug and args.end_token == 50118 and args.max_decoding_step == 128
    assert PRECISIONS["fp16"] == "bfloat16" and PRECISIONS["fp32"] == "float32"
