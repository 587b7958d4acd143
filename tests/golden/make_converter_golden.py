#!/usr/bin/env python3
"""Runs the reference's own weight converter on a tiny random OPT model and keeps what it wrote.

    python tests/golden/make_converter_golden.py --reference <checkout of LLMServe/SwiftTransformer> [--out FILE]

The reference's model code needs a GPU, MPI and a missing submodule and cannot run here; its offline weight
converter (scripts/lib/converter_lib.py: convertWeight, divideWeightAndSave) is plain PyTorch and can.  It
defines the layout the reference's kernels read: q|k|v fused from the K,V,Q order of the original checkpoint
and stored [in, out] (converter_lib.py:259-262,278-281), out_proj transposed (276-277), the two unused rows cut
off the position table (271), the output projection a copy of the embedding (272), everything cut in eight
along the dimension tensor parallelism uses (164-245).  This script

  1. writes a tiny random model with this package (config.json + model.safetensors, checkpoint names),
  2. restates it in the original checkpoint's form (decoder.* names, one qkv_proj tensor in K,V,Q order),
  3. runs the reference's convertWeight on that, reads its eight-way pieces back and joins them,
  4. stores the converted tensors and a digest of every source tensor in opt_converter_tiny.npz.

tests/test_golden_converter.py compares what this package's loader makes of the same model with the stored
result (and, when a checkout of the reference is given, with a fresh run of the converter).
"""
import argparse
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

# the converter guesses head_dim = 64 from ffn_dim <= 8192 (converter_lib.py:264-268) and cuts by eight
CONFIG = dict(vocab_size=16, hidden_size=64, num_hidden_layers=2, ffn_dim=24, num_attention_heads=1,
              max_position_embeddings=8, do_layer_norm_before=True, word_embed_proj_dim=64, enable_bias=True,
              layer_norm_elementwise_affine=True, activation_function="relu")
SEED, STD = 11, 0.05


def write_tiny_model(model_dir):
    from swifttransformer_b200.config import OptConfig
    from swifttransformer_b200.models import write_random_model
    write_random_model(model_dir, OptConfig.from_dict(dict(CONFIG)), seed=SEED, std=STD)
    import plain_opt
    return plain_opt.read_safetensors(os.path.join(model_dir, "model.safetensors"))


def source_digest(t):
    import hashlib
    return hashlib.sha256(np.ascontiguousarray(np.asarray(t, dtype=np.float32)).tobytes()).hexdigest()[:16]


def original_form(src):
    """Checkpoint names (model.decoder..., q_proj/k_proj/v_proj) -> the original form the converter reads."""
    out = {"decoder.version": np.zeros(1)}
    for name, t in src.items():
        name = name[len("model."):] if name.startswith("model.") else name
        if name == "decoder.final_layer_norm.weight" or name == "decoder.final_layer_norm.bias":
            out[name.replace("final_layer_norm", "layer_norm")] = t
        elif ".self_attn.q_proj." in name or ".self_attn.k_proj." in name or ".self_attn.v_proj." in name:
            continue
        elif name == "lm_head.weight":
            continue
        else:
            out[name] = t
    for i in range(CONFIG["num_hidden_layers"]):
        p = f"decoder.layers.{i}.self_attn."
        for kind in ("weight", "bias"):
            out[p + "qkv_proj." + kind] = np.concatenate(
                [src[f"model.{p}{x}_proj.{kind}"] for x in ("k", "v", "q")], axis=0)
    return out


def run_converter(reference, tensors):
    """convertWeight of the reference on a dict of arrays; returns its output joined again, as float32 arrays."""
    import torch
    sys.path.insert(0, os.path.join(reference, "scripts", "lib"))
    import converter_lib
    nh = CONFIG["num_attention_heads"]
    with tempfile.TemporaryDirectory() as out_dir:
        converter_lib.convertWeight(out_dir, {k: torch.tensor(np.asarray(v, dtype=np.float32)) for k, v in tensors.items()},
                                    torch.float32, "opt")
        files = sorted(os.listdir(out_dir))

        def load(fname, key):
            return getattr(torch.jit.load(os.path.join(out_dir, fname)), key)

        keys = sorted({f.split(".tp_")[0] if ".tp_" in f else f[:-3] for f in files})
        joined = {}
        for key in keys:
            if key + ".pt" in files:
                joined[key] = load(key + ".pt", key)
                continue
            pieces = [load(f"{key}.tp_{r}.pt", key) for r in range(8)]
            if "qkv_proj" in key:
                # piece r holds its share of the q heads, then of the k heads, then of the v heads
                dim = pieces[0].dim() - 2
                shares = [nh // 8] * 8 if nh % 8 == 0 else [nh // 8] * 7 + [nh - (nh // 8) * 7]
                q = [p.narrow(dim, 0, s) for p, s in zip(pieces, shares)]
                k = [p.narrow(dim, s, s) for p, s in zip(pieces, shares)]
                v = [p.narrow(dim, 2 * s, s) for p, s in zip(pieces, shares)]
                t = torch.cat(q + k + v, dim=dim)
                joined[key] = t.reshape(*t.shape[:dim], -1)
            elif key.endswith("fc2.weight"):
                joined[key] = torch.cat(pieces, dim=1)
            else:
                joined[key] = torch.cat(pieces, dim=0)
        return {k: v.detach().to(torch.float32).numpy() for k, v in joined.items()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of LLMServe/SwiftTransformer")
    ap.add_argument("--out", default=os.path.join(HERE, "opt_converter_tiny.npz"))
    args = ap.parse_args()
    with tempfile.TemporaryDirectory() as model_dir:
        src = write_tiny_model(model_dir)
    converted = run_converter(args.reference, original_form(src))
    # the converted tensors, and a digest of each source tensor (the test regenerates the model from the seed)
    arrays = {k: v for k, v in converted.items()}
    digests = {k: source_digest(v) for k, v in src.items()}
    arrays["meta"] = np.frombuffer(json.dumps(dict(config=CONFIG, seed=SEED, std=STD, source=digests)).encode(),
                                   dtype=np.uint8)
    np.savez_compressed(args.out, **arrays)
    print(f"wrote {args.out}: {len(src)} source and {len(converted)} converted tensors, "
          f"{os.path.getsize(args.out)} bytes")


if __name__ == "__main__":
    main()
