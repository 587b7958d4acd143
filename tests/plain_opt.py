"""A plain, slow OPT: whole sequences, no cache, one function per part.

This file is the tests' oracle.  It shares no code with the package: it has
its own safetensors reader, its own config handling and computes with numpy
(float64 by default).  It rests on the reference's formulas (the reference's
model code needs a GPU, MPI and a missing submodule, so it cannot be run or
compiled on a CPU); each function cites the lines it restates.  What of the
reference does run on a CPU is (1) its offline weight converter: its output for a
tiny random model is kept under tests/golden/, and tests/test_golden_converter.py
checks that this file's logits equal those of the reference's order of
operations on the converter's tensors (fused q|k|v, transposes, cut positions);
and (2) the LibTorch attention oracle its kernel tests use
(src/unittest/kernel/attention_ref.cc), compiled unchanged for the host: its
inputs and outputs are kept under tests/golden/ too, and
tests/test_golden_attention.py holds ``causal_attention`` to them.  Where the
reference has no code for an option (post-LN, project_in/out, no bias, no
affine), the definition used is stated in the function.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np

_NP = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def read_safetensors(path):
    """name -> float64 / int array."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        b, e = rec["data_offsets"]
        raw = data[b:e]
        if rec["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            arr = u.view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(raw, dtype=_NP[rec["dtype"]])
            if arr.dtype.kind == "f":
                arr = arr.astype(np.float64)
        out[name] = arr.reshape(rec["shape"])
    return out


def load_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    for fn in sorted(os.listdir(model_dir)):
        if fn.endswith(".safetensors"):
            w.update(read_safetensors(os.path.join(model_dir, fn)))
    return cfg, w


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def embed_tokens(ids, table):
    """x[t] = embed_tokens[id[t]]  (src/csrc/kernel/embedding.cu:25-33)."""
    return table[np.asarray(ids)]


def learned_positions(positions, table, offset):
    """embed_positions[pos + offset]: the reference cuts the first `offset`=2
    rows off the table offline (scripts/lib/converter_lib.py:271) and indexes
    with the 0-based position (src/csrc/model/gpt/gpt.cc:87-104); reading the
    uncut table at pos+offset is the same thing."""
    return table[np.asarray(positions) + offset]


def layer_norm(x, gamma, beta, eps):
    """y = (x - mean) * rsqrt(var + eps) * gamma + beta over the last axis
    (src/csrc/kernel/layernorm.cu:34-51,78-96; the reference uses the
    one-pass E[x^2]-mean^2, here the two-pass variance of the same quantity).
    gamma/beta None = layer_norm_elementwise_affine false (gamma 1, beta 0)."""
    mean = x.mean(-1, keepdims=True)
    var = ((x - mean) ** 2).mean(-1, keepdims=True)
    y = (x - mean) / np.sqrt(var + eps)
    if gamma is not None:
        y = y * gamma
    if beta is not None:
        y = y + beta
    return y


def linear(x, w, b=None):
    """y = x . w^T + b with w stored [out, in]  (fc1/fc2: src/csrc/layer/ffn.cc:71-124;
    the reference keeps qkv/out_proj pre-transposed, src/csrc/layer/attention.cc:102-130,255-288,
    which is the same product)."""
    y = x @ w.T
    if b is not None:
        y = y + b
    return y


def activation(x, name):
    """ReLU = x>0 ? x : 0 (src/csrc/kernel/activations.cuh:12-14); gelu is the
    erf form (activations.cuh:18-25 is the reference's GELU for GPT-2)."""
    if name == "relu":
        return np.maximum(x, 0)
    if name == "gelu":
        from math import erf
        return 0.5 * x * (1.0 + np.vectorize(erf)(x / np.sqrt(2.0)))
    raise ValueError(name)


def causal_attention(q, k, v, num_heads, window=None):
    """Per head: S = q k^T / sqrt(d); keys j > i are masked; P = softmax(S); o = P v
    (src/csrc/layer/attention.cc:91 scale; src/csrc/kernel/fused_context_stage_attention.cu:226-265,
    313-334,345-404; decode form src/csrc/kernel/fused_decoding_stage_attention_mha.cu:159-252).
    Masked keys are left out of the softmax (the reference adds -10000 and 1e-6 to the
    denominator, quirks of its kernels that change nothing at working precision).
    q,k,v: [T, heads*d].  window W (not an OPT option) keeps keys i-W < j <= i."""
    T, H = q.shape
    d = H // num_heads
    out = np.zeros_like(q)
    scale = 1.0 / np.sqrt(d)
    for h in range(num_heads):
        qs, ks, vs = (a[:, h * d:(h + 1) * d] for a in (q, k, v))
        s = (qs @ ks.T) * scale
        i = np.arange(T)[:, None]
        j = np.arange(T)[None, :]
        mask = j > i
        if window is not None:
            mask |= j <= i - window
        s = np.where(mask, -np.inf, s)
        s = s - s.max(-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(-1, keepdims=True)
        out[:, h * d:(h + 1) * d] = p @ vs
    return out


def attention_block(x, w, prefix, cfg):
    """q,k,v projections with bias, causal attention, output projection with bias
    (src/csrc/layer/attention.cc:102-130 qkv+bias, 179-246 attention, 255-288 out+bias)."""
    def b(name):
        return w.get(prefix + name + ".bias") if cfg.get("enable_bias", True) else None
    q = linear(x, w[prefix + "q_proj.weight"], b("q_proj"))
    k = linear(x, w[prefix + "k_proj.weight"], b("k_proj"))
    v = linear(x, w[prefix + "v_proj.weight"], b("v_proj"))
    o = causal_attention(q, k, v, cfg["num_attention_heads"])
    return linear(o, w[prefix + "out_proj.weight"], b("out_proj"))


def feed_forward(x, w, prefix, cfg):
    """z = act(x fc1^T + b1) fc2^T + b2  (src/csrc/layer/ffn.cc:71-124)."""
    bias = cfg.get("enable_bias", True)
    u = linear(x, w[prefix + "fc1.weight"], w.get(prefix + "fc1.bias") if bias else None)
    u = activation(u, cfg.get("activation_function", "relu"))
    return linear(u, w[prefix + "fc2.weight"], w.get(prefix + "fc2.bias") if bias else None)


def decoder_layer(x, w, i, cfg):
    """Pre-LN (do_layer_norm_before): r = x + attn(LN1(x)); x' = r + ffn(LN2(r))
    (src/csrc/model/gpt/gpt.cc:304-503: LN 325-335, attention, residual+LN 423-436, ffn, add 496-501).
    Post-LN (the reference throws, gpt.cc:238-240; defined here as the same sublayers with
    the norm after the residual sum): r = LN1(x + attn(x)); x' = LN2(r + ffn(r))."""
    p = f"model.decoder.layers.{i}."
    eps = cfg.get("layer_norm_eps", 1e-5)
    affine = cfg.get("layer_norm_elementwise_affine", True)

    def ln(name, t):
        return layer_norm(t, w[p + name + ".weight"] if affine else None,
                          w[p + name + ".bias"] if affine else None, eps)
    if cfg.get("do_layer_norm_before", True):
        r = x + attention_block(ln("self_attn_layer_norm", x), w, p + "self_attn.", cfg)
        return r + feed_forward(ln("final_layer_norm", r), w, p, cfg)
    r = ln("self_attn_layer_norm", x + attention_block(x, w, p + "self_attn.", cfg))
    return ln("final_layer_norm", r + feed_forward(r, w, p, cfg))


def forward(cfg, w, ids, dtype=np.float64, rows=None):
    """Logits [T, vocab] for one whole sequence `ids` (with `rows`: only at those positions, [len(rows), vocab];
    the sequence is computed whole all the same).

    x = embed_tokens[id] (project_in when word_embed_proj_dim != hidden) + positions;
    layers; final LayerNorm only for pre-LN models; project_out; logits = h . embed_tokens^T
    (tied; src/csrc/model/gpt/gpt.cc:112-145 embedding, 614-624 final LN, 175-201 LM head)."""
    w = {k: (v.astype(dtype, copy=False) if v.dtype.kind == "f" else v) for k, v in w.items()}
    ids = np.asarray(ids)
    H = cfg["hidden_size"]
    E = cfg.get("word_embed_proj_dim", H) or H
    x = embed_tokens(ids, w["model.decoder.embed_tokens.weight"])
    if E != H:
        x = linear(x, w["model.decoder.project_in.weight"])
    x = x + learned_positions(np.arange(len(ids)), w["model.decoder.embed_positions.weight"],
                              cfg.get("position_offset", 2))
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, cfg)
    if cfg.get("do_layer_norm_before", True) and not cfg.get("_remove_final_layer_norm", False):
        affine = cfg.get("layer_norm_elementwise_affine", True)
        x = layer_norm(x, w["model.decoder.final_layer_norm.weight"] if affine else None,
                       w["model.decoder.final_layer_norm.bias"] if affine else None,
                       cfg.get("layer_norm_eps", 1e-5))
    if rows is not None:
        x = x[np.asarray(rows)]
    if E != H:
        x = linear(x, w["model.decoder.project_out.weight"])
    head = w["model.decoder.embed_tokens.weight"] if cfg.get("tie_word_embeddings", True) else w["lm_head.weight"]
    return linear(x, head)


def greedy_generate(cfg, w, prompt, n_new):
    """Append argmax tokens one by one, recomputing the whole sequence each time
    (greedy: src/csrc/model/gpt/gpt.cc:205-210; ties -> lowest id)."""
    ids = list(prompt)
    for _ in range(n_new):
        logits = forward(cfg, w, ids)
        ids.append(int(np.argmax(logits[-1])))
    return ids[len(prompt):]


def softmax_sample(logits, temperature, u, top_k=0):
    """Inverse-CDF draw from softmax(logits / temperature) (restricted to the top_k
    largest when top_k > 0) with a given uniform number u in [0,1)."""
    z = np.asarray(logits, dtype=np.float64) / temperature
    if top_k and top_k < len(z):
        kth = np.sort(z)[-top_k]
        z = np.where(z >= kth, z, -np.inf)
    p = np.exp(z - z.max())
    c = np.cumsum(p)
    return int(min(np.searchsorted(c, u * c[-1], side="right"), len(z) - 1))
