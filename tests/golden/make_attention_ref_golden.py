#!/usr/bin/env python3
"""Runs the reference's own attention oracle on the CPU and keeps its inputs and outputs.

    python tests/golden/make_attention_ref_golden.py --reference <checkout of LLMServe/SwiftTransformer> [--out FILE]

The reference tests its attention kernels against a LibTorch restatement,
``st::reference::kernel::attentionKernelRef`` (src/unittest/kernel/attention_ref.cc:13-141): per request, whole
prompts (53-88: q k^T, scale, an additive -10000 above the diagonal, torch::softmax, P v) and single decode
tokens over a paged cache gathered through the block table (89-141).  The file names ``torch::kCUDA`` for the
tensors it makes, nothing else in it needs a GPU.  This script compiles that file **unchanged** into a small
extension: a wrapper translation unit includes the LibTorch headers first, then defines ``kCUDA`` as ``kCPU``
and includes the reference's source, so the same statements run on the host.  It then calls the oracle on a few
small cases (multi-head and grouped heads, prompts of several lengths beside decode tokens, a shuffled block
table, a cache that holds stale values past each request's length) and stores inputs and outputs in
attention_ref_tiny.npz.  tests/test_golden_attention.py holds the plain implementation's attention to them.

The reference's model code itself (src/csrc/model/gpt/gpt.cc) cannot be compiled or run without a GPU, MPI
headers and a submodule that is not in the tree; of its numerical code, this oracle and the weight converter
(make_converter_golden.py) are what runs on a CPU.
"""
import argparse
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

WRAPPER = r"""
#include <torch/extension.h>
#include <torch/torch.h>
// the reference's file, unchanged; the device it names for new tensors becomes the host
#define kCUDA kCPU
#include "unittest/kernel/attention_ref.cc"
#undef kCUDA

torch::Tensor run(torch::Tensor k_cache, torch::Tensor v_cache, torch::Tensor qkvs, double scale,
                  torch::Tensor block_table, torch::Tensor input_len, torch::Tensor is_context) {
    torch::Tensor result;
    st::reference::kernel::attentionKernelRef(result, k_cache, v_cache, qkvs, (float)scale, block_table,
                                              input_len, is_context, true, true);
    return result;
}
PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) { m.def("run", &run); }
"""

# (name, query heads, key/value heads, head size, block size, [(is prompt, input_len)])
# input_len of a prompt: its tokens; of a decode token: the tokens already in the cache (attention_ref.cc:50,96)
CASES = [
    ("mha", 3, 3, 8, 4, [(True, 5), (False, 6), (True, 1), (False, 11), (True, 9), (False, 0)]),
    ("grouped", 4, 2, 16, 8, [(False, 17), (True, 12), (False, 8), (True, 3)]),
    ("one_head", 1, 1, 32, 16, [(True, 33), (False, 32), (False, 15)]),
]
SEED = 5


def make_case(nq, nkv, d, bs, reqs, rng):
    """Random inputs in the oracle's layout: qkvs [tokens, nq + 2 nkv, d]; caches [blocks, 1, nkv, bs, d]
    filled everywhere (so values past a request's length are stale numbers, not zeros); a shuffled block table."""
    n_tokens = sum(n if ctx else 1 for ctx, n in reqs)
    blocks_of = [-(-(n + 1) // bs) for _, n in reqs]
    max_blocks = max(blocks_of)
    num_blocks = sum(blocks_of) + 3
    ids = rng.permutation(num_blocks)[:sum(blocks_of)]
    table = np.full((len(reqs), max_blocks), 0, dtype=np.int64)
    k = 0
    for r, nb in enumerate(blocks_of):
        table[r, :nb] = ids[k:k + nb]
        k += nb
    return dict(
        qkvs=rng.standard_normal((n_tokens, nq + 2 * nkv, d)).astype(np.float32),
        k_cache=rng.standard_normal((num_blocks, 1, nkv, bs, d)).astype(np.float32),
        v_cache=rng.standard_normal((num_blocks, 1, nkv, bs, d)).astype(np.float32),
        block_table=table,
        input_len=np.asarray([n for _, n in reqs], dtype=np.int64),
        is_context=np.asarray([c for c, _ in reqs], dtype=bool))


def build_oracle(reference):
    import torch.utils.cpp_extension as ext
    build = tempfile.mkdtemp(prefix="attention_ref_")
    src = os.path.join(build, "attention_ref_on_host.cc")
    with open(src, "w") as f:
        f.write(WRAPPER)
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")   # util/cuda_utils.h wants cuda_runtime.h
    return ext.load(name="attention_ref_on_host", sources=[src], build_directory=build, verbose=False,
                    extra_include_paths=[os.path.join(reference, "src"), os.path.join(reference, "src", "csrc"),
                                         cuda_inc])


def run_oracle(oracle, case, d):
    import torch
    t = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in case.items()}
    out = oracle.run(t["k_cache"].clone(), t["v_cache"].clone(), t["qkvs"], 1.0 / float(np.sqrt(d)),
                     t["block_table"], t["input_len"], t["is_context"])
    return out.to(torch.float32).numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of LLMServe/SwiftTransformer")
    ap.add_argument("--out", default=os.path.join(HERE, "attention_ref_tiny.npz"))
    args = ap.parse_args()
    oracle = build_oracle(args.reference)
    rng = np.random.default_rng(SEED)
    arrays = {}
    for name, nq, nkv, d, bs, reqs in CASES:
        case = make_case(nq, nkv, d, bs, reqs, rng)
        case["result"] = run_oracle(oracle, case, d)
        for k, v in case.items():
            arrays[f"{name}.{k}"] = v
    arrays["meta"] = np.frombuffer(json.dumps(dict(cases=[[c[0], c[1], c[2], c[3], c[4]] for c in CASES],
                                                   seed=SEED)).encode(), dtype=np.uint8)
    np.savez_compressed(args.out, **arrays)
    print(f"wrote {args.out}: {len(CASES)} cases, {os.path.getsize(args.out)} bytes")


if __name__ == "__main__":
    sys.exit(main())
