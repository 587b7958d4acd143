"""``run_gpt``: load a model, feed it the given input sequences, print the generated tokens.

The command line follows the reference's program of the same name
(src/examples/run_gpt.cc:163-196): positional ``model_path model_name precision
input_path`` and the options ``-v/--vocab_json_path`` and ``-d/--debug``; the input
file holds one line of space-separated token ids per request (run_gpt.cc:72-90);
the output lines ``[ i] (prompt) generated  (n tokens generated)`` and the timing
block are the reference's (run_gpt.cc:122-149).  Its compile-time constants
(END_TOKEN, MAX_DECODING_STEP, block size 16, run_gpt.cc:21-24,93-96) are options here.

``model_path`` is a folder with config.json and safetensors, or ``dummy`` for random
weights of the size named by ``model_name`` (as ``-m dummy`` of the reference's
benchmark program).  ``precision`` is ``bf16`` or ``fp32``; ``fp16``, the reference's
half precision, selects the 16-bit path, which is bfloat16 here.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Optional

PRECISIONS = {"fp32": "float32", "float32": "float32", "bf16": "bfloat16", "bfloat16": "bfloat16",
              "fp16": "bfloat16"}


def read_input(path: str) -> List[List[int]]:
    prompts = []
    with open(path, "r", encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line:
                prompts.append([int(t) for t in line.split()])
    return prompts


class VocabDecoder:
    """id -> token string from a vocab.json (token -> id), as the reference's SimpleVocabDecoder
    (src/examples/lib/simple_vocab_decoder.h:14-41); for looking at output only."""

    def __init__(self, path: str):
        with open(path, "r", encoding="utf-8") as f:
            self.by_id = {int(i): t for t, i in json.load(f).items()}

    def decode(self, token: int) -> str:
        return self.by_id.get(token, f"<{token}>").replace("Ġ", " ").replace("Ċ", "\n")


def build_parser(prog: str = "run_gpt") -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog=prog, description="This program loads a model, feeds it with given input "
                                 "sequences, and prints the generated tokens.")
    ap.add_argument("model_path", help="Path to the model folder (config.json + safetensors), or 'dummy'")
    ap.add_argument("model_name", help="Name of the model (e.g. opt_1.3b); decides the sizes when model_path is 'dummy'")
    ap.add_argument("precision", help="Precision used for inference (bf16 or fp32)")
    ap.add_argument("input_path", help="Path to the input file: one line of token ids per request")
    ap.add_argument("-v", "--vocab_json_path", default="", help="Path to the vocab json file")
    ap.add_argument("-d", "--debug", action="store_true", help="Enable debug mode (prints every step)")
    ap.add_argument("--end_token", type=int, default=50118, help="generation of a request stops at this token id")
    ap.add_argument("--max_decoding_step", type=int, default=128, help="most tokens generated per request")
    ap.add_argument("--block_size", type=int, default=16, help="positions per cache block")
    ap.add_argument("--num_total_blocks", type=int, default=0, help="cache blocks (0: sized from free memory)")
    ap.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    ap.add_argument("--top_k", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--max_batch_tokens", type=int, default=2048, help="token budget of one step")
    ap.add_argument("--chunk_size", type=int, default=2048, help="longest prompt portion in one step")
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.precision.lower() not in PRECISIONS:
        print(f"Invalid precision: {args.precision}\nValid precision: bf16, fp32")
        return 1
    if args.precision.lower() == "fp16":
        print("note: the 16-bit path of this engine is bfloat16", file=sys.stderr)
    dtype = PRECISIONS[args.precision.lower()]
    try:
        prompts = read_input(args.input_path)
    except OSError:
        print(f"Failed to open input file: {args.input_path}")
        return 1

    import torch
    from ..config import opt_preset
    from ..engine.engine import LLMEngine
    from ..models import load_model, random_model
    from ..sampling import SamplingParams

    print("Loading model...")
    if args.model_path == "dummy":
        model = random_model(opt_preset(args.model_name), seed=0, dtype=dtype, device="cuda")
    else:
        model = load_model(args.model_path, dtype, "cuda")
    eng = LLMEngine(model, page_size=args.block_size, num_pages=args.num_total_blocks or None,
                    max_batch_tokens=args.max_batch_tokens, chunk_size=args.chunk_size)
    params = [SamplingParams(temperature=args.temperature, top_k=args.top_k, seed=args.seed + i,
                             max_new_tokens=args.max_decoding_step, eos_id=args.end_token)
              for i in range(len(prompts))]
    ids = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    t_context = None
    step = 0
    while eng.has_work():
        eng.step()
        step += 1
        if args.debug:
            print(f"step {step}: running {len(eng.scheduler.running)} waiting {len(eng.scheduler.waiting)} "
                  f"free pages {eng.cache.free_pages}")
        if t_context is None and all(r.n_computed >= len(r.prompt) or r.state == "finished"
                                     for r in eng.requests.values()):
            torch.cuda.synchronize()
            t_context = time.perf_counter()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    dec = VocabDecoder(args.vocab_json_path) if args.vocab_json_path else None

    def show(tokens):
        return "".join(dec.decode(t) for t in tokens) if dec else "".join(f"{t} " for t in tokens)
    for i, rid in enumerate(ids):
        r = eng.requests[rid]
        print(f"[{i:2d}] ({show(r.prompt)}){show(r.output)}  ({len(r.output)} tokens generated)")
    t_context = t_context or t1
    print("Time usage:")
    print(f"\tContext stage: {(t_context - t0) * 1e3:.2f} ms")
    print(f"\tRegression stage: {(t1 - t_context) * 1e3:.2f} ms")
    print(f"\tTotal: {(t1 - t0) * 1e3:.2f} ms")
    print("Done!")
    return 0


if __name__ == "__main__":
    sys.exit(main())
