"""``benchmark_all_input_same``: time a static batch in which every request has the same prompt.

Command line as the reference's program (src/examples/benchmark_all_input_same.cc:372-386):
positional ``model_name precision exp_params_name`` and ``-m/--model_path`` (default ``dummy``:
random weights), ``-v/--vocab_json_path``.  An experiment is a list of
``(input_len, batch_size, block_size, num_decoding_step)`` (benchmark_all_input_same.cc:29-141);
the named lists live in ``experiments.json`` beside this file, and ``exp_params_name`` may also be
given directly as ``input_len,batch_size,block_size,num_decoding_step[;...]``.  For every line it
runs one warm-up and one timed pass (benchmark_all_input_same.cc:268-296) and prints the
milliseconds of the context stage, the decoding stage and the total.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List, Optional, Tuple

from .run_gpt import PRECISIONS

_EXPERIMENTS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "experiments.json")


def experiments(name: str) -> List[Tuple[int, int, int, int]]:
    with open(_EXPERIMENTS) as f:
        table = json.load(f)
    if name in table:
        return [tuple(x) for x in table[name]]
    try:
        out = [tuple(int(v) for v in part.split(",")) for part in name.split(";") if part]
        if out and all(len(x) == 4 for x in out):
            return out
    except ValueError:
        pass
    raise SystemExit(f"unknown experiment '{name}'; known: {', '.join(sorted(table))} "
                     "(or give input_len,batch_size,block_size,num_decoding_step)")


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="benchmark_all_input_same")
    ap.add_argument("model_name", help="Name of this model")
    ap.add_argument("precision", help="Precision used for inference (bf16 or fp32)")
    ap.add_argument("exp_params_name", help="Name of the experiment parameters")
    ap.add_argument("-m", "--model_path", default="dummy",
                    help="Path to the model folder (type 'dummy' to use dummy weights)")
    ap.add_argument("-v", "--vocab_json_path", default="")
    args = ap.parse_args(argv)
    if args.precision.lower() not in PRECISIONS:
        print(f"Invalid precision: {args.precision}\nValid precision: bf16, fp32")
        return 1
    dtype = PRECISIONS[args.precision.lower()]

    import numpy as np
    import torch
    from ..config import opt_preset
    from ..engine.engine import LLMEngine
    from ..models import load_model, random_model
    from ..sampling import SamplingParams

    if args.model_path == "dummy":
        model = random_model(opt_preset(args.model_name), seed=0, dtype=dtype, device="cuda")
    else:
        model = load_model(args.model_path, dtype, "cuda")
    rng = np.random.default_rng(0)
    rows = []
    for input_len, batch, block_size, n_steps in experiments(args.exp_params_name):
        prompt = rng.integers(3, model.vocab_size, input_len).tolist()
        pages = batch * ((input_len + n_steps) // block_size + 2)
        # steps are not launched ahead here: the two stages are timed separately, and a decode step that
        # is already on the GPU when the context stage is read off would count towards the wrong one
        eng = LLMEngine(model, page_size=block_size, num_pages=pages, max_batch_tokens=max(2048, input_len),
                        chunk_size=max(2048, input_len), max_num_seqs=batch, pipeline=False)
        sp = SamplingParams(max_new_tokens=n_steps, ignore_eos=True)
        for timed in (False, True):
            for _ in range(batch):
                eng.add_request(prompt, SamplingParams(**vars(sp)))
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            t_ctx = None
            while eng.has_work():
                eng.step()
                if t_ctx is None and all(r.n_computed >= len(r.prompt) for r in eng.scheduler.running):
                    torch.cuda.synchronize()
                    t_ctx = time.perf_counter()
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            eng.requests.clear()
        rows.append((input_len, batch, block_size, n_steps, (t_ctx - t0) * 1e3, (t1 - t_ctx) * 1e3, (t1 - t0) * 1e3))
    print(f"{'input_len':>9} {'batch':>6} {'block':>6} {'steps':>6} {'context_ms':>11} {'decoding_ms':>12} {'total_ms':>10}")
    for r in rows:
        print(f"{r[0]:>9} {r[1]:>6} {r[2]:>6} {r[3]:>6} {r[4]:>11.2f} {r[5]:>12.2f} {r[6]:>10.2f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
