#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: OPT-1.3B layer sizes with random bfloat16 weights, a batch of 8 requests with 512-token
prompts that then decode; ``value`` is decoded tokens per second over K decode steps timed with CUDA
events on the device; ``e2e`` is the same through ``LLMEngine.step`` (host token ids in, sampled ids
out, wall clock).  Also reported: a 2,048-token prefill, the decode step's HBM roofline fraction, and
decode at batch 1 and 64.  Prints ONE JSON line.  For --gpus > 1 it says that the engine is
single-GPU and exits with 2.

``--only decode|prefill`` run one small measurement (for profiling); ``--only mixed`` runs a continuous
batch of requests of random lengths (prompt portions of 512 tokens beside decoded tokens) through
``LLMEngine.generate`` and reports tokens per second, steps and preemptions.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
        out = dict(FALLBACK_PEAKS)
        for k in out:
            if isinstance(raw.get(k), (int, float)) and raw[k] > 0:
                out[k] = float(raw[k])
        out["source"] = "measured"
        return out
    except Exception:
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6 and parts[0].isdigit():
                self.rows.append(parts)

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": int(statistics.median(int(r[0]) for r in self.rows)),
                "sm_max_mhz": int(self.rows[0][1]), "reasons": reasons, "samples": len(self.rows)}


def prefill_flops(cfg, n_layers, n):
    H, F, V = cfg.hidden_size, cfg.ffn_dim, cfg.vocab_size
    per_layer = 2 * n * H * 3 * H + 2 * n * H * H + 2 * 2 * n * H * F
    attn = 2 * 2 * H * n * (n + 1) // 2            # QK^T and PV over the causal half
    return n_layers * (per_layer + attn) + 2 * H * V   # + the output product for the one wanted row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model-name", default="opt_1.3b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the model has (0: all)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 and prefill measurements")
    ap.add_argument("--no-big", action="store_true", help="skip the OPT-6.7B and OPT-30B points (13 and 60 GB of random weights)")
    ap.add_argument("--launch-floor", action="store_true",
                    help="with --only decode: same number of layers and kernels, but hidden size 64, so that the "
                         "step time is what the chain of dependent launches costs by itself")
    ap.add_argument("--rows", type=int, nargs="*", default=[16, 32, 64], help="with --only products: token counts")
    ap.add_argument("--only", default="", choices=["", "decode", "prefill", "mixed", "products"],
                    help="run just the device-timed decode loop or just the prefill (for profiling small cases), or "
                         "the mixed continuous batch: --requests requests with prompt lengths uniform in [16,1536] "
                         "and output lengths uniform in [16,512], prompt portions of 512 tokens beside decoded "
                         "tokens, through LLMEngine.generate (host token ids in and out, wall clock); or products: "
                         "the model's five matrix products alone at --rows tokens, each 16 times in a recorded graph "
                         "with weights taken in turn from copies larger than L2, by the library, the tcgen05 "
                         "weight-streaming kernel and (up to 32 rows) the mma.sync one")
    ap.add_argument("--requests", type=int, default=64, help="requests of the mixed continuous batch")
    ap.add_argument("--set", action="append", default=[], metavar="MODULE.NAME=VALUE",
                    help="set a tuning constant of the package before the run, e.g. ops.SKINNY_MAX_ROWS=32 or "
                         "parts.attention.KEYS_PER_BLOCK=512 (for A/B measurements; may be repeated)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "LLMServe/SwiftTransformer cannot be built offline: its xformers submodule is empty, "
                          "CMake fetches googletest/json/argparse from the network, and it needs MPI headers"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import dataclasses
    import gc
    import numpy as np
    import torch
    from swifttransformer_b200 import ops
    from swifttransformer_b200.config import opt_preset
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.engine.step import StepEntry
    from swifttransformer_b200.models import random_model
    from swifttransformer_b200.sampling import SamplingParams

    for item in args.set:
        import importlib
        target, value = item.split("=", 1)
        module, name = target.rsplit(".", 1)
        mod = importlib.import_module("swifttransformer_b200." + module)
        if not hasattr(mod, name):
            raise SystemExit(f"bench.py: swifttransformer_b200.{module} has no constant {name}")
        setattr(mod, name, json.loads(value))
    peaks = load_peaks()
    cfg = opt_preset(args.model_name)
    full_layers = cfg.num_hidden_layers
    if args.layers and args.layers < full_layers:
        cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers)
    if args.launch_floor:
        cfg = dataclasses.replace(cfg, hidden_size=64, ffn_dim=256, num_attention_heads=1, word_embed_proj_dim=64,
                                  vocab_size=512)
    torch.cuda.set_device(0)
    model = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    P, K, W = args.prompt_len, args.steps, args.warmup
    ctx_max = cfg.max_position_embeddings
    gen_room = min(ctx_max - P, 2 * (K + W) + 16)
    rng = np.random.default_rng(0)

    def new_engine(batch):
        # an engine that went out of scope lies in a reference cycle with its recorded steps: collect it, and
        # hand its pool back to the device, before the next one asks for its own
        gc.collect()
        torch.cuda.empty_cache()
        pages = batch * ((P + gen_room + 15) // 16 + 1) + (2048 // 16 + 2)
        return LLMEngine(model, page_size=16, num_pages=pages, max_batch_tokens=max(2048, batch * P if batch * P <= 8192 else 4096),
                         chunk_size=2048, max_num_seqs=max(batch, 1))

    def prompts(batch, n):
        return [rng.integers(3, cfg.vocab_size, n).tolist() for _ in range(batch)]

    def decode_device(batch, steps, warmup):
        """Device-timed decode: prompts prefilled through the runner, then `steps` recorded decode steps."""
        eng = new_engine(batch)
        slots = [eng.cache.alloc_slot() for _ in range(batch)]
        lens = [0] * batch
        for i, p in enumerate(prompts(batch, P)):
            eng.runner.step([StepEntry(slots[i], p, 0, [])])
            lens[i] = P
        toks = rng.integers(3, cfg.vocab_size, (warmup + steps, batch)).tolist()

        def one(k):
            entries = [StepEntry(slots[i], [toks[k][i]], lens[i], [0]) for i in range(batch)]
            logits = eng.runner.step(entries)
            ops.argmax(logits)
            for i in range(batch):
                lens[i] += 1
        for k in range(warmup):
            one(k)
        torch.cuda.synchronize()
        launches0 = ops.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(warmup, warmup + steps):
            one(k)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        kernels = eng.runner.kernels_last_step + 1
        mean_ctx = P + warmup + steps / 2
        step_bytes = model.step_param_bytes() + batch * mean_ctx * eng.cache.bytes_per_token()
        eng.runner.check_status()
        return dict(ms=ms, tok_s=batch / ms * 1e3, kernels_per_step=kernels, bytes=step_bytes,
                    graph_steps=eng.runner.graph_steps)

    def decode_e2e(batch, steps, warmup):
        """The same through LLMEngine.step: host ids in, sampled ids out, wall clock."""
        eng = new_engine(batch)
        sp = SamplingParams(max_new_tokens=warmup + steps + 8, ignore_eos=True)
        for p in prompts(batch, P):
            eng.add_request(p, dataclasses.replace(sp))
        while any(r.n_computed < len(r.prompt) for r in eng.requests.values()):
            eng.step()
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        h2d0 = eng.runner.h2d_bytes
        t0 = time.perf_counter()
        for _ in range(steps):
            eng.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        return dict(tok_s=batch * steps / dt, ms=dt / steps * 1e3,
                    h2d=(eng.runner.h2d_bytes - h2d0) / steps, d2h=batch * 4)

    def prefill(n):
        eng = new_engine(1)
        times = []
        for it in range(5):
            slot = eng.cache.alloc_slot()
            p = prompts(1, n)[0]
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            logits = eng.runner.step([StepEntry(slot, p, 0, [n - 1])])
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
            eng.cache.free_slot(slot)
        eng.runner.check_status()        # a kernel that gave up a wait or met a hole in a block table raises here
        ms = min(times[2:])
        fl = prefill_flops(cfg, cfg.num_hidden_layers, n)
        return dict(value=n / ms * 1e3, tokens=n, ms=ms, frac=fl / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12))

    def mixed(n_req):
        """Continuous batching: every request is admitted at once, prompts run in portions of 512 tokens beside
        the decoded tokens of the others.  Run twice with different tokens of the same lengths; the second
        run (whose step shapes are mostly recorded already) is timed."""
        chunk = 512
        lens = [(int(rng.integers(16, 1537)), int(rng.integers(16, 513))) for _ in range(n_req)]
        lens = [(p, min(o, ctx_max - p)) for p, o in lens]
        pages = sum((p + o + 15) // 16 + 1 for p, o in lens)
        eng = LLMEngine(model, page_size=16, num_pages=pages, max_batch_tokens=chunk + n_req, chunk_size=chunk,
                        max_num_seqs=n_req)
        result = {}
        for rep in range(2):
            ps = [rng.integers(3, cfg.vocab_size, p).tolist() for p, _ in lens]
            sp = [SamplingParams(max_new_tokens=o, ignore_eos=True) for _, o in lens]
            steps0, pre0 = eng.stats["steps"], eng.scheduler.num_preemptions
            graphs0, eager0 = eng.runner.graph_steps + eng.runner.padded_graph_steps, eng.runner.steps_run
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            outs = eng.generate(ps, sp)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            n_in, n_out = sum(p for p, _ in lens), sum(len(o) for o in outs)
            steps = eng.stats["steps"] - steps0
            replayed = eng.runner.graph_steps + eng.runner.padded_graph_steps - graphs0
            result = {"only": "mixed", "model": args.model_name, "requests": n_req, "prompt_tokens": n_in,
                      "generated_tokens": n_out, "seconds": round(dt, 4), "total_tok_s": round((n_in + n_out) / dt, 1),
                      "generated_tok_s": round(n_out / dt, 1), "steps": steps, "ms_per_step": round(dt / steps * 1e3, 3),
                      "preemptions": eng.scheduler.num_preemptions - pre0, "replayed_steps": replayed,
                      "eager_steps": eng.runner.steps_run - eager0 - replayed,
                      "recorded_shapes": len(eng.runner._graphs) + len(eng.runner._step_graphs),
                      "first_run_seconds": result.get("seconds")}
        eng.runner.check_status()
        return result

    if args.only == "products":
        H, F, V = cfg.hidden_size, cfg.ffn_dim, cfg.vocab_size

        def graph_us(fn, calls=16, reps=20):
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for i in range(3):
                    fn(i)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for i in range(calls):
                        fn(i)
                for _ in range(3):
                    g.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    g.replay()
                e1.record()
                torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps / calls * 1e3
        for m in args.rows:
            for n, k, name in ((3 * H, H, "qkv"), (H, H, "out"), (F, H, "fc1"), (H, F, "fc2"), (V, H, "head")):
                copies = max(4, int(600e6 / (n * k * 2)))
                ws = [torch.randn(n, k, device="cuda").to(torch.bfloat16) for _ in range(copies)]
                x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
                us = {"library": graph_us(lambda i: torch.mm(x, ws[i % copies].t()))}
                if m <= 128:
                    us["stream_tc"] = graph_us(lambda i: ops.gemm_stream_tc(x, ws[i % copies]))
                if m > ops.SKINNY_MAX_ROWS and ops.linear_parts_slices(m, ws[0]) > 1:
                    us["stream_tc_parts"] = graph_us(lambda i: ops.linear_parts(x, ws[i % copies]))
                if m <= 32:
                    us["skinny"] = graph_us(lambda i: ops.gemm_skinny(x, ws[i % copies]))
                print(json.dumps({"only": "products", "rows": m, "product": name, "n": n, "k": k,
                                  "us": {a: round(b, 1) for a, b in us.items()},
                                  "tb_s": {a: round(n * k * 2 / b / 1e6, 2) for a, b in us.items()}}))
                del ws
        return 0
    if args.only == "decode":
        r = decode_device(args.batch, K, W)
        print(json.dumps({"only": "decode", "ms_per_step": round(r["ms"], 4), "tok_s": round(r["tok_s"], 1)}))
        return 0
    if args.only == "prefill":
        print(json.dumps(dict(prefill(2048), only="prefill")))
        return 0
    if args.only == "mixed":
        print(json.dumps(mixed(args.requests)))
        return 0
    with ClockSampler(0) as clocks:
        dev = decode_device(args.batch, K, W)
    e2e = decode_e2e(args.batch, K, W)
    out = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2048 tokens (OPT-1.3B fp16)",
        "value": round(dev["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(dev["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), token ids uniform in [3,vocab))",
        "impl": "ours",
        "config": {"model": args.model_name, "global_batch": args.batch, "seq_len": ctx_max,
                   "parallelism": "single-gpu", "prompt_len": P, "layers": cfg.num_hidden_layers,
                   "layers_full": full_layers, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "head_dim": cfg.head_dim, "ffn_dim": cfg.ffn_dim, "vocab": cfg.vocab_size, "page_size": 16,
                   "cuda_graphs": dev["graph_steps"] > 0, "l2": "inputs larger than L2 (weights read every step)",
                   "peaks": peaks["source"]},
        "clocks": clocks.summary(),
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "ms_per_step": round(e2e["ms"], 4),
                "h2d_bytes_per_step": int(e2e["h2d"]), "d2h_bytes_per_step": int(e2e["d2h"])},
        "gpu_launches": int(dev["kernels_per_step"] * K),
        "roofline": {"bound": "hbm", "achieved": round(dev["bytes"] / (dev["ms"] * 1e-3) / 1e9, 1),
                     "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(dev["bytes"] / (dev["ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)},
    }
    if not args.no_points:
        pf = prefill(2048)
        out["prefill"] = {"value": round(pf["value"], 1), "tokens": pf["tokens"], "ms": round(pf["ms"], 3),
                          "frac": round(pf["frac"], 4)}
        pts = {}
        for b in (1, 64):
            r = decode_device(b, min(K, 64), W)
            pts[f"decode_b{b}"] = round(r["tok_s"], 1)
            pts[f"decode_b{b}_hbm_frac"] = round(r["bytes"] / (r["ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
        if args.model_name == "opt_1.3b" and not args.layers and not args.launch_floor and not args.no_big:
            # The same two measurements at the OPT-6.7B sizes (head size 128: another set of attention kernels) and at
            # the OPT-30B sizes (60 GB of weights, 56 heads of 128; prompts of 1024 tokens).  A GPU that has no room
            # for them (someone else's memory on it) costs these points, not the line.
            for name, key, prompt, steps in (("opt_6.7b", "opt6.7b", P, 32), ("opt_30b", "opt30b", 1024, 16)):
                model = None
                gc.collect()
                torch.cuda.empty_cache()
                free = torch.cuda.mem_get_info()[0]
                cfg = opt_preset(name)
                need = 2 * 12 * cfg.num_hidden_layers * cfg.hidden_size ** 2 * 1.25
                if free < need:
                    pts[f"{key}_skipped"] = f"{free >> 30} GiB free on the device"
                    continue
                try:
                    model = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
                    P = prompt
                    gen_room = min(ctx_max - P, 2 * (K + W) + 16)
                    r = decode_device(8, min(K, steps), W)
                    pts[f"{key}_decode_b8"] = round(r["tok_s"], 1)
                    pts[f"{key}_decode_b8_hbm_frac"] = round(r["bytes"] / (r["ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
                    pf = prefill(2048)
                    pts[f"{key}_prefill_2048_ms"] = round(pf["ms"], 3)
                    pts[f"{key}_prefill_frac"] = round(pf["frac"], 4)
                except torch.cuda.OutOfMemoryError:
                    pts[f"{key}_skipped"] = "out of device memory"
        out["points"] = pts
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
