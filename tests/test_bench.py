"""bench.py: what it answers without a GPU, and its small modes on one."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")


def run(*args, timeout=600):
    return subprocess.run([sys.executable, BENCH, *args], capture_output=True, text=True, timeout=timeout)


def test_more_than_one_gpu_is_refused_in_one_line():
    r = run("--gpus", "2")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_reference_arm_says_why_it_is_unavailable():
    r = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip())
    assert line["impl"] == "reference" and line["unavailable"]


@pytest.mark.gpu
def test_mixed_continuous_batch_mode():
    r = run("--only", "mixed", "--layers", "1", "--requests", "5")
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["only"] == "mixed" and line["requests"] == 5
    assert line["generated_tokens"] > 0 and line["total_tok_s"] > 0 and line["preemptions"] == 0
    assert line["replayed_steps"] + line["eager_steps"] == line["steps"]


@pytest.mark.gpu
def test_small_decode_and_prefill_modes():
    r = run("--only", "decode", "--layers", "1", "--steps", "4", "--warmup", "3", "--batch", "2")
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1])["tok_s"] > 0
    r = run("--only", "prefill", "--layers", "1")
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    # the fraction is the step's flops / its time / the tensor peak: recompute it from the sizes of one layer of
    # OPT-1.3B (4 products, the causal half of the attention, one row of the output product) and the time printed
    T, H, F, V = 2048, 2048, 8192, 50272
    flops = 2 * T * H * 3 * H + 2 * T * H * H + 4 * T * H * F + 4 * H * T * (T + 1) // 2 + 2 * H * V
    peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"] \
        if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 1590.0
    assert line["tokens"] == T and 0.05 < line["frac"] < 1.0
    assert abs(line["frac"] - flops / (line["ms"] * 1e-3) / (peak * 1e12)) < 0.02 * line["frac"]
