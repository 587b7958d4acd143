"""Each CUDA kernel alone against its plain reference (tests/cpu_ops.py), at sizes other than the engine's."""
import math

import numpy as np
import pytest
import torch

import cpu_ops
from swifttransformer_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def close(got, ref, dtype, what, rel=None):
    got, ref = got.double().cpu(), ref.double().cpu()
    rel = rel if rel is not None else (2e-6 if dtype == torch.float32 else 1e-2)
    tol = rel * max(ref.abs().max().item(), 1e-6)
    err = (got - ref).abs().max().item()
    assert err <= tol, f"{what}: max error {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [24, 1000, 2048])
def test_embed(dtype, width):
    vocab, n, off = 301, 37, 2
    table, ptab = rnd((vocab, width), dtype, 1), rnd((50 + off, width), dtype, 2)
    ids = torch.randint(0, vocab, (n,), dtype=torch.int32)
    pos = torch.randint(0, 50, (n,), dtype=torch.int32)
    for out_dtype in {torch.float32, dtype}:
        ref = cpu_ops.embed(ids, table, torch.empty(n, width, dtype=out_dtype), pos, ptab, off)
        got = ops.embed(ids.to(DEV), table.to(DEV), torch.empty(n, width, dtype=out_dtype, device=DEV),
                        pos.to(DEV), ptab.to(DEV), off)
        close(got, ref, out_dtype, "embed+pos", rel=1e-6 if out_dtype == torch.float32 else 4e-3)
        ref = cpu_ops.embed(ids, table, torch.empty(n, width, dtype=out_dtype))
        got = ops.embed(ids.to(DEV), table.to(DEV), torch.empty(n, width, dtype=out_dtype, device=DEV))
        assert torch.equal(got.cpu(), ref)
    x = rnd((n, width), dtype, 3)
    ref = cpu_ops.add_positions(x, pos, ptab, off, torch.empty(n, width))
    got = ops.add_positions(x.to(DEV), pos.to(DEV), ptab.to(DEV), off, torch.empty(n, width, device=DEV))
    close(got, ref, torch.float32, "add_positions", rel=1e-6)
    # padding tokens of a fixed-shape step stand at position -1: with an offset of zero their row would lie
    # before the table, so they get none (the table here is the tail of a larger tensor whose head is huge:
    # a kernel that read the row before it would show 1e30 in its output)
    big = torch.cat([torch.full((4, width), 1e30).to(dtype), rnd((50, width), dtype, 4)]).to(DEV)
    pad_pos = pos.clone(); pad_pos[::3] = -1
    got = ops.embed(ids.to(DEV), table.to(DEV), torch.empty(n, width, dtype=torch.float32, device=DEV),
                    pad_pos.to(DEV), big[4:], 0)
    ref = cpu_ops.embed(ids, table, torch.empty(n, width), pad_pos.clamp(min=0), big[4:].cpu(), 0)
    keep = pad_pos >= 0
    close(got[keep], ref[keep], torch.float32, "embed beside padding", rel=1e-6)
    assert torch.equal(got[~keep].cpu(), table[ids[~keep].long()].float()), "a padding token gets no position row"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm", "none"])
@pytest.mark.parametrize("width", [40, 777, 7168])
def test_add_norm(dtype, kind, width):
    n = 19
    # a row offset far from zero shows a one-pass variance; the two-pass one must not care
    x = rnd((n, width), torch.float32, 4) + 30.0
    delta, dbias = rnd((n, width), dtype, 5), rnd((width,), torch.float32, 6)
    gamma, beta = 1 + rnd((width,), torch.float32, 7, 0.1), rnd((width,), torch.float32, 8, 0.1)
    eps = 3e-4
    # pre-norm use: residual updated, normalised copy out
    xr = x.clone()
    ref_out = torch.empty(n, width, dtype=dtype)
    cpu_ops.add_norm(xr, delta=delta, delta_bias=dbias, resid_out=xr, gamma=gamma, beta=beta, eps=eps, kind=kind,
                     out_act=ref_out)
    xg = x.to(DEV)
    got_out = torch.empty(n, width, dtype=dtype, device=DEV)
    ops.add_norm(xg, delta=delta.to(DEV), delta_bias=dbias.to(DEV), resid_out=xg, gamma=gamma.to(DEV),
                 beta=beta.to(DEV), eps=eps, kind=kind, out_act=got_out)
    close(xg, xr, torch.float32, "residual", rel=1e-6)
    close(got_out, ref_out, dtype, f"{kind} out", rel=5e-5 if dtype == torch.float32 else 8e-3)
    # post-norm use: residual replaced by the normalised row; and a gather of rows without affine
    xr = x.clone()
    cpu_ops.add_norm(xr, delta=delta, eps=eps, kind=kind, out_act=ref_out, out_f32=xr)
    xg = x.to(DEV)
    ops.add_norm(xg, delta=delta.to(DEV), eps=eps, kind=kind, out_act=got_out, out_f32=xg)
    close(xg, xr, torch.float32, "normalised residual", rel=5e-5)
    rows = torch.tensor([3, 0, 18, 3], dtype=torch.int32)
    ref_g = torch.empty(4, width, dtype=dtype)
    cpu_ops.add_norm(x, delta=delta, delta_bias=dbias, gamma=gamma, beta=beta, eps=eps, kind=kind, rows=rows,
                     out_act=ref_g)
    got_g = torch.empty(4, width, dtype=dtype, device=DEV)
    xg = x.to(DEV)
    ops.add_norm(xg, delta=delta.to(DEV), delta_bias=dbias.to(DEV), gamma=gamma.to(DEV), beta=beta.to(DEV),
                 eps=eps, kind=kind, rows=rows.to(DEV), out_act=got_g)
    close(got_g, ref_g, dtype, "gathered rows", rel=5e-5 if dtype == torch.float32 else 8e-3)
    assert torch.equal(xg.cpu(), x), "a gathered norm must not touch the residual stream"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["none", "relu", "gelu"])
def test_bias_act(dtype, act):
    y, b = rnd((33, 530), dtype, 9), rnd((530,), torch.float32, 10)
    ref = cpu_ops.bias_act(y.clone(), b, act)
    got = ops.bias_act(y.to(DEV), b.to(DEV), act)
    close(got, ref, dtype, "bias_act", rel=1e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 50, 24), (5, 130, 77), (70, 333, 520), (129, 64, 2048)])
def test_gemm_plain(dtype, shape):
    n, m, k = shape
    a, w, b = rnd((n, k), dtype, 11), rnd((m, k), dtype, 12, 0.1), rnd((m,), torch.float32, 13)
    for act in ("none", "relu"):
        ref = cpu_ops.linear(a, w, b, act, torch.float32)
        got = ops.gemm_plain(a.to(DEV), w.to(DEV), b.to(DEV), act, torch.float32)
        close(got, ref, torch.float32, "gemm_plain", rel=3e-6)
    got = ops.linear(a.to(DEV), w.to(DEV), b.to(DEV), "relu")
    ref = cpu_ops.linear(a, w, b, "relu")
    close(got, ref, dtype, "linear", rel=3e-6 if dtype == torch.float32 else 1e-2)
    # float32 logits out of bfloat16 operands (the output head)
    got = ops.linear(a.to(DEV), w.to(DEV), out_dtype=torch.float32)
    close(got, cpu_ops.linear(a, w, out_dtype=torch.float32), torch.float32, "linear f32 out",
          rel=3e-6 if dtype == torch.float32 else 1e-5)


def test_gemm_plain_rows_do_not_depend_on_the_batch():
    a, w = rnd((70, 200), torch.float32, 14).to(DEV), rnd((90, 200), torch.float32, 15).to(DEV)
    full = ops.gemm_plain(a, w)
    one = ops.gemm_plain(a[37:38].contiguous(), w)
    assert torch.equal(full[37:38], one)


def make_cache(dtype, n_seqs, lens, nkv, d, page_size, n_layers, seed, shuffle=True):
    """A pool with random contents (stale values everywhere), random page assignment, and the true K/V."""
    g = torch.Generator().manual_seed(seed)
    max_pages = max((l + page_size - 1) // page_size for l in lens) + 1
    num_pages = sum((l + page_size - 1) // page_size for l in lens) + 3
    pool = (torch.randn((num_pages, n_layers, 2, nkv, page_size, d), generator=g) * 3).to(dtype)
    perm = torch.randperm(num_pages, generator=g).tolist() if shuffle else list(range(num_pages))
    bt = torch.full((n_seqs + 2, max_pages), -1, dtype=torch.int32)
    slots = torch.randperm(n_seqs + 2, generator=g)[:n_seqs].to(torch.int32)
    for i, l in enumerate(lens):
        for j in range((l + page_size - 1) // page_size):
            bt[int(slots[i]), j] = perm.pop()
    return pool, bt, slots


@pytest.mark.parametrize("dtype", DTYPES)
def test_qkv_to_cache(dtype):
    nh, nkv, d, ps, L = 6, 2, 24, 8, 3
    lens, new = [13, 40, 1], [5, 40, 1]
    pool, bt, slots = make_cache(dtype, 3, lens, nkv, d, ps, L, 20)
    pos, seq = [], []
    for i, (l, n) in enumerate(zip(lens, new)):
        pos += list(range(l - n, l)); seq += [i] * n
    n = len(pos)
    pos, seq = torch.tensor(pos, dtype=torch.int32), torch.tensor(seq, dtype=torch.int32)
    qkv, bias = rnd((n, (nh + 2 * nkv) * d), dtype, 21), rnd(((nh + 2 * nkv) * d,), torch.float32, 22)
    ref_pool, ref_q, st = pool.clone(), torch.empty(n, nh * d, dtype=dtype), torch.zeros(1, dtype=torch.int32)
    cpu_ops.qkv_to_cache(qkv, bias, ref_q, ref_pool, 1, pos, seq, slots, bt, nh, nkv, d, st)
    gp, gq, gst = pool.to(DEV), torch.empty(n, nh * d, dtype=dtype, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.qkv_to_cache(qkv.to(DEV), bias.to(DEV), gq, gp, 1, pos.to(DEV), seq.to(DEV), slots.to(DEV), bt.to(DEV),
                     nh, nkv, d, gst)
    assert int(gst.item()) == 0
    close(gq, ref_q, dtype, "q", rel=1e-6 if dtype == torch.float32 else 8e-3)
    close(gp, ref_pool, dtype, "pool", rel=1e-6 if dtype == torch.float32 else 8e-3)
    assert torch.equal(gp[:, 0].cpu(), pool[:, 0]) and torch.equal(gp[:, 2].cpu(), pool[:, 2]), "other layers untouched"
    # the queries may stay where they are: only keys and values move, without a bias, bit for bit
    for head_dim in (24, 3):                                   # 16-byte pieces, and single elements
        nh2, nkv2 = (nh, nkv) if head_dim == 24 else (5, 3)
        pool2, bt_2, slots2 = make_cache(dtype, 3, lens, nkv2, head_dim, ps, L, 23)
        wide = rnd((n, (nh2 + 2 * nkv2) * head_dim), dtype, 24)
        want = pool2.clone()
        cpu_ops.qkv_to_cache(wide, None, None, want, 1, pos, seq, slots2, bt_2, nh2, nkv2, head_dim, st)
        got = pool2.to(DEV)
        ops.qkv_to_cache(wide.to(DEV), None, None, got, 1, pos.to(DEV), seq.to(DEV), slots2.to(DEV), bt_2.to(DEV),
                         nh2, nkv2, head_dim, gst)
        assert torch.equal(got.cpu(), want) and not torch.equal(want, pool2)
    # a hole in the block table is reported, not written through
    bt2 = bt.clone(); bt2[int(slots[1]), 2] = -1
    ops.qkv_to_cache(qkv.to(DEV), bias.to(DEV), gq, gp, 1, pos.to(DEV), seq.to(DEV), slots.to(DEV), bt2.to(DEV),
                     nh, nkv, d, gst)
    assert int(gst.item()) == 1


def attention_case(dtype, nh, nkv, d, ps, lens, new, seed, window=0):
    L = 2
    pool, bt, slots = make_cache(dtype, len(lens), lens, nkv, d, ps, L, seed)
    pos, seq, q_start = [], [], [0]
    for i, (l, n) in enumerate(zip(lens, new)):
        pos += list(range(l - n, l)); seq += [i] * n; q_start.append(q_start[-1] + n)
    n = len(pos)
    t = dict(pos=torch.tensor(pos, dtype=torch.int32), seq=torch.tensor(seq, dtype=torch.int32),
             q_start=torch.tensor(q_start, dtype=torch.int32),
             start=torch.tensor([l - m for l, m in zip(lens, new)], dtype=torch.int32))
    q = rnd((n, nh * d), dtype, seed + 1)
    scale = 1 / math.sqrt(d)
    ref = torch.zeros(n, nh * d, dtype=dtype)
    cpu_ops.attention_plain(q, pool, 1, ref, t["pos"], t["seq"], slots, bt, nh, scale, window)
    return pool, bt, slots, t, q, scale, ref


ATT_SHAPES = [  # nh, nkv, d, page_size
    (4, 4, 16, 8), (3, 3, 32, 16), (5, 5, 48, 32), (6, 2, 64, 16), (2, 1, 80, 4), (4, 4, 128, 16), (2, 2, 256, 64),
    (3, 1, 64, 8), (2, 2, 128, 64), (5, 5, 64, 32), (40, 2, 32, 16),     # the last: 20 query heads per kv head
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ATT_SHAPES)
@pytest.mark.parametrize("window", [0, 37])
def test_attention_plain(dtype, shape, window):
    nh, nkv, d, ps = shape
    lens, new = [150, 9, 300, 1], [150, 2, 1, 1]
    pool, bt, slots, t, q, scale, ref = attention_case(dtype, nh, nkv, d, ps, lens, new, 30, window)
    out = torch.zeros_like(ref, device=DEV)
    ops.attention_plain(q.to(DEV), pool.to(DEV), 1, out, t["pos"].to(DEV), t["seq"].to(DEV), slots.to(DEV),
                        bt.to(DEV), nh, scale, window)
    close(out, ref, dtype, "attention_plain", rel=3e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("shape", ATT_SHAPES)
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("n_splits", [1, 3, 8])
@pytest.mark.parametrize("kernel", ["mma", "mma8", "lanes"])
def test_attention_decode(shape, window, n_splits, kernel):
    nh, nkv, d, ps = shape
    if kernel.startswith("mma") and (d % 16 or d > 128):
        pytest.skip("the tensor-core kernel takes head sizes that are multiples of 16 up to 128")
    warps = 8 if kernel == "mma8" else 4
    kernel = kernel[:3] if kernel.startswith("mma") else kernel
    dtype = torch.bfloat16
    lens, new = [150, 9, 700, 1, 64], [1, 2, 1, 1, 3]
    pool, bt, slots, t, q, scale, ref = attention_case(dtype, nh, nkv, d, ps, lens, new, 40, window)
    n = q.shape[0]
    items = torch.tensor([i for i in range(n) if i != 2], dtype=torch.int32)   # token 2 is left to "another kernel"
    out = torch.full_like(ref, 7.0, device=DEV)
    partial = torch.empty(ops.attention_decode_scratch(len(items), nh, d, n_splits) + 1, device=DEV)
    ops.attention_decode(q.to(DEV), pool.to(DEV), 1, out, items.to(DEV), len(items), t["pos"].to(DEV),
                         t["seq"].to(DEV), slots.to(DEV), bt.to(DEV), nh, scale, window, n_splits, partial,
                         kernel=kernel, warps=warps)
    close(out[items.long()], ref[items.long()], dtype, "attention_decode", rel=1e-2)
    assert torch.all(out[2] == 7.0), "a token that is not in the item list must not be written"
    # told which keys earlier steps wrote, the kernel starts copying those before its wait: same result
    early = torch.full_like(ref, 7.0, device=DEV)
    ops.attention_decode(q.to(DEV), pool.to(DEV), 1, early, items.to(DEV), len(items), t["pos"].to(DEV),
                         t["seq"].to(DEV), slots.to(DEV), bt.to(DEV), nh, scale, window, n_splits, partial,
                         kernel=kernel, warps=warps, start_pos=t["start"].to(DEV))
    assert torch.equal(early, out)


@pytest.mark.parametrize("shape", [sh for sh in ATT_SHAPES if sh[2] % 16 == 0 and sh[2] <= 128])
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("n_splits,warps", [(1, 4), (3, 4), (1, 8), (8, 8)])
def test_attention_decode_from_the_fused_projection(shape, window, n_splits, warps):
    """The single-token kernel given the q|k|v product instead of queries: it takes this step's keys and values from
    the product's rows (the pages hold stale values at their places until it writes them: a read from the cache
    there would show), writes each token's rows into its page exactly as the cache-write kernel would, and skips a
    padding token.  Requests bring one to three tokens; one starts at position 0."""
    nh, nkv, d, ps = shape
    dtype = torch.bfloat16
    lens, new = [150, 9, 700, 1, 64, 33], [1, 2, 1, 1, 3, 1]
    pool, bt, slots, t, _, scale, _ = attention_case(dtype, nh, nkv, d, ps, lens, new, 60, window)
    pos = torch.cat([t["pos"], torch.tensor([-1], dtype=torch.int32)])          # the last token is padding
    seq = torch.cat([t["seq"], torch.tensor([0], dtype=torch.int32)])
    n = pos.shape[0]
    width = (nh + 2 * nkv) * d
    qkv = rnd((n, width), dtype, 61)
    bias = None
    ref_pool, ref_q, st = pool.clone(), torch.zeros(n, nh * d, dtype=dtype), torch.zeros(1, dtype=torch.int32)
    cpu_ops.qkv_to_cache(qkv, bias, ref_q, ref_pool, 1, pos, seq, slots, bt, nh, nkv, d, st)
    ref = torch.zeros(n, nh * d, dtype=dtype)
    cpu_ops.attention_plain(ref_q, ref_pool, 1, ref, pos, seq, slots, bt, nh, scale, window)
    for write_kv in (True, False):
        gp, out = pool.to(DEV), torch.full((n, nh * d), 7.0, dtype=dtype, device=DEV)
        gst = torch.zeros(1, dtype=torch.int32, device=DEV)
        partial = torch.empty(ops.attention_decode_scratch(n, nh, d, n_splits) + 1, device=DEV)
        ops.attention_decode_qkv(qkv.to(DEV), gp, 1, out, None, n, pos.to(DEV),
                                 seq.to(DEV), slots.to(DEV), t["start"].to(DEV), bt.to(DEV), nh, scale, window, n_splits,
                                 partial, warps=warps, write_kv=write_kv, status=gst)
        assert int(gst.item()) == 0
        close(out[:n - 1], ref[:n - 1], dtype, "attention_decode_qkv", rel=1e-2)
        assert torch.all(out[n - 1] == 7.0), "a padding token must not be written"
        assert torch.equal(gp.cpu(), ref_pool if write_kv else pool), "the pages after the step"


@pytest.mark.parametrize("shape", ATT_SHAPES)
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("kernel", ["tmap", "tma", "tma3", "tc", "mma"])
def test_attention_prefill(shape, window, kernel):
    nh, nkv, d, ps = shape
    if kernel == "tc" and d > 128:
        pytest.skip("the tcgen05 kernel takes head sizes up to 128")
    if kernel == "tmap" and not (d == 64 and ps in (8, 16, 32, 64)):
        pytest.skip("the persistent TMA-fed kernel takes head size 64 and pages of 8 to 64 positions")
    if kernel in ("tma", "tma3") and not (d in (64, 128) and ps in (8, 16, 32, 64)):
        pytest.skip("the TMA-fed kernel takes head sizes 64 and 128 and pages of 8 to 64 positions")
    if kernel == "tma3" and d != 64:
        pytest.skip("three warpgroups fit tensor memory at head size 64 only")
    dtype = torch.bfloat16
    lens, new = [150, 200, 300, 64, 17, 400], [150, 70, 16, 64, 17, 300]
    pool, bt, slots, t, q, scale, ref = attention_case(dtype, nh, nkv, d, ps, lens, new, 50, window)
    tiles = []
    for i, m in enumerate(new):
        if i == 2:
            continue                                   # request 2 is left to "another kernel"
        tiles += [(i, off) for off in range(0, m, ops.attention_prefill_tile_rows())]
    tiles_t = torch.tensor(tiles, dtype=torch.int32).flatten()
    out = torch.full_like(ref, 7.0, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.attention_prefill(q.to(DEV), pool.to(DEV), 1, out, tiles_t.to(DEV), len(tiles), t["q_start"].to(DEV),
                          t["start"].to(DEV), slots.to(DEV), bt.to(DEV), nh, scale, window, status=status,
                          kernel=kernel)
    assert int(status.item()) == 0
    keep = t["seq"] != 2
    close(out[keep], ref[keep], dtype, "attention_prefill", rel=1.5e-2)
    assert torch.all(out[~keep] == 7.0)
    # the queries as the first columns of a wider tensor (the fused q|k|v product), read with the row's stride
    wide = torch.cat([q, rnd((q.shape[0], 2 * nkv * d), dtype, 51)], dim=1).to(DEV)
    strided = torch.full_like(ref, 7.0, device=DEV)
    ops.attention_prefill(wide, pool.to(DEV), 1, strided, tiles_t.to(DEV), len(tiles), t["q_start"].to(DEV),
                          t["start"].to(DEV), slots.to(DEV), bt.to(DEV), nh, scale, window, status=status,
                          kernel=kernel, q_stride=wide.shape[1])
    assert torch.equal(strided, out)


@pytest.mark.parametrize("window", [0, 200])
@pytest.mark.parametrize("ps", [16, 64])
def test_attention_prefill_persistent_kernel_walks_through_many_tiles(ps, window):
    """More (tile, head) pairs than the GPU has SMs, so that every block of the persistent kernel goes through
    several pairs: long and short tiles, a request whose keys lie mostly in the cache, tiles of a single key
    tile (the second warpgroup has none), padding tiles between real ones."""
    nh, nkv, d = 6, 3, 64
    dtype = torch.bfloat16
    lens, new = [2048, 700, 129, 1500, 40], [2048, 300, 129, 1000, 40]
    pool, bt, slots, t, q, scale, ref = attention_case(dtype, nh, nkv, d, ps, lens, new, 55, window)
    tr = ops.attention_prefill_tile_rows()
    tiles = []
    for i, m in enumerate(new):
        tiles += [(lens[i] - m + min(off + tr, m), i, off) for off in range(0, m, tr)]
    tiles.sort(reverse=True)                          # the longest key range first, as the engine lists them
    flat = []
    for j, (_, i, off) in enumerate(tiles):
        flat += [i, off]
        if j % 5 == 2:
            flat += [0, 1 << 24]                      # a padding tile: an offset past any request's tokens
    n_tiles = len(flat) // 2
    assert n_tiles * nh > 148 * 1.2
    out = torch.full_like(ref, 7.0, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.attention_prefill(q.to(DEV), pool.to(DEV), 1, out, torch.tensor(flat, dtype=torch.int32, device=DEV), n_tiles,
                          t["q_start"].to(DEV), t["start"].to(DEV), slots.to(DEV), bt.to(DEV), nh, scale, window,
                          status=status, kernel="tmap")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    close(out, ref, dtype, "persistent attention_prefill", rel=1.5e-2)
    same = torch.full_like(ref, 7.0, device=DEV)
    ops.attention_prefill(q.to(DEV), pool.to(DEV), 1, same, torch.tensor(flat, dtype=torch.int32, device=DEV), n_tiles,
                          t["q_start"].to(DEV), t["start"].to(DEV), slots.to(DEV), bt.to(DEV), nh, scale, window,
                          status=status, kernel="tma")
    assert torch.equal(out, same), "the persistent kernel does the arithmetic of the kernel with one block per pair"


def test_attention_kernels_drop_keys_behind_a_hole_in_the_block_table():
    """A page missing from a request's block table (-1) must not be read through: every attention kernel
    treats the keys of that page as absent (zeros or dropped), leaves the other requests' results exact,
    returns finite numbers for the request with the hole, and sets the status word to 1 so that the host
    hears of it (ModelRunner.check_status then raises: the step's bookkeeping is broken)."""
    nh, nkv, d, ps = 4, 2, 64, 16
    dtype = torch.bfloat16
    lens, new = [200, 150, 300], [200, 1, 300]
    pool, bt, slots, t, q, scale, ref = attention_case(dtype, nh, nkv, d, ps, lens, new, 70)
    bt2 = bt.clone()
    bt2[int(slots[0]), 3] = -1          # request 0, prefill: positions 48..63 missing
    bt2[int(slots[1]), 5] = -1          # request 1, decode
    n = q.shape[0]
    dev = dict(pos=t["pos"].to(DEV), seq=t["seq"].to(DEV), slots=slots.to(DEV), bt=bt2.to(DEV), q=q.to(DEV),
               pool=pool.to(DEV), q_start=t["q_start"].to(DEV), start=t["start"].to(DEV))
    keep = t["seq"] == 2
    tr = ops.attention_prefill_tile_rows()
    tiles = torch.tensor([v for i in (0, 2) for off in range(0, new[i], tr) for v in (i, off)], dtype=torch.int32).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for kernel in ("tmap", "tma", "tma3", "tc", "mma"):
        out = torch.zeros_like(ref, device=DEV)
        ops.attention_prefill(dev["q"], dev["pool"], 1, out, tiles, tiles.numel() // 2, dev["q_start"], dev["start"],
                              dev["slots"], dev["bt"], nh, scale, 0, status=status, kernel=kernel)
        assert int(status.item()) == 1, f"prefill {kernel}: the hole must be reported"
        status.zero_()
        assert torch.isfinite(out.float()).all()
        close(out[keep], ref[keep], dtype, f"prefill {kernel} beside a hole", rel=1.5e-2)
    # without a hole the word stays 0
    clean = bt.to(DEV)
    for kernel in ("tmap", "tma", "tc", "mma"):
        out = torch.zeros_like(ref, device=DEV)
        ops.attention_prefill(dev["q"], dev["pool"], 1, out, tiles, tiles.numel() // 2, dev["q_start"], dev["start"],
                              dev["slots"], clean, nh, scale, 0, status=status, kernel=kernel)
        assert int(status.item()) == 0, kernel
    item = torch.tensor([200], dtype=torch.int32, device=DEV)     # request 1's token
    for kernel, splits in (("mma", 1), ("lanes", 1), ("mma", 3), ("lanes", 3)):
        out = torch.zeros_like(ref, device=DEV)
        partial = torch.empty(max(ops.attention_decode_scratch(1, nh, d, splits), 1), device=DEV)
        ops.attention_decode(dev["q"], dev["pool"], 1, out, item, 1, dev["pos"], dev["seq"], dev["slots"], dev["bt"],
                             nh, scale, n_splits=splits, partial=partial, kernel=kernel, status=status)
        assert int(status.item()) == 1, f"decode {kernel}/{splits}: the hole must be reported"
        status.zero_()
        assert torch.isfinite(out.float()).all() and float(out[200].float().abs().max()) > 0
        ops.attention_decode(dev["q"], dev["pool"], 1, out, item, 1, dev["pos"], dev["seq"], dev["slots"], clean,
                             nh, scale, n_splits=splits, partial=partial, kernel=kernel, status=status)
        assert int(status.item()) == 0
    out = torch.zeros_like(ref, device=DEV)
    ops.attention_plain(dev["q"], dev["pool"], 1, out, dev["pos"], dev["seq"], dev["slots"], dev["bt"], nh, scale,
                        status=status)
    assert int(status.item()) == 1 and torch.isfinite(out.float()).all()
    status.zero_()
    close(out[keep], ref[keep], dtype, "plain beside a hole", rel=1e-2)
    # a request none of whose pages is there: zeros or finite numbers, never NaN
    none = torch.full_like(dev["bt"], -1)
    for kernel in ("lanes", "mma"):
        out = torch.zeros_like(ref, device=DEV)
        ops.attention_decode(dev["q"], dev["pool"], 1, out, item, 1, dev["pos"], dev["seq"], dev["slots"], none,
                             nh, scale, kernel=kernel, status=status)
        assert torch.isfinite(out.float()).all() and int(status.item()) == 1, kernel
    out = torch.full_like(ref, 7.0, device=DEV)
    ops.attention_plain(dev["q"], dev["pool"], 1, out, dev["pos"], dev["seq"], dev["slots"], none, nh, scale)
    assert bool((out == 0).all())


def test_attention_finds_a_far_key_among_hundreds():
    """One key far back is made to dominate: a kernel that skips or misplaces it shows at once."""
    nh, nkv, d, ps = 2, 2, 64, 16
    for dtype in DTYPES:
        lens, new = [600], [1]
        pool, bt, slots, t, q, scale, _ = attention_case(dtype, nh, nkv, d, ps, lens, new, 60)
        far = 37
        page = int(bt[int(slots[0]), far // ps])
        pool[page, 1, 0, :, far % ps, :] = (q[0].float().view(nh, d) * 4).to(dtype)   # key aligned with the query
        pool[page, 1, 1, :, far % ps, :] = 100.0
        ref = torch.zeros(1, nh * d, dtype=dtype)
        cpu_ops.attention_plain(q, pool, 1, ref, t["pos"], t["seq"], slots, bt, nh, scale)
        assert ref.float().mean() > 90
        args = (t["pos"].to(DEV), t["seq"].to(DEV), slots.to(DEV), bt.to(DEV), nh, scale)
        out = torch.zeros_like(ref, device=DEV)
        ops.attention_plain(q.to(DEV), pool.to(DEV), 1, out, *args)
        close(out, ref, dtype, "plain far key", rel=3e-6 if dtype == torch.float32 else 1e-2)
        if dtype == torch.bfloat16:
            for ns in (1, 4):
                out = torch.zeros_like(ref, device=DEV)
                partial = torch.empty(ops.attention_decode_scratch(1, nh, d, ns) + 1, device=DEV)
                ops.attention_decode(q.to(DEV), pool.to(DEV), 1, out, None, 1, *args, 0, ns, partial)
                close(out, ref, dtype, "decode far key", rel=1e-2)


def test_argmax_and_sample():
    g = torch.Generator().manual_seed(70)
    logits = torch.randn((9, 50272), generator=g) * 3
    logits[3, 100] = logits[3, 40000] = 50.0          # a tie: the lowest id wins
    got = ops.argmax(logits.to(DEV)).cpu()
    assert torch.equal(got, cpu_ops.argmax(logits)) and int(got[3]) == 100
    n = logits.shape[0]
    temps = torch.tensor([0.0, 0.8, 1.0, 0.0, 1.5, 0.7, 1.0, 0.3, 2.0])
    topk = torch.tensor([0, 0, 50, 0, 5, 1, 0, 1000, 0], dtype=torch.int32)
    seeds = torch.arange(n, dtype=torch.int64) + 1234
    same = 0
    for step in range(20):
        counters = torch.full((n,), step, dtype=torch.int64)
        ref = cpu_ops.sample(logits, temps, topk, seeds, counters)
        got = ops.sample(logits.to(DEV), temps.to(DEV), topk.to(DEV), seeds.to(DEV), counters.to(DEV)).cpu()
        for r in range(n):
            if int(got[r]) == int(ref[r]):
                same += 1
            else:
                # float32 vs float64 CDF: a draw that lands within rounding of a boundary may
                # pick the neighbouring kept id; it must still be a kept id of similar mass
                assert temps[r] > 0
                k = int(topk[r])
                if k > 0:
                    kth = torch.sort(logits[r], descending=True).values[k - 1]
                    assert logits[r, int(got[r])] >= kth
    assert same >= 20 * n - 2
    assert int(got[5]) == int(torch.argmax(logits[5]))   # top_k = 1 is greedy
    assert abs(ops.uniform(5, 9) - cpu_ops.uniform(5, 9)) == 0.0


def test_sampling_distribution():
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5]]).repeat(4000, 1)
    n = logits.shape[0]
    got = ops.sample(logits.to(DEV), torch.full((n,), 0.7, device=DEV), torch.zeros(n, dtype=torch.int32, device=DEV),
                     torch.full((n,), 99, dtype=torch.int64, device=DEV),
                     torch.arange(n, dtype=torch.int64, device=DEV)).cpu()
    freq = torch.bincount(got.long(), minlength=5).double() / n
    p = torch.softmax(logits[0].double() / 0.7, 0)
    assert (freq - p).abs().max() < 0.03


def test_cpu_tensors_are_refused():
    with pytest.raises(ops.KernelError):
        ops.bias_act(torch.zeros(2, 2), torch.zeros(2), "relu")


@pytest.mark.parametrize("shape", [(1, 50, 24), (3, 2048, 2048), (8, 777, 520), (9, 130, 8192), (16, 96, 72),
                                   (17, 1000, 264), (32, 6144, 2048)])
def test_gemm_skinny(shape):
    n, m, k = shape
    dtype = torch.bfloat16
    a, w, b = rnd((n, k), dtype, 80), rnd((m, k), dtype, 81, 0.1), rnd((m,), torch.float32, 82)
    for act in ("none", "relu", "gelu"):
        got = ops.gemm_skinny(a.to(DEV), w.to(DEV), b.to(DEV), act, torch.float32)
        close(got, cpu_ops.linear(a, w, b, act, torch.float32), torch.float32, f"gemm_skinny {act}", rel=2e-5)
    got = ops.gemm_skinny(a.to(DEV), w.to(DEV))
    close(got, cpu_ops.linear(a, w), dtype, "gemm_skinny bf16 out", rel=8e-3)
    with pytest.raises(ops.KernelError):
        ops.gemm_skinny(rnd((33, k), dtype, 83).to(DEV), w.to(DEV))
    # a row's result does not depend on the other rows in the batch
    one = ops.gemm_skinny(a[n - 1:n].to(DEV).contiguous(), w.to(DEV), b.to(DEV), "none", torch.float32)
    full = ops.gemm_skinny(a.to(DEV), w.to(DEV), b.to(DEV), "none", torch.float32)
    assert torch.equal(one[0], full[n - 1])


@pytest.mark.parametrize("shape", [(1, 130, 64), (2, 96, 96), (3, 1000, 544), (5, 2048, 2048), (8, 6144, 2048),
                                   (8, 512, 4096), (7, 300, 7168), (4, 33, 8192), (8, 777, 1024)])
@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm", "none"])
def test_gemm_skinny_with_the_norm_in_front(shape, kind, monkeypatch):
    """norm(x) . w^T for a few float rows x in one kernel: every count of rows (clusters of 1, 2, 4, 8 blocks that
    share the normalised rows through distributed shared memory), widths that need 1, 2, 4 and 8 pieces of a row
    per thread, feature counts that leave a cluster partly empty, with and without gain and shift.  The
    reference rounds the normalised rows to bfloat16 where the kernel does."""
    monkeypatch.setattr(ops, "FUSE_NORM", True)          # the kernel itself (the engine runs norm and product apart)
    n, m, k = shape
    x = rnd((n, k), torch.float32, 90) * 3 + 0.7
    x[0, 1] = 40.0                                       # one large element, as residual streams have
    w, b = rnd((m, k), torch.bfloat16, 91, 0.1), rnd((m,), torch.float32, 92)
    gamma, beta = 1 + 0.2 * rnd((k,), torch.float32, 93), 0.3 * rnd((k,), torch.float32, 94)
    assert ops.fused_norm_applies(n, k, w.to(DEV))
    for g, be, act in ((gamma, beta, "relu"), (None, None, "none"), (gamma, None, "gelu")):
        ref = cpu_ops.norm_linear(x, kind, g, be, 1e-5, w, b, act, torch.float32)
        got = ops.norm_linear(x.to(DEV), kind, g.to(DEV) if g is not None else None,
                              be.to(DEV) if be is not None else None, 1e-5, w.to(DEV), b.to(DEV), act, torch.float32)
        # the normalised rows are rounded to bfloat16 in both; a value that lies near the middle between two
        # bfloat16 numbers may round the other way after float rather than double arithmetic
        close(got, ref, torch.float32, f"norm_linear {kind} {act}", rel=2e-3)
    got = ops.norm_linear(x.to(DEV), kind, gamma.to(DEV), beta.to(DEV), 1e-5, w.to(DEV), None, "none")
    close(got, cpu_ops.norm_linear(x, kind, gamma, beta, 1e-5, w), torch.bfloat16, "norm_linear bf16 out", rel=1e-2)
    # a row's result does not depend on the other rows of the step, nor on their number
    full = ops.norm_linear(x.to(DEV), kind, gamma.to(DEV), beta.to(DEV), 1e-5, w.to(DEV), b.to(DEV), "none", torch.float32)
    one = ops.norm_linear(x[n - 1:n].to(DEV).contiguous(), kind, gamma.to(DEV), beta.to(DEV), 1e-5, w.to(DEV),
                          b.to(DEV), "none", torch.float32)
    assert torch.equal(one[0], full[n - 1])
    # and equals the two kernels it replaces, bit for bit up to the order of the norm's sums
    h = torch.empty((n, k), dtype=torch.bfloat16, device=DEV)
    ops.add_norm(x.to(DEV), gamma=gamma.to(DEV), beta=beta.to(DEV), eps=1e-5, kind=kind, out_act=h)
    two = ops.gemm_skinny(h, w.to(DEV), b.to(DEV), "none", torch.float32)
    close(full, two, torch.float32, "fused against norm kernel + product", rel=2e-3)


def test_fused_norm_is_refused_where_it_does_not_apply(monkeypatch):
    monkeypatch.setattr(ops, "FUSE_NORM", True)
    w = rnd((64, 80), torch.bfloat16, 95).to(DEV)
    assert not ops.fused_norm_applies(9, 64, w) and not ops.fused_norm_applies(4, 80, w)
    assert not ops.fused_norm_applies(4, 16384, w) and not ops.fused_norm_applies(4, 64, w.float())
    with pytest.raises(ops.KernelError):
        ops.norm_linear(rnd((4, 80), torch.float32, 96).to(DEV), "layernorm", None, None, 1e-5, w)


@pytest.mark.parametrize("shape", [(1, 2048, 2048), (8, 2048, 8192), (3, 130, 64), (6, 1000, 520), (8, 96, 4096)])
def test_gemm_skinny_with_the_residual_sum_behind(shape):
    """x += a . w^T + bias in float, in place: with and without slices of k that meet in a cluster."""
    n, m, k = shape
    a, w, b = rnd((n, k), torch.bfloat16, 97), rnd((m, k), torch.bfloat16, 98, 0.1), rnd((m,), torch.float32, 99)
    x = rnd((n, m), torch.float32, 100) * 5
    for bias in (b, None):
        got = x.to(DEV).clone()
        ops.linear_add(a.to(DEV), w.to(DEV), bias.to(DEV) if bias is not None else None, got)
        ref = x.double() + cpu_ops.linear(a, w, bias, "none", torch.float32).double()
        close(got, ref, torch.float32, "linear_add", rel=2e-5)


@pytest.mark.parametrize("n", [1, 5, 8])
def test_norm_qkv_product_and_cache_write_in_one_kernel(n, monkeypatch):
    """The fused first kernel of the attention layer against norm kernel + product + cache write."""
    monkeypatch.setattr(ops, "FUSE_NORM", True)
    nh, nkv, d, ps, L = 6, 2, 64, 16, 3
    k = 384
    lens = [40 + 17 * i for i in range(n)]
    pool, bt, slots = make_cache(torch.bfloat16, n, lens, nkv, d, ps, L, 101)
    x = rnd((n, k), torch.float32, 102) * 2
    w, b = rnd(((nh + 2 * nkv) * d, k), torch.bfloat16, 103, 0.1), rnd(((nh + 2 * nkv) * d,), torch.float32, 104)
    gamma, beta = 1 + 0.2 * rnd((k,), torch.float32, 105), 0.3 * rnd((k,), torch.float32, 106)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32)
    pos[n // 2] = -1 if n > 1 else pos[0]                      # a padding token of a fixed-shape step writes nothing
    seq = torch.arange(n, dtype=torch.int32)
    status = torch.zeros(1, dtype=torch.int32)
    ref_pool, ref_q = pool.clone(), torch.zeros(n, nh * d, dtype=torch.bfloat16)
    cpu_ops.norm_qkv_linear_to_cache(x, "layernorm", gamma, beta, 1e-5, w, b, ref_q, ref_pool, 1, pos, seq, slots, bt,
                                     nh, nkv, d, status)
    got_pool, got_q = pool.to(DEV), torch.zeros(n, nh * d, dtype=torch.bfloat16, device=DEV)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.norm_qkv_linear_to_cache(x.to(DEV), "layernorm", gamma.to(DEV), beta.to(DEV), 1e-5, w.to(DEV), b.to(DEV), got_q,
                                 got_pool, 1, pos.to(DEV), seq.to(DEV), slots.to(DEV), bt.to(DEV), nh, nkv, d, st)
    assert int(st.item()) == 0
    live = pos >= 0
    close(got_q[live.to(DEV)], ref_q[live], torch.bfloat16, "fused q", rel=1.2e-2)
    close(got_pool, ref_pool, torch.bfloat16, "fused cache write", rel=1.2e-2)
    changed = (got_pool.cpu() != pool).any(dim=-1).sum().item()
    assert changed == int(live.sum()) * 2 * nkv, "one key row and one value row per live token and kv head, nothing else"


@pytest.mark.parametrize("shape", [(9, 130, 64), (16, 2048, 2048), (33, 777, 576), (48, 300, 8192), (64, 6144, 2048),
                                   (100, 1000, 320), (128, 4096, 1024), (12, 50272, 512)])
def test_gemm_stream_tc(shape):
    """The tcgen05 + TMA weight-streaming product: every count of tokens up to 128, feature counts that are
    no multiple of its 64- or 128-row tiles (the last shape takes the 128-row tiles), k that is no multiple of its
    stages of 256 (128) elements, and more stages of k than its rings hold.  An inner dimension that is no multiple
    of 64 is refused."""
    n, m, k = shape
    dtype = torch.bfloat16
    a, w, b = rnd((n, k), dtype, 84), rnd((m, k), dtype, 85, 0.1), rnd((m,), torch.float32, 86)
    for act in ("none", "relu", "gelu"):
        got = ops.gemm_stream_tc(a.to(DEV), w.to(DEV), b.to(DEV), act, torch.float32)
        close(got, cpu_ops.linear(a, w, b, act, torch.float32), torch.float32, f"gemm_stream_tc {act}", rel=2e-5)
    got = ops.gemm_stream_tc(a.to(DEV), w.to(DEV))
    close(got, cpu_ops.linear(a, w), dtype, "gemm_stream_tc bf16 out", rel=8e-3)
    assert ops.kernel_status(DEV) == 0
    with pytest.raises(ops.KernelError):
        ops.gemm_stream_tc(rnd((129, k), dtype, 87).to(DEV), w.to(DEV))
    with pytest.raises(ops.KernelError):
        ops.gemm_stream_tc(rnd((n, k + 8), dtype, 88).to(DEV), rnd((m, k + 8), dtype, 89).to(DEV))
    # a row's result does not depend on the other rows in the batch
    one = ops.gemm_stream_tc(a[n - 1:n].to(DEV).contiguous(), w.to(DEV), b.to(DEV), "none", torch.float32)
    full = ops.gemm_stream_tc(a.to(DEV), w.to(DEV), b.to(DEV), "none", torch.float32)
    assert torch.equal(one[0], full[n - 1])


@pytest.mark.parametrize("shape", [(64, 2048, 8192), (9, 2048, 2048), (33, 1000, 2112), (16, 96, 4096),
                                   (128, 4096, 16384), (48, 130, 576), (20, 12288, 4096)])
def test_linear_parts_of_the_tcgen05_product_and_the_norm_that_adds_them(shape):
    """More tokens than the mma.sync kernel serves: the tcgen05 product cut over k leaves its slices' float sums
    (blocks of their own, no bias), and the norm kernel behind adds them in slice order with the bias and the
    residual rows."""
    n, m, k = shape
    a, w, b = rnd((n, k), torch.bfloat16, 215), rnd((m, k), torch.bfloat16, 216, 0.1), rnd((m,), torch.float32, 217)
    x = rnd((n, m), torch.float32, 218) * 3
    slices = int(ops.lib().st_gemm_stream_tc_slices(m, k))
    stage = 256 if (m + 63) // 64 <= ops.sm_count() else 128       # elements of k per stage: tiles of 64 or 128 rows
    stages = (k + stage - 1) // stage
    per = (stages + slices - 1) // slices * stage
    parts = torch.empty((slices, n, m), dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ga, gw = a.to(DEV), w.to(DEV)
    rc = ops.lib().st_gemm_stream_tc_parts(ops._p(ga), ops._p(gw), ops._p(parts), n, m, k, ops._p(status), ops._stream())
    assert rc == 0 and int(status.item()) == 0
    ref_parts = torch.zeros(slices, n, m)
    for sl in range(slices):
        lo, hi = min(k, sl * per), min(k, (sl + 1) * per)
        if lo < hi:
            ref_parts[sl] = (a[:, lo:hi].double() @ w[:, lo:hi].double().T).float()
    close(parts, ref_parts, torch.float32, "parts of the tcgen05 product", rel=2e-5)
    if ops.linear_parts_slices(n, w.to(DEV)) > 1:             # what the engine calls for this shape: the same parts
        assert torch.equal(ops.linear_parts(a.to(DEV), w.to(DEV)), parts)
    gamma, beta = 1 + 0.2 * rnd((m,), torch.float32, 219), 0.3 * rnd((m,), torch.float32, 220)
    got_x, got_h = x.to(DEV).clone(), torch.empty((n, m), dtype=torch.bfloat16, device=DEV)
    ops.add_norm(got_x, parts=parts, delta_bias=b.to(DEV), resid_out=got_x, gamma=gamma.to(DEV), beta=beta.to(DEV),
                 eps=1e-5, kind="layernorm", out_act=got_h)
    close(got_x, x.double() + cpu_ops.linear(a, w, b, "none", torch.float32).double(), torch.float32,
          "parts add up to the product", rel=3e-5)
    ref_x, ref_h = x.clone(), torch.empty((n, m), dtype=torch.bfloat16)
    cpu_ops.add_norm(ref_x, parts=ref_parts, delta_bias=b, resid_out=ref_x, gamma=gamma, beta=beta, eps=1e-5,
                     kind="layernorm", out_act=ref_h)
    close(got_h, ref_h, torch.bfloat16, "norm of rows with parts", rel=1e-2)


@pytest.mark.parametrize("shape", [(5, 6144, 2048), (8, 5000, 576), (2, 8192, 1056), (1, 4768, 1024)])
def test_gemm_skinny_with_all_weights_on_chip_before_its_wait(shape, monkeypatch):
    """Few tokens, an inner dimension of 544 to 2048 and more than 296 tiles of 16 features (no slices of k): the
    product copies what its two register rounds do not hold into shared memory ahead of its dependency wait.  Sizes:
    the engine's own, a feature count that is no multiple of 16, an inner dimension of an odd number of blocks of
    32, the fewest features that still run uncut.  The same launch with the variant switched off gives the same bits
    (the arithmetic per output is the same: a warp's k-blocks in the same order)."""
    n, m, k = shape
    a, w, b = rnd((n, k), torch.bfloat16, 180), rnd((m, k), torch.bfloat16, 181, 0.1), rnd((m,), torch.float32, 182)
    for act in ("none", "relu"):
        got = ops.gemm_skinny(a.to(DEV), w.to(DEV), b.to(DEV), act, torch.float32)
        close(got, cpu_ops.linear(a, w, b, act, torch.float32), torch.float32, f"gemm_skinny on chip {act}", rel=2e-5)
    one = ops.gemm_skinny(a[n - 1:n].to(DEV).contiguous(), w.to(DEV), b.to(DEV), "none", torch.float32)
    full = ops.gemm_skinny(a.to(DEV), w.to(DEV), b.to(DEV), "none", torch.float32)
    assert torch.equal(one[0], full[n - 1])


@pytest.mark.parametrize("shape", [(3, 1000, 1024), (8, 130, 2048), (7, 2040, 800), (8, 6144, 1536)])
def test_linear_add_uncut_with_all_weights_on_chip(shape):
    """The residual sum behind a product of 544 to 2048 inner elements: one block per 16 features over the whole of k
    (never cut into cluster slices), weights on chip before the wait."""
    n, m, k = shape
    a, w, b = rnd((n, k), torch.bfloat16, 185), rnd((m, k), torch.bfloat16, 186, 0.1), rnd((m,), torch.float32, 187)
    x = rnd((n, m), torch.float32, 188) * 5
    got = x.to(DEV).clone()
    ops.linear_add(a.to(DEV), w.to(DEV), b.to(DEV), got)
    ref = x.double() + cpu_ops.linear(a, w, b, "none", torch.float32).double()
    close(got, ref, torch.float32, "linear_add on chip", rel=2e-5)


@pytest.mark.parametrize("shape", [(8, 2048, 8192), (1, 2048, 8192), (5, 4096, 4096), (3, 1000, 2080), (8, 96, 4096),
                                   (7, 1536, 6240), (6, 2000, 4640), (4, 1200, 2240)])
def test_linear_parts_and_the_norm_that_adds_them(shape):
    """A product cut over k leaves the slices' sums as float parts (no cluster, no bias); the norm kernel behind adds
    them in slice order with the bias and the residual rows: together they equal x + a . w^T + bias, normalised.
    The first two shapes are fc2 of OPT-1.3B; the last three have a shorter last slice."""
    n, m, k = shape
    a, w, b = rnd((n, k), torch.bfloat16, 195), rnd((m, k), torch.bfloat16, 196, 0.1), rnd((m,), torch.float32, 197)
    x = rnd((n, m), torch.float32, 198) * 3
    slices = ops.linear_parts_slices(n, w.to(DEV))
    assert slices == int(ops.lib().st_gemm_skinny_parts_slices(m, k))
    if slices == 1:
        pytest.skip("this product is not cut on this GPU")
    parts = ops.linear_parts(a.to(DEV), w.to(DEV))
    assert parts.shape == (slices, n, m) and parts.dtype == torch.float32
    ref_parts = cpu_ops.linear_parts(a, w, slices)
    close(parts, ref_parts, torch.float32, "linear_parts", rel=2e-5)
    gamma, beta = 1 + 0.2 * rnd((m,), torch.float32, 199), 0.3 * rnd((m,), torch.float32, 200)
    for width_ok in (True,):
        got_x, got_h = x.to(DEV).clone(), torch.empty((n, m), dtype=torch.bfloat16, device=DEV)
        ops.add_norm(got_x, parts=parts, delta_bias=b.to(DEV), resid_out=got_x, gamma=gamma.to(DEV), beta=beta.to(DEV),
                     eps=1e-5, kind="layernorm", out_act=got_h)
        ref_x, ref_h = x.clone(), torch.empty((n, m), dtype=torch.bfloat16)
        cpu_ops.add_norm(ref_x, parts=ref_parts, delta_bias=b, resid_out=ref_x, gamma=gamma, beta=beta, eps=1e-5,
                         kind="layernorm", out_act=ref_h)
        close(got_x, ref_x, torch.float32, "residual rows with parts", rel=2e-5)
        close(got_x, x.double() + cpu_ops.linear(a, w, b, "none", torch.float32).double(), torch.float32,
              "parts add up to the product", rel=3e-5)
        close(got_h, ref_h, torch.bfloat16, "norm of rows with parts", rel=1e-2)


@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm", "none"])
@pytest.mark.parametrize("width", [128, 640, 2048, 2176, 200])
def test_add_norm_of_many_rows(kind, width):
    """More rows than the launch has blocks (prompt portions): every block takes several rows, the next row's loads
    under this row's reductions.  Both uses: residual updated with a normalised copy out (with and without delta,
    bias, gain and shift), and the residual replaced by the normalised row."""
    dtype = torch.bfloat16
    n = 700
    x = rnd((n, width), torch.float32, 230) + 20.0
    delta, dbias = rnd((n, width), dtype, 231), rnd((width,), torch.float32, 232)
    gamma, beta = 1 + rnd((width,), torch.float32, 233, 0.1), rnd((width,), torch.float32, 234, 0.1)
    dev = lambda t: None if t is None else t.to(DEV)
    for dl, db, ga, be in ((delta, dbias, gamma, beta), (None, None, gamma, None), (delta, None, None, None)):
        xr, ref_out = x.clone(), torch.empty(n, width, dtype=dtype)
        cpu_ops.add_norm(xr, delta=dl, delta_bias=db, resid_out=xr, gamma=ga, beta=be, eps=1e-5, kind=kind, out_act=ref_out)
        xg, got_out = x.to(DEV), torch.empty(n, width, dtype=dtype, device=DEV)
        ops.add_norm(xg, delta=dev(dl), delta_bias=dev(db), resid_out=xg, gamma=dev(ga), beta=dev(be), eps=1e-5, kind=kind,
                     out_act=got_out)
        close(xg, xr, torch.float32, "residual of many rows", rel=1e-6)
        close(got_out, ref_out, dtype, f"{kind} of many rows", rel=8e-3)
    xr, ref_out = x.clone(), torch.empty(n, width, dtype=dtype)
    cpu_ops.add_norm(xr, delta=delta, delta_bias=dbias, gamma=gamma, beta=beta, eps=1e-5, kind=kind, out_act=ref_out, out_f32=xr)
    xg, got_out = x.to(DEV), torch.empty(n, width, dtype=dtype, device=DEV)
    ops.add_norm(xg, delta=dev(delta), delta_bias=dev(dbias), gamma=dev(gamma), beta=dev(beta), eps=1e-5, kind=kind,
                 out_act=got_out, out_f32=xg)
    close(xg, xr, torch.float32, "normalised residual of many rows", rel=5e-5)
    close(got_out, ref_out, dtype, f"{kind} of many rows, normalised residual", rel=8e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [40, 777, 2048, 7168, 12288])
def test_add_norm_with_parts_and_a_delta_and_a_row_gather(dtype, width):
    """Every form of the norm kernel (row in shared memory, two or four vectors per thread in registers) with float
    parts beside a delta in the activation type, a bias, and a gather of rows (the final norm of a step)."""
    n, n_parts = 9, 3
    x = rnd((n, width), torch.float32, 205) * 2
    delta, bias = rnd((n, width), dtype, 206), rnd((width,), torch.float32, 207)
    parts = rnd((n_parts, n, width), torch.float32, 208)
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    gamma, beta = 1 + 0.2 * rnd((width,), torch.float32, 209), 0.3 * rnd((width,), torch.float32, 210)
    for kind in ("layernorm", "rmsnorm", "none"):
        got = torch.empty((3, width), dtype=dtype, device=DEV)
        ops.add_norm(x.to(DEV), delta=delta.to(DEV), delta_bias=bias.to(DEV), parts=parts.to(DEV), gamma=gamma.to(DEV),
                     beta=beta.to(DEV), eps=1e-5, kind=kind, rows=rows.to(DEV), out_act=got)
        ref = torch.empty((3, width), dtype=dtype)
        cpu_ops.add_norm(x.clone(), delta=delta, delta_bias=bias, parts=parts, gamma=gamma, beta=beta, eps=1e-5, kind=kind,
                         rows=rows, out_act=ref)
        close(got, ref, dtype, f"add_norm with parts, {kind}", rel=2e-5 if dtype == torch.float32 else 1e-2)


def test_qkv_linear_to_cache_with_all_weights_on_chip():
    """The fused q|k|v product at a size that takes the on-chip variant (6144 features, 1024 inner elements, 7 tokens
    of which one is padding): queries and pages as the plain reference leaves them."""
    dtype = torch.bfloat16
    n, nh, nkv, d, ps, L, K = 7, 32, 32, 64, 16, 2, 1024
    lens = [33 + 5 * i for i in range(n)]
    pool, bt, slots = make_cache(dtype, n, lens, nkv, d, ps, L, 190)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32)
    pos[3] = -1
    seq = torch.arange(n, dtype=torch.int32)
    h, w = rnd((n, K), dtype, 191), rnd(((nh + 2 * nkv) * d, K), dtype, 192, 0.1)
    bias = rnd(((nh + 2 * nkv) * d,), torch.float32, 193)
    ref_pool, ref_q, st = pool.clone(), torch.zeros(n, nh * d, dtype=dtype), torch.zeros(1, dtype=torch.int32)
    cpu_ops.qkv_linear_to_cache(h, w, bias, ref_q, ref_pool, 1, pos, seq, slots, bt, nh, nkv, d, st)
    gp, gq = pool.to(DEV), torch.zeros(n, nh * d, dtype=dtype, device=DEV)
    gst = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.qkv_linear_to_cache(h.to(DEV), w.to(DEV), bias.to(DEV), gq, gp, 1, pos.to(DEV), seq.to(DEV), slots.to(DEV),
                            bt.to(DEV), nh, nkv, d, gst)
    assert int(gst.item()) == 0
    live = pos >= 0
    close(gq[live.to(DEV)], ref_q[live], dtype, "q on chip", rel=1e-2)
    close(gp, ref_pool, dtype, "pool on chip", rel=1e-2)
    changed = (gp.cpu() != pool).any(dim=-1).sum().item()
    assert changed <= 2 * nkv * (n - 1)


@pytest.mark.parametrize("n", [1, 8, 13, 32])
def test_qkv_linear_to_cache(n):
    dtype = torch.bfloat16
    nh, nkv, d, ps, L, K = 6, 2, 24, 8, 3, 136
    lens = [40 + i for i in range(n)]
    pool, bt, slots = make_cache(dtype, n, lens, nkv, d, ps, L, 90)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32)
    pos[n // 2] = -1 if n > 1 else pos[0]                      # one padding token
    seq = torch.arange(n, dtype=torch.int32)
    h, w = rnd((n, K), dtype, 91), rnd(((nh + 2 * nkv) * d, K), dtype, 92, 0.2)
    bias = rnd(((nh + 2 * nkv) * d,), torch.float32, 93)
    ref_pool, ref_q, st = pool.clone(), torch.zeros(n, nh * d, dtype=dtype), torch.zeros(1, dtype=torch.int32)
    cpu_ops.qkv_linear_to_cache(h, w, bias, ref_q, ref_pool, 2, pos, seq, slots, bt, nh, nkv, d, st)
    gp, gq = pool.to(DEV), torch.zeros(n, nh * d, dtype=dtype, device=DEV)
    gst = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.qkv_linear_to_cache(h.to(DEV), w.to(DEV), bias.to(DEV), gq, gp, 2, pos.to(DEV), seq.to(DEV), slots.to(DEV),
                            bt.to(DEV), nh, nkv, d, gst)
    assert int(gst.item()) == 0
    close(gq, ref_q, dtype, "q", rel=1e-2)
    close(gp, ref_pool, dtype, "pool", rel=1e-2)
    changed = (gp.cpu() != pool).any(dim=-1).sum().item()
    assert changed <= 2 * nkv * n, "only the new tokens' rows of layer 2 may change"
