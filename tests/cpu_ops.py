"""The plain reference of every device operation, in torch on the CPU.

Each function has the signature of its namesake in ``swifttransformer_b200.ops``
and computes the same thing the slow, obvious way (float64 inside where that
is free).  The kernel tests compare each CUDA kernel with its function here;
the CPU tests patch these over ``ops`` to exercise the engine's host logic
(step building, cache manager, scheduler) where there is no GPU.  Nothing in
the package imports this file.
"""
from __future__ import annotations

import math

import torch


def _act(y, act):
    if act == "relu":
        return torch.relu(y)
    if act == "gelu":
        return 0.5 * y * (1 + torch.erf(y / math.sqrt(2.0)))
    return y


def embed(ids, table, out, positions=None, pos_table=None, pos_offset=0):
    v = table[ids.long()].double()
    if pos_table is not None:
        live = (positions >= 0).unsqueeze(1)       # padding tokens (position -1) get no position row
        v = v + pos_table[(positions.long() + pos_offset).clamp(min=0)].double() * live
    out.copy_(v.to(out.dtype))
    return out


def add_positions(x, positions, pos_table, pos_offset, out):
    live = (positions >= 0).unsqueeze(1)
    out.copy_((x.double() + pos_table[(positions.long() + pos_offset).clamp(min=0)].double() * live).to(out.dtype))
    return out


def add_norm(x, *, delta=None, delta_bias=None, resid_out=None, gamma=None, beta=None, eps=1e-5,
             kind="layernorm", rows=None, out_act=None, out_f32=None, act_dtype=None, parts=None):
    idx = rows.long() if rows is not None else torch.arange(x.shape[0])
    s = x[idx].float()
    if delta is not None or parts is not None:
        d = delta[idx].float() if delta is not None else torch.zeros_like(s)
        if parts is not None:
            for p in parts:
                d = d + p[idx].float()
        s = s + d
    if delta_bias is not None:
        s = s + delta_bias.float()
    if resid_out is not None:
        resid_out[idx] = s
    sd = s.double()
    if kind == "layernorm":
        mean = sd.mean(-1, keepdim=True)
        var = ((sd - mean) ** 2).mean(-1, keepdim=True)
        y = (sd - mean) / torch.sqrt(var + eps)
    elif kind == "rmsnorm":
        y = sd / torch.sqrt((sd ** 2).mean(-1, keepdim=True) + eps)
    else:
        y = sd
    if kind != "none":
        if gamma is not None:
            y = y * gamma.double()
        if beta is not None:
            y = y + beta.double()
    if out_act is not None:
        out_act.copy_(y.to(out_act.dtype))
    if out_f32 is not None:
        out_f32.copy_(y.float())


def bias_act(y, bias, act):
    v = y.float()
    if bias is not None:
        v = v + bias
    y.copy_(_act(v, act).to(y.dtype))
    return y


def scatter_i32(dst, idx, val, count, max_count):
    n = int(count[0])
    dst.view(-1)[idx[:n].long()] = val[:n]


def gather_where_i32(dst, src_index, src):
    m = src_index >= 0
    dst[m] = src[src_index[m].long()]


def lossless_bf16(v):
    return None


def linear(a, w, bias=None, act="none", out_dtype=None, bias_bf16=None):
    y = a.double() @ w.double().t()
    if bias is not None:
        y = y + bias.double()
    return _act(y, act).to(out_dtype or a.dtype)


gemm_plain = linear
gemm_skinny = linear
gemm_stream_tc = linear
STREAM_TC_MAX_ROWS = 0


def stream_tc_applies(n_rows, w):
    return False


def kernel_status(device):
    return 0
SKINNY_MAX_ROWS = 8


FUSED_MAX_ROWS = 8
UNCUT_MAX_INNER = 2048
FUSE_NORM = False


def fused_norm_applies(n_rows, k, w):
    return False        # the CPU runs of the engine take the unfused path


def _norm_rows(x, kind, gamma, beta, eps, dtype, delta=None, delta_bias=None, parts=None):
    out = torch.empty(x.shape, dtype=dtype)
    pending = delta is not None or delta_bias is not None or parts is not None
    add_norm(x, delta=delta, delta_bias=delta_bias, parts=parts, resid_out=x if pending else None, gamma=gamma,
             beta=beta, eps=eps, kind=kind, out_act=out)
    return out


def norm_linear(x, kind, gamma, beta, eps, w, bias=None, act="none", out_dtype=None, delta=None, delta_bias=None,
                parts=None):
    return linear(_norm_rows(x, kind, gamma, beta, eps, w.dtype, delta, delta_bias, parts), w, bias, act,
                  out_dtype or w.dtype)


def linear_add(a, w, bias, x):
    x += linear(a, w, bias, "none", torch.float32)


def linear_parts_slices(n_rows, w):
    return 1            # the CPU runs of the engine do not cut products


def linear_parts(a, w, slices=4):
    """The sums of a @ w.T over `slices` equal ranges of 32-element blocks of the inner dimension, float32
    [slices, rows, out] (the kernel's cut: blocks of 32 dealt out in equal runs, the last run shorter)."""
    k = a.shape[1]
    nkb = (k + 31) // 32
    per = (nkb + slices - 1) // slices
    out = torch.zeros(slices, a.shape[0], w.shape[0], dtype=torch.float32)
    for s in range(slices):
        lo, hi = min(k, s * per * 32), min(k, (s + 1) * per * 32)
        if lo < hi:
            out[s] = (a[:, lo:hi].double() @ w[:, lo:hi].double().T).float()
    return out


def norm_qkv_linear_to_cache(x, kind, gamma, beta, eps, w, bias, q_out, pool, layer, positions, seq_of_token, slots,
                             block_table, nh, nkv, d, status, write_kv=True, delta=None, delta_bias=None, parts=None):
    qkv_linear_to_cache(_norm_rows(x, kind, gamma, beta, eps, w.dtype, delta, delta_bias, parts), w, bias, q_out, pool,
                        layer, positions, seq_of_token, slots, block_table, nh, nkv, d, status, write_kv)


def qkv_linear_to_cache(h, w, bias, q_out, pool, layer, positions, seq_of_token, slots, block_table, nh, nkv, d,
                        status, write_kv=True):
    qkv = linear(h, w)
    qkv_to_cache(qkv, bias, q_out, pool, layer, positions, seq_of_token, slots, block_table, nh, nkv, d, status,
                 write_kv)


def qkv_to_cache(qkv, bias, q_out, pool, layer, positions, seq_of_token, slots, block_table, nh, nkv, d,
                 status, write_kv=True):
    n = qkv.shape[0]
    v = qkv.float()
    if bias is not None:
        v = v + bias
    if q_out is not None:
        q_out.copy_(v[:, :nh * d].to(q_out.dtype))
    if not write_kv:
        return
    ps = pool.shape[4]
    for t in range(n):
        pos = int(positions[t])
        if pos < 0:
            continue
        slot = int(slots[int(seq_of_token[t])])
        page = int(block_table[slot, pos // ps])
        if page < 0 or page >= pool.shape[0]:
            status[0] = 1
            continue
        pool[page, layer, 0, :, pos % ps, :] = v[t, nh * d:(nh + nkv) * d].view(nkv, d).to(pool.dtype)
        pool[page, layer, 1, :, pos % ps, :] = v[t, (nh + nkv) * d:].view(nkv, d).to(pool.dtype)


def attention_plain(q, pool, layer, out, positions, seq_of_token, slots, block_table, nh, scale, window=0, status=None):
    n = q.shape[0]
    _, _, _, nkv, ps, d = pool.shape
    g = nh // nkv
    for t in range(n):
        pos = int(positions[t])
        if pos < 0:
            continue
        slot = int(slots[int(seq_of_token[t])])
        lo = max(0, pos - window + 1) if window > 0 else 0
        keys = torch.arange(lo, pos + 1)
        pages = block_table[slot, (keys // ps).long()].long()
        k = pool[pages, layer, 0, :, (keys % ps).long(), :].double()    # [keys, nkv, d]
        v = pool[pages, layer, 1, :, (keys % ps).long(), :].double()
        qt = q[t].double().view(nh, d)
        for h in range(nh):
            s = (k[:, h // g, :] @ qt[h]) * scale
            p = torch.softmax(s, 0)
            out[t, h * d:(h + 1) * d] = (p @ v[:, h // g, :]).to(out.dtype)
    return out


def sm_count(device=None):
    return 148


def decode_warps(n_items, nkv, d, n_splits, max_kv):
    return 4


def attention_decode_scratch(n_items, nh, d, n_splits):
    return n_items * nh * n_splits * (d + 2) if n_splits > 1 else 0


def attention_decode(q, pool, layer, out, items, n_items, positions, seq_of_token, slots, block_table, nh,
                     scale, window=0, n_splits=1, partial=None, fused_merge=True, kernel="auto", warps=4, status=None, start_pos=None):
    idx = items[:n_items].long() if items is not None else torch.arange(n_items)
    tmp = torch.zeros_like(out)
    pos = torch.full_like(positions, -1)
    pos[idx] = positions[idx]
    attention_plain(q, pool, layer, tmp, pos, seq_of_token, slots, block_table, nh, scale, window)
    keep = idx[positions[idx] >= 0]
    out[keep] = tmp[keep]
    return out


DECODE_FROM_PROJECTION = True


def attention_decode_qkv_applies(qkv, pool, n_items, nh, n_splits):
    return False        # the CPU runs of the engine keep the cache write apart


def attention_decode_qkv(qkv, pool, layer, out, items, n_items, positions, seq_of_token, slots, start_pos,
                         block_table, nh, scale, window=0, n_splits=1, partial=None, warps=4, write_kv=True, status=None):
    """The cache write of every token of the step, then single-token attention for the items."""
    nkv, d = pool.shape[3], pool.shape[5]
    q = torch.zeros(qkv.shape[0], nh * d, dtype=qkv.dtype)
    st = status if status is not None else torch.zeros(1, dtype=torch.int32)
    qkv_to_cache(qkv, None, q, pool, layer, positions, seq_of_token, slots, block_table, nh, nkv, d, st, write_kv)
    return attention_decode(q, pool, layer, out, items, n_items, positions, seq_of_token, slots, block_table, nh,
                            scale, window)


TILE_ROWS = 128


def attention_prefill_tile_rows():
    return TILE_ROWS


def attention_prefill(q, pool, layer, out, tiles, n_tiles, q_start, start_pos, slots, block_table, nh, scale,
                      window=0, status=None, kernel="auto", q_stride=0):
    if q_stride:
        q = q[:, :out.shape[1]]
    n = q.shape[0]
    pos = torch.full((n,), -1, dtype=torch.int32)
    seq_of = torch.zeros(n, dtype=torch.int32)
    for i in range(n_tiles):
        seq, off = int(tiles[2 * i]), int(tiles[2 * i + 1])
        a = int(q_start[seq]) + off
        b = min(a + TILE_ROWS, int(q_start[seq + 1]))
        pos[a:b] = torch.arange(int(start_pos[seq]) + off, int(start_pos[seq]) + off + (b - a), dtype=torch.int32)
        seq_of[a:b] = seq
    tmp = torch.zeros_like(out)
    attention_plain(q, pool, layer, tmp, pos, seq_of, slots, block_table, nh, scale, window)
    out[pos >= 0] = tmp[pos >= 0]
    return out


def argmax(logits, out=None):
    r = torch.argmax(logits, dim=-1).to(torch.int32)   # torch returns the first maximal index
    if out is not None:
        out.copy_(r)
        return out
    return r


def _uniform(seed, counter):
    m = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + (counter + 1) * 0xBF58476D1CE4E5B9) & m
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & m
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & m
    z ^= z >> 31
    return float(z >> 40) / 16777216.0


def uniform(seed, counter):
    return _uniform(int(seed) & ((1 << 64) - 1), int(counter) & ((1 << 64) - 1))


def sample(logits, temperatures, top_k, seeds, counters, out=None):
    n, v = logits.shape
    res = torch.empty(n, dtype=torch.int32)
    for r in range(n):
        z = logits[r].double()
        t = float(temperatures[r])
        if t <= 0:
            res[r] = int(torch.argmax(z))
            continue
        k = int(top_k[r])
        if 0 < k < v:
            kth = torch.sort(z, descending=True).values[k - 1]
            z = torch.where(z >= kth, z, torch.full_like(z, -float("inf")))
        p = torch.exp((z - z.max()) / t)
        c = torch.cumsum(p, 0)
        u = uniform(int(seeds[r]), int(counters[r]))
        res[r] = min(int(torch.searchsorted(c, torch.tensor(u * float(c[-1]), dtype=c.dtype), right=True)), v - 1)
    if out is not None:
        out.copy_(res)
        return out
    return res


ALL = ["sm_count", "fused_norm_applies", "norm_linear", "linear_add", "linear_parts_slices", "linear_parts", "norm_qkv_linear_to_cache", "embed", "add_positions", "add_norm", "bias_act", "scatter_i32", "gather_where_i32", "linear", "gemm_plain", "gemm_skinny", "gemm_stream_tc", "kernel_status",
       "qkv_linear_to_cache", "qkv_to_cache",
       "attention_plain", "attention_decode_scratch", "decode_warps", "attention_decode", "attention_prefill_tile_rows",
       "attention_prefill", "argmax", "sample", "uniform"]


def install(monkeypatch):
    """Patch every operation of the package with its CPU reference (tests only)."""
    import sys
    from swifttransformer_b200 import ops
    this = sys.modules[__name__]
    for name in ALL:
        monkeypatch.setattr(ops, name, getattr(this, name))
