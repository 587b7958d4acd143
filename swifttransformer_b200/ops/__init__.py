"""The engine's device operations.

Every function here launches hand-written sm_100a kernels from ``csrc/``
through the C entry points of ``libst_b200.so`` (loaded with ctypes; built on
first use by ``ops.build``), on torch's current CUDA stream, on tensors the
caller owns.  The only library calls are the bfloat16 matrix products, which
go to cuBLAS through ``torch`` (the reference uses cuBLAS for the same five
products, src/csrc/util/cublas_wrapper.cc:29-53).

There is no CPU path: a tensor that is not on a CUDA device is an error, and
so is a missing or unbuildable library.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import build as _build

_LIB = None

ACT_CODES = {"none": 0, "relu": 1, "gelu": 2}
NORM_CODES = {"layernorm": 0, "rmsnorm": 1, "none": 2}

_ERRORS = {-1: "unsupported dtype", -2: "unsupported size", -3: "size beyond the kernel's limit",
           -4: "invalid argument"}


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded kernel library (built on first use)."""
    global _LIB
    if _LIB is None:
        path = _build.ensure_built()
        try:
            _LIB = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load {path}: {e}") from None
        _LIB.st_attention_decode_scratch_floats.restype = ctypes.c_longlong
        _LIB.st_uniform_host.restype = ctypes.c_float
        _LIB.st_uniform_host.argtypes = [ctypes.c_longlong, ctypes.c_longlong]
    return _LIB


def library_path() -> str:
    return _build.ensure_built()


_LAUNCHES = 0


def launch_count() -> int:
    """How many kernel launchers of this library have been called so far (recorded launches count once)."""
    return _LAUNCHES


def _check(rc: int, what: str) -> None:
    global _LAUNCHES
    _LAUNCHES += 1
    if rc == 0:
        return
    if rc < 0:
        raise KernelError(f"{what}: refused ({_ERRORS.get(rc, rc)})")
    raise KernelError(f"{what}: CUDA error {rc} at launch")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"unsupported tensor type {t.dtype} (float32 or bfloat16)")


def _p(t: Optional[torch.Tensor]):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("this engine runs on a CUDA device only; got a CPU tensor")
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream of the current device as a handle for the library.  torch.cuda.current_stream()
    costs ~15 us of host time per call (a fifth of the host's time for a step of eager launches); the raw
    query behind it is used where this torch has it."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _f(x: float):
    return ctypes.c_float(x)


_SM_COUNT = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of a CUDA device (the current one by default); asked once per device."""
    index = device.index if isinstance(device, torch.device) and device.index is not None \
        else torch.cuda.current_device()
    if index not in _SM_COUNT:
        _SM_COUNT[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _SM_COUNT[index]


# ------------------------------------------------------------------ embedding
def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, positions: Optional[torch.Tensor] = None,
          pos_table: Optional[torch.Tensor] = None, pos_offset: int = 0) -> torch.Tensor:
    """out[t] = table[ids[t]] (+ pos_table[positions[t] + pos_offset]); out is float32 or table's type."""
    n, width = ids.numel(), table.shape[1]
    assert out.shape == (n, width) and out.is_contiguous() and table.is_contiguous()
    if pos_table is not None:
        assert pos_table.shape[1] == width and pos_table.dtype == table.dtype
    _check(lib().st_embed(_p(ids), _p(table), n, width, _p(positions) if pos_table is not None else None,
                          _p(pos_table), pos_offset, _p(out), _dt(table), int(out.dtype == torch.float32),
                          _stream()), "embed")
    return out


def add_positions(x: torch.Tensor, positions: torch.Tensor, pos_table: torch.Tensor, pos_offset: int,
                  out: torch.Tensor) -> torch.Tensor:
    """out[t] = x[t] + pos_table[positions[t] + pos_offset]."""
    n, width = x.shape
    assert pos_table.shape[1] == width and x.dtype == pos_table.dtype and out.shape == x.shape
    _check(lib().st_add_positions(_p(x), n, width, _p(positions), _p(pos_table), pos_offset, _p(out),
                                  _dt(x), int(out.dtype == torch.float32), _stream()), "add_positions")
    return out


# ------------------------------------------------------------ residual + norm
def add_norm(x: torch.Tensor, *, delta: Optional[torch.Tensor] = None, delta_bias: Optional[torch.Tensor] = None,
             resid_out: Optional[torch.Tensor] = None, gamma: Optional[torch.Tensor] = None,
             beta: Optional[torch.Tensor] = None, eps: float = 1e-5, kind: str = "layernorm",
             rows: Optional[torch.Tensor] = None, out_act: Optional[torch.Tensor] = None,
             out_f32: Optional[torch.Tensor] = None, act_dtype: Optional[torch.dtype] = None,
             parts: Optional[torch.Tensor] = None) -> None:
    """s = x[i] + (delta[i] + parts[0][i] + parts[1][i] + ...) + delta_bias; resid_out[i] = s; y = norm(s);
    out_act[r] = y; out_f32[r] = y.

    ``x`` is the float32 residual stream; ``i = rows[r]`` when ``rows`` is given, else ``r``.  ``parts``: float32
    [n, rows of x, width], further addends (the slices of k of a product, see ``linear_parts``).
    """
    assert x.dtype == torch.float32 and x.is_contiguous()
    if parts is not None:
        assert parts.dtype == torch.float32 and parts.dim() == 3 and parts.shape[1:] == x.shape
        assert parts.stride(2) == 1 and parts.stride(1) == x.shape[1]
    width = x.shape[1]
    n = rows.numel() if rows is not None else x.shape[0]
    if out_act is not None:
        code = _dt(out_act)
    elif delta is not None:
        code = _dt(delta)
    else:
        code = 0 if act_dtype in (None, torch.float32) else 1
    if delta is not None and out_act is not None:
        assert delta.dtype == out_act.dtype
    _check(lib().st_add_norm(_p(x), _p(rows), _p(delta), _p(delta_bias), _p(parts),
                             parts.shape[0] if parts is not None else 0,
                             ctypes.c_longlong(parts.stride(0) if parts is not None else 0), _p(resid_out), _p(gamma), _p(beta),
                             _f(eps), NORM_CODES[kind], n, width, _p(out_act), _p(out_f32), code, _stream()),
           "add_norm")


def bias_act(y: torch.Tensor, bias: Optional[torch.Tensor], act: str) -> torch.Tensor:
    """y = act(y + bias) in place."""
    if bias is None and act == "none":
        return y
    assert y.is_contiguous()
    _check(lib().st_bias_act(_p(y), _p(bias), ACT_CODES[act], y.shape[0], y.shape[1], _dt(y), _stream()), "bias_act")
    return y


def scatter_i32(dst: torch.Tensor, idx: torch.Tensor, val: torch.Tensor, count: torch.Tensor, max_count: int) -> None:
    """dst.flatten()[idx[i]] = val[i] for i < count[0] (count lives on the device)."""
    _check(lib().st_scatter_i32(_p(dst), _p(idx), _p(val), _p(count), max_count, _stream()), "scatter_i32")


def gather_where_i32(dst: torch.Tensor, src_index: torch.Tensor, src: torch.Tensor) -> None:
    """dst[i] = src[src_index[i]] wherever src_index[i] >= 0 (int32 tensors on the device)."""
    assert dst.dtype == src.dtype == src_index.dtype == torch.int32 and dst.numel() == src_index.numel()
    _check(lib().st_gather_where_i32(_p(dst), _p(src_index), _p(src), dst.numel(), src.numel(), _stream()),
           "gather_where_i32")


# ------------------------------------------------------------ matrix products
_tc_status = {}


def _tc_status_word(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _tc_status:
        _tc_status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_status[key]


def lossless_bf16(v: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """A bfloat16 copy of a float vector if every element survives the rounding unchanged, else None."""
    if v is None or v.dtype != torch.float32:
        return None
    low = v.to(torch.bfloat16)
    return low if bool(torch.equal(low.float(), v)) else None


_addmm_activation = getattr(torch, "_addmm_activation", None)    # the library product with bias and ReLU in its epilogue


def linear(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
           out_dtype: Optional[torch.dtype] = None, bias_bf16: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(a @ w.T + bias); w is [out, in].  float32: the plain fused-multiply-add kernel (true 32-bit).
    bfloat16, few rows: the weight-streaming kernel.  bfloat16, more rows: the library product with float
    accumulation; bias and ReLU ride in its epilogue when ``bias_bf16`` (a lossless bfloat16 copy of
    ``bias``, see lossless_bf16) is given, else the bias/activation kernel follows."""
    assert a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1] and a.dtype == w.dtype
    out_dtype = out_dtype or a.dtype
    n, m = a.shape[0], w.shape[0]
    if a.dtype == torch.float32:
        return gemm_plain(a, w, bias, act, out_dtype)
    if not a.is_cuda:
        raise KernelError("this engine runs on a CUDA device only; got a CPU tensor")
    if n == 0:
        return torch.empty((0, m), dtype=out_dtype, device=a.device)
    if n <= SKINNY_MAX_ROWS and a.shape[1] % 8 == 0:
        return gemm_skinny(a, w, bias, act, out_dtype)
    if stream_tc_applies(n, w):
        return gemm_stream_tc(a, w, bias, act, out_dtype)
    if out_dtype == torch.float32:
        y = torch.mm(a, w.t(), out_dtype=torch.float32)
    elif bias_bf16 is not None and (act == "none" or (act == "relu" and _addmm_activation is not None)):
        if act == "relu":
            return _addmm_activation(bias_bf16, a, w.t(), use_gelu=False)
        return torch.addmm(bias_bf16, a, w.t())
    else:
        y = torch.mm(a, w.t())
    return bias_act(y, bias, act)


# Up to this many tokens the weight-streaming kernel serves bfloat16 products.  The kernel itself takes up
# to 32 rows; from 9 rows on the library product is ahead (at 16 rows: on four of the model's five products).
SKINNY_MAX_ROWS = 8
SKINNY_KERNEL_MAX_ROWS = 32


# Up to this many tokens (and above SKINNY_MAX_ROWS) the tcgen05 weight-streaming kernel serves the bfloat16
# products that it runs in one wave of blocks; 0: off, the library product takes over from SKINNY_MAX_ROWS + 1 on.
# Off: the library is ahead at every row count (OPT-1.3B decode step at batch 16 / 64: 1.42 / 2.33 ms against 1.77 /
# 2.93 with this kernel; per layer 34 against 44 microseconds at 16 tokens, 35 against 54 at 64).
STREAM_TC_MAX_ROWS = 0


def stream_tc_applies(n_rows: int, w: torch.Tensor) -> bool:
    """Whether ``linear`` / ``linear_parts`` give a product of n_rows tokens with w [out, in] to the tcgen05
    weight-streaming kernel: bfloat16 on the device, more tokens than the mma.sync kernel serves, an inner dimension
    that is a multiple of 64, and few enough features for one block per SM (the output head is not)."""
    return (w.is_cuda and w.dtype == torch.bfloat16 and SKINNY_MAX_ROWS < n_rows <= min(STREAM_TC_MAX_ROWS, 128)
            and w.shape[1] % 64 == 0 and bool(lib().st_gemm_stream_tc_one_wave(w.shape[0])))


def gemm_stream_tc(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
                   out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """act(a @ w.T + bias) for at most 128 rows of bfloat16 ``a`` on tcgen05 fed by TMA; w is [out, in] with
    in % 64 == 0.  A wait that expires inside the kernel shows in ``kernel_status``."""
    out_dtype = out_dtype or a.dtype
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_stream_tc is a bfloat16 kernel")
    a = a.contiguous()
    assert w.is_contiguous()
    n, k = a.shape
    m = w.shape[0]
    out = torch.empty((n, m), dtype=out_dtype, device=a.device)
    _check(lib().st_gemm_stream_tc(_p(a), _p(w), _p(bias), _p(out), n, m, k, ACT_CODES[act],
                                   int(out_dtype == torch.float32), _p(_tc_status_word(a.device)), _stream()),
           "gemm_stream_tc")
    return out


def kernel_status(device: torch.device) -> int:
    """The status word of kernels that have no step context to report to (0: fine; 5: the tcgen05 product
    gave up waiting); reading it synchronises and clears it."""
    word = _tc_status_word(torch.device(device))
    code = int(word.item())
    if code:
        word.zero_()
    return code


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """act(a @ w.T + bias) for at most SKINNY_KERNEL_MAX_ROWS rows of bfloat16 ``a``; w is [out, in] with in % 8 == 0."""
    out_dtype = out_dtype or a.dtype
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny is a bfloat16 kernel")
    a = a.contiguous()
    assert w.is_contiguous()
    n, k = a.shape
    m = w.shape[0]
    out = torch.empty((n, m), dtype=out_dtype, device=a.device)
    _check(lib().st_gemm_skinny(_p(a), _p(w), _p(bias), _p(out), n, m, k, ACT_CODES[act],
                                int(out_dtype == torch.float32), _stream()), "gemm_skinny")
    return out


# ---- the same products with their neighbours fused (steps of a few tokens) ----
# The residual sum behind a product (out[m, n] += ..., in float, in the product's epilogue) is used: a decode
# step gains 4 %.  The norm in front of a product (five kernels per pre-norm layer instead of seven) is built
# and tested but off: measured in the recorded step it loses, at batch 8 by 10 %, because the small norm
# kernel between two products is what lets the second product start all at once on an idle GPU with its
# first loads already under way.  With a switch off, the operation runs as
# the separate kernels it replaces.
FUSED_MAX_ROWS = 8
FUSE_NORM = False
FUSE_RESIDUAL = True
LINEAR_PARTS = True       # a product cut over k leaves its slices' sums for the next norm kernel (decode steps)
UNCUT_MAX_INNER = 2048    # up to this inner dimension ``linear_add`` runs uncut with its weights on chip: no parts


def fused_norm_applies(n_rows: int, k: int, w: torch.Tensor) -> bool:
    """Whether ``norm_linear`` / ``norm_qkv_linear_to_cache`` / ``linear_add`` take a step of n_rows tokens
    with inner dimension k and weights w."""
    return (w.is_cuda and w.dtype == torch.bfloat16 and 1 <= n_rows <= min(FUSED_MAX_ROWS, SKINNY_MAX_ROWS)
            and bool(lib().st_gemm_skinny_norm_applies(n_rows, k)))


def norm_linear(x: torch.Tensor, kind: str, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor], eps: float,
                w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
                out_dtype: Optional[torch.dtype] = None, delta: Optional[torch.Tensor] = None,
                delta_bias: Optional[torch.Tensor] = None, parts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(norm(x) @ w.T + bias) for at most FUSED_MAX_ROWS float32 rows x (the residual stream) and bfloat16
    w [out, in]: the norm of ``add_norm`` (statistics in float, two passes; its result rounded to bfloat16 as
    ``add_norm`` stores it) in front of the weight-streaming product, in one kernel.  ``delta`` / ``delta_bias`` /
    ``parts``: what is still to be added to x (``add_norm`` adds it, x is updated); only with FUSE_NORM off."""
    assert x.dtype == torch.float32 and x.is_contiguous() and w.is_contiguous() and x.shape[1] == w.shape[1]
    n, k = x.shape
    m = w.shape[0]
    out_dtype = out_dtype or w.dtype
    pending = delta is not None or delta_bias is not None or parts is not None
    assert not (FUSE_NORM and pending)
    if not FUSE_NORM:
        h = torch.empty((n, k), dtype=w.dtype, device=x.device)
        add_norm(x, delta=delta, delta_bias=delta_bias, parts=parts, resid_out=x if pending else None, gamma=gamma,
                 beta=beta, eps=eps, kind=kind, out_act=h)
        return gemm_skinny(h, w, bias, act, out_dtype)
    out = torch.empty((n, m), dtype=out_dtype, device=x.device)
    _check(lib().st_gemm_skinny_norm(_p(x), _p(gamma), _p(beta), _f(eps), NORM_CODES[kind], _p(w), _p(bias), _p(out),
                                     n, m, k, ACT_CODES[act], int(out_dtype == torch.float32), _stream()),
           "norm_linear")
    return out


def linear_add(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], x: torch.Tensor) -> None:
    """x += a @ w.T + bias in place, for at most FUSED_MAX_ROWS bfloat16 rows a and float32 x (the residual
    stream): the residual sum behind the weight-streaming product, in float, in one kernel."""
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dtype == torch.float32
    assert a.is_contiguous() and w.is_contiguous() and x.is_contiguous()
    assert a.shape[1] == w.shape[1] and x.shape == (a.shape[0], w.shape[0])
    if not FUSE_RESIDUAL:
        add_norm(x, delta=gemm_skinny(a, w), delta_bias=bias, resid_out=x, kind="none", act_dtype=a.dtype)
        return
    _check(lib().st_gemm_skinny_add(_p(a), _p(w), _p(bias), _p(x), a.shape[0], w.shape[0], a.shape[1], _stream()),
           "linear_add")


_parts_scratch = {}


def linear_parts_slices(n_rows: int, w: torch.Tensor) -> int:
    """Into how many slices of k ``linear_parts`` cuts a product with w [out, in] for n_rows tokens (1: it does not
    apply: more than FUSED_MAX_ROWS tokens, weights that are not bfloat16 on the device, an inner dimension that is
    no multiple of 32, or a product that is not cut)."""
    if not (LINEAR_PARTS and w.is_cuda and w.dtype == torch.bfloat16 and n_rows >= 1):
        return 1
    if n_rows <= FUSED_MAX_ROWS:
        return int(lib().st_gemm_skinny_parts_slices(w.shape[0], w.shape[1]))
    if stream_tc_applies(n_rows, w):
        return int(lib().st_gemm_stream_tc_slices(w.shape[0], w.shape[1]))
    return 1


def linear_parts(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """The slices' sums of a @ w.T for bfloat16 rows (as many as ``linear_parts_slices`` answers for with more than
    one slice): float32 [slices, rows, out], to be added in slice order (``add_norm(parts=...)`` does, in the kernel
    that reads the residual rows anyway).  Up to FUSED_MAX_ROWS rows the mma.sync kernel, beyond it the tcgen05
    kernel.  The result lives in a buffer that the next call for the same sizes overwrites."""
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous()
    assert a.shape[1] == w.shape[1]
    n, m = a.shape[0], w.shape[0]
    slices = linear_parts_slices(n, w)
    cap = FUSED_MAX_ROWS if n <= FUSED_MAX_ROWS else 128
    key = (a.device.index, slices, m, cap)
    if key not in _parts_scratch:
        _parts_scratch[key] = torch.zeros(slices * cap * m, dtype=torch.float32, device=a.device)
    parts = _parts_scratch[key][:slices * n * m].view(slices, n, m)
    if n <= FUSED_MAX_ROWS:
        _check(lib().st_gemm_skinny_parts(_p(a), _p(w), _p(parts), n, m, a.shape[1], _stream()), "linear_parts")
    else:
        _check(lib().st_gemm_stream_tc_parts(_p(a), _p(w), _p(parts), n, m, a.shape[1],
                                             _p(_tc_status_word(a.device)), _stream()), "linear_parts")
    return parts


def norm_qkv_linear_to_cache(x: torch.Tensor, kind: str, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor],
                             eps: float, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                             pool: torch.Tensor, layer: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                             slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int, d: int,
                             status: torch.Tensor, write_kv: bool = True, delta: Optional[torch.Tensor] = None,
                             delta_bias: Optional[torch.Tensor] = None, parts: Optional[torch.Tensor] = None) -> None:
    """``qkv_linear_to_cache`` of norm(x) for float32 rows x: norm, product, bias and cache write in one kernel.
    ``delta`` / ``delta_bias`` / ``parts``: as in ``norm_linear``."""
    assert x.dtype == torch.float32 and x.is_contiguous() and w.is_contiguous() and pool.dtype == torch.bfloat16
    num_pages, n_layers, _, pnkv, page_size, pd = pool.shape
    assert pnkv == nkv and pd == d and w.shape[0] == (nh + 2 * nkv) * d
    pending = delta is not None or delta_bias is not None or parts is not None
    assert not (FUSE_NORM and pending)
    if not FUSE_NORM:
        h = torch.empty(x.shape, dtype=w.dtype, device=x.device)
        add_norm(x, delta=delta, delta_bias=delta_bias, parts=parts, resid_out=x if pending else None, gamma=gamma,
                 beta=beta, eps=eps, kind=kind, out_act=h)
        return qkv_linear_to_cache(h, w, bias, q_out, pool, layer, positions, seq_of_token, slots, block_table, nh, nkv,
                                   d, status, write_kv)
    _check(lib().st_gemm_skinny_norm_qkv(_p(x), _p(gamma), _p(beta), _f(eps), NORM_CODES[kind], _p(w), _p(bias),
                                         _p(q_out), _p(pool), _p(positions), _p(seq_of_token), _p(slots),
                                         _p(block_table), block_table.shape[1], num_pages, n_layers, layer,
                                         x.shape[0], x.shape[1], nh, nkv, d, page_size, int(write_kv), _p(status),
                                         _stream()), "norm_qkv_linear_to_cache")


def qkv_linear_to_cache(h: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                        pool: torch.Tensor, layer: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                        slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int, d: int,
                        status: torch.Tensor, write_kv: bool = True) -> None:
    """The fused form of ``linear`` + ``qkv_to_cache`` for at most SKINNY_KERNEL_MAX_ROWS bfloat16 tokens:
    q_out = (h @ w.T + bias)[:, :nh*d]; the k and v parts go straight into the paged cache."""
    if h.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16:
        raise KernelError("qkv_linear_to_cache is a bfloat16 kernel")
    num_pages, n_layers, _, pnkv, page_size, pd = pool.shape
    assert pnkv == nkv and pd == d and w.shape[0] == (nh + 2 * nkv) * d and h.is_contiguous() and w.is_contiguous()
    _check(lib().st_gemm_skinny_qkv(_p(h), _p(w), _p(bias), _p(q_out), _p(pool), _p(positions), _p(seq_of_token),
                                    _p(slots), _p(block_table), block_table.shape[1], num_pages, n_layers, layer,
                                    h.shape[0], h.shape[1], nh, nkv, d, page_size, int(write_kv), _p(status),
                                    _stream()), "qkv_linear_to_cache")


def gemm_plain(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
               out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """The plain kernel for either storage type (float arithmetic, fixed summation order)."""
    out_dtype = out_dtype or a.dtype
    a = a.contiguous()
    assert w.is_contiguous()
    n, k = a.shape
    m = w.shape[0]
    out = torch.empty((n, m), dtype=out_dtype, device=a.device)
    _check(lib().st_gemm_plain(_p(a), _p(w), _p(bias), _p(out), n, m, k, ACT_CODES[act], _dt(a),
                               int(out_dtype == torch.float32), _stream()), "gemm_plain")
    return out


# ------------------------------------------------------------------ attention
def qkv_to_cache(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_out: Optional[torch.Tensor], pool: torch.Tensor,
                 layer: int, positions: torch.Tensor, seq_of_token: torch.Tensor, slots: torch.Tensor,
                 block_table: torch.Tensor, nh: int, nkv: int, d: int, status: torch.Tensor,
                 write_kv: bool = True) -> None:
    """q_out = q + bias; pool[page, layer, 0/1, head, pos % page, :] = k/v + bias.  ``q_out`` None: the queries
    stay where they are (in ``qkv``), only keys and values move.

    pool: [pages, layers, 2, nkv, page_size, d]; block_table: [slots, max_pages] int32."""
    n = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * d and pool.dtype == qkv.dtype
    num_pages, n_layers, _, pnkv, page_size, pd = pool.shape
    assert pnkv == nkv and pd == d
    _check(lib().st_qkv_to_cache(_p(qkv), _p(bias), _p(q_out), _p(pool), _p(positions), _p(seq_of_token),
                                 _p(slots), _p(block_table), block_table.shape[1], num_pages, n_layers, layer,
                                 n, nh, nkv, d, page_size, int(write_kv), _p(status), _dt(qkv), _stream()),
           "qkv_to_cache")


def attention_plain(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, positions: torch.Tensor,
                    seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int,
                    scale: float, window: int = 0, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Paged causal attention, one block per (token, head), float arithmetic, any sizes.  ``status`` (as for
    the other attention kernels) is set to 1 when a key a query needs has no page in the block table."""
    n = q.shape[0]
    _, n_layers, _, nkv, page_size, d = pool.shape
    _check(lib().st_attention_plain(_p(q), _p(pool), _p(out), _p(positions), _p(seq_of_token), _p(slots),
                                    _p(block_table), block_table.shape[1], n_layers, layer, n, nh, nkv, d,
                                    page_size, _f(scale), window, _dt(q), _p(status), _stream()), "attention_plain")
    return out


_DECODE_COUNTERS = 1 << 16
DECODE_MMA_MIN_BLOCKS = 2048     # (token, kv head) pairs from which the tensor-core decode attention serves head sizes above 64
_decode_counter_buffers = {}


def _decode_counters(device: torch.device) -> torch.Tensor:
    """Per-device arrival counters of the split decode attention (zero between launches)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _decode_counter_buffers:
        _decode_counter_buffers[key] = torch.zeros(_DECODE_COUNTERS, dtype=torch.int32, device=device)
    return _decode_counter_buffers[key]


def attention_decode_scratch(n_items: int, nh: int, d: int, n_splits: int) -> int:
    return int(lib().st_attention_decode_scratch_floats(n_items, nh, d, n_splits))


def attention_decode(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor,
                     items: Optional[torch.Tensor], n_items: int, positions: torch.Tensor,
                     seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int,
                     scale: float, window: int = 0, n_splits: int = 1,
                     partial: Optional[torch.Tensor] = None, fused_merge: bool = True,
                     kernel: str = "auto", warps: int = 4, status: Optional[torch.Tensor] = None,
                     start_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bfloat16 paged attention for single query tokens; ``items`` lists the token indices it serves
    (None: tokens 0..n_items-1).  A token whose position is negative is skipped.

    kernel: "mma" = the tensor-core kernel (head sizes that are multiples of 16 up to 128; with several
    splits it needs the fused merge), "lanes" = the kernel with eight lanes per key (multiples of 8 up to
    256), "auto" = the first that applies.  warps: warps per block of the tensor-core kernel, 4 or 8 (8 pays
    for few and long blocks with head sizes up to 64, see decode_warps).  start_pos: per request of the step, the
    tokens it had in the cache before the step: the tensor-core kernel starts copying those keys before the
    kernel that writes this step's keys has finished (None: it waits first)."""
    _, n_layers, _, nkv, page_size, d = pool.shape
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_decode is a bfloat16 kernel")
    if n_splits > 1:
        need = attention_decode_scratch(n_items, nh, d, n_splits)
        if partial is None or partial.numel() < need or partial.dtype != torch.float32:
            raise KernelError(f"attention_decode: needs {need} floats of scratch for {n_splits} splits")
    counters = _decode_counters(q.device) if (n_splits > 1 and fused_merge
                                              and n_items * nh <= _DECODE_COUNTERS) else None
    mma_ok = bool(lib().st_attention_decode_mma_applies(d)) and (n_splits == 1 or counters is not None)
    if kernel == "auto":
        # Head sizes up to 64: the tensor-core kernel; beyond, it holds fewer blocks per SM than the lanes
        # kernel and pays only for many blocks; grouped queries always gain from it (the group shares one
        # read of the keys and values).
        # (OPT-6.7B decode step, tensor-core / lanes kernel, ms: batch 1 2.98 / 3.08, batch 8 3.68 / 3.70, batch 16
        # 3.88 / 3.76, batch 64 the tensor-core kernel either way: it also serves launches of up to two blocks per SM)
        busy = n_items * nkv >= DECODE_MMA_MIN_BLOCKS
        few = n_items * nkv * n_splits <= 2 * sm_count(q.device)
        kernel = "mma" if mma_ok and (d <= 64 or nh != nkv or busy or few) else "lanes"
    if kernel == "mma":
        if not mma_ok:
            raise KernelError("attention_decode: the tensor-core kernel takes head sizes that are multiples of "
                              "16 up to 128 and merges its splits itself")
        _check(lib().st_attention_decode_mma(_p(q), _p(pool), _p(out), _p(partial), _p(items), n_items,
                                             _p(positions), _p(seq_of_token), _p(slots), _p(start_pos),
                                             _p(block_table), block_table.shape[1], n_layers, layer, nh, nkv, d,
                                             page_size, _f(scale), window, n_splits, _p(counters),
                                             warps if d <= 64 else 4,
                                             _p(status), _stream()), "attention_decode_mma")
    elif kernel == "lanes":
        _check(lib().st_attention_decode(_p(q), _p(pool), _p(out), _p(partial), _p(items), n_items, _p(positions),
                                         _p(seq_of_token), _p(slots), _p(block_table), block_table.shape[1],
                                         n_layers, layer, nh, nkv, d, page_size, _f(scale), window, n_splits,
                                         _p(counters), _p(status), _stream()), "attention_decode")
    else:
        raise KernelError(f"attention_decode: no kernel named {kernel!r}")
    return out


# Decode steps of more tokens than the weight-streaming product serves: the attention kernel works from the library's
# q|k|v product and writes the cache itself (False: a cache-write kernel between the two, for measurements).
DECODE_FROM_PROJECTION = True


def attention_decode_qkv_applies(qkv: torch.Tensor, pool: torch.Tensor, n_items: int, nh: int, n_splits: int) -> bool:
    """Whether ``attention_decode_qkv`` takes this step: bfloat16 on the device, a head size the tensor-core kernel
    takes, and (with several splits) few enough (token, head) pairs for its arrival counters."""
    d = pool.shape[-1]
    return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16
            and bool(lib().st_attention_decode_mma_applies(d)) and (n_splits == 1 or n_items * nh <= _DECODE_COUNTERS))


def attention_decode_qkv(qkv: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, items: Optional[torch.Tensor], n_items: int, positions: torch.Tensor,
                         seq_of_token: torch.Tensor, slots: torch.Tensor, start_pos: torch.Tensor,
                         block_table: torch.Tensor, nh: int, scale: float, window: int = 0, n_splits: int = 1,
                         partial: Optional[torch.Tensor] = None, warps: int = 4, write_kv: bool = True,
                         status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Single-token attention straight from the fused projection: ``qkv`` [tokens, (nh + 2 nkv) d] holds the q, k and
    v features of ALL the step's tokens as the product left them (bias included), every token of the step is an item,
    and ``start_pos`` says where each request's tokens of this step begin.  The kernel writes each token's key and
    value into its page (``write_kv``) and attends over the cache and the step's own rows: the step needs no
    cache-write kernel.  Only for steps in which no other kernel reads this step's keys from the cache (no prompt
    tiles)."""
    _, n_layers, _, nkv, page_size, d = pool.shape
    if not attention_decode_qkv_applies(qkv, pool, n_items, nh, n_splits):
        raise KernelError("attention_decode_qkv: bfloat16, head sizes that are multiples of 16 up to 128")
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * d and out.shape == (qkv.shape[0], nh * d)
    counters = None
    if n_splits > 1:
        need = attention_decode_scratch(n_items, nh, d, n_splits)
        if partial is None or partial.numel() < need or partial.dtype != torch.float32:
            raise KernelError(f"attention_decode_qkv: needs {need} floats of scratch for {n_splits} splits")
        counters = _decode_counters(qkv.device)
    _check(lib().st_attention_decode_mma_qkv(_p(qkv), _p(pool), _p(out), _p(partial), _p(items), n_items,
                                             _p(positions), _p(seq_of_token), _p(slots), _p(start_pos),
                                             _p(block_table), block_table.shape[1], pool.shape[0], n_layers, layer,
                                             nh, nkv, d, page_size, _f(scale), window, n_splits, _p(counters),
                                             warps if d <= 64 else 4, int(write_kv), _p(status), _stream()),
           "attention_decode_qkv")
    return out


def decode_warps(n_items: int, nkv: int, d: int, n_splits: int, max_kv: int) -> int:
    """Warps per block for the tensor-core decode attention.  Eight when the launch is at most two blocks per
    SM and the key ranges are long: a warp's chain of groups is then half as long; with many blocks four are
    better (OPT-1.3B decode steps, eight against four warps: batch 8 1.256 / 1.299 ms, batch 64 2.61 / 2.46)."""
    return 8 if (d <= 64 and n_items * nkv * n_splits <= 2 * sm_count() and max_kv >= 256) else 4


# "auto", or the name of one prompt-attention kernel for every call that says "auto" (measurements)
PREFILL_KERNEL = "auto"


def attention_prefill_tile_rows() -> int:
    return int(lib().st_attention_prefill_tile_rows())


def attention_prefill(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, tiles: torch.Tensor,
                      n_tiles: int, q_start: torch.Tensor, start_pos: torch.Tensor, slots: torch.Tensor,
                      block_table: torch.Tensor, nh: int, scale: float, window: int = 0,
                      status: Optional[torch.Tensor] = None, kernel: str = "auto", q_stride: int = 0) -> torch.Tensor:
    """bfloat16 tensor-core paged attention over tiles of 128 query tokens; tiles: int32 [n_tiles, 2] =
    (request index in the step, offset of the tile among the request's new tokens).  ``q_stride``: elements
    between the query rows of consecutive tokens when ``q`` is part of a wider tensor (the q|k|v product), 0 for
    a dense [tokens, nh * d] tensor.

    kernel: "tmap" = the persistent tcgen05 kernel fed by TMA (head size 64, pages of 8 to 64 positions: one block
    per SM walks through the (tile, head) pairs), "tma" = the same with one block per pair (head sizes 64 and 128;
    "tma3" = the same with three softmax warpgroups per block instead of two, at head size 64 only),
    "tc" = the tcgen05 kernel fed by asynchronous copies (head sizes up to 128), "mma" = the mma.sync
    kernel (up to 256), "auto" = the first of these that applies.  ``status`` receives 3 if a tcgen05
    kernel gave up waiting, and 1 from any of them when a key a query needs has no page in the block table."""
    n_pages, n_layers, _, nkv, page_size, d = pool.shape
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill is a bfloat16 kernel")
    if kernel == "auto":
        kernel = PREFILL_KERNEL
    if kernel == "auto":
        if lib().st_attention_prefill_tmap_applies(d, page_size):
            kernel = "tmap"
        elif lib().st_attention_prefill_tma_applies(d, page_size):
            kernel = "tma"
        else:
            kernel = "tc" if d <= 128 else "mma"
    if kernel == "tmap":
        st = status if status is not None else _tc_status_word(q.device)
        _check(lib().st_attention_prefill_tmap(_p(q), _p(pool), ctypes.c_longlong(n_pages), _p(out), _p(tiles),
                                               n_tiles, _p(q_start), _p(start_pos), _p(slots), _p(block_table),
                                               block_table.shape[1], n_layers, layer, nh, nkv, d, page_size,
                                               _f(scale), window, q_stride, _p(st), _stream()), "attention_prefill_tmap")
        return out
    if kernel in ("tma", "tma3"):
        st = status if status is not None else _tc_status_word(q.device)
        lib().st_attention_prefill_tma_warpgroups(3 if kernel == "tma3" else 2)
        _check(lib().st_attention_prefill_tma(_p(q), _p(pool), ctypes.c_longlong(n_pages), _p(out), _p(tiles),
                                              n_tiles, _p(q_start), _p(start_pos), _p(slots), _p(block_table),
                                              block_table.shape[1], n_layers, layer, nh, nkv, d, page_size,
                                              _f(scale), window, q_stride, _p(st), _stream()), "attention_prefill_tma")
        return out
    if kernel == "tc":
        st = status if status is not None else _tc_status_word(q.device)
        _check(lib().st_attention_prefill_tc(_p(q), _p(pool), _p(out), _p(tiles), n_tiles, _p(q_start),
                                             _p(start_pos), _p(slots), _p(block_table), block_table.shape[1],
                                             n_layers, layer, nh, nkv, d, page_size, _f(scale), window, q_stride,
                                             _p(st), _stream()), "attention_prefill_tc")
        return out
    if kernel != "mma":
        raise KernelError(f"attention_prefill: no kernel named {kernel!r}")
    _check(lib().st_attention_prefill(_p(q), _p(pool), _p(out), _p(tiles), n_tiles, _p(q_start), _p(start_pos),
                                      _p(slots), _p(block_table), block_table.shape[1], n_layers, layer, nh, nkv,
                                      d, page_size, _f(scale), window, q_stride, _p(status), _stream()),
           "attention_prefill")
    return out


# ------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Lowest index of the largest value of each row of float32 logits -> int32 [rows]."""
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    n, v = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(lib().st_argmax(_p(logits), n, v, _p(out), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperatures: torch.Tensor, top_k: torch.Tensor, seeds: torch.Tensor,
           counters: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row r: temperature <= 0 -> greedy; else draw from softmax(logits/temperature) restricted to the
    top_k[r] largest (<= 0: all) with the uniform number ``uniform(seeds[r], counters[r])``."""
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    assert temperatures.dtype == torch.float32 and top_k.dtype == torch.int32
    assert seeds.dtype == torch.int64 and counters.dtype == torch.int64
    n, v = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(lib().st_sample(_p(logits), n, v, _p(temperatures), _p(top_k), _p(seeds), _p(counters), _p(out),
                           _stream()), "sample")
    return out


def uniform(seed: int, counter: int) -> float:
    """The uniform number in [0,1) that `sample` uses for (seed, counter); computed on the host."""
    return float(lib().st_uniform_host(seed, counter))
