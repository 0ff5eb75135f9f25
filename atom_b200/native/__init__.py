"""ctypes binding of the sm_100a kernel library.

``lib()`` builds the library on first use (see ``build.py``) and loads it; every kernel
wrapper below takes torch tensors, passes raw device pointers and the current stream, and
raises if the kernel refuses its arguments.  There is no fallback: without the library the
product path does not run.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

from .build import NativeBuildError, build, build_variant

F32, BF16 = 0, 1
_ERR = {1: "argument the kernel does not take", 2: "CUDA launch failed", 3: "library call failed"}

_lib = None
_lock = threading.Lock()
launches = 0        # launches of this library's own kernels made by this process
library_gemms = 0   # calls into the vendor GEMM library (counted apart from own kernels)


class NativeError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise NativeError(f"kernels take float32 or bfloat16, not {dt}")


def lib():
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = build()
                try:
                    _lib = ctypes.CDLL(path)
                except OSError as e:  # pragma: no cover
                    raise NativeBuildError(f"cannot load {path}: {e}") from e
                _declare(_lib)
    return _lib


def lib_path() -> str:
    return build(verbose=False)


_vp, _i, _i64, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t

_SIGNATURES = {
    "atom_embedding": [_vp, _vp, _i, _vp, _i, _i, _i, _vp],
    "atom_add_rmsnorm": [_vp, _i, _vp, _vp, _vp, _i, _f, _vp, _i, _i, _vp],
    "atom_rmsnorm": [_vp, _vp, _i, _vp, _i, _f, _i, _i, _vp],
    "atom_silu_mul": [_vp, _vp, _i, _i, _i, _vp],
    "atom_qknorm_rope_kvwrite": [_vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _f, _vp, _i, _i, _vp, _vp,
                                 _vp, _i, _i, _vp, _vp, _i64, _vp, _vp],
    "atom_qk_headnorm": [_vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _f, _vp, _vp],
    "atom_paged_attention_generic": [_vp, _vp, _i64, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i,
                                     _i, _i, _f, _i, _vp],
    "atom_gemm_f32": [_vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i64, _vp],
    "atom_gemm_bf16": [_vp, _i, _vp, _vp, _i, _i, _i, _i64, _vp, _sz, _vp],
    "atom_add_bias": [_vp, _i, _vp, _i, _i, _i, _vp],
    "atom_gemm_rows": [_vp, _i, _vp, _vp],
    "atom_gemm_rows_grid": [],
    "atom_gemm_rows_supports": [_i, _i, _i, _i64],
    "atom_gemm_pairs": [_vp, _i64, _vp, _vp, _i64, _i, _i, _i, _i, _vp, _vp],
    "atom_gemm_pairs_resident": [],
    "atom_gemm_pairs_supports": [_i, _i, _i, _i64, _i64],
    "atom_set_option": [_i, _i],
    "atom_copy_rows_h2d": [_vp, _i64, _vp, _i64, _i64, _i64, _vp],
}


def _declare(l) -> None:
    for name, args in _SIGNATURES.items():
        if not hasattr(l, name):
            continue  # optional kernels are declared by the module that owns them
        fn = getattr(l, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int64 if name.endswith("_bytes") else ctypes.c_int


def declare(name: str, args) -> None:
    """Declares the signature of one more exported function (used by kernel modules)."""
    _SIGNATURES[name] = args
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int


# Choices the launch code otherwise makes by itself (csrc/common.cuh, ATOM_OPT_*): for measurements
# and for tests of both sides of a choice.  They hold for launches made after the call; a captured
# graph keeps what it was recorded with.
OPTIONS = {"pdl": 0, "decode_tma": 1, "decode_ktw": 2}
_option_values = {}


def set_option(name: str, value: int) -> None:
    """Sets an option in every loaded library of the package (and in those loaded later)."""
    key = OPTIONS[name]
    _option_values[key] = int(value)
    if lib().atom_set_option(key, int(value)) != 0:
        raise NativeError(f"option {name!r} was refused")
    for l in _flash_libs.values():
        l.atom_flash_set_option(key, int(value))


def reset_options() -> None:
    for name, default in (("pdl", 1), ("decode_tma", 1), ("decode_ktw", 0)):
        set_option(name, default)
    _option_values.clear()


def copy_rows_h2d(dst: torch.Tensor, dst_pitch: int, src: torch.Tensor, src_pitch: int, row_elems: int,
                  rows: int) -> None:
    """rows x row_elems elements from pinned host memory (rows src_pitch elements apart) to the device
    (rows dst_pitch elements apart), asynchronously on the current stream."""
    es = dst.element_size()
    assert dst.is_cuda and not src.is_cuda and src.element_size() == es     # (src: pinned memory)
    assert rows == 0 or (dst.numel() >= (rows - 1) * dst_pitch + row_elems and src.numel() >= (rows - 1) * src_pitch + row_elems)
    code = lib().atom_copy_rows_h2d(dst.data_ptr(), dst_pitch * es, src.data_ptr(), src_pitch * es, row_elems * es,
                                    rows, _stream())
    if code != 0:
        raise NativeError(f"copy_rows_h2d: {_ERR.get(code, code)}")


def _check(code: int, name: str, own: bool = True) -> None:
    global launches, library_gemms
    if own:
        launches += 1
    else:
        library_gemms += 1
    if code != 0:
        raise NativeError(f"{name}: {_ERR.get(code, f'error {code}')}")


def add_launches(n: int) -> None:
    """Counts kernels that ran without passing through the wrappers (a replayed CUDA graph)."""
    global launches
    launches += n


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of the current CUDA stream of the current device (the raw query is an order of
    magnitude cheaper than building a torch.cuda.Stream object for every launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NativeError("kernels take CUDA tensors only (there is no CPU path)")


# --------------------------------------------------------------------------- wrappers


def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
    """out[t] = table[ids[t]] widened to float32.  out [T,H] f32, table [V,H], ids [T] i32."""
    _cuda(out, table, ids)
    T, H = out.shape
    assert out.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == H
    assert out.is_contiguous() and table.is_contiguous() and ids.numel() >= T
    _check(lib().atom_embedding(out.data_ptr(), table.data_ptr(), dtype_code(table.dtype),
                                ids.data_ptr(), T, H, table.shape[0], _stream()), "embedding")


def add_rmsnorm(out: torch.Tensor, residual: torch.Tensor, delta: Optional[torch.Tensor],
                weight: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None) -> None:
    """residual (+= delta); out = rmsnorm(residual) * weight.  With ``rows`` (int32 indices)
    only those rows are normalised, written densely to ``out``, and residual is left as is."""
    _cuda(out, residual, delta, weight, rows)
    H = residual.shape[-1]
    assert residual.dtype == torch.float32 and residual.is_contiguous() and out.is_contiguous()
    assert weight.numel() == H and (delta is None or (delta.dtype == out.dtype and delta.is_contiguous()))
    n = (rows.numel() if n_rows is None else n_rows) if rows is not None else residual.shape[0]
    assert out.shape[0] >= n and out.shape[-1] == H
    _check(lib().atom_add_rmsnorm(out.data_ptr(), dtype_code(out.dtype), residual.data_ptr(),
                                  _ptr(delta), weight.data_ptr(), dtype_code(weight.dtype),
                                  float(eps), _ptr(rows), n, H, _stream()), "add_rmsnorm")


def rmsnorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    _cuda(out, x, weight)
    H = x.shape[-1]
    assert x.is_contiguous() and out.is_contiguous() and out.dtype == x.dtype and weight.numel() == H
    _check(lib().atom_rmsnorm(out.data_ptr(), x.data_ptr(), dtype_code(x.dtype), weight.data_ptr(),
                              dtype_code(weight.dtype), float(eps), x.numel() // H, H, _stream()),
           "rmsnorm")


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _cuda(out, gate_up)
    T, I2 = gate_up.shape
    assert I2 % 2 == 0 and out.shape == (T, I2 // 2) and out.dtype == gate_up.dtype
    assert out.is_contiguous() and gate_up.is_contiguous()
    _check(lib().atom_silu_mul(out.data_ptr(), gate_up.data_ptr(), dtype_code(out.dtype), T, I2 // 2,
                               _stream()), "silu_mul")


def qknorm_rope_kvwrite(qkv: torch.Tensor, nh: int, nkv: int, hd: int,
                        q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                        eps: float, cos_sin: Optional[torch.Tensor], rotary_dim: int,
                        positions: torch.Tensor, seq_of_token: torch.Tensor,
                        block_table: torch.Tensor, page_size: int,
                        k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                        status: torch.Tensor) -> None:
    """Per-head q/k norm, rotation and cache write for the packed [T, (nh+2nkv)*hd] projection."""
    _cuda(qkv, q_weight, k_weight, cos_sin, positions, seq_of_token, block_table, k_pages, v_pages, status)
    T = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * hd
    assert (q_weight is None) == (k_weight is None)
    wd = dtype_code(q_weight.dtype) if q_weight is not None else F32
    if q_weight is not None:
        assert k_weight.dtype == q_weight.dtype and q_weight.numel() == hd and k_weight.numel() == hd
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] == rotary_dim
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    num_pages = 0
    if k_pages is not None:
        assert k_pages.dtype == qkv.dtype and k_pages.is_contiguous() and v_pages.is_contiguous()
        assert tuple(k_pages.shape[1:]) == (nkv, page_size, hd) and v_pages.shape == k_pages.shape
        num_pages = k_pages.shape[0]
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
    assert positions.dtype == torch.int32 and seq_of_token.dtype == torch.int32
    assert status.dtype == torch.int32
    _check(lib().atom_qknorm_rope_kvwrite(
        qkv.data_ptr(), dtype_code(qkv.dtype), T, nh, nkv, hd, _ptr(q_weight), _ptr(k_weight), wd,
        float(eps), _ptr(cos_sin), rotary_dim, max_pos, positions.data_ptr(), seq_of_token.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], page_size, _ptr(k_pages), _ptr(v_pages),
        num_pages, status.data_ptr(), _stream()), "qknorm_rope_kvwrite")


def qk_headnorm(qkv: torch.Tensor, nh: int, nkv: int, hd: int, q_weight: torch.Tensor, k_weight: torch.Tensor,
                eps: float, seq_of_token: torch.Tensor) -> None:
    """Per-head RMSNorm of the q and k heads of the packed [T, (nh+2nkv)*hd] projection, in place."""
    _cuda(qkv, q_weight, k_weight, seq_of_token)
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * hd
    assert k_weight.dtype == q_weight.dtype and q_weight.numel() == hd and k_weight.numel() == hd
    _check(lib().atom_qk_headnorm(qkv.data_ptr(), dtype_code(qkv.dtype), qkv.shape[0], nh, nkv, hd,
                                  q_weight.data_ptr(), k_weight.data_ptr(), dtype_code(q_weight.dtype), float(eps),
                                  seq_of_token.data_ptr(), _stream()), "qk_headnorm")


def paged_attention_generic(out: torch.Tensor, q: torch.Tensor, q_stride: int,
                            k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                            positions: torch.Tensor, seq_of_token: torch.Tensor, T: int, nh: int,
                            nkv: int, hd: int, scale: float, window: int) -> None:
    """out[T, nh*hd]: causal attention of every token over its request's pages (any sizes)."""
    _cuda(out, q, k_pages, v_pages, block_table, positions, seq_of_token)
    page_size = k_pages.shape[2]
    assert out.is_contiguous() and out.dtype == q.dtype == k_pages.dtype
    assert tuple(k_pages.shape[1:]) == (nkv, page_size, hd) and k_pages.is_contiguous() and v_pages.is_contiguous()
    _check(lib().atom_paged_attention_generic(
        out.data_ptr(), q.data_ptr(), q_stride, dtype_code(q.dtype), k_pages.data_ptr(),
        v_pages.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size,
        positions.data_ptr(), seq_of_token.data_ptr(), T, nh, nkv, hd, float(scale), int(window),
        _stream()), "paged_attention_generic")


def gemm_f32(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T (+ bias) in true 32-bit arithmetic."""
    _cuda(out, a, w, bias)
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == w.dtype == out.dtype == torch.float32 and w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous()
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == N)
    _check(lib().atom_gemm_f32(out.data_ptr(), a.data_ptr(), w.data_ptr(), _ptr(bias), M, N, K,
                               a.stride(0), out.stride(0), _stream()), "gemm_f32")


_workspaces = {}


def _workspace(device: torch.device) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.empty(32 << 20, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def gemm_bf16(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """out[M,N] (bf16 or f32) = a[M,K] @ w[N,K]^T, bf16 operands, 32-bit accumulation (cuBLAS)."""
    _cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == w.dtype == torch.bfloat16 and w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and out.is_contiguous() and w.is_contiguous()
    ws = _workspace(out.device)
    _check(lib().atom_gemm_bf16(out.data_ptr(), dtype_code(out.dtype), a.data_ptr(), w.data_ptr(), M, N,
                                K, a.stride(0), ws.data_ptr(), ws.numel(), _stream()), "gemm_bf16",
           own=False)


_device_flags = {}


def device_flags(device: torch.device) -> torch.Tensor:
    """Two device ints that kernels raise and the host reads after a step (0: all well):
    [0] a bounded wait ran out, [1] a token position had no cache page."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    f = _device_flags.get(key)
    if f is None:
        f = _device_flags[key] = torch.zeros(2, dtype=torch.int32, device=device)
    return f


def error_flag(device: torch.device) -> torch.Tensor:
    """The device int that kernels with bounded waits set when a wait ran out."""
    return device_flags(device)[0:1]


def status_flag(device: torch.device) -> torch.Tensor:
    """The device int that kernels set when they meet a token position without a cache page."""
    return device_flags(device)[1:2]


FLAG_MESSAGES = ("a kernel's bounded wait ran out", "a kernel found a token position without a cache page")


def flash_has_tc(hd: int) -> bool:
    """Whether the attention library of this head size has the tcgen05 kernel for long portions."""
    return flash_supports(hd, torch.bfloat16) and bool(flash_lib(hd).atom_flash_has_tc())


def check_error_flags() -> None:
    """Raises if a kernel gave up a bounded wait or met a position without a page (synchronises the
    device); the flags are cleared, so the next check speaks of what ran after this one."""
    for f in _device_flags.values():
        v = f.tolist()
        if any(v):
            f.zero_()
            raise NativeError("; ".join(m for m, x in zip(FLAG_MESSAGES, v) if x))
    for hd, l in _flash_libs.items():      # (a device on which the library still uses its own flag)
        if l.atom_flash_take_error() != 0:
            raise NativeError(f"a bounded wait of the attention kernels (head size {hd}) ran out")


class _RowsOpC(ctypes.Structure):
    """csrc/gemm_rows.h: AtomRowsOp."""
    _fields_ = [("X", _vp), ("lda", _i64), ("W", _vp), ("out", _vp), ("out_dtype", _i), ("ldc", _i64),
                ("bias", _vp), ("bias_dtype", _i), ("N", _i), ("K", _i), ("gated", _i),
                ("ssq_in", _vp), ("ssq_parts", _i), ("norm_size", _i), ("norm_eps", _f),
                ("residual", _vp), ("norm_w", _vp), ("norm_w_dtype", _i), ("xout", _vp), ("ssq_out", _vp)]


ROWS_M = 16     # rows up to which the weight-streaming product is used (parts/linear.py: streams)


def gemm_rows_grid() -> int:
    """CTAs of a ``gemm_rows`` launch: a residual product writes one part of the rows' sums of squares per CTA."""
    return int(lib().atom_gemm_rows_grid())


def gemm_rows_supports(M: int, N: int, K: int, lda: int) -> bool:
    return bool(lib().atom_gemm_rows_supports(M, N, K, lda))


def gemm_rows(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
              bias: Optional[torch.Tensor] = None, gated: bool = False, ssq_in: Optional[torch.Tensor] = None,
              norm_size: int = 0, norm_eps: float = 0.0, residual: Optional[torch.Tensor] = None,
              norm_w: Optional[torch.Tensor] = None, xout: Optional[torch.Tensor] = None,
              ssq_out: Optional[torch.Tensor] = None) -> None:
    """out[M, N] = x[M, K] w[N, K]^T for at most 16 rows of bf16 x, with one of the epilogues of
    csrc/gemm_rows.h: plain (+ bias; out bf16 or float32); ``gated`` (w = [gate ; up] of 2N rows);
    ``residual`` (float32 [M, N], += product in place, with ``xout`` = bf16(residual * norm_w) and the CTAs'
    sums of squares in ``ssq_out`` [gemm_rows_grid(), 16]).  ``ssq_in`` (such sums, of ``norm_size`` columns):
    every output row is first multiplied by its rstd."""
    M, K = x.shape
    res = residual is not None
    N = residual.shape[1] if res else out.shape[1]
    _cuda(x, w, out, bias, ssq_in, residual, norm_w, xout, ssq_out)
    assert x.dtype == w.dtype == torch.bfloat16 and w.shape[1] == K and w.is_contiguous() and x.stride(1) == 1
    assert w.shape[0] == (2 * N if gated else N)
    c = _RowsOpC()
    if res:
        assert residual.dtype == torch.float32 and residual.is_contiguous() and residual.shape[0] == M
        assert xout.dtype == torch.bfloat16 and xout.is_contiguous() and xout.shape == residual.shape
        assert ssq_out.dtype == torch.float32 and ssq_out.shape == (gemm_rows_grid(), 16) and ssq_out.is_contiguous()
        assert norm_w.numel() == N and norm_w.is_contiguous()
    else:
        assert out.shape[0] == M and out.stride(1) == 1
    if ssq_in is not None:
        assert ssq_in.dtype == torch.float32 and ssq_in.is_contiguous() and ssq_in.shape[-1] == 16
    c.X, c.lda, c.W = x.data_ptr(), x.stride(0), w.data_ptr()
    c.out = _ptr(out)
    c.out_dtype = dtype_code(out.dtype) if out is not None else BF16
    c.ldc = out.stride(0) if out is not None else 0
    c.bias, c.bias_dtype = _ptr(bias), (dtype_code(bias.dtype) if bias is not None else F32)
    c.N, c.K, c.gated = N, K, int(gated)
    c.ssq_in = _ptr(ssq_in)
    c.ssq_parts = ssq_in.numel() // 16 if ssq_in is not None else 0
    c.norm_size, c.norm_eps = int(norm_size), float(norm_eps)
    c.residual, c.norm_w = _ptr(residual), _ptr(norm_w)
    c.norm_w_dtype = dtype_code(norm_w.dtype) if norm_w is not None else F32
    c.xout, c.ssq_out = _ptr(xout), _ptr(ssq_out)
    _check(lib().atom_gemm_rows(ctypes.byref(c), M, error_flag(x.device).data_ptr(), _stream()), "gemm_rows")


def gemm_pairs_supports(M: int, N: int, K: int, lda: int, ldc: int) -> bool:
    return bool(lib().atom_gemm_pairs_supports(M, N, K, lda, ldc)) and gemm_pairs_resident() > 0


_pairs_resident = None


def gemm_pairs_resident() -> int:
    """Pairs of CTAs of a ``gemm_pairs`` launch: as many as the device holds at once."""
    global _pairs_resident
    if _pairs_resident is None:
        _pairs_resident = int(lib().atom_gemm_pairs_resident())
    return _pairs_resident


def gemm_pairs_waves(M: int, N: int, gated: bool) -> float:
    """How well the tiles of a ``gemm_pairs`` product fill the device: tiles / (waves x pairs), where the
    last, ragged wave counts 0.72 when it is handed out in halves (csrc/gemm_pairs.cu: plan_items; a half
    tile runs at about 0.72 of a whole one's time)."""
    pairs = gemm_pairs_resident()
    if pairs < 1:
        return 0.0
    tiles = -(-M // 256) * (-(-N // 256) if gated else -(-N // 512))
    full, rem = divmod(tiles, pairs)
    waves = full + (0.0 if rem == 0 else (0.72 if full > 0 and 2 * rem <= pairs else 1.0))
    return tiles / (waves * pairs)


def gemm_pairs(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False) -> None:
    """out[M, N] = x[M, K] w[N, K]^T in bf16 on tcgen05 with two CTAs to a tile; ``gated``: w = [gate ; up]
    of 2N rows, out = silu(x gate^T) * (x up^T) (csrc/gemm_pairs.cu)."""
    M, K = x.shape
    N = out.shape[1]
    _cuda(x, w, out)
    assert x.dtype == w.dtype == out.dtype == torch.bfloat16 and w.shape[1] == K and w.is_contiguous()
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == M and w.shape[0] == (2 * N if gated else N)
    _check(lib().atom_gemm_pairs(x.data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0), M, N, K,
                                 int(gated), error_flag(x.device).data_ptr(), _stream()), "gemm_pairs")


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    _cuda(out, bias)
    M, N = out.shape
    assert out.is_contiguous() and bias.numel() == N
    _check(lib().atom_add_bias(out.data_ptr(), dtype_code(out.dtype), bias.data_ptr(),
                               dtype_code(bias.dtype), M, N, _stream()), "add_bias")


# --------------------------------------------------------------------------- tensor-core attention

_flash_libs = {}
_FLASH_SIG = [_vp, _vp, _i64, _vp, _vp, _i64, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _i,
              _i, _vp, _vp]
_FLASH_ROT_SIG = [_vp, _vp, _i64, _vp, _vp, _i64, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _vp,
                  _vp, _vp, _i, _i, _vp, _vp, _i, _f, _i, _vp, _vp]
LONG_ROWS = 128    # packed rows from which a request runs on the tcgen05 attention kernel
ROTATE_IN_DECODE = True    # decode steps leave q/k norm, rotation and cache write to the attention kernel where it takes them


def flash_supports(hd: int, dtype: torch.dtype) -> bool:
    """The tensor-core attention takes bfloat16 and head sizes that are multiples of 16 up to 256."""
    return dtype == torch.bfloat16 and hd % 16 == 0 and 16 <= hd <= 256


def flash_lib(hd: int):
    """The attention library compiled for this head size (built on first use)."""
    l = _flash_libs.get(hd)
    if l is None:
        with _lock:
            l = _flash_libs.get(hd)
            if l is None:
                path = build_variant("attention_flash.cu", {"ATOM_HD": hd})
                l = ctypes.CDLL(path)
                l.atom_flash_attention.argtypes = _FLASH_SIG
                l.atom_flash_attention.restype = ctypes.c_int
                l.atom_flash_scratch_bytes.argtypes = [_i, _i, _i]
                l.atom_flash_scratch_bytes.restype = ctypes.c_int64
                l.atom_flash_attention_rotating.argtypes = _FLASH_ROT_SIG
                l.atom_flash_attention_rotating.restype = ctypes.c_int
                l.atom_flash_rotating_supports.argtypes = [_i, _i64, _i, _i, _i]
                l.atom_flash_rotating_supports.restype = ctypes.c_int
                l.atom_flash_take_error.restype = ctypes.c_int
                l.atom_flash_has_tc.restype = ctypes.c_int
                if l.atom_flash_head_dim() != hd:
                    raise NativeBuildError(f"{path} was built for another head size")
                # bounded waits of this library report into the device's shared flag word, which the
                # engine reads back with every step's tokens (other devices keep the library's own flag)
                l.atom_flash_set_option.argtypes = [_i, _i]
                l.atom_flash_set_option.restype = ctypes.c_int
                for k, v in _option_values.items():
                    l.atom_flash_set_option(k, v)
                l.atom_flash_set_error_flag.argtypes = [_vp]
                l.atom_flash_set_error_flag.restype = ctypes.c_int
                if torch.cuda.is_available():
                    l.atom_flash_set_error_flag(error_flag(torch.device("cuda", torch.cuda.current_device())).data_ptr())
                _flash_libs[hd] = l
    return l


_sm_counts = {}


def sm_count() -> int:
    dev = torch.cuda.current_device()
    if dev not in _sm_counts:
        _sm_counts[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sm_counts[dev]


def flash_plan(q_lens, group: int, nkv: int, max_ctx: int, sms: Optional[int] = None, long_rows: int = 0):
    """Host-side launch plan: (64-row tiles of the mid-size requests, any short request?,
    splits[, 128-row tiles of the long requests when long_rows > 0]).

    Short requests (at most 16 packed rows) are split along their keys.  Two CTAs fit an SM.
    Measured on B200: one wave of CTAs (at most 2 per SM) is best, with splits no shorter than
    256 keys; when even one split per (request, kv head) is more than a wave, a larger split
    count (up to 8) only where it fills whole waves at least 15 % better (every split costs a
    pass of the merge kernel over its partial sums)."""
    sms = sms or sm_count()
    tiles, short, long_tiles = 0, 0, 0
    for n in q_lens:
        rows = n * group
        if long_rows and rows >= long_rows:
            long_tiles += -(-rows // 128)
        elif rows > 16:
            tiles += -(-rows // 64)
        elif rows > 0:
            short += 1
    splits = 1
    if short:
        slots = 2 * sms
        pairs = max(1, len(q_lens) * nkv)
        longest = max(1, -(-max_ctx // 256))
        if pairs <= slots:
            splits = max(1, min(slots // pairs, longest, 64))
        else:
            best = 0.0
            for s in range(1, min(8, longest) + 1):
                ctas = pairs * s
                eff = ctas / (-(-ctas // slots) * slots)
                if eff > best * 1.15:
                    best, splits = eff, s
    if long_rows:
        return tiles, short > 0, splits, long_tiles
    return tiles, short > 0, splits


def flash_plan_for_any(tokens: int, seqs: int, group: int, nkv: int, max_ctx: int, sms: Optional[int] = None,
                       long_rows: int = 0):
    """A launch plan that holds for every batch of at most ``tokens`` tokens in at most ``seqs`` requests
    (for a step recorded once and replayed for batches of other makeups): tile counts are upper bounds
    (the kernels find their tile from the step's arrays; a CTA without one leaves at once), short
    requests are always provided for, with the splits of ``seqs`` short requests."""
    rows = tokens * group
    n_long = min(seqs, rows // long_rows) if long_rows else 0
    long_tiles = rows // 128 + 1 + n_long if long_rows else 0
    tiles = rows // 64 + 1 + min(seqs, max(1, rows // 17))
    splits = flash_plan([1] * seqs, group, nkv, max_ctx, sms)[2]
    if long_rows:
        return tiles, True, splits, long_tiles
    return tiles, True, splits


def flash_attention(out: torch.Tensor, q: torch.Tensor, q_stride: int, k_pages: torch.Tensor,
                    v_pages: torch.Tensor, block_table: torch.Tensor, cu_q: torch.Tensor,
                    ctx_len: torch.Tensor, seq_of_token: torch.Tensor, T: int, num_seqs: int, nh: int,
                    nkv: int, hd: int, scale: float, window: int, plan, scratch: Optional[torch.Tensor]) -> None:
    """out[T, nh*hd] (bf16): causal attention of every token over its request's pages, on the
    tensor cores.  ``plan`` comes from ``flash_plan``; ``scratch`` (float32) must hold
    ``flash_scratch_elems`` elements when the plan has more than one split."""
    _cuda(out, q, k_pages, v_pages, block_table, cu_q, ctx_len, seq_of_token, scratch)
    page_size = k_pages.shape[2]
    assert out.dtype == q.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16
    assert out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert tuple(k_pages.shape[1:]) == (nkv, page_size, hd) and v_pages.shape == k_pages.shape
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
    assert cu_q.dtype == ctx_len.dtype == seq_of_token.dtype == torch.int32
    tiles, has_short, splits = plan[:3]
    long_tiles = plan[3] if len(plan) > 3 else 0
    if splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32
        assert scratch.numel() >= flash_scratch_elems(T, nh, hd, splits)
    l = flash_lib(hd)
    _check(l.atom_flash_attention(
        out.data_ptr(), q.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
        block_table.data_ptr(), block_table.shape[1], page_size, cu_q.data_ptr(), ctx_len.data_ptr(),
        seq_of_token.data_ptr(), T, num_seqs, nh, nkv, hd, float(scale), int(window), int(long_tiles),
        LONG_ROWS, int(tiles), int(has_short), int(splits), _ptr(scratch), _stream()), "flash_attention")
    # (one kernel for the long portions, one for the others, one for the short requests, one that merges their splits)
    add_launches(int(long_tiles > 0) + int(tiles > 0) + int(bool(has_short)) + int(bool(has_short) and splits > 1) - 1)


def flash_rotating_supports(hd: int, page_size: int, num_pages: int, nh: int, nkv: int, rotary_dim: int) -> bool:
    """A decode step of these sizes can leave the heads' norm, the rotation and the cache write of its new
    tokens to the decode attention kernel (``flash_attention_rotating``)."""
    return ROTATE_IN_DECODE and flash_supports(hd, torch.bfloat16) and bool(
        flash_lib(hd).atom_flash_rotating_supports(page_size, num_pages, nh, nkv, rotary_dim))


def flash_attention_rotating(out: torch.Tensor, qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                             block_table: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor,
                             seq_of_token: torch.Tensor, T: int, num_seqs: int, nh: int, nkv: int, hd: int,
                             scale: float, window: int, splits: int, scratch: Optional[torch.Tensor],
                             table: torch.Tensor, rotary_dim: int, rows: torch.Tensor,
                             q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                             write_cache: bool, status: torch.Tensor) -> None:
    """Decode attention of a step in which every request brings one token, over the raw projection
    qkv[T, (nh + 2 nkv) * hd]: the kernel normalises each query and key head (weights or None), rotates it
    by row rows[t] of ``table`` [positions, rotary_dim] (cos, then sin), stores the new key and value in the
    token's page (``write_cache``; a token without a page sets ``status``) and attends.  out[T, nh*hd]."""
    _cuda(out, qkv, k_pages, v_pages, block_table, cu_q, ctx_len, seq_of_token, scratch, table, rows, q_weight,
          k_weight, status)
    page_size = k_pages.shape[2]
    assert out.dtype == qkv.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16 and T == num_seqs
    assert out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous() and qkv.stride(1) == 1
    assert qkv.shape[1] == (nh + 2 * nkv) * hd
    assert tuple(k_pages.shape[1:]) == (nkv, page_size, hd) and v_pages.shape == k_pages.shape
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
    assert cu_q.dtype == ctx_len.dtype == seq_of_token.dtype == rows.dtype == status.dtype == torch.int32
    assert table.dtype == torch.float32 and table.is_contiguous() and table.shape[1] == rotary_dim
    w = q_weight if q_weight is not None else k_weight
    if w is not None:
        assert all(x is None or (x.dtype == w.dtype and x.numel() == hd and x.is_contiguous()) for x in (q_weight, k_weight))
    if splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32
        assert scratch.numel() >= flash_scratch_elems(T, nh, hd, splits)
    l = flash_lib(hd)
    _check(l.atom_flash_attention_rotating(
        out.data_ptr(), qkv.data_ptr(), qkv.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
        block_table.data_ptr(), block_table.shape[1], page_size, cu_q.data_ptr(), ctx_len.data_ptr(),
        seq_of_token.data_ptr(), T, num_seqs, nh, nkv, hd, float(scale), int(window), int(splits), _ptr(scratch),
        table.data_ptr(), rows.data_ptr(), int(rotary_dim), table.shape[0], _ptr(q_weight), _ptr(k_weight),
        dtype_code(w.dtype) if w is not None else F32, float(eps), int(write_cache), status.data_ptr(), _stream()),
        "flash_attention_rotating")
    add_launches(int(splits > 1))      # (the kernel that merges the splits)


def flash_scratch_elems(T: int, nh: int, hd: int, splits: int) -> int:
    return 0 if splits <= 1 else T * nh * splits * (hd + 2)
