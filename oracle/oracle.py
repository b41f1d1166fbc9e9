"""ctypes front end of the CPU oracle (test infrastructure only).

Only the test-suite, the smoke check and the benchmark's CPU legs may import this
module; the product package never does.  Every function takes and returns numpy
arrays and mirrors one `extern "C"` entry of nvfp4_oracle.cpp, which cites the
reference source lines it restates.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import c_float, c_int, c_uint8, c_uint32, c_uint64, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libnvfp4_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile next to this file."""
    src = os.path.join(_HERE, "nvfp4_oracle.cpp")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B" if force else "-s", "libnvfp4_oracle.so"])
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_e2m1_decode.restype = c_float
        _lib.oracle_e2m1_decode.argtypes = [c_uint8]
        _lib.oracle_e4m3_decode.restype = c_float
        _lib.oracle_e4m3_decode.argtypes = [c_uint8]
        _lib.oracle_e2m1_encode.restype = c_uint8
        _lib.oracle_e2m1_encode.argtypes = [c_float]
        _lib.oracle_e4m3_encode.restype = c_uint8
        _lib.oracle_e4m3_encode.argtypes = [c_float]
        _lib.oracle_hash_u32.restype = c_uint32
        _lib.oracle_hash_u32.argtypes = [c_uint32]
        _lib.oracle_quartet_scale_override.restype = c_float
        _lib.oracle_four_six_global_scale.restype = c_float
        _lib.oracle_four_six_global_scale.argtypes = [c_float]
        _lib.oracle_ms_eden_global_scale.restype = c_float
        _lib.oracle_ms_eden_global_scale.argtypes = [c_float]
        _lib.oracle_scale_packed_offset.restype = c_uint64
        _lib.oracle_scale_packed_offset.argtypes = [c_uint32, c_uint32, c_uint32]
        _lib.oracle_max_threads.restype = c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


QUARTET_SO = None


def quartet_scale_override() -> float:
    return float(lib().oracle_quartet_scale_override())


def set_threads(n: int) -> None:
    lib().oracle_set_threads(c_int(n))


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def e2m1_decode(n):
    return float(lib().oracle_e2m1_decode(c_uint8(n)))


def e4m3_decode(b):
    return float(lib().oracle_e4m3_decode(c_uint8(b)))


def e2m1_encode(x):
    return int(lib().oracle_e2m1_encode(c_float(x)))


def e4m3_encode(x):
    return int(lib().oracle_e4m3_encode(c_float(x)))


def hash_u32(v):
    return int(lib().oracle_hash_u32(c_uint32(v & 0xFFFFFFFF)))


def four_six_global_scale(amax):
    return float(lib().oracle_four_six_global_scale(c_float(amax)))


def ms_eden_global_scale(amax):
    return float(lib().oracle_ms_eden_global_scale(c_float(amax)))


def padded_k(k: int) -> int:
    """utils/nvfp4_tc_matmul/args.rs:37-39: K padded to a multiple of 64."""
    return (k + 63) // 64 * 64


def row_amax(x):
    x = _f32(x)
    rows, cols = x.shape
    out = np.empty(rows, np.float32)
    lib().oracle_row_amax_f32(_p(x), _p(out), c_uint32(rows), c_uint32(cols))
    return out


def stochastic_e4m3_scale(value: float, seed: int, group: int) -> int:
    """utils/nvfp4/quant/kernels/ms_eden/pack/scale.rs:7-30: E4M3 code of `value`, rounded stochastically."""
    fn = lib().oracle_stochastic_e4m3_scale
    fn.restype = ctypes.c_uint8
    return int(fn(c_float(value), c_uint32(seed & 0xFFFFFFFF), c_uint32(group & 0xFFFFFFFF)))


def hash_u32(v: int) -> int:
    fn = lib().oracle_hash_u32
    fn.restype = c_uint32
    return int(fn(c_uint32(v & 0xFFFFFFFF)))


def relu2_backward(pre_activation, d_out):
    """gpt/mlp/kernels.rs:72-104: d_pre = d_out * 2 * relu(pre), f32."""
    p, d = _f32(pre_activation).reshape(-1), _f32(d_out).reshape(-1)
    out = np.empty(p.size, np.float32)
    lib().oracle_relu2_backward(_p(p), _p(d), _p(out), c_uint64(p.size))
    return out


def schedule_free_value(z_master, x_master, beta: float):
    """gpt/optimizer/schedule_free/value.rs:4-9: y = z + beta * (x - z) in f32."""
    z, x = _f32(z_master).reshape(-1), _f32(x_master).reshape(-1)
    out = np.empty(z.size, np.float32)
    lib().oracle_schedule_free_value(_p(z), _p(x), c_float(beta), c_uint64(z.size), _p(out))
    return out


def tensor_amax(x):
    """Returns (chunk_amax[ceil(n/1024)], amax[1])."""
    x = _f32(x).reshape(-1)
    chunks = np.empty((x.size + 1023) // 1024, np.float32)
    out = np.empty(1, np.float32)
    lib().oracle_tensor_amax_f32(_p(x), _p(chunks), _p(out), c_uint64(x.size))
    return chunks, out


def nvfp4_amax(bytes_, scales, gscales, rows, cols, rowwise):
    bytes_, scales, gscales = _u8(bytes_), _u8(scales), _f32(gscales)
    n = rows * cols
    chunks = np.empty((n + 1023) // 1024, np.float32)
    out = np.empty(1, np.float32)
    lib().oracle_nvfp4_amax(_p(bytes_), _p(scales), _p(gscales), c_uint64(n), c_uint32(cols if rowwise else 0),
                            _p(chunks), _p(out))
    return chunks, out


def four_six(x, amax, rowwise: bool):
    """x [rows, cols] f32, amax [rows] (rowwise) or [1].  Returns (bytes, scales, global_scales)."""
    x = _f32(x)
    rows, cols = x.shape
    assert cols % 16 == 0
    amax = _f32(amax)
    fp4 = np.empty(rows * cols // 2, np.uint8)
    scales = np.empty(rows * cols // 16, np.uint8)
    gs = np.empty(rows if rowwise else 1, np.float32)
    lib().oracle_four_six(_p(x), _p(amax), c_uint64(x.size), c_uint32(cols if rowwise else 0), _p(fp4),
                          _p(scales), _p(gs))
    return fp4, scales, gs


def four_six_padded(x, amax, padded_rows, padded_cols, transposed: bool):
    x = _f32(x)
    rows, cols = x.shape
    amax = _f32(amax)
    n = padded_rows * padded_cols
    fp4 = np.empty(n // 2, np.uint8)
    scales = np.empty(n // 16, np.uint8)
    gs = np.empty(1, np.float32)
    lib().oracle_four_six_padded(_p(x), _p(amax), c_uint32(rows), c_uint32(cols), c_uint32(padded_rows),
                                 c_uint32(padded_cols), c_int(1 if transposed else 0), _p(fp4), _p(scales),
                                 _p(gs))
    return fp4, scales, gs


def ms_eden(kind, src, out_rows, dst_row_len, gs, sign_seed, scale_seed, so=None, col_offset=0,
            group_offset=0, want_chunk_amax=True):
    """MS-EDEN quantizer.

    kind 0: src = f32 [out_rows, src_row_len]                       (rows, zero padded to dst_row_len)
    kind 1: src = f32 [source_rows, source_cols], out_rows = source_cols (transpose)
    kind 2: src = (bytes, scales, gscale[1], source_rows, source_cols)   NVFP4 tensor scale, transposed
    kind 3: src = (bytes, scales, gscales[source_rows], source_rows, source_cols) NVFP4 rowwise, transposed
    Returns (bytes, scales, global_scales[out_rows], chunk_amax or None).
    """
    so = quartet_scale_override() if so is None else so
    assert dst_row_len % 32 == 0 and group_offset % 2 == 0
    x = b = s = g = None
    if kind in (0, 1):
        x = _f32(src)
        a = x.shape[1] if kind == 0 else x.shape[0]
        bb = 0 if kind == 0 else x.shape[1]
    else:
        b, s, g, a, bb = src
        b, s, g = _u8(b), _u8(s), _f32(g)
    n = out_rows * dst_row_len
    fp4 = np.empty(n // 2, np.uint8)
    scales = np.empty(n // 16, np.uint8)
    gsc = np.empty(out_rows, np.float32)
    ca = np.empty(n // 32, np.float32) if want_chunk_amax else None
    lib().oracle_ms_eden(c_int(kind), _p(x), _p(b), _p(s), _p(g), c_uint32(a), c_uint32(bb), c_uint32(out_rows),
                         c_uint32(dst_row_len), c_float(gs), c_float(so), c_uint32(sign_seed),
                         c_uint32(scale_seed), c_uint32(col_offset), c_uint32(group_offset), _p(fp4), _p(scales),
                         _p(gsc), _p(ca))
    return fp4, scales, gsc, ca


def scale_packed_len(mn: int, k: int) -> int:
    return (mn + 127) // 128 * (k // 64) * 512


def scale_pack(logical, mn, k):
    logical = _u8(logical)
    packed = np.empty(scale_packed_len(mn, k), np.uint8)
    lib().oracle_scale_pack(_p(logical), _p(packed), c_uint32(mn), c_uint32(k))
    return packed


def scale_packed_offset(mn, k_group, k):
    return int(lib().oracle_scale_packed_offset(c_uint32(mn), c_uint32(k_group), c_uint32(k)))


def decode(bytes_, scales, gscales, rows, cols, rowwise: bool, transpose: bool):
    bytes_, scales, gscales = _u8(bytes_), _u8(scales), _f32(gscales)
    out = np.empty((cols, rows) if transpose else (rows, cols), np.float32)
    lib().oracle_decode(_p(bytes_), _p(scales), _p(gscales), c_uint32(rows), c_uint32(cols),
                        c_int(1 if rowwise else 0), c_int(1 if transpose else 0), _p(out))
    return out


def gemm(a, b, m, k, n, mode, weight=1.0, bias=None, epi=0, residual=None, ldo=None, want_pre=False):
    """a = (bytes, scales_logical, global[rows or 1]); b likewise (tensor scale).  Returns out [m, ldo]
    (and the pre-activation when want_pre).  epi: 0 raw, 1 +bias, 2 relu^2, 3 residual add."""
    ldo = n if ldo is None else ldo
    ab, asc, ag = _u8(a[0]), _u8(a[1]), _f32(a[2])
    bb, bsc, bg = _u8(b[0]), _u8(b[1]), _f32(b[2])
    out = np.zeros((m, ldo), np.float32) if residual is None else _f32(residual).copy().reshape(m, ldo)
    pre = np.zeros((m, ldo), np.float32) if want_pre else None
    bias_ = None if bias is None else _f32(bias)
    lib().oracle_gemm(_p(ab), _p(asc), _p(ag), _p(bb), _p(bsc), _p(bg), c_uint32(m), c_uint32(k), c_uint32(n),
                      c_uint32(ldo), c_int(mode), c_float(weight), _p(bias_), c_int(epi), _p(out), _p(pre))
    return (out, pre) if want_pre else out


def bias_grad(e):
    e = _f32(e)
    tokens, n = e.shape
    out = np.empty(n, np.float32)
    lib().oracle_bias_grad(_p(e), _p(out), c_uint32(tokens), c_uint32(n))
    return out


def bias_grad_tiled(e):
    """Column sums in the order of the fused GPU path (128-row tiles; see nvfp4_oracle.cpp)."""
    e = _f32(e)
    tokens, n = e.shape
    out = np.empty(n, np.float32)
    lib().oracle_bias_grad_tiled(_p(e), _p(out), c_uint32(tokens), c_uint32(n))
    return out


def linear_forward_backward(x, w, bias, dy, sign_seed, scale_seed, epi=1):
    """One projection, forward and backward, entirely on the CPU oracle: the composition of
    crates/gpt2-nvfp4/src/types/l3_mlp/forward.rs:15-67 (quantize X rowwise, W tensor scale, GEMM +
    epilogue) and crates/cuda-kernels/src/gpt/linear_backward/ms_eden.rs:15-55 (dbias, MS-EDEN of
    dY rows / dY^T / W^T / X^T, dX and dW GEMMs).  x [T, K], w [N, K], dy [T, N] float32 arrays.
    Returns (y, dx, dw, dbias)."""
    x, w, dy = _f32(x), _f32(w), _f32(dy)
    tokens, in_dim = x.shape
    out_dim = w.shape[0]
    xq = four_six(x, row_amax(x), rowwise=True)
    wq = four_six(w, tensor_amax(w)[1], rowwise=False)
    y = gemm(xq, wq, tokens, in_dim, out_dim, mode=2, bias=bias, epi=epi if bias is not None else 0)
    dbias = bias_grad(dy)
    ok, tk = padded_k(out_dim), padded_k(tokens)
    gs_e = ms_eden_global_scale(float(tensor_amax(dy)[1][0]))
    e_h = ms_eden(0, dy, tokens, ok, gs_e, sign_seed, scale_seed, want_chunk_amax=False)
    e_t = ms_eden(1, dy, out_dim, tk, gs_e, sign_seed, scale_seed ^ 0x85EBCA6B, want_chunk_amax=False)
    gs_w = ms_eden_global_scale(float(nvfp4_amax(*wq, out_dim, in_dim, False)[1][0]))
    w_t = ms_eden(2, (*wq, out_dim, in_dim), in_dim, ok, gs_w, sign_seed, scale_seed ^ 0x9E3779B9,
                  want_chunk_amax=False)
    gs_x = ms_eden_global_scale(float(nvfp4_amax(*xq, tokens, in_dim, True)[1][0]))
    x_t = ms_eden(3, (*xq, tokens, in_dim), in_dim, tk, gs_x, sign_seed, scale_seed ^ 0xC2B2AE35,
                  want_chunk_amax=False)
    dx = gemm(e_h[:3], (w_t[0], w_t[1], np.array([gs_w], np.float32)), tokens, ok, in_dim, mode=2)
    dw = gemm(e_t[:3], (x_t[0], x_t[1], np.array([gs_x], np.float32)), out_dim, tk, in_dim, mode=2)
    return y, dx, dw, dbias
