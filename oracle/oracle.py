"""ctypes front end of the CPU oracle (oracle/illatio_oracle.c).

Test infrastructure: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg only.  Nothing in the illatio_b200 package imports
this module.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")

Q8_0, Q4_K, Q6_K, Q2_K, IQ2_XXS = range(5)

_c = ctypes
_u8p = _c.POINTER(_c.c_uint8)
_i8p = _c.POINTER(_c.c_int8)
_f32p = _c.POINTER(_c.c_float)
_i32p = _c.POINTER(_c.c_int32)


def build(force=False):
    """Compile liboracle.so with the Makefile beside this file."""
    srcs = [os.path.join(HERE, f) for f in ("illatio_oracle.c", "illatio_oracle_simd.c", "iq2xxs_tables.h", "Makefile")]
    if force or not os.path.exists(LIB) or any(os.path.getmtime(LIB) < os.path.getmtime(f) for f in srcs):
        subprocess.check_call(["make", "-C", HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        L = ctypes.CDLL(LIB)
        L.orc_half_to_single.restype = _c.c_float
        L.orc_half_to_single.argtypes = [_c.c_uint16]
        L.orc_single_to_half.restype = _c.c_uint16
        L.orc_single_to_half.argtypes = [_c.c_float]
        L.orc_silu.restype = _c.c_float
        L.orc_silu.argtypes = [_c.c_float]
        L.orc_dequant_row.argtypes = [_c.c_int, _u8p, _c.c_int, _f32p]
        L.orc_quantize_q8_0.argtypes = [_f32p, _c.c_int64, _i8p, _f32p, _c.c_int]
        L.orc_rmsnorm.argtypes = [_f32p, _f32p, _c.c_int64, _c.c_float, _f32p]
        L.orc_f32mv.argtypes = [_f32p, _c.c_int, _c.c_int, _f32p, _f32p]
        L.orc_quantize_q8k.argtypes = [_f32p, _c.c_int64, _i8p, _f32p, _i32p]
        L.orc_row_dot.restype = _c.c_float
        L.orc_row_dot.argtypes = [_c.c_int, _u8p, _c.c_int, _i8p, _f32p, _i32p]
        for name in ("orc_iq2xxs_row_dot_x86",):
            getattr(L, name).restype = _c.c_float
            getattr(L, name).argtypes = [_u8p, _c.c_int, _i8p, _f32p]
        L.orc_q2k_row_dot_x86.restype = _c.c_float
        L.orc_q2k_row_dot_x86.argtypes = [_u8p, _c.c_int, _i8p, _f32p, _i32p]
        L.orc_matvec.argtypes = [_c.c_int, _u8p, _c.c_int, _c.c_int, _i8p, _f32p, _i32p, _c.c_int, _f32p,
                                 _f32p, _c.c_int]
        L.orc_route.argtypes = [_f32p, _c.c_int, _c.c_int, _c.c_int, _f32p, _c.c_float, _i32p, _f32p]
        L.orc_moe_routed.argtypes = [_c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _u8p, _u8p, _u8p, _f32p,
                                     _i32p, _f32p, _c.c_float, _f32p, _f32p, _c.c_int]
        L.orc_set_fast.restype = _c.c_int
        L.orc_set_fast.argtypes = [_c.c_int]
        L.orc_simd_available.restype = _c.c_int
        L.orc_row_dot_simd.restype = _c.c_float
        L.orc_row_dot_simd.argtypes = [_c.c_int, _u8p, _c.c_int, _i8p, _f32p, _i32p]
        L.orc_moe_shared.argtypes = [_c.c_int, _c.c_int, _u8p, _u8p, _u8p, _f32p, _c.c_float, _f32p, _c.c_int]
        _lib = L
    return _lib


BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210, Q2_K: 84, IQ2_XXS: 66}
BLOCK_WEIGHTS = {Q8_0: 32, Q4_K: 256, Q6_K: 256, Q2_K: 256, IQ2_XXS: 256}


def row_bytes(fmt, cols):
    return cols // BLOCK_WEIGHTS[fmt] * BLOCK_BYTES[fmt]


def _p(a, t):
    return a.ctypes.data_as(t) if a is not None else None


def _c_(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


def half_to_single(h):
    return lib().orc_half_to_single(int(h))


def single_to_half(x):
    return lib().orc_single_to_half(float(x))


def dequant(fmt, w, rows, cols):
    """rows x cols floats from raw GGUF blocks (uint8 array)."""
    w = _c_(w, np.uint8).reshape(-1)
    rb = row_bytes(fmt, cols)
    assert w.size >= rows * rb
    out = np.empty((rows, cols), np.float32)
    L = lib()
    for r in range(rows):
        L.orc_dequant_row(fmt, _p(w[r * rb:], _u8p), cols, _p(out[r], _f32p))
    return out


def f32mv(w, x):
    """F32MV!: out[r] = row r of W (floats, [rows, cols]) . x."""
    w, x = _c_(w, np.float32), _c_(x, np.float32).reshape(-1)
    rows, cols = w.shape
    out = np.empty(rows, np.float32)
    lib().orc_f32mv(_p(w, _f32p), rows, cols, _p(x, _f32p), _p(out, _f32p))
    return out


def rmsnorm(x, w, eps):
    """RMSNORM! of one row."""
    x, w = _c_(x, np.float32).reshape(-1), _c_(w, np.float32).reshape(-1)
    out = np.empty(x.size, np.float32)
    lib().orc_rmsnorm(_p(x, _f32p), _p(w, _f32p), x.size, float(eps), _p(out, _f32p))
    return out


def quantize_q8_0(x, f16_scale=True):
    x = _c_(x, np.float32).reshape(-1)
    q = np.empty(x.size, np.int8)
    s = np.empty(x.size // 32, np.float32)
    lib().orc_quantize_q8_0(_p(x, _f32p), x.size, _p(q, _i8p), _p(s, _f32p), 1 if f16_scale else 0)
    return q, s


def quantize_q8k(x):
    x = _c_(x, np.float32).reshape(-1)
    q = np.empty(x.size, np.int8)
    d = np.empty(x.size // 256, np.float32)
    bs = np.empty(x.size // 16, np.int32)
    lib().orc_quantize_q8k(_p(x, _f32p), x.size, _p(q, _i8p), _p(d, _f32p), _p(bs, _i32p))
    return q, d, bs


def quantize_act(fmt, x, f16_scale=True):
    """(xq, xs, bsums-or-None) in the activation format FMT's products take."""
    if fmt == Q8_0:
        q, s = quantize_q8_0(x, f16_scale)
        return q, s, None
    return quantize_q8k(x)


def matvec(fmt, w, rows, cols, act, n=1, bias=None, threads=1):
    """out[t, r] = row r . token t.  ACT = (xq, xs, bsums) for n tokens, flat."""
    xq, xs, bs = act
    w = _c_(w, np.uint8).reshape(-1)
    out = np.empty((n, rows), np.float32)
    b = _c_(bias, np.float32) if bias is not None else None
    lib().orc_matvec(fmt, _p(w, _u8p), rows, cols, _p(xq, _i8p), _p(xs, _f32p), _p(bs, _i32p), n,
                     _p(out, _f32p), _p(b, _f32p), threads)
    return out


def simd_available():
    """Whether this CPU runs the AVX2 row dots."""
    return bool(lib().orc_simd_available())


def set_fast(on):
    """The timed CPU baseline's form: AVX2 row dots (IQ2_XXS / Q2_K in the x86 float order) on a pool of pinned
    threads.  Off (the default) for every parity check.  Returns the previous setting."""
    return lib().orc_set_fast(1 if on else 0)


def row_dot_simd(fmt, w_row, cols, act):
    xq, xs, bs = act
    w_row = _c_(w_row, np.uint8)
    return lib().orc_row_dot_simd(fmt, _p(w_row, _u8p), cols, _p(xq, _i8p), _p(xs, _f32p), _p(bs, _i32p))


def row_dot_x86(fmt, w_row, cols, act):
    xq, xs, bs = act
    w_row = _c_(w_row, np.uint8)
    if fmt == IQ2_XXS:
        return lib().orc_iq2xxs_row_dot_x86(_p(w_row, _u8p), cols // 256, _p(xq, _i8p), _p(xs, _f32p))
    assert fmt == Q2_K
    return lib().orc_q2k_row_dot_x86(_p(w_row, _u8p), cols // 256, _p(xq, _i8p), _p(xs, _f32p), _p(bs, _i32p))


def route(logits, nu, mode=2, bias=None, scale=1.0):
    """(sel [n, nu] int32, w [n, nu] float32) for n tokens' router logits."""
    logits = _c_(logits, np.float32)
    if logits.ndim == 1:
        logits = logits[None]
    n, ne = logits.shape
    sel = np.empty((n, nu), np.int32)
    w = np.empty((n, nu), np.float32)
    b = _c_(bias, np.float32) if bias is not None else None
    L = lib()
    for t in range(n):
        L.orc_route(_p(logits[t], _f32p), ne, nu, mode, _p(b, _f32p), scale, _p(sel[t], _i32p), _p(w[t], _f32p))
    return sel, w


def moe_routed(d, ff, gate_fmt, down_fmt, gate, up, down, norm, sel, wts, clamp=0.0, threads=1, want_mid=False):
    """The routed experts of one token (see orc_moe_routed)."""
    nu = len(sel)
    norm = _c_(norm, np.float32)
    sel = _c_(sel, np.int32)
    wts = _c_(wts, np.float32)
    moe = np.empty(d, np.float32)
    mid = np.empty(nu * ff, np.float32) if want_mid else None
    lib().orc_moe_routed(d, ff, nu, gate_fmt, down_fmt, _p(gate, _u8p), _p(up, _u8p), _p(down, _u8p),
                         _p(norm, _f32p), _p(sel, _i32p), _p(wts, _f32p), clamp, _p(moe, _f32p),
                         _p(mid, _f32p), threads)
    return (moe, mid) if want_mid else moe


def moe_shared(d, ff, gate, up, down, norm, clamp=0.0, threads=1):
    norm = _c_(norm, np.float32)
    out = np.empty(d, np.float32)
    lib().orc_moe_shared(d, ff, _p(gate, _u8p), _p(up, _u8p), _p(down, _u8p), _p(norm, _f32p), clamp,
                         _p(out, _f32p), threads)
    return out
