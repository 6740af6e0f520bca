"""numpy front end of oracle/dtas_oracle.c (plain C restatement of the workload PrimFuncs).

TEST INFRASTRUCTURE, not product.  Functions take and return numpy arrays; fp16 data is
numpy float16.  See dtas_oracle.c for the reference citations of each function.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "dtas_oracle.c")
_SO = os.path.join(_HERE, "_build", "libdtas_oracle.so")
_lib = None


def build(force=False):
    """gcc -O2 -fopenmp; rebuilt when the source is newer than the library."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        os.makedirs(os.path.dirname(_SO), exist_ok=True)
        cmd = ["gcc", "-O2", "-mf16c", "-fopenmp", "-shared", "-fPIC", "-Wall", "-o", _SO, _SRC, "-lm"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("building the oracle failed:\n" + res.stderr)
    return _SO


def _c():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.oracle_max_threads.restype = ctypes.c_int
    return _lib


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data)


def _i64(v):
    return ctypes.c_int64(int(v))


def set_threads(n):
    _c().oracle_set_threads(ctypes.c_int(int(n)))


def max_threads():
    return int(_c().oracle_max_threads())


def _2d(a):
    a = np.ascontiguousarray(a)
    return a.reshape(-1, a.shape[-1])


def cast(a, dst_dtype):
    a2 = _2d(a)
    m, h = a2.shape
    dst_dtype = np.dtype(dst_dtype)
    out = np.empty((m, h), dst_dtype)
    if a2.dtype == np.float32 and dst_dtype == np.float16:
        _c().oracle_cast_f32_f16(_ptr(a2), _ptr(out), _i64(m), _i64(h))
    elif a2.dtype == np.float16 and dst_dtype == np.float32:
        _c().oracle_cast_f16_f32(_ptr(a2), _ptr(out), _i64(m), _i64(h))
    else:
        raise ValueError(f"cast {a2.dtype} -> {dst_dtype} is not a workload of the path")
    return out.reshape(a.shape)


def add(a, b):
    a2, b2 = _2d(a), _2d(b)
    assert a2.shape == b2.shape and a2.dtype == b2.dtype
    m, h = a2.shape
    out = np.empty_like(a2)
    fn = {np.dtype(np.float16): "oracle_add_f16", np.dtype(np.float32): "oracle_add_f32",
          np.dtype(np.int8): "oracle_add_i8"}[a2.dtype]
    getattr(_c(), fn)(_ptr(a2), _ptr(b2), _ptr(out), _i64(m), _i64(h))
    return out.reshape(a.shape)


def copy(a):
    a2 = _2d(a)
    m, h = a2.shape
    out = np.empty_like(a2)
    _c().oracle_copy(_ptr(a2), _ptr(out), _i64(m), _i64(h), _i64(a2.dtype.itemsize))
    return out.reshape(a.shape)


def rms_norm(x, w, eps=1e-6):
    x2 = _2d(x)
    assert x2.dtype == np.float16 and w.dtype == np.float16
    m, h = x2.shape
    w = np.ascontiguousarray(w)
    out = np.empty((m, h), np.float16)
    _c().oracle_rms_norm_f16(_ptr(x2), _ptr(w), _ptr(out), _i64(m), _i64(h), ctypes.c_float(eps))
    return out.reshape(x.shape)


def softmax(x):
    x2 = _2d(x)
    assert x2.dtype in (np.float16, np.float32)
    m, h = x2.shape
    out = np.empty((m, h), np.float16)
    scratch = np.empty(2 * h * max(1, max_threads()), np.float32)
    _c().oracle_softmax(_ptr(x2), _ptr(out), _i64(m), _i64(h), ctypes.c_int(int(x2.dtype == np.float16)),
                        _ptr(scratch))
    return out.reshape(x.shape)


def layer_norm(x, gamma, beta, eps=1e-5):
    x2 = _2d(x)
    assert x2.dtype in (np.float16, np.float32)
    m, h = x2.shape
    gamma = np.ascontiguousarray(gamma, np.float32)
    beta = np.ascontiguousarray(beta, np.float32)
    out = np.empty((m, h), np.float16)
    _c().oracle_layer_norm(_ptr(x2), _ptr(gamma), _ptr(beta), _ptr(out), _i64(m), _i64(h), ctypes.c_float(eps),
                           ctypes.c_int(int(x2.dtype == np.float16)))
    return out.reshape(x.shape)


def gemv(x, w, bias=None):
    x = np.ascontiguousarray(x).reshape(-1)
    w = np.ascontiguousarray(w)
    assert x.dtype == np.float16 and w.dtype == np.float16
    n, k = w.shape
    assert x.shape[0] == k
    out = np.empty((1, n), np.float16)
    b = None if bias is None else np.ascontiguousarray(bias)
    _c().oracle_gemv_f16(_ptr(x), _ptr(w), _ptr(b) if b is not None else None, _ptr(out), _i64(n), _i64(k))
    return out


def gemm_nt(x, w, bias=None, rows=None, cols=None, out=None):
    """Y = X W^T.  `rows=(r0, r1)`, `cols=(c0, c1)` restrict the computed block (the rest of
    the returned array is left as passed in `out`, or zero)."""
    x2 = _2d(x)
    w = np.ascontiguousarray(w)
    assert x2.dtype == np.float16 and w.dtype == np.float16
    m, k = x2.shape
    n = w.shape[0]
    assert w.shape[1] == k
    if out is None:
        out = np.zeros((m, n), np.float16)
    r0, r1 = rows if rows is not None else (0, m)
    c0, c1 = cols if cols is not None else (0, n)
    b = None if bias is None else np.ascontiguousarray(bias)
    _c().oracle_gemm_nt_f16(_ptr(x2), _ptr(w), _ptr(b) if b is not None else None, _ptr(out), _i64(m), _i64(n),
                            _i64(k), _i64(n), _i64(r0), _i64(r1), _i64(c0), _i64(c1))
    return out


def gemm_nt_f16acc(x, w, bias=None, rows=None):
    """Y = X W^T (+ bias) with the fp16 accumulator the reference's own matmul PrimFuncs declare
    (one rounding per update, bias added by a second rounded stage).  `rows=(r0, r1)` restricts the
    computed rows; a single-row x gives the reference's GEMV."""
    x2 = _2d(x)
    w = np.ascontiguousarray(w)
    assert x2.dtype == np.float16 and w.dtype == np.float16
    m, k = x2.shape
    n = w.shape[0]
    assert w.shape[1] == k
    out = np.zeros((m, n), np.float16)
    r0, r1 = rows if rows is not None else (0, m)
    b = None if bias is None else np.ascontiguousarray(bias)
    _c().oracle_gemm_nt_f16acc(_ptr(x2), _ptr(w), _ptr(b) if b is not None else None, _ptr(out), _i64(n), _i64(k),
                               _i64(r0), _i64(r1))
    return out


def gemm_nt_fused(x, w, bias=None, res1=None, res2=None, act=None, out_dtype=np.float16, rows=None, cols=None, out=None):
    """The fused matmul forms of the model workloads with the reference's stage-by-stage fp16
    rounding: y = cast(((res1 + gelu?(X W^T + bias)) + res2)).  rows / cols restrict the block."""
    x2 = _2d(x)
    w = np.ascontiguousarray(w)
    assert x2.dtype == np.float16 and w.dtype == np.float16
    m, k = x2.shape
    n = w.shape[0]
    assert w.shape[1] == k and act in (None, "gelu") and np.dtype(out_dtype) in (np.dtype(np.float16), np.dtype(np.float32))
    if out is None:
        out = np.zeros((m, n), out_dtype)
    r0, r1 = rows if rows is not None else (0, m)
    c0, c1 = cols if cols is not None else (0, n)
    opt = [None if t is None else np.ascontiguousarray(t) for t in (bias, res1, res2)]
    for r in opt[1:]:
        assert r is None or (r.dtype == np.float16 and r.size == m * n)
    ptrs = [_ptr(t) if t is not None else None for t in opt]
    _c().oracle_gemm_nt_fused_f16(_ptr(x2), _ptr(w), ptrs[0], ptrs[1], ptrs[2], _ptr(out), _i64(m), _i64(n), _i64(k),
                                  _i64(n), _i64(n), ctypes.c_int(1 if act == "gelu" else 0),
                                  ctypes.c_int(1 if np.dtype(out_dtype) == np.dtype(np.float32) else 0),
                                  _i64(r0), _i64(r1), _i64(c0), _i64(c1))
    return out


def gemv_fused(x, w, bias=None, res1=None, res2=None, act=None, out_dtype=np.float16):
    x = np.ascontiguousarray(x).reshape(1, -1)
    return gemm_nt_fused(x, w, bias, res1, res2, act, out_dtype)
