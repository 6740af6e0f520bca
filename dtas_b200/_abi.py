"""ctypes binding of the C ABI declared in include/dtas_b200.h.

The reference reaches its kernels through TVM packed functions (`rt_mod["cast"](x, y)`,
experiment/dtas_tuned/elementwise/cast/profile_cast.py:8-20; generated host code
experiment/dtas_tuned/elementwise/cast/top10_256/host.cc:42-131).  Here the same call is a
plain C function taking device pointers; this module owns the library handle, the prototypes
and the error translation.  There is no fallback: if the shared library is missing the import
of any op raises.
"""
import ctypes
import os

from .build import LIB_PATH

OK, EINVAL, EALIGN, ECUDA, ETIMEOUT, EUNSUPPORTED = 0, 1, 2, 3, 4, 5
F16, F32, I8 = 0, 1, 2
ACT_NONE, ACT_GELU = 0, 1

_ERR_NAMES = {
    EINVAL: "DTAS_EINVAL", EALIGN: "DTAS_EALIGN", ECUDA: "DTAS_ECUDA",
    ETIMEOUT: "DTAS_ETIMEOUT", EUNSUPPORTED: "DTAS_EUNSUPPORTED",
}


class DtasError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code, message):
        super().__init__(f"{_ERR_NAMES.get(code, code)}: {message}")
        self.code = code


_p, _i64, _i, _f = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float

# name -> (restype, argtypes); every symbol include/dtas_b200.h declares.
PROTOTYPES = {
    "dtas_cast": (_i, [_p, _p, _i64, _i64, _i, _i, _i, _p]),
    "dtas_add": (_i, [_p, _p, _p, _i64, _i64, _i, _i, _p]),
    "dtas_copy": (_i, [_p, _p, _i64, _i64, _i, _i, _p]),
    "dtas_rms_norm": (_i, [_p, _p, _p, _i64, _i64, _f, _i, _i, _p]),
    "dtas_softmax": (_i, [_p, _p, _i64, _i64, _i, _i, _p]),
    "dtas_layer_norm": (_i, [_p, _p, _p, _p, _i64, _i64, _f, _i, _i, _p]),
    "dtas_gemv": (_i, [_p, _p, _p, _p, _i64, _i64, _i, _i, _p]),
    "dtas_gemm_nt": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i, _i, _p]),
    "dtas_gemm_nt_fused": (_i, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i, _p]),
    "dtas_gemv_fused": (_i, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i, _i, _i, _i, _p]),
    "dtas_gemm_nt_static_scratch": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i, _i, _i, _p, _p]),
    "dtas_gemm_nt_static_scratch_plan": (_i, [_i64, _i64, _i64, _i, ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "dtas_bucket_of": (_i, [ctypes.c_char_p, _i64]),
    "dtas_bucket_count": (_i, [ctypes.c_char_p]),
    "dtas_variant_of": (_i, [ctypes.c_char_p, _i64, _i64, _i64, _i, ctypes.c_char_p, _i]),
    "dtas_gemm_set_override": (_i, [_i, _i]),
    "dtas_gemm_table_set": (_i, [_i64, _i64, _i64, _i64, _i, _i]),
    "dtas_gemm_table_clear": (_i, []),
    "dtas_ew_set_override": (_i, [_i, _i, _i]),
    "dtas_row_set_override": (_i, [_i]),
    "dtas_gemv_set_override": (_i, [_i, _i]),
    "dtas_set_pdl": (_i, [_i]),
    "dtas_peer_push": (_i, [_p, ctypes.POINTER(ctypes.c_void_p), _i, _i64, _i, _p]),
    "dtas_gemm_nt_scatter": (_i, [_p, _p, _p, _p, ctypes.POINTER(ctypes.c_void_p), _i, _i64, _i64, _i64, _i64, _i, _i, _p]),
    "dtas_gemm_nt_scatter_multicast": (_i, [_p, _p, _p, _p, ctypes.POINTER(ctypes.c_void_p), _i, _p, _i64, _i64, _i64, _i64,
                                            _i, _i, _p]),
    "dtas_last_error": (ctypes.c_char_p, []),
    "dtas_launch_count": (_i64, []),
    "dtas_poll_status": (_i, [_i]),
    "dtas_selftest_wait_timeout": (_i, [_i, _p, _i64]),
    "dtas_shutdown": (_i, []),
    "dtas_version": (ctypes.c_char_p, []),
}

_lib = None


def lib():
    """Loads lib/libdtas_b200.so once and installs the prototypes."""
    global _lib
    if _lib is None:
        path = os.environ.get("DTAS_B200_LIB") or LIB_PATH    # another build of the same ABI, e.g. for A/B timing
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m dtas_b200.build` "
                "(or __graft_entry__.build()); dtas_b200 has no fallback path")
        handle = ctypes.CDLL(path)
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
        _install_default_tables(handle)
    return _lib


DEFAULT_GEMM_TABLE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tables", "b200_gemm.json")


def _install_default_tables(handle):
    """Installs the shipped measured GEMM table (written by `python -m dtas_b200.retune`) unless
    DTAS_B200_NO_TABLE is set.  Shapes it does not cover fall back to the cost model."""
    if os.environ.get("DTAS_B200_NO_TABLE") or not os.path.exists(DEFAULT_GEMM_TABLE):
        return 0
    import json
    with open(DEFAULT_GEMM_TABLE) as f:
        rec = json.load(f)
    count = 0
    for shape in rec.get("gemm", []):
        for r in shape["rows"]:
            if handle.dtas_gemm_table_set(shape["n"], shape["k"], r["m_lo"], r["m_hi"], r["bn"], r["split"]) == OK:
                count += 1
    return count


def check(status):
    if status != OK:
        raise DtasError(status, lib().dtas_last_error().decode())


def bucket_of(op, m):
    return lib().dtas_bucket_of(op.encode(), int(m))


def variant_of(op, m, n, k=0, device=-1):
    buf = ctypes.create_string_buffer(128)
    check(lib().dtas_variant_of(op.encode(), int(m), int(n), int(k), int(device), buf, 128))
    return buf.value.decode()


def launch_count():
    return int(lib().dtas_launch_count())
