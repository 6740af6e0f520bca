"""C-ABI checks that need no GPU: the library loads, exports everything the header declares,
and rejects bad arguments before it touches a device."""
import ctypes
import os
import re

import pytest

from dtas_b200 import _abi
from dtas_b200.build import LIB_PATH, build_library

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build_library()
    return _abi.lib()


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "dtas_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(dtas_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_abi.PROTOTYPES), (declared ^ set(_abi.PROTOTYPES))
    raw = ctypes.CDLL(LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), f"{name} is declared in include/dtas_b200.h but not exported"
    assert lib.dtas_version().decode().startswith("dtas_b200")


def test_bucket_index_is_total_monotone_and_clamped(lib):
    # bucket = min((m-1)/256, last): 1-based ranges, no off-by-one at multiples of the width
    assert _abi.bucket_of("cast", 1) == 0
    assert _abi.bucket_of("cast", 256) == 0
    assert _abi.bucket_of("cast", 257) == 1
    assert _abi.bucket_of("gemm", 4096) == 15
    count = lib.dtas_bucket_count(b"gemm")
    assert count == 32
    prev = 0
    for m in range(1, 2 * 8192 + 2, 7):
        b = _abi.bucket_of("gemm", m)
        assert 0 <= b < count and b >= prev
        prev = b
    assert _abi.bucket_of("gemm", 10 ** 9) == count - 1          # clamp above the bound
    assert _abi.bucket_of("gemm", 0) == -1 and _abi.bucket_of("gemm", -5) == -1
    assert _abi.bucket_of("nonsense", 5) == -1


def test_variant_names(lib):
    lib.dtas_gemm_table_clear()          # the cost model's own choices, not a shipped table's
    assert _abi.variant_of("cast", 1, 4096) == "ew_vec16_unroll1"
    assert _abi.variant_of("add", 8192, 11008) == "ew_vec16_unroll1"     # two loads per vector already
    assert _abi.variant_of("copy", 8192, 11008) == "ew_vec16_unroll2"
    assert _abi.variant_of("copy", 1, 11008) == "ew_vec16_unroll1"
    assert "softmax_regs" in _abi.variant_of("softmax", 4096, 4096)
    assert "generic" in _abi.variant_of("rms_norm", 4, 101)
    assert _abi.variant_of("gemv", 1, 4096, 4096) == "gemv_stream_s16_rows1"       # 33.5 MB: the streaming kernel
    assert _abi.variant_of("gemv", 1, 32000, 2560) == "gemv_stream_s16_rows2"     # short rows: 16 shallow stages
    assert _abi.variant_of("gemv", 1, 32000, 4096) == "gemv_stream_s8_rows2"      # long band: two 8 KB rows per copy
    assert _abi.variant_of("gemv", 1, 4096, 11008) == "gemv_stream_s8_rows1"
    assert _abi.variant_of("gemv", 1, 512, 4096).startswith("gemv_vec16")          # 4 MB: the per-row kernel
    assert _abi.variant_of("gemv", 1, 4096, 16384).startswith("gemv_vec16")        # a row does not fit a stage
    assert _abi.variant_of("gemm", 8192, 22016, 4096) == "gemm_tcgen05_2cta_bm256_bn256_bk64_s6"
    assert _abi.variant_of("gemm", 16, 22016, 4096).startswith("gemm_tcgen05_swap_n128_m16")
    assert _abi.variant_of("gemm", 255, 22016, 4096).startswith("gemm_tcgen05_bm128_bn")
    assert _abi.variant_of("gemm", 33, 70, 101) == "gemm_simt_fallback"
    with pytest.raises(_abi.DtasError):
        _abi.variant_of("nope", 1, 1)
    _abi._install_default_tables(lib)


def test_gemm_table_overrides_cost_model(lib):
    lib.dtas_gemm_table_clear()
    try:
        base = _abi.variant_of("gemm", 16, 4096, 4096)
        assert lib.dtas_gemm_table_set(4096, 4096, 1, 32, 128, 2) == _abi.OK
        assert _abi.variant_of("gemm", 16, 4096, 4096) == "gemm_tcgen05_bm128_bn128_bk64_s6_splitk2"
        assert _abi.variant_of("gemm", 33, 4096, 4096) == _abi.variant_of("gemm", 33, 4096, 4096)
        assert _abi.variant_of("gemm", 16, 4096, 11008) != "gemm_tcgen05_bm128_bn128_bk64_s6_splitk2"   # other shape untouched
        assert lib.dtas_gemm_set_override(256, 1) == _abi.OK                       # the global override wins
        assert _abi.variant_of("gemm", 16, 4096, 4096) == "gemm_tcgen05_bm128_bn256_bk64_s4_splitk1"
        lib.dtas_gemm_set_override(0, 0)
        assert lib.dtas_gemm_table_set(4096, 4096, 0, 32, 128, 2) == _abi.EINVAL
        assert lib.dtas_gemm_table_set(4096, 4096, 1, 32, 100, 2) == _abi.EINVAL
        lib.dtas_gemm_table_clear()
        assert _abi.variant_of("gemm", 16, 4096, 4096) == base
    finally:
        lib.dtas_gemm_set_override(0, 0)
        lib.dtas_gemm_table_clear()
        _abi._install_default_tables(lib)


def test_argument_validation_needs_no_device(lib):
    buf = (ctypes.c_char * 64)()
    p = ctypes.addressof(buf)
    # m <= 0 is rejected (the reference asserts dynamic dims > 0)
    assert lib.dtas_cast(p, p, 0, 4096, _abi.F32, _abi.F16, 0, None) == _abi.EINVAL
    assert b"m must be > 0" in lib.dtas_last_error()
    assert lib.dtas_add(p, p, p, -3, 8, _abi.F16, 0, None) == _abi.EINVAL
    assert lib.dtas_copy(p, p, 1, 0, _abi.F16, 0, None) == _abi.EINVAL
    assert lib.dtas_copy(p, p, 1, 8, 99, 0, None) == _abi.EUNSUPPORTED
    # null pointers
    assert lib.dtas_cast(None, p, 1, 8, _abi.F32, _abi.F16, 0, None) == _abi.EINVAL
    assert b"NULL" in lib.dtas_last_error()
    assert lib.dtas_rms_norm(p, None, p, 1, 8, 1e-6, _abi.F16, 0, None) == _abi.EINVAL
    assert lib.dtas_softmax(p, p, 0, 8, _abi.F16, 0, None) == _abi.EINVAL
    assert lib.dtas_gemv(p, p, None, p, 0, 8, _abi.F16, 0, None) == _abi.EINVAL
    assert lib.dtas_gemv(p, p, None, p, 8, 8, _abi.F32, 0, None) == _abi.EUNSUPPORTED
    assert lib.dtas_gemm_nt(p, p, None, p, 0, 8, 8, 8, _abi.F16, 0, None) == _abi.EINVAL
    assert lib.dtas_gemm_nt(p, p, None, p, 4, 8, 8, 4, _abi.F16, 0, None) == _abi.EINVAL   # ldy < n
    assert lib.dtas_gemm_set_override(100, 0) == _abi.EINVAL
    assert lib.dtas_gemm_set_override(0, 0) == _abi.OK
    with pytest.raises(_abi.DtasError) as e:
        _abi.check(lib.dtas_cast(p, p, -1, 8, _abi.F32, _abi.F16, 0, None))
    assert e.value.code == _abi.EINVAL


def test_ops_reject_cpu_tensors():
    import torch
    from dtas_b200 import ops
    a = torch.zeros(2, 8)
    with pytest.raises(_abi.DtasError):
        ops.cast(a, torch.zeros(2, 8, dtype=torch.float16))
    with pytest.raises(_abi.DtasError):
        ops.gemm_nt(a.half(), a.half(), torch.zeros(2, 2, dtype=torch.float16))


def test_shipped_gemm_table_installs_and_decides(lib):
    """Every row of the shipped measured table is accepted, the ranges of a shape tile 1 .. 2^30
    without gaps, and with the table installed the dispatch answers with the row's variant.  It
    covers the Llama-2-7B shapes with their column shards and the reference model's own weight
    shapes (experiment/ModelIR/dolly-v2-3b-q0f16/before_dl.py: hidden size 2560, vocabulary 50280)."""
    import json
    with open(_abi.DEFAULT_GEMM_TABLE) as f:
        rec = json.load(f)
    shapes = {(s["n"], s["k"]): s["rows"] for s in rec["gemm"]}
    for nk in [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008), (2752, 4096), (512, 11008),
               (7680, 2560), (2560, 2560), (10240, 2560), (2560, 10240), (50280, 2560)]:
        assert nk in shapes, nk
    lib.dtas_gemm_table_clear()
    try:
        assert _abi._install_default_tables(lib) == sum(len(r) for r in shapes.values())
        for (n, k), rows in shapes.items():
            assert rows[0]["m_lo"] == 1 and rows[-1]["m_hi"] == 1 << 30
            for a, b in zip(rows, rows[1:]):
                assert b["m_lo"] == a["m_hi"] + 1
            for r in rows:
                m = min(r["m_hi"], 8192)
                got = _abi.variant_of("gemm", m, n, k)
                # the padded-m suffix of the swapped kernel depends on m inside the range, and the ring depth
                # in a name (_s<stages>) is a property of the build, not of the choice
                norm = lambda v: re.sub(r"_s\d+", "", v.split("_m")[0])
                assert norm(got) == norm(r["variant"]), (n, k, m, got, r["variant"])
    finally:
        lib.dtas_gemm_table_clear()
        _abi._install_default_tables(lib)


def test_a_new_table_range_overrides_the_shipped_ranges(lib):
    """A freshly tuned range wins over whatever an earlier table held for the same weight shape, whatever
    ranges that table used: overlapping entries are trimmed, the part outside the new range survives."""
    lib.dtas_gemm_table_clear()
    _abi._install_default_tables(lib)
    try:
        shipped_16 = _abi.variant_of("gemm", 16, 12288, 4096)
        shipped_300 = _abi.variant_of("gemm", 300, 12288, 4096)
        _abi.check(lib.dtas_gemm_table_set(12288, 4096, 1, 256, 256, 1))
        assert _abi.variant_of("gemm", 16, 12288, 4096) == "gemm_tcgen05_bm128_bn256_bk64_s4_splitk1" != shipped_16
        assert _abi.variant_of("gemm", 256, 12288, 4096) == "gemm_tcgen05_bm128_bn256_bk64_s4_splitk1"
        assert _abi.variant_of("gemm", 300, 12288, 4096) == shipped_300      # outside the new range: untouched
        # a range cut out of the middle of an entry leaves both ends in place
        lib.dtas_gemm_table_clear()
        _abi.check(lib.dtas_gemm_table_set(1024, 1024, 1, 1000, 128, 1))
        _abi.check(lib.dtas_gemm_table_set(1024, 1024, 100, 200, 64, 1))
        assert "bn128" in _abi.variant_of("gemm", 50, 1024, 1024)
        assert "bn64" in _abi.variant_of("gemm", 150, 1024, 1024)
        assert "bn128" in _abi.variant_of("gemm", 500, 1024, 1024)
    finally:
        lib.dtas_gemm_table_clear()
        _abi._install_default_tables(lib)


def test_reference_import_lines_resolve():
    """The import lines of the reference's driver scripts (tuning_test/tune_cast.py:35-36 and the
    package surface python/dtas/__init__.py:1-8) resolve to this library."""
    import dtas
    from dtas.arch import B200, RTX3090
    from dtas.codegen.runtime_packer import load_module_from_file
    from dtas.common.config import Config
    from dtas.engine.tuner import Engine
    import dtas_b200
    assert Engine is dtas_b200.Engine and load_module_from_file is dtas_b200.load_module_from_file
    assert RTX3090(7).dev_id == 7 and B200(0).num_sm == 148 and Config is dtas_b200.Config
    dtas.set_log_level(dtas.get_log_level())
