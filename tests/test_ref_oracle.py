"""Pins the C oracle against the reference's own PrimFunc text, as built by TVM for the CPU
(tests/golden/make_ref_golden.py writes the fixtures from the reference files; their paths, line
spans and text hashes are in tests/golden/ref_golden_meta.json).  CPU only.

  * cast fp16->fp32 (tuning_test/tune_cast.py), int8 add (tune_ele_add.py), fp32 copy
    (tune_ele_copy.py): bit for bit on the kept rows, and the SHA-256 of the whole oracle output
    equals the one recorded from the TVM build;
  * NT matmul + bias with the fp16 accumulator the reference declares (experiment/testIR/GEMM/dlight.py,
    experiment/testIR/GEMV/m1n2560k10240/dlight_gemv.py): bit for bit;
  * layer norm and softmax (experiment/dtas_tuned/general_reduction/*/profile_dlight.py): to
    rounding (TVM's C backend prints fp32 constants with 7 digits).
"""
import hashlib
import json
import os
import zlib

import numpy as np
import pytest

import oracle
from tests import util
from tests.golden.ref_cases import EXACT, SOURCES, make_inputs, n_values


def _meta():
    with open(os.path.join(util.GOLDEN_DIR, "ref_golden_meta.json")) as f:
        return json.load(f)


def run_oracle(key, ins, rows=None):
    """Oracle output of one reference PrimFunc as [rows, cols]; `rows` restricts a matmul to the rows
    a fixture keeps (rows are independent in every PrimFunc)."""
    if key == "cast":
        out = oracle.cast(ins[0], np.float32)
    elif key == "add":
        out = oracle.add(ins[0], ins[1])
    elif key == "copy":
        out = oracle.copy(ins[0])
    elif key == "layer_norm":
        out = oracle.layer_norm(ins[0], ins[1], ins[2], 1e-5)
    elif key == "softmax":
        out = oracle.softmax(ins[0])
    elif key in ("gemm", "gemv"):
        x = ins[0].reshape(-1, ins[0].shape[-1])
        if rows is not None:
            x = np.ascontiguousarray(x[rows])
        return oracle.gemm_nt_f16acc(x, ins[1], ins[2])
    else:
        raise KeyError(key)
    out = out.reshape(-1, out.shape[-1])
    return out if rows is None else out[rows]


CASES = [(k, n) for k in SOURCES for n in n_values(k)]


@pytest.mark.parametrize("key,n", CASES, ids=[f"{k}-n{n}" for k, n in CASES])
def test_oracle_matches_reference_text(key, n):
    meta = _meta()[key]["cases"][str(n)]
    ins, _ = make_inputs(key, n)
    crcs = [zlib.crc32(np.ascontiguousarray(a).tobytes()) for a in ins]
    assert crcs == meta["input_crc32"], "seeded inputs differ from the ones the fixture was made with"
    gold = util.load_ref_golden(key)
    want, rows = gold[f"n{n}"], gold[f"n{n}_rows"]
    if key in EXACT:
        full = run_oracle(key, ins)
        util.assert_bit_exact(full[rows], want, f"{key} n={n}")
        assert hashlib.sha256(np.ascontiguousarray(full).tobytes()).hexdigest() == meta["output_sha256"]
    elif key in ("gemm", "gemv"):
        util.assert_bit_exact(run_oracle(key, ins, rows), want, f"{key} n={n}")
    else:
        got = run_oracle(key, ins, rows)
        abs_floor = 1e-6 if key == "layer_norm" else 0.0
        util.assert_reduction_close(got, want, f"{key} n={n}", abs_floor=abs_floor)
        mism = np.mean(util.bits(got) != util.bits(want))
        assert mism < 0.02, f"{key} n={n}: {mism:.3%} of elements differ from the TVM build by an fp16 ULP"


def _tvm():
    try:
        import tilelang  # noqa: F401
        from tilelang import tvm
        return tvm
    except Exception:  # noqa: BLE001
        return None


@pytest.mark.parametrize("key", sorted(SOURCES))
def test_module_fixture_is_the_reference_text(key):
    """The IRModule fixtures the GPU tests hand to Engine.tune_module are the reference's text: the hash
    of the text cut from the reference file equals the recorded one and parsing it gives a module
    structurally equal to the fixture.  Needs a checkout of the reference and a TVM."""
    tree, tvm = util.reference_tree(), _tvm()
    if tree is None or tvm is None:
        pytest.skip("no checkout of the reference, or no TVM")
    from tests.golden import make_ref_golden as gen
    meta = _meta()[key]
    text, span = gen.module_text(os.path.join(tree, meta["source"]))
    assert list(span) == meta["lines"]
    assert hashlib.sha256(text.encode()).hexdigest() == meta["module_text_sha256"]
    parsed = gen.parse_module(text, f"chk_{key}")
    with open(os.path.join(util.GOLDEN_DIR, "ref_modules", f"{key}.json")) as f:
        stored = tvm.ir.load_json(f.read())
    tvm.ir.assert_structural_equal(parsed, stored)


@pytest.mark.parametrize("key", sorted(SOURCES))
def test_engine_classifies_the_reference_modules(key):
    """Engine.tune_module, called the way the reference's scripts call it (tuning_test/tune_cast.py:35-43),
    binds each reference PrimFunc to the operator, dtypes and static dims its text states."""
    tvm = _tvm()
    if tvm is None:
        pytest.skip("no TVM")
    from dtas.arch import RTX3090
    from dtas.engine.tuner import Engine
    with open(os.path.join(util.GOLDEN_DIR, "ref_modules", f"{key}.json")) as f:
        mod = tvm.ir.load_json(f.read())
    rt_mod = Engine(1, parallel_build=True, work_dir=None).tune_module(mod, arch=RTX3090(7), range_div_factor=256)
    spec = rt_mod[SOURCES[key]["func"]].spec
    want = {
        "cast": ("cast", "float16", "float32", 2560, 0), "add": ("add", "int8", "int8", 2560, 0),
        "copy": ("copy", "float32", "float32", 2560, 0), "layer_norm": ("layer_norm", "float32", "float16", 2560, 0),
        "softmax": ("softmax", "float32", "float16", 0, 0), "gemm": ("gemm", "float16", "float16", 10240, 2560),
        "gemv": ("gemv", "float16", "float16", 2560, 10240),
    }[key]
    assert (spec.op, spec.in_dtype, spec.out_dtype, spec.cols, spec.k) == want
    if key in ("gemm", "gemv"):
        assert spec.bias and not spec.residuals and not spec.act
    if key == "layer_norm":
        assert abs(spec.eps - 1e-5) < 1e-12
