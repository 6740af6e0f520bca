"""Pins the C oracle (oracle/dtas_oracle.c) against the golden fixtures, i.e. against the
workload PrimFuncs as built by TVM (tests/golden/make_golden.py).  CPU only."""
import json
import os
import zlib

import numpy as np
import pytest

import oracle
from tests import util
from tests.golden.golden_cases import CASES, make_inputs

EXACT_OPS = {"cast", "add", "copy"}


def run_oracle(case, ins):
    op = case["op"]
    if op == "cast":
        return oracle.cast(ins[0], case["dst"])
    if op == "add":
        return oracle.add(ins[0], ins[1])
    if op == "copy":
        return oracle.copy(ins[0])
    if op == "rms_norm":
        return oracle.rms_norm(ins[0], ins[1], case["eps"])
    if op in ("softmax", "softmax_dyn"):
        return oracle.softmax(ins[0])
    if op == "layer_norm":
        return oracle.layer_norm(ins[0], ins[1], ins[2], case["eps"])
    if op == "gemv":
        return oracle.gemv(ins[0], ins[1])
    if op == "gemm":
        return oracle.gemm_nt(ins[0], ins[1])
    if op in ("gemm_fused", "gemv_fused"):
        return oracle.gemm_nt_fused(*util.fused_operands(case, ins), act=case.get("act"),
                                    out_dtype=case.get("out", "float16"))
    raise ValueError(op)


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_tvm_golden(name):
    case = CASES[name]
    ins, _ = make_inputs(case)
    with open(os.path.join(util.GOLDEN_DIR, "golden_meta.json")) as f:
        meta = json.load(f)
    crcs = [zlib.crc32(np.ascontiguousarray(a).tobytes()) for a in ins]
    assert crcs == meta[name]["input_crc32"], "seeded inputs differ from the ones the fixture was made with"
    want = util.load_golden(case["op"])[name]
    got = np.asarray(run_oracle(case, ins)).reshape(want.shape)
    if case["op"] in EXACT_OPS:
        util.assert_bit_exact(got, want, name)
    elif case["op"] in ("gemv", "gemm"):
        # Same k-ordered fp32 accumulation as TVM's C output: identical bits expected.
        util.assert_bit_exact(got, want, name)
    elif case["op"] in ("gemm_fused", "gemv_fused"):
        # The tail is restated stage by stage with the reference's fp16 rounding: identical bits,
        # except where libm's erff and the one TVM's build linked differ in the last place.
        if case.get("act"):
            util.assert_matmul_close(got, want.astype(np.float32), name)
            assert np.mean(util.bits(got) != util.bits(want)) < 1e-3
        else:
            util.assert_bit_exact(got, want, name)
    else:
        # TVM's C backend prints fp32 constants with 7 significant digits (1/H is not exact
        # in its output), so the reductions agree to rounding, not bit for bit.
        util.assert_reduction_close(got, want, name)
        mism = np.mean(util.bits(got) != util.bits(want))
        assert mism < 0.02, f"{name}: {mism:.3%} of elements differ from the TVM build by an fp16 ULP"


def test_thread_count_does_not_change_results():
    case = CASES["softmax_m33"]
    ins, _ = make_inputs(case)
    oracle.set_threads(1)
    a = oracle.softmax(ins[0])
    oracle.set_threads(oracle.max_threads() if oracle.max_threads() > 1 else 4)
    b = oracle.softmax(ins[0])
    util.assert_bit_exact(a, b, "softmax 1 thread vs many")
