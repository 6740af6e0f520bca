"""GPU parity against the reference's own PrimFunc text.

Each test loads one IRModule fixture (the `@I.ir_module class Module` of a reference file, parsed by
TVM and stored by tests/golden/make_ref_golden.py), hands that module object to the engine through the
reference's own import lines and call shape (tuning_test/tune_cast.py:35-43):

    from dtas.engine.tuner import Engine
    from dtas.arch import RTX3090
    rt_mod = Engine(1, parallel_build=True, work_dir=...).tune_module(mod, arch=..., range_div_factor=256)
    rt_mod["cast"](x, y)

and compares the result with what a TVM build of the same text produced on the same seeded inputs.

Rules:
  * cast fp16->fp32, int8 add, fp32 copy: bit for bit - the SHA-256 of the whole device output equals
    the recorded one, and the kept rows are compared element by element;
  * layer norm, softmax: 1e-3 relative + 1 fp16 ULP on the kept rows;
  * NT matmul + bias (GEMM N = 10240, K = 2560; GEMV N = 2560, K = 10240).  The reference text
    accumulates in fp16; the kernels here accumulate in fp32, which the parity rule of this library
    names as the yardstick.  So two checks: (1) 1e-2 relative (+ 1e-2 rms floor) against the
    fp32-accumulated oracle; (2) against the reference-text vectors with the error an fp16 accumulator
    makes added to the bound: every one of the K updates rounds the running sum to fp16, a random walk
    of sigma = ULP_fp16(rms) * sqrt(K / 12), taken at eight sigma (tests/util.py:fp16_accumulation_bound).
"""
import hashlib
import json
import os
import tempfile

import numpy as np
import pytest
import torch

import oracle
from tests import util
from tests.golden.ref_cases import EXACT, SOURCES, make_inputs, n_values

pytestmark = pytest.mark.gpu


def _tvm():
    try:
        import tilelang  # noqa: F401
        from tilelang import tvm
        return tvm
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"no TVM to load the IRModule fixtures with: {e}")


_modules = {}


def _runtime_module(key):
    """Engine.tune_module on the fixture module, once per key; called as the reference's scripts do."""
    if key not in _modules:
        tvm = _tvm()
        from dtas.arch import B200
        from dtas.engine.tuner import Engine
        with open(os.path.join(util.GOLDEN_DIR, "ref_modules", f"{key}.json")) as f:
            mod = tvm.ir.load_json(f.read())
        work_dir = tempfile.mkdtemp(prefix=f"dtas_ref_{key}_")
        engine = Engine(1, parallel_build=True, work_dir=work_dir)
        _modules[key] = (engine.tune_module(mod, arch=B200(0), range_div_factor=256), work_dir)
    return _modules[key]


CASES = [(k, n) for k in SOURCES for n in n_values(k)]


@pytest.mark.parametrize("key,n", CASES, ids=[f"{k}-n{n}" for k, n in CASES])
def test_reference_module_on_gpu(key, n, cuda_device):
    rt_mod, _ = _runtime_module(key)
    func = SOURCES[key]["func"]
    with open(os.path.join(util.GOLDEN_DIR, "ref_golden_meta.json")) as f:
        meta = json.load(f)[key]["cases"][str(n)]
    ins, out = make_inputs(key, n)
    dev_ins = [torch.from_numpy(a).to(cuda_device) for a in ins]
    dev_out = torch.full(out.shape, 77, dtype=torch.from_numpy(out).dtype, device=cuda_device)
    rt_mod[func](*dev_ins, dev_out)
    torch.cuda.synchronize()
    got_full = dev_out.cpu().numpy()
    assert list(got_full.shape) == meta["shape"] and str(got_full.dtype) == meta["dtype"]
    gold = util.load_ref_golden(key)
    want, rows = gold[f"n{n}"], gold[f"n{n}_rows"]
    got = got_full.reshape(-1, got_full.shape[-1])[rows]
    what = f"{SOURCES[key]['path']}:{func} n={n}"
    if key in EXACT:
        util.assert_bit_exact(got, want, what)
        assert hashlib.sha256(np.ascontiguousarray(got_full).tobytes()).hexdigest() == meta["output_sha256"], what
    elif key in ("layer_norm", "softmax"):
        util.assert_reduction_close(got, want, what, abs_floor=1e-6 if key == "layer_norm" else 0.0)
    else:
        x = ins[0].reshape(-1, ins[0].shape[-1])
        k = x.shape[1]
        x_rows = np.ascontiguousarray(x[rows])
        exact = oracle.gemm_nt(x_rows, ins[1], bias=ins[2]).astype(np.float32)
        util.assert_matmul_close(got, exact, what + " vs fp32-accumulated oracle")
        w32 = want.astype(np.float32)
        rms = float(np.sqrt(np.mean(w32.astype(np.float64) ** 2)))
        tol = 1e-2 * np.abs(w32) + 1e-2 * rms + util.fp16_accumulation_bound(k, rms)
        err = np.abs(got.astype(np.float32) - w32)
        assert (err <= tol).all(), f"{what}: worst {err.max()} against bound {tol[err.argmax()]} (rms {rms})"
        # the reference-text vectors themselves sit inside the same model around the exact result
        assert (np.abs(w32 - exact) <= 1e-2 * rms + util.fp16_accumulation_bound(k, rms)).all()


def test_reference_script_flow(cuda_device):
    """The remaining lines of the reference's driver scripts: a reloaded module from work_dir and the
    timing call (tuning_test/tune_cast.py:44-58, experiment/dtas_tuned/elementwise/cast/profile_cast.py:8-20)."""
    from dtas.codegen.runtime_packer import load_module_from_file
    rt_mod, work_dir = _runtime_module("cast")
    again = load_module_from_file(work_dir)
    x = torch.rand((1, 100, 2560), device=cuda_device).to(torch.float16)
    y = torch.empty((1, 100, 2560), dtype=torch.float32, device=cuda_device)
    again["cast"](x, y)
    assert torch.equal(y, x.float())
    timer = rt_mod.time_evaluator(func_name="cast", dev=cuda_device, number=5, min_repeat_ms=5)
    res = timer(x, y)
    assert res.mean > 0 and res.min <= res.mean
