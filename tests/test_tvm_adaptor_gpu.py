"""The kernels called from a TVM runtime: as registered global functions on TVM tensors, and from a
Relax VM program through R.call_dps_packed with a symbolic row count (the reference's call path,
tuning_test/tune_cast.py:24-32).  Skipped where no CUDA-enabled TVM is importable."""
import numpy as np
import pytest
import torch

import oracle
from dtas_b200.reference import seeded_normal
from tests import util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tvm_cuda():
    try:
        from dtas_b200.workloads.tir_defs import _tvm
        tvm = _tvm()
    except ImportError:
        pytest.skip("no TVM in this environment")
    dev = tvm.cuda(0)
    if not dev.exist:
        pytest.skip("this TVM runtime has no CUDA device")
    return tvm, dev


@pytest.fixture(scope="module")
def module(tvm_cuda):
    import dtas_b200
    from dtas_b200 import Engine, arch, tvm_adaptor
    from dtas_b200.workloads import OpSpec
    dtas_b200.set_log_level(0)
    specs = [OpSpec("cast", "cast", "float32", "float16", cols=1024),
             OpSpec("rms_norm", "rms_norm", cols=1024, eps=1e-6),
             OpSpec("proj", "gemm", cols=512, k=1024, bias=True, residuals=1, act="gelu")]
    rt = Engine(1, True, None).tune_module(specs, arch=arch.B200(0), range_div_factor=256)
    return rt, tvm_adaptor.register_module(rt, prefix="dtas_b200_test")


def to_tvm(tvm, dev, a):
    make = tvm.runtime.tensor if hasattr(tvm.runtime, "tensor") else tvm.nd.array
    return make(np.ascontiguousarray(a), device=dev)


def test_registered_functions_on_tvm_tensors(cuda_device, tvm_cuda, module):
    tvm, dev = tvm_cuda
    _, names = module
    x = seeded_normal((1, 37, 1024), 1, "float32").numpy()
    y = to_tvm(tvm, dev, np.zeros((1, 37, 1024), "float16"))
    tvm.get_global_func(names["cast"])(to_tvm(tvm, dev, x), y)
    torch.cuda.synchronize()
    util.assert_bit_exact(y.numpy(), oracle.cast(x, "float16").reshape(y.shape), "cast through a TVM global function")


def test_relax_vm_calls_the_kernels(cuda_device, tvm_cuda, module):
    tvm, dev = tvm_cuda
    _, names = module
    from tvm import relax
    from tvm.script import ir as I, relax as R, tir as T

    cast_fn, norm_fn, proj_fn = names["cast"], names["rms_norm"], names["proj"]

    @I.ir_module
    class Block:
        @R.function
        def main(x: R.Tensor((1, "n", 1024), "float32"), g: R.Tensor((1024,), "float16"),
                 w: R.Tensor((512, 1024), "float16"), b: R.Tensor((512,), "float16"),
                 res: R.Tensor((1, "n", 512), "float16")) -> R.Tensor((1, "n", 512), "float16"):
            n = T.int64()
            with R.dataflow():
                h = R.call_dps_packed(cast_fn, (x,), out_sinfo=R.Tensor((1, n, 1024), "float16"))
                a = R.call_dps_packed(norm_fn, (h, g), out_sinfo=R.Tensor((1, n, 1024), "float16"))
                y = R.call_dps_packed(proj_fn, (a, w, b, res), out_sinfo=R.Tensor((1, n, 512), "float16"))
                R.output(y)
            return y

    vm = relax.VirtualMachine(relax.build(Block, target="c"), dev)
    g = seeded_normal((1024,), 3, "float16", scale=0.1, mean=1.0).numpy()
    w = seeded_normal((512, 1024), 4, "float16", scale=0.03).numpy()
    b = seeded_normal((512,), 5, "float16", scale=0.5).numpy()
    for m in (1, 19, 300):                       # one compiled program, any row count
        x = seeded_normal((1, m, 1024), 10 + m, "float32").numpy()
        res = seeded_normal((1, m, 512), 20 + m, "float16").numpy()
        y = vm["main"](*[to_tvm(tvm, dev, t) for t in (x, g, w, b, res)])
        torch.cuda.synchronize()
        h = oracle.cast(x, "float16")
        a = oracle.rms_norm(h, g, 1e-6)
        want = oracle.gemm_nt_fused(np.asarray(a).reshape(m, 1024), w, b, res.reshape(m, 512), None, act="gelu")
        util.assert_matmul_close(y.numpy().reshape(m, 512), want.astype(np.float32), f"relax block m={m}")
