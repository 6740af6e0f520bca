"""Fused GEMM / GEMV tails (bias, GELU, residual adds, fp32 output) against the CPU oracle, which
restates the reference's stage-by-stage fp16 arithmetic
(experiment/ModelIR/dolly-v2-3b-q0f16/before_dl.py:163-318), and against the TVM-made fixtures.
Tolerance: the GEMM rule, 1e-2 relative to an fp32-accumulated reference (tests/util.py)."""
import numpy as np
import pytest
import torch

import oracle
from dtas_b200 import _abi, ops
from dtas_b200.reference import seeded_normal
from tests import util
from tests.golden.golden_cases import CASES, make_inputs

pytestmark = pytest.mark.gpu

TAILS = {
    "bias": dict(bias=True),
    "gelu": dict(bias=True, act="gelu"),
    "res2": dict(bias=True, residuals=2),
    "res2_f32": dict(bias=True, residuals=2, out=torch.float32),
    "res1_nobias": dict(bias=False, residuals=1),
    "gelu_res1_f32": dict(bias=True, act="gelu", residuals=1, out=torch.float32),
}


def operands(m, n, k, tail, seed, device):
    x = seeded_normal((m, k), seed, "float16")
    w = seeded_normal((n, k), seed + 1, "float16", scale=0.03)
    bias = seeded_normal((n,), seed + 2, "float16", scale=0.5) if tail.get("bias") else None
    res = [seeded_normal((m, n), seed + 3 + i, "float16") for i in range(tail.get("residuals", 0))] + [None, None]
    host = (x, w, bias, res[0], res[1])
    dev = tuple(None if t is None else t.to(device) for t in host)
    return host, dev


def expected(host, tail, rows=None, cols=None):
    x, w, bias, r1, r2 = [None if t is None else t.numpy() for t in host]
    out_dtype = np.float32 if tail.get("out") == torch.float32 else np.float16
    return oracle.gemm_nt_fused(x, w, bias, r1, r2, act=tail.get("act"), out_dtype=out_dtype, rows=rows, cols=cols)


def run_gemm(dev, tail, m, n, device, ld=None):
    out_dtype = tail.get("out", torch.float16)
    ld = ld or n
    big = torch.full((m, ld), 7.0, dtype=out_dtype, device=device)
    y = big[:, :n]
    ops.gemm_nt(dev[0], dev[1], y, bias=dev[2], res1=dev[3], res2=dev[4], act=tail.get("act"))
    ops.poll_status()
    if ld > n:
        assert bool((big[:, n:] == 7.0).all()), "wrote outside its column slab"
    return y.cpu().numpy()


@pytest.mark.parametrize("tail", sorted(TAILS))
@pytest.mark.parametrize("m,n,k", [(16, 512, 1024), (64, 384, 512), (300, 520, 264), (1100, 768, 512)])
def test_gemm_fused_tails_default_dispatch(cuda_device, tail, m, n, k):
    """Every tail through whatever kernel the dispatch picks for the shape (swapped operands at
    m <= 64, single-CTA tiles, the two-CTA kernel at m = 1100)."""
    t = TAILS[tail]
    host, dev = operands(m, n, k, t, 100 + m, cuda_device)
    got = run_gemm(dev, t, m, n, cuda_device, ld=n + 24)
    what = f"gemm {tail} m={m} n={n} k={k} [{_abi.variant_of('gemm', m, n, k)}]"
    util.assert_matmul_close(got, expected(host, t).astype(np.float32), what)
    if t.get("out") == torch.float32:   # the fp32 output is an fp16 value widened
        assert np.array_equal(got, got.astype(np.float16).astype(np.float32)), what


@pytest.mark.parametrize("bn,split", [(64, 1), (128, 3), (256, 2), (512, 1), (1024, 1), (1024, 4), (2048, 0), (4224, 0), (8320, 0)])
@pytest.mark.parametrize("tail", ["gelu", "res2_f32"])
def test_gemm_fused_tails_every_kernel(cuda_device, tail, bn, split):
    """The tail is applied in five places (direct and reduced epilogues of the tiled and swapped
    kernels, the two-CTA kernel): force each with ragged sizes."""
    t = TAILS[tail]
    m, n, k = (200, 520, 1160) if bn < 1024 or bn > 2048 else (40, 520, 1160)   # the swapped kernel takes m <= 256
    if bn == 512:
        m = 300
    host, dev = operands(m, n, k, t, 900 + bn + split, cuda_device)
    lib = _abi.lib()
    lib.dtas_gemm_table_clear()
    try:
        _abi.check(lib.dtas_gemm_set_override(bn, split))
        got = run_gemm(dev, t, m, n, cuda_device)
        what = f"gemm {tail} bn={bn} split={split} [{_abi.variant_of('gemm', m, n, k)}]"
    finally:
        lib.dtas_gemm_set_override(0, 0)
        _abi._install_default_tables(lib)
    util.assert_matmul_close(got, expected(host, t).astype(np.float32), what)


@pytest.mark.parametrize("tail", ["res2", "res1_nobias"])
def test_gemm_fused_residuals_as_own_pass(cuda_device, tail):
    """From m = 2048 up (contiguous fp16 output) the residuals are added by a streaming pass behind
    the GEMM instead of inside its epilogue; a column slab keeps them in the epilogue."""
    t = TAILS[tail]
    m, n, k = 2100, 264, 520
    host, dev = operands(m, n, k, t, 1700, cuda_device)
    want = expected(host, t).astype(np.float32)
    before = _abi.launch_count()
    got = run_gemm(dev, t, m, n, cuda_device)
    assert _abi.launch_count() - before == 2
    util.assert_matmul_close(got, want, f"gemm {tail} m={m} own pass")
    before = _abi.launch_count()
    got = run_gemm(dev, t, m, n, cuda_device, ld=n + 8)
    assert _abi.launch_count() - before == 1
    util.assert_matmul_close(got, want, f"gemm {tail} m={m} slab")


def test_gemm_fused_unaligned_falls_back(cuda_device):
    """K not a multiple of 8 (no TMA) and an odd N (no 16-byte stores or residual loads)."""
    t = TAILS["res2"]
    for m, n, k in [(9, 201, 100), (130, 201, 264)]:
        host, dev = operands(m, n, k, t, 1300 + m, cuda_device)
        got = run_gemm(dev, t, m, n, cuda_device)
        util.assert_matmul_close(got, expected(host, t).astype(np.float32), f"gemm res2 m={m} n={n} k={k}")


@pytest.mark.parametrize("bn", [128, 512])
@pytest.mark.parametrize("tail", ["bias", "gelu"])
def test_gemm_bias_at_an_odd_address(cuda_device, tail, bn):
    """The row-wise tails read the bias with 16-byte loads where its address allows; a bias that starts one
    element into a buffer takes the two-byte loads and gives the same result bit for bit (single-CTA tiles
    and the two-CTA kernel, plain and GELU tails, ragged last column chunk)."""
    t = TAILS[tail]
    m, n, k = 300, 1064, 520
    host, dev = operands(m, n, k, t, 3100 + bn, cuda_device)
    shifted = torch.empty(n + 1, dtype=torch.float16, device=cuda_device)
    shifted[1:] = dev[2]
    lib = _abi.lib()
    try:
        _abi.check(lib.dtas_gemm_set_override(bn, 1))
        got = run_gemm(dev, t, m, n, cuda_device)
        got_shifted = run_gemm((dev[0], dev[1], shifted[1:], dev[3], dev[4]), t, m, n, cuda_device)
    finally:
        lib.dtas_gemm_set_override(0, 0)
    util.assert_matmul_close(got, expected(host, t).astype(np.float32), f"gemm {tail} bn={bn}")
    util.assert_bit_exact(got_shifted, got, f"gemm {tail} bn={bn}, bias one element into its buffer")


def test_gemm_fused_linearity_in_residual(cuda_device):
    """Full-size property: y(res1) - y(0) == res1 up to fp16 rounding, at m=1024, N=K=4096."""
    m, n, k = 1024, 4096, 4096
    t = TAILS["bias"]
    host, dev = operands(m, n, k, t, 1500, cuda_device)
    r = seeded_normal((m, n), 1510, "float16").to(cuda_device)
    y0 = torch.empty((m, n), dtype=torch.float16, device=cuda_device)
    y1 = torch.empty_like(y0)
    ops.gemm_nt(dev[0], dev[1], y0, bias=dev[2])
    ops.gemm_nt(dev[0], dev[1], y1, bias=dev[2], res1=r)
    ops.poll_status()
    diff = (y1.float() - y0.float() - r.float()).abs()
    bound = 2.0 ** -10 * (y0.float().abs() + y1.float().abs()) + 1e-6   # one rounding of each result
    assert bool((diff <= bound).all()), f"max excess {(diff - bound).max().item()}"


@pytest.mark.parametrize("tail", sorted(TAILS))
@pytest.mark.parametrize("n,k", [(2560, 2560), (10240, 2560), (2560, 10240), (33, 1001)])
def test_gemv_fused_tails(cuda_device, tail, n, k):
    t = TAILS[tail]
    host, dev = operands(1, n, k, t, 2000 + n % 97, cuda_device)
    y = torch.zeros((1, n), dtype=t.get("out", torch.float16), device=cuda_device)
    ops.gemv(dev[0], dev[1], y, bias=dev[2], res1=dev[3], res2=dev[4], act=t.get("act"))
    torch.cuda.synchronize()
    util.assert_matmul_close(y.cpu().numpy(), expected(host, t).astype(np.float32), f"gemv {tail} n={n} k={k}")


@pytest.mark.parametrize("name", sorted(c for c in CASES if CASES[c]["op"] in ("gemm_fused", "gemv_fused")))
def test_fused_against_tvm_golden(cuda_device, name):
    case = CASES[name]
    ins, out = make_inputs(case)
    want = util.load_golden(case["op"])[name]
    x, w, bias, r1, r2 = [None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)
                          for a in util.fused_operands(case, ins)]
    y = torch.zeros(out.shape[1:], dtype=torch.float32 if case.get("out") == "float32" else torch.float16,
                    device=cuda_device)
    flat = lambda t: None if t is None else t.reshape(-1, t.shape[-1])   # noqa: E731
    if case["op"] == "gemv_fused":
        ops.gemv(flat(x), w, y, bias=bias, res1=flat(r1), res2=flat(r2), act=case.get("act"))
    else:
        ops.gemm_nt(flat(x), w, y, bias=bias, res1=flat(r1), res2=flat(r2), act=case.get("act"))
    ops.poll_status()
    util.assert_matmul_close(y.cpu().numpy().reshape(want.shape), want.astype(np.float32), name)


def test_fused_argument_errors(cuda_device):
    f16 = dict(dtype=torch.float16, device=cuda_device)
    x, w, y = torch.zeros((4, 64), **f16), torch.zeros((32, 64), **f16), torch.zeros((4, 32), **f16)
    r = torch.zeros((4, 32), **f16)
    with pytest.raises(_abi.DtasError):
        ops.gemm_nt(x, w, y, res2=r)                       # res2 without res1
    with pytest.raises(_abi.DtasError):
        ops.gemm_nt(x, w, y, act="relu")                   # unknown activation
    with pytest.raises(_abi.DtasError):
        ops.gemm_nt(x, w, y, res1=torch.zeros((4, 16), **f16))   # residual of the wrong shape
    with pytest.raises(_abi.DtasError):
        ops.gemm_nt(x, w, torch.zeros((4, 32), dtype=torch.int8, device=cuda_device))
    lib = _abi.lib()
    rc = lib.dtas_gemm_nt_fused(x.data_ptr(), w.data_ptr(), None, r.data_ptr(), None, y.data_ptr(), 4, 32, 64, 32, 16,
                                0, _abi.F16, _abi.F16, cuda_device.index or 0, None)
    assert rc == _abi.EINVAL and b"ldr" in lib.dtas_last_error()
