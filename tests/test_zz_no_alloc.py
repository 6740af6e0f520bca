"""dtas_gemm_nt_static_scratch: the split-K GEMM for callers that cannot allocate device
memory at call time (a runtime whose pool already owns the device, a process with a memory
budget fixed at load).  Its scratch is an array inside the library image, so the test only
has to show that it computes what dtas_gemm_nt computes - twice in a row, because the array
keeps the previous call's contents - and that it refuses work that does not fit the array.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  It must pass alone in a fresh process and after the other tests.
"""
import ctypes


import pytest
import torch

from dtas_b200 import _abi
from dtas_b200.reference import seeded_normal
from tests import util


def _static(x, w, y, split_k, bias=None, status=None):
    m, k = x.shape
    n = w.shape[0]
    dev = x.device.index or 0
    st = torch.cuda.current_stream(dev).cuda_stream
    return _abi.lib().dtas_gemm_nt_static_scratch(
        x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None, y.data_ptr(),
        m, n, k, y.stride(0), split_k, _abi.F16, dev, st, status.data_ptr() if status is not None else None)


def _plan(m, n, k, split_k):
    """(return code, tile width, split) the entry point would use for this shape."""
    tile, splits = ctypes.c_int(), ctypes.c_int()
    rc = _abi.lib().dtas_gemm_nt_static_scratch_plan(m, n, k, split_k, ctypes.byref(tile), ctypes.byref(splits))
    return rc, tile.value, splits.value


def _dynamic(x, w, y, bias=None):
    m, k = x.shape
    n = w.shape[0]
    dev = x.device.index or 0
    st = torch.cuda.current_stream(dev).cuda_stream
    return _abi.lib().dtas_gemm_nt(x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
                                   y.data_ptr(), m, n, k, y.stride(0), _abi.F16, dev, st)


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,split_k", [(16, 4096, 4096, 4), (64, 1000, 2120, 3), (200, 512, 4096, 0)])
def test_static_scratch_matches_workspace_gemm_twice(cuda_device, m, n, k, split_k):
    x = seeded_normal((m, k), 7000 + m, "float16").to(cuda_device)
    w = seeded_normal((n, k), 7001 + n, "float16", scale=0.02).to(cuda_device)
    b = seeded_normal((n,), 7002, "float16", scale=0.1).to(cuda_device)
    want = torch.empty((m, n), dtype=torch.float16, device=cuda_device)
    rc, _, planned = _plan(m, n, k, split_k)
    assert rc == _abi.OK
    # every case here goes through the array: with split_k = 0 the library's own choice is a real split
    assert planned > 1 and (split_k == 0 or planned == split_k)
    # the existing entry point, forced to the same split so both run the same arithmetic
    _abi.check(_abi.lib().dtas_gemm_set_override(0, planned))
    try:
        _abi.check(_dynamic(x, w, want, bias=b))
        _abi.check(_abi.lib().dtas_poll_status(0))
    finally:
        _abi.check(_abi.lib().dtas_gemm_set_override(0, 0))
    ref32 = x.float().cpu().numpy() @ w.float().cpu().numpy().T + b.float().cpu().numpy()
    util.assert_matmul_close(want.cpu().numpy(), ref32, "workspace gemm vs fp32")
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    for call in (1, 2):                       # the second call sees the first call's leftovers
        got = torch.full((m, n), float("nan"), dtype=torch.float16, device=cuda_device)
        _abi.check(_static(x, w, got, split_k, bias=b, status=status))
        torch.cuda.synchronize()
        assert int(status.item()) == 0, f"a bounded wait gave up (code {int(status.item()):#x})"
        util.assert_matmul_close(got.cpu().numpy(), want.float().cpu().numpy(), f"static scratch call {call} vs dtas_gemm_nt")
        util.assert_matmul_close(got.cpu().numpy(), ref32, f"static scratch call {call} vs fp32")
    # without a status word of the caller's, the code would sit in the library's own array, where
    # dtas_poll_status looks for it; after clean calls there is nothing to report
    got = torch.full((m, n), float("nan"), dtype=torch.float16, device=cuda_device)
    _abi.check(_static(x, w, got, split_k, bias=b, status=None))
    _abi.check(_abi.lib().dtas_poll_status(0))
    util.assert_matmul_close(got.cpu().numpy(), ref32, "static scratch with the built-in status word vs fp32")


def test_static_scratch_rejects_what_does_not_fit():
    """Argument checks run before any device is touched, so this part needs no GPU."""
    lib = _abi.lib()
    buf = (ctypes.c_char * 64)()
    p = ctypes.addressof(buf) & ~15
    # 4 slices of a 255 x 22016 fp32 tile = 90 MB > the 8 MiB built into the library
    rc = lib.dtas_gemm_nt_static_scratch(p, p, None, p, 255, 22016, 4096, 22016, 4, _abi.F16, 0, None, None)
    assert rc == _abi.EINVAL
    msg = lib.dtas_last_error().decode()
    assert "needs" in msg and "built-in" in msg
    assert lib.dtas_gemm_nt_static_scratch(p, p, None, p, 0, 8, 8, 8, 0, _abi.F16, 0, None, None) == _abi.EINVAL
    assert lib.dtas_gemm_nt_static_scratch(None, p, None, p, 1, 8, 8, 8, 0, _abi.F16, 0, None, None) == _abi.EINVAL
    assert lib.dtas_gemm_nt_static_scratch(p, p, None, p, 4, 8, 12, 8, 0, _abi.F16, 0, None, None) == _abi.EALIGN
    assert lib.dtas_gemm_nt_static_scratch(p, p, None, p, 4, 8, 8, 8, 65, _abi.F16, 0, None, None) == _abi.EINVAL


def test_static_scratch_plan_always_fits_when_the_library_chooses():
    """split_k = 0 is never refused for size: the split is lowered until the partial sums fit 8 MiB and
    1024 counters.  The global override and the measured table do not reach this entry point."""
    lib = _abi.lib()
    for m, n, k in [(255, 22016, 4096), (255, 4096, 4096), (512, 12288, 4096), (16, 4096, 4096), (200, 512, 4096),
                    (8192, 22016, 4096), (1, 8, 8)]:
        rc, tile, splits = _plan(m, n, k, 0)
        assert rc == _abi.OK and tile in (64, 128, 256) and splits >= 1
        n_pad = -(-n // tile) * tile
        tiles = -(-m // 128) * (n_pad // tile)
        assert splits == 1 or (splits * m * n_pad * 4 <= 8 << 20 and tiles <= 1024)
    assert _plan(200, 512, 4096, 0)[2] > 1             # a shape where the library's own choice is a real split
    before = _plan(16, 4096, 4096, 0)
    _abi.check(lib.dtas_gemm_set_override(256, 8))
    _abi.check(lib.dtas_gemm_table_set(4096, 4096, 1, 64, 128, 16))
    try:
        assert _plan(16, 4096, 4096, 0) == before
    finally:
        _abi.check(lib.dtas_gemm_set_override(0, 0))
        lib.dtas_gemm_table_clear()
        _abi._install_default_tables(lib)
    assert _plan(255, 22016, 4096, 4)[0] == _abi.EINVAL
