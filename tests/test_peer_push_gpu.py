"""dtas_peer_push on one GPU: the destinations are ordinary buffers of the same device, which the
kernel cannot tell from mapped peer memory.  Bit-exact copies, ragged byte counts, argument errors.
The two-GPU path (real peer buffers) is in tests/test_dist_gpu.py."""
import ctypes

import pytest
import torch

from dtas_b200 import _abi, ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_dsts", [1, 3, 7])
@pytest.mark.parametrize("numel", [8, 4096, 1 << 20, (1 << 22) + 8])
def test_peer_push_copies_to_every_destination(cuda_device, n_dsts, numel):
    g = torch.Generator(device=cuda_device).manual_seed(numel + n_dsts)
    src = torch.randn(numel, generator=g, device=cuda_device).half()
    dsts = [torch.zeros_like(src) for _ in range(n_dsts)]
    before = _abi.launch_count()
    ops.peer_push(src, dsts)
    torch.cuda.synchronize()
    assert _abi.launch_count() - before == 1
    for d in dsts:
        assert torch.equal(d.view(torch.int16), src.view(torch.int16))


def test_peer_push_ragged_bytes_and_guard_band(cuda_device):
    """A byte count that is not a multiple of 16, and nothing written past it."""
    lib = _abi.lib()
    src = torch.arange(0, 256, dtype=torch.uint8, device=cuda_device).repeat(5)          # 1280 bytes
    dsts = [torch.full((1280,), 0xEE, dtype=torch.uint8, device=cuda_device) for _ in range(2)]
    nbytes = 1000 + 7
    ptrs = (ctypes.c_void_p * 2)(*[d.data_ptr() for d in dsts])
    _abi.check(lib.dtas_peer_push(src.data_ptr(), ptrs, 2, nbytes, cuda_device.index or 0, None))
    torch.cuda.synchronize()
    for d in dsts:
        assert torch.equal(d[:nbytes], src[:nbytes])
        assert bool((d[nbytes:] == 0xEE).all())


def test_peer_push_argument_errors(cuda_device):
    lib = _abi.lib()
    dev = cuda_device.index or 0
    src = torch.zeros(64, dtype=torch.float16, device=cuda_device)
    dst = torch.zeros(80, dtype=torch.float16, device=cuda_device)
    one = (ctypes.c_void_p * 1)(dst.data_ptr())
    assert lib.dtas_peer_push(src.data_ptr(), one, 0, 128, dev, None) == _abi.EINVAL
    assert lib.dtas_peer_push(src.data_ptr(), one, 8, 128, dev, None) == _abi.EINVAL
    assert lib.dtas_peer_push(src.data_ptr(), one, 1, 0, dev, None) == _abi.EINVAL
    assert lib.dtas_peer_push(None, one, 1, 128, dev, None) == _abi.EINVAL
    odd = (ctypes.c_void_p * 1)(dst.data_ptr() + 2)
    assert lib.dtas_peer_push(src.data_ptr(), odd, 1, 128, dev, None) == _abi.EALIGN
    same = (ctypes.c_void_p * 1)(src.data_ptr())
    assert lib.dtas_peer_push(src.data_ptr(), same, 1, 128, dev, None) == _abi.EINVAL
    with pytest.raises(_abi.DtasError):
        ops.peer_push(src, [dst])                       # another size


@pytest.mark.parametrize("m,n,k,n_peers", [(129, 512, 1024, 1), (300, 1000, 2120, 3), (1024, 2752, 4096, 7), (2500, 520, 264, 2)])
def test_gemm_scatter_writes_every_peer(cuda_device, m, n, k, n_peers):
    """dtas_gemm_nt_scatter on one GPU: the peer buffers are ordinary buffers of the same device.  Y and
    every peer copy hold the bits dtas_gemm_nt produces with the same kernel, column slabs of wider
    buffers are respected, and rows too few for the two-CTA kernel are refused."""
    from dtas_b200.reference import seeded_normal
    x = seeded_normal((m, k), 501, "float16").to(cuda_device)
    w = seeded_normal((n, k), 502, "float16", scale=0.02).to(cuda_device)
    b = seeded_normal((n,), 503, "float16", scale=0.1).to(cuda_device)
    want = torch.empty((m, n), dtype=torch.float16, device=cuda_device)
    _abi.check(_abi.lib().dtas_gemm_set_override(512, 0))          # the kernel the scatter entry point uses
    try:
        ops.gemm_nt(x, w, want, bias=b)
    finally:
        _abi.check(_abi.lib().dtas_gemm_set_override(0, 0))
    wide = [torch.full((m, n + 16), 7.0, dtype=torch.float16, device=cuda_device) for _ in range(n_peers + 1)]
    views = [t[:, 8:8 + n] for t in wide]
    ops.gemm_nt_scatter(x, w, views[0], views[1:], bias=b)
    ops.poll_status()
    ref = x.float() @ w.float().T + b.float()
    rms = ref.double().pow(2).mean().sqrt().item()
    assert (((want.float() - ref).abs() - (1e-2 * ref.abs() + 1e-2 * rms)).max().item()) <= 0
    for t, v in zip(wide, views):
        assert torch.equal(v, want)
        assert bool((t[:, :8] == 7.0).all()) and bool((t[:, 8 + n:] == 7.0).all()), "wrote outside its column slab"
    small = torch.empty((64, n), dtype=torch.float16, device=cuda_device)
    with pytest.raises(_abi.DtasError):
        ops.gemm_nt_scatter(x[:64], w, small, [torch.empty_like(small)])


def test_gemm_scatter_multicast_argument_errors(cuda_device):
    """dtas_gemm_nt_scatter_multicast refuses, before any launch, a multicast address that is y itself or
    not 16-byte aligned.  (The route itself needs an NVLink multicast mapping over several GPUs: it is
    covered by the two-GPU test of the gather engines.)"""
    m, n, k = 256, 256, 256
    x = torch.zeros((m, k), dtype=torch.float16, device=cuda_device)
    w = torch.zeros((n, k), dtype=torch.float16, device=cuda_device)
    y = torch.empty((m, n), dtype=torch.float16, device=cuda_device)
    peer = torch.empty_like(y)
    other = torch.empty((m * n + 8,), dtype=torch.float16, device=cuda_device)
    before = _abi.launch_count()
    with pytest.raises(_abi.DtasError) as e:
        ops.gemm_nt_scatter(x, w, y, [peer], multicast=y.data_ptr())
    assert e.value.code == _abi.EINVAL
    with pytest.raises(_abi.DtasError) as e:
        ops.gemm_nt_scatter(x, w, y, [peer], multicast=other.data_ptr() + 2)
    assert e.value.code == _abi.EALIGN
    assert _abi.launch_count() == before
