"""Parity of the CUDA kernels against the CPU oracle and the TVM-made golden fixtures.

Every call goes through the C ABI (dtas_b200.ops -> ctypes -> libdtas_b200.so).  Rules:
cast / add / copy bit-exact; reductions within 1e-3 relative + 1 fp16 ULP; GEMV / GEMM within
1e-2 relative of an fp32-accumulated reference (tests/util.py).
"""
import numpy as np
import pytest
import torch

import oracle
from dtas_b200 import _abi, ops
from dtas_b200.reference import config_seed, seeded_normal
from tests import util
from tests.golden.golden_cases import CASES, make_inputs

pytestmark = pytest.mark.gpu

GUARD = 2048  # elements of guard band on each side of every output


def guarded(shape, dtype, device, fill):
    """Output tensor carved out of a larger buffer whose borders hold a sentinel."""
    n = int(np.prod(shape))
    pad = GUARD + (-n) % 8  # keeps the payload 16-byte aligned for every dtype
    big = torch.full((GUARD + n + pad,), fill, dtype=dtype, device=device)
    return big, big[GUARD:GUARD + n].view(*shape)


def assert_guards(big, n, fill, what):
    head, tail = big[:GUARD], big[GUARD + n:]
    assert bool((head == fill).all()) and bool((tail == fill).all()), f"{what}: wrote outside its output"


def np_of(t):
    return t.detach().cpu().numpy()


# ---------------------------------------------------------------------------------------
# elementwise
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("m", [1, 17, 128, 4096])
def test_cast_f32_f16_baseline(cuda_device, m):
    x = seeded_normal((m, 4096), config_seed(0, 0), "float32")
    big, y = guarded((m, 4096), torch.float16, cuda_device, 7.0)
    ops.cast(x.to(cuda_device), y)
    torch.cuda.synchronize()
    util.assert_bit_exact(np_of(y), oracle.cast(x.numpy(), np.float16), f"cast m={m}")
    assert_guards(big, m * 4096, 7.0, f"cast m={m}")


@pytest.mark.parametrize("m", [1, 7, 64, 512, 8192])
def test_add_copy_f16_baseline(cuda_device, m):
    a = seeded_normal((m, 11008), config_seed(1, 0), "float16")
    b = seeded_normal((m, 11008), config_seed(1, 1), "float16")
    ad, bd = a.to(cuda_device), b.to(cuda_device)
    big, c = guarded((m, 11008), torch.float16, cuda_device, 7.0)
    ops.add(ad, bd, c)
    torch.cuda.synchronize()
    util.assert_bit_exact(np_of(c), oracle.add(a.numpy(), b.numpy()), f"add m={m}")
    assert_guards(big, m * 11008, 7.0, f"add m={m}")
    big, c = guarded((m, 11008), torch.float16, cuda_device, 7.0)
    ops.copy(ad, c)
    torch.cuda.synchronize()
    util.assert_bit_exact(np_of(c), oracle.copy(a.numpy()), f"copy m={m}")
    assert_guards(big, m * 11008, 7.0, f"copy m={m}")


def test_elementwise_reference_signature_and_dtypes(cuda_device):
    """The reference's own shapes: [1, n, 2560], cast fp16->fp32, add int8 / fp32, copy fp32."""
    n = 300
    a16 = seeded_normal((1, n, 2560), 5, "float16")
    out = torch.empty((1, n, 2560), dtype=torch.float32, device=cuda_device)
    ops.cast(a16.to(cuda_device), out)
    util.assert_bit_exact(np_of(out), oracle.cast(a16.numpy(), np.float32), "cast f16->f32")
    for dt in ("int8", "float32", "float16"):
        a = seeded_normal((1, n, 2560), 6, dt)
        b = seeded_normal((1, n, 2560), 7, dt)
        out = torch.empty_like(a, device=cuda_device)
        ops.add(a.to(cuda_device), b.to(cuda_device), out)
        util.assert_bit_exact(np_of(out), oracle.add(a.numpy(), b.numpy()), f"add {dt}")
        ops.copy(a.to(cuda_device), out)
        util.assert_bit_exact(np_of(out), a.numpy(), f"copy {dt}")


@pytest.mark.parametrize("m,h", [(1, 1), (1, 3), (1, 4), (1, 5), (7, 37), (1, 2051), (300, 2560), (4096, 2560), (3, 70001)])
def test_cast_f16_f32_lengths(cuda_device, m, h):
    """fp16 -> fp32 (the reference's cast, tuning_test/tune_cast.py:10-21) moves 4-element vectors:
    tails of 0..3 elements, one full-size case, and a view that starts 2 bytes off alignment."""
    x = seeded_normal((m, h), 400 + h, "float16")
    big, y = guarded((m, h), torch.float32, cuda_device, 3.0)
    ops.cast(x.to(cuda_device), y)
    torch.cuda.synchronize()
    util.assert_bit_exact(np_of(y), oracle.cast(x.numpy(), np.float32), f"cast f16->f32 {m}x{h}")
    assert_guards(big, m * h, 3.0, f"cast f16->f32 {m}x{h}")
    if m == 1:
        src = torch.zeros(h + 1, dtype=torch.float16, device=cuda_device)
        src[1:] = x.to(cuda_device).view(-1)
        out = torch.empty((1, h), dtype=torch.float32, device=cuda_device)
        ops.cast(src[1:].view(1, h), out)
        util.assert_bit_exact(np_of(out), oracle.cast(x.numpy(), np.float32), f"cast f16->f32 misaligned {h}")


def test_elementwise_ragged_lengths_and_misalignment(cuda_device):
    """Every m in 1..40 at a tiny odd H (tails shorter than a vector), a few random
    lengths up to ~70k elements, and buffers that start 2 bytes off a 16-byte boundary."""
    rng = np.random.default_rng(0)
    shapes = [(m, 37) for m in range(1, 41)] + [(1, int(v)) for v in rng.integers(1, 70000, 12)]
    for (m, h) in shapes:
        a = seeded_normal((m, h), 100 + m + h, "float16")
        b = seeded_normal((m, h), 200 + m + h, "float16")
        big, c = guarded((m, h), torch.float16, cuda_device, 3.0)
        ops.add(a.to(cuda_device), b.to(cuda_device), c)
        util.assert_bit_exact(np_of(c), oracle.add(a.numpy(), b.numpy()), f"add {m}x{h}")
        assert_guards(big, m * h, 3.0, f"add {m}x{h}")
        x = seeded_normal((m, h), 300 + m + h, "float32")
        big, y = guarded((m, h), torch.float16, cuda_device, 3.0)
        ops.cast(x.to(cuda_device), y)
        util.assert_bit_exact(np_of(y), oracle.cast(x.numpy(), np.float16), f"cast {m}x{h}")
        assert_guards(big, m * h, 3.0, f"cast {m}x{h}")
    # misaligned: views starting one element into a buffer
    m, h = 9, 1001
    a = seeded_normal((m * h + 1,), 1, "float16")
    b = seeded_normal((m * h + 1,), 2, "float16")
    ad, bd = a.to(cuda_device)[1:].view(m, h), b.to(cuda_device)[1:].view(m, h)
    outbuf = torch.full((m * h + 2,), 3.0, dtype=torch.float16, device=cuda_device)
    c = outbuf[1:1 + m * h].view(m, h)
    ops.add(ad, bd, c)
    util.assert_bit_exact(np_of(c), oracle.add(a.numpy()[1:].reshape(m, h), b.numpy()[1:].reshape(m, h)), "add misaligned")
    assert float(outbuf[0]) == 3.0 and float(outbuf[-1]) == 3.0
    ops.copy(ad, c)
    util.assert_bit_exact(np_of(c), a.numpy()[1:].reshape(m, h), "copy misaligned")


# ---------------------------------------------------------------------------------------
# row reductions
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("m", [1, 33, 256, 4096])
def test_rms_norm_softmax_baseline(cuda_device, m):
    x = seeded_normal((m, 4096), config_seed(2, 0), "float16")
    w = seeded_normal((4096,), config_seed(2, 1), "float16", scale=0.1, mean=1.0)
    xd, wd = x.to(cuda_device), w.to(cuda_device)
    big, y = guarded((m, 4096), torch.float16, cuda_device, 9.0)
    ops.rms_norm(xd, wd, y, eps=1e-6)
    torch.cuda.synchronize()
    util.assert_reduction_close(np_of(y), oracle.rms_norm(x.numpy(), w.numpy(), 1e-6), f"rms_norm m={m}")
    assert_guards(big, m * 4096, 9.0, f"rms_norm m={m}")
    big, y = guarded((m, 4096), torch.float16, cuda_device, 9.0)
    ops.softmax(xd, y)
    torch.cuda.synchronize()
    util.assert_reduction_close(np_of(y), oracle.softmax(x.numpy()), f"softmax m={m}")
    assert_guards(big, m * 4096, 9.0, f"softmax m={m}")


@pytest.mark.parametrize("m,h", [(3, 8), (5, 264), (2, 8192), (3, 32000), (2, 65536), (4, 101), (3, 1000), (2, 70000)])
def test_row_ops_other_row_lengths(cuda_device, m, h):
    """Short, long (vocabulary-sized), non-multiple-of-8 and over-long rows: register path
    with every threads-per-row choice and the generic path."""
    x = seeded_normal((m, h), 50 + h, "float16")
    w = seeded_normal((h,), 51 + h, "float16", scale=0.1, mean=1.0)
    xd = x.to(cuda_device)
    y = torch.empty_like(xd)
    ops.rms_norm(xd, w.to(cuda_device), y)
    util.assert_reduction_close(np_of(y), oracle.rms_norm(x.numpy(), w.numpy(), 1e-6), f"rms_norm {m}x{h}")
    ops.softmax(xd, y)
    util.assert_reduction_close(np_of(y), oracle.softmax(x.numpy()), f"softmax {m}x{h}")


@pytest.mark.parametrize("dtype", ["float16", "float32"])
@pytest.mark.parametrize("m,h", [(1, 1), (700, 17), (9, 255), (37, 257), (5, 1023), (130, 1025), (3, 2047), (66, 2049),
                                 (7, 4095), (3, 4097), (2, 5001)])
def test_row_ops_ragged_row_lengths(cuda_device, m, h, dtype):
    """Row lengths that are not a multiple of 8 (the reference sweeps softmax over 17, 1025, 2049:
    experiment/dtas_tuned/general_reduction/softmax/profile_dlight.py:8-52): every configuration of
    the scalar register kernel (rows up to 256 / 1024 / 2048 / 4096 columns), rows sharing a CTA with
    the last CTA partly empty, and the one-CTA-per-row kernel beyond 4096; nothing written past the
    end."""
    x = seeded_normal((m, h), 90 + h, dtype)
    xd = x.to(cuda_device)
    name = _abi.variant_of("softmax", m, h)
    assert ("elems" in name) == (h <= 4096) and "generic" in name, name
    big, y = guarded((m, h), torch.float16, cuda_device, 9.0)
    ops.softmax(xd, y)
    torch.cuda.synchronize()
    util.assert_reduction_close(np_of(y), oracle.softmax(x.numpy()), f"softmax {dtype} {m}x{h}")
    assert_guards(big, m * h, 9.0, f"softmax {m}x{h}")
    if dtype == "float16":
        w = seeded_normal((h,), 91 + h, "float16", scale=0.1, mean=1.0)
        big, y = guarded((m, h), torch.float16, cuda_device, 9.0)
        ops.rms_norm(xd, w.to(cuda_device), y)
        torch.cuda.synchronize()
        util.assert_reduction_close(np_of(y), oracle.rms_norm(x.numpy(), w.numpy(), 1e-6), f"rms_norm {m}x{h}")
        assert_guards(big, m * h, 9.0, f"rms_norm {m}x{h}")
    else:
        g = seeded_normal((h,), 92 + h, "float32", scale=0.1, mean=1.0)
        b = seeded_normal((h,), 93 + h, "float32", scale=0.1)
        big, y = guarded((m, h), torch.float16, cuda_device, 9.0)
        ops.layer_norm(xd, g.to(cuda_device), b.to(cuda_device), y, eps=1e-5)
        torch.cuda.synchronize()
        util.assert_reduction_close(np_of(y), oracle.layer_norm(x.numpy(), g.numpy(), b.numpy(), 1e-5),
                                    f"layer_norm {m}x{h}", abs_floor=1e-6)
        assert_guards(big, m * h, 9.0, f"layer_norm {m}x{h}")


def test_reference_reduction_workloads_fp32_in(cuda_device):
    """The reference's own reductions: LayerNorm and softmax read fp32 and write fp16."""
    for m in (1, 300):
        x = seeded_normal((1, m, 2560), 60, "float32")
        g = seeded_normal((2560,), 61, "float32", scale=0.1, mean=1.0)
        b = seeded_normal((2560,), 62, "float32", scale=0.1)
        y = torch.empty((1, m, 2560), dtype=torch.float16, device=cuda_device)
        ops.layer_norm(x.to(cuda_device), g.to(cuda_device), b.to(cuda_device), y, eps=1e-5)
        util.assert_reduction_close(np_of(y), oracle.layer_norm(x.numpy(), g.numpy(), b.numpy(), 1e-5), f"layer_norm m={m}",
                                    abs_floor=1e-6)
        ops.softmax(x.to(cuda_device), y)
        util.assert_reduction_close(np_of(y), oracle.softmax(x.numpy()), f"softmax f32 m={m}")


def test_reductions_row_permutation_invariance(cuda_device):
    """Full-size property: permuting rows permutes the result, bit for bit."""
    m = 4096
    x = seeded_normal((m, 4096), 70, "float16").to(cuda_device)
    perm = torch.randperm(m, generator=torch.Generator().manual_seed(1)).to(cuda_device)
    y1, y2 = torch.empty_like(x), torch.empty_like(x)
    ops.softmax(x, y1)
    ops.softmax(x[perm].contiguous(), y2)
    assert torch.equal(y1[perm], y2)
    s = y1.float().sum(-1)
    assert float((s - 1).abs().max()) < 2e-3


# ---------------------------------------------------------------------------------------
# GEMV
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("n,k", [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)])
def test_gemv_baseline(cuda_device, n, k):
    x = seeded_normal((1, k), config_seed(3, 0), "float16")
    w = seeded_normal((n, k), config_seed(3, 1), "float16", scale=0.02)
    big, y = guarded((1, n), torch.float16, cuda_device, 5.0)
    ops.gemv(x.to(cuda_device), w.to(cuda_device), y)
    torch.cuda.synchronize()
    want = x.float().numpy() @ w.float().numpy().T
    util.assert_matmul_close(np_of(y), want, f"gemv {n}x{k} vs fp32")
    util.assert_matmul_close(np_of(y), oracle.gemv(x.numpy(), w.numpy()).astype(np.float32), f"gemv {n}x{k} vs oracle")
    assert_guards(big, n, 5.0, f"gemv {n}x{k}")


@pytest.mark.parametrize("n,k", [(512, 4096), (1376, 4096), (4000, 4096), (512, 11008), (7, 40), (33, 1001), (100, 264)])
def test_gemv_sharded_and_odd_shapes(cuda_device, n, k):
    """Per-rank shapes of 8-way column sharding (multi-warp rows), tiny and unaligned K."""
    x = seeded_normal((1, k), 80, "float16")
    w = seeded_normal((n, k), 81, "float16", scale=0.02)
    b = seeded_normal((n,), 82, "float16", scale=0.1)
    y = torch.empty((1, n), dtype=torch.float16, device=cuda_device)
    ops.gemv(x.to(cuda_device), w.to(cuda_device), y, bias=b.to(cuda_device))
    want = x.float().numpy() @ w.float().numpy().T + b.float().numpy()
    util.assert_matmul_close(np_of(y), want, f"gemv+bias {n}x{k}")


@pytest.mark.parametrize("n,k", [(4096, 4096), (4096, 11008), (8, 8), (9, 264), (1000, 5632), (300, 11264), (20000, 1024), (50280, 2560), (1187, 512)])
def test_gemv_streaming_kernel(cuda_device, n, k):
    """The bulk-copy-fed persistent kernel, forced (code 16) on shapes at its limits: one row per consumer
    warp, the longest rows each ring depth takes, ragged bands; with a bias, and twice (barrier phases)."""
    x = seeded_normal((1, k), 60, "float16")
    w = seeded_normal((n, k), 61, "float16", scale=0.02)
    b = seeded_normal((n,), 62, "float16", scale=0.3)
    big, y = guarded((1, n), torch.float16, cuda_device, 5.0)
    lib = _abi.lib()
    _abi.check(lib.dtas_gemv_set_override(16, 0))
    try:
        assert _abi.variant_of("gemv", 1, n, k).startswith("gemv_stream_s")
        ops.gemv(x.to(cuda_device), w.to(cuda_device), y, bias=b.to(cuda_device))
        first = y.clone()
        ops.gemv(x.to(cuda_device), w.to(cuda_device), y, bias=b.to(cuda_device))
        ops.poll_status()
    finally:
        lib.dtas_gemv_set_override(0, 0)
    assert torch.equal(first, y)
    assert_guards(big, n, 5.0, f"gemv stream n={n} k={k}")
    util.assert_matmul_close(np_of(y), oracle.gemv(x.numpy(), w.numpy(), b.numpy()).astype(np.float32), f"gemv stream n={n} k={k}")


# ---------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------
GEMM_SHAPES = [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)]


def _check_gemm_tiles(y_np, x, w, m, n, k, what, n_tiles=64):
    """fp32-accumulated reference on 128x128 tiles: every tile for m <= 255, else at least 64 sampled
    ones, always including the last (partial) row / column tiles."""
    if m <= 255:
        n_tiles = 1 << 30
    rng = np.random.default_rng(m * 131 + n)
    mt, nt = (m + 127) // 128, (n + 127) // 128
    picks = {(mt - 1, nt - 1), (0, 0), (mt - 1, 0), (0, nt - 1)}
    while len(picks) < min(n_tiles, mt * nt):
        picks.add((int(rng.integers(mt)), int(rng.integers(nt))))
    xn, wn = x.numpy(), w.numpy()
    for (i, j) in sorted(picks):
        r0, r1, c0, c1 = i * 128, min(m, i * 128 + 128), j * 128, min(n, j * 128 + 128)
        want = xn[r0:r1].astype(np.float32) @ wn[c0:c1].astype(np.float32).T
        util.assert_matmul_close(y_np[r0:r1, c0:c1], want, f"{what} tile ({i},{j})")


@pytest.mark.parametrize("n,k", GEMM_SHAPES)
@pytest.mark.parametrize("m", [16, 64, 255, 1024, 4096, 8192])
def test_gemm_baseline(cuda_device, m, n, k):
    x = seeded_normal((m, k), config_seed(4, 0), "float16")
    w = seeded_normal((n, k), config_seed(4, 1), "float16", scale=0.02)
    xd, wd = x.to(cuda_device), w.to(cuda_device)
    big, y = guarded((m, n), torch.float16, cuda_device, 5.0)
    ops.gemm_nt(xd, wd, y)
    ops.poll_status()
    y_np = np_of(y)
    assert_guards(big, m * n, 5.0, f"gemm m={m} n={n} k={k}")
    _check_gemm_tiles(y_np, x, w, m, n, k, f"gemm m={m} n={n} k={k} [{_abi.variant_of('gemm', m, n, k)}]")
    # Whole-matrix cross-check against the library GEMM (checker only, never the product path), under
    # the same rule as the tiles: 1e-2 relative + 1e-2 rms, evaluated on the device.
    ref = (xd @ wd.T).float()
    rms = ref.double().pow(2).mean().sqrt().item()
    excess = ((y.float() - ref).abs() - (1e-2 * ref.abs() + 1e-2 * rms)).max().item()
    assert excess <= 0, f"gemm m={m} n={n} k={k}: an element is {excess} outside 1e-2 rel + 1e-2 rms of the library GEMM"


def test_gemm_small_m_full_oracle(cuda_device):
    """m <= 255 at (4096, 4096): every element against the C oracle (k-ordered fp32 sum)."""
    n, k = 4096, 4096
    w = seeded_normal((n, k), config_seed(4, 1), "float16", scale=0.02)
    wd = w.to(cuda_device)
    for m in (1, 16, 255):
        x = seeded_normal((m, k), config_seed(4, 0), "float16")
        y = torch.empty((m, n), dtype=torch.float16, device=cuda_device)
        ops.gemm_nt(x.to(cuda_device), wd, y)
        ops.poll_status()
        util.assert_matmul_close(np_of(y), oracle.gemm_nt(x.numpy(), w.numpy()).astype(np.float32), f"gemm m={m} full")


@pytest.mark.parametrize("bn,split", [(64, 1), (128, 1), (256, 1), (64, 4), (128, 3), (256, 2), (128, 16), (512, 1),
                                      (1024, 1), (1024, 4), (1024, 7), (2048, 0), (4160, 0), (4224, 0), (4352, 0), (8256, 0), (8320, 0)])
def test_gemm_every_tile_width_and_split(cuda_device, bn, split):
    """Forces each kernel instantiation and split factor on ragged shapes (m, n, k not
    multiples of the tile), with a bias, writing into a column slab of a wider buffer."""
    m, n, k = 200, 1000, 2120
    x = seeded_normal((m, k), 90, "float16")
    w = seeded_normal((n, k), 91, "float16", scale=0.02)
    b = seeded_normal((n,), 92, "float16", scale=0.1)
    wide = torch.full((m, n + 24), 5.0, dtype=torch.float16, device=cuda_device)
    y = wide[:, 8:8 + n]
    _abi.check(_abi.lib().dtas_gemm_set_override(bn, split))
    try:
        ops.gemm_nt(x.to(cuda_device), w.to(cuda_device), y, bias=b.to(cuda_device))
        ops.poll_status()
        ops.gemm_nt(x.to(cuda_device), w.to(cuda_device), y, bias=b.to(cuda_device))  # counters re-armed?
        ops.poll_status()
    finally:
        _abi.check(_abi.lib().dtas_gemm_set_override(0, 0))
    want = x.float().numpy() @ w.float().numpy().T + b.float().numpy()
    util.assert_matmul_close(np_of(y), want, f"gemm bn={bn} split={split}")
    assert bool((wide[:, :8] == 5.0).all()) and bool((wide[:, 8 + n:] == 5.0).all()), "wrote outside its column slab"


@pytest.mark.parametrize("code", [512, 513])
@pytest.mark.parametrize("m,n,k", [(1024, 4096, 4096), (4096, 12288, 4096), (1000, 2752, 11008), (300, 520, 72),
                                   (4096, 512, 4096), (200, 22016, 1024), (130, 1000, 2120), (2304, 2304, 512),
                                   (255, 22016, 4096)])
def test_gemm_two_cta_kernel(cuda_device, m, n, k, code):
    """The cta_group::2 kernel (256 x 256 tiles on CTA pairs), forced, on full and ragged shapes: tiles
    dealt out whole (512) and with the last, partial wave cut stream-K fashion and finished through the
    workspace (513; tile counts below, just above (81, 86) and far above the number of pairs)."""
    x = seeded_normal((m, k), 97, "float16")
    w = seeded_normal((n, k), 98, "float16", scale=0.02)
    xd, wd = x.to(cuda_device), w.to(cuda_device)
    big, y = guarded((m, n), torch.float16, cuda_device, 5.0)
    _abi.check(_abi.lib().dtas_gemm_set_override(code, 0))
    try:
        assert "2cta" in _abi.variant_of("gemm", m, n, k) and ("streamk" in _abi.variant_of("gemm", m, n, k)) == (code == 513)
        ops.gemm_nt(xd, wd, y)
        ops.poll_status()
        y2 = torch.empty_like(y)
        ops.gemm_nt(xd, wd, y2)
        ops.poll_status()
    finally:
        _abi.check(_abi.lib().dtas_gemm_set_override(0, 0))
    assert_guards(big, m * n, 5.0, f"2cta gemm m={m} n={n} k={k}")
    assert torch.equal(y, y2), "two runs differ"
    _check_gemm_tiles(np_of(y), x, w, m, n, k, f"2cta gemm m={m} n={n} k={k}")
    ref = (xd @ wd.T).float()
    err = (y.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item()


@pytest.mark.parametrize("slices", [2, 3, 4])
@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (16, 4096, 11008), (17, 1000, 1096), (32, 520, 320), (5, 136, 256),
                                   (33, 1000, 1096), (64, 4096, 4096)])
def test_gemm_swapped_kernel_cluster_k_split(cuda_device, m, n, k, slices):
    """Swapped operands with K cut in 2..4 slices inside a cluster (codes 16386..16388): ragged n and k,
    slices of unequal length (k = 320: five k-blocks) down to an empty one, bias, strided output."""
    x = seeded_normal((m, k), 87, "float16")
    w = seeded_normal((n, k), 88, "float16", scale=0.02)
    b = seeded_normal((n,), 89, "float16", scale=0.1)
    xd, wd, bd = x.to(cuda_device), w.to(cuda_device), b.to(cuda_device)
    wide = torch.full((m, n + 16), 5.0, dtype=torch.float16, device=cuda_device)
    y = wide[:, :n]
    _abi.check(_abi.lib().dtas_gemm_set_override(16384 + slices, 0))
    try:
        assert f"k{slices}cluster" in _abi.variant_of("gemm", m, n, k)
        ops.gemm_nt(xd, wd, y, bias=bd)
        ops.poll_status()
        first = y.clone()
        ops.gemm_nt(xd, wd, y, bias=bd)
        ops.poll_status()
    finally:
        _abi.check(_abi.lib().dtas_gemm_set_override(0, 0))
    assert torch.equal(first, y), "two runs differ"
    assert bool((wide[:, n:] == 5.0).all()), "wrote outside its column slab"
    want = x.float().numpy() @ w.float().numpy().T + b.float().numpy()
    util.assert_matmul_close(np_of(y), want, f"swap kc gemm m={m} n={n} k={k} slices={slices}")


@pytest.mark.parametrize("code", [8256, 8320])
@pytest.mark.parametrize("m,n,k", [(255, 4096, 4096), (512, 4096, 11008), (130, 200, 136), (1, 64, 128), (300, 1000, 72), (2000, 520, 1160)])
def test_gemm_cluster_k_split_kernel(cuda_device, m, n, k, code):
    """K cut in two inside a two-CTA cluster, the second half handed over through distributed shared
    memory: full and ragged shapes, odd k-block counts (k = 72: the halves are 1 and 1 with zero fill),
    several waves of clusters (m = 2000), bias, strided output; two runs are bit-identical."""
    x = seeded_normal((m, k), 77, "float16")
    w = seeded_normal((n, k), 78, "float16", scale=0.02)
    b = seeded_normal((n,), 79, "float16", scale=0.1)
    xd, wd, bd = x.to(cuda_device), w.to(cuda_device), b.to(cuda_device)
    wide = torch.full((m, n + 16), 5.0, dtype=torch.float16, device=cuda_device)
    y = wide[:, :n]
    _abi.check(_abi.lib().dtas_gemm_set_override(code, 0))
    try:
        assert "k2cluster" in _abi.variant_of("gemm", m, n, k)
        ops.gemm_nt(xd, wd, y, bias=bd)
        ops.poll_status()
        first = y.clone()
        ops.gemm_nt(xd, wd, y, bias=bd)
        ops.poll_status()
    finally:
        _abi.check(_abi.lib().dtas_gemm_set_override(0, 0))
    assert torch.equal(first, y), "two runs differ"
    assert bool((wide[:, n:] == 5.0).all()), "wrote outside its column slab"
    want = x.float().numpy() @ w.float().numpy().T + b.float().numpy()
    util.assert_matmul_close(np_of(y), want, f"k2 cluster gemm m={m} n={n} k={k} code={code}")


@pytest.mark.parametrize("m", [1, 15, 16, 17, 33, 100, 129, 256])
@pytest.mark.parametrize("split", [0, 1, 5, "streamk"])
def test_gemm_swapped_operand_kernel(cuda_device, m, split):
    """The m <= 256 kernel at every padded X-tile height, ragged n and k, bias, strided output;
    K cut into fixed slices or dealt out stream-K fashion."""
    n, k = 1000, 1096
    x = seeded_normal((m, k), 99, "float16")
    w = seeded_normal((n, k), 100, "float16", scale=0.02)
    b = seeded_normal((n,), 101, "float16", scale=0.1)
    wide = torch.full((m, n + 16), 5.0, dtype=torch.float16, device=cuda_device)
    y = wide[:, 8:8 + n]
    code, split = (2048, 0) if split == "streamk" else (1024, split)
    _abi.check(_abi.lib().dtas_gemm_set_override(code, split))
    try:
        assert "swap" in _abi.variant_of("gemm", m, n, k)
        assert ("streamk" in _abi.variant_of("gemm", m, n, k)) == (code == 2048)
        for _ in range(2):
            ops.gemm_nt(x.to(cuda_device), w.to(cuda_device), y, bias=b.to(cuda_device))
            ops.poll_status()
    finally:
        _abi.check(_abi.lib().dtas_gemm_set_override(0, 0))
    want = x.float().numpy() @ w.float().numpy().T + b.float().numpy()
    util.assert_matmul_close(np_of(y), want, f"swap gemm m={m} split={split}")
    assert bool((wide[:, :8] == 5.0).all()) and bool((wide[:, 8 + n:] == 5.0).all()), "wrote outside its column slab"


def test_gemm_unaligned_k_uses_fallback(cuda_device):
    m, n, k = 33, 70, 101
    x = seeded_normal((m, k), 93, "float16")
    w = seeded_normal((n, k), 94, "float16", scale=0.02)
    y = torch.empty((m, n), dtype=torch.float16, device=cuda_device)
    ops.gemm_nt(x.to(cuda_device), w.to(cuda_device), y)
    util.assert_matmul_close(np_of(y), x.float().numpy() @ w.float().numpy().T, "gemm simt fallback")


def test_gemm_linearity_full_size(cuda_device):
    """Size-independent properties at the largest shape: X -> 2X doubles Y exactly wherever Y
    is a normal fp16 number (a power of two commutes with every rounding except the fixed
    2^-24 grid of fp16 subnormals, where it may move the result by one grid step); the same
    call twice gives the same bits, with and without split-K."""
    m, n, k = 8192, 22016, 4096
    x = seeded_normal((m, k), 95, "float16").to(cuda_device)
    w = seeded_normal((n, k), 96, "float16", scale=0.02).to(cuda_device)
    y1 = torch.empty((m, n), dtype=torch.float16, device=cuda_device)
    y2 = torch.empty_like(y1)
    ops.gemm_nt(x, w, y1)
    ops.gemm_nt(x * 2, w, y2)
    ops.poll_status()
    normal = y1.abs() >= 2.0 ** -14
    assert torch.equal((y1 * 2)[normal], y2[normal])
    assert float(((y1 * 2)[~normal].float() - y2[~normal].float()).abs().max()) <= 2.0 ** -24 + 1e-12
    ops.gemm_nt(x, w, y2)
    ops.gemm_nt(x, w, y2)
    ops.poll_status()
    assert torch.equal(y1, y2), "two runs of the same GEMM differ"
    del y1, y2, normal
    xs = x[:64].contiguous()
    a = torch.empty((64, n), dtype=torch.float16, device=cuda_device)
    b = torch.empty_like(a)
    ops.gemm_nt(xs, w, a)
    ops.gemm_nt(xs, w, b)
    ops.poll_status()
    assert torch.equal(a, b)


# ---------------------------------------------------------------------------------------
# golden fixtures (outputs of the TVM build of the PrimFuncs)
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", sorted(c for c in CASES if not CASES[c]["op"].endswith("_fused")))   # fused: test_fused_gpu.py
def test_against_tvm_golden(cuda_device, name):
    case = CASES[name]
    ins, out = make_inputs(case)
    want = util.load_golden(case["op"])[name]
    d = [torch.from_numpy(a).to(cuda_device) for a in ins]
    y = torch.from_numpy(out).to(cuda_device)
    op = case["op"]
    if op == "cast":
        ops.cast(d[0], y)
    elif op == "add":
        ops.add(d[0], d[1], y)
    elif op == "copy":
        ops.copy(d[0], y)
    elif op == "rms_norm":
        ops.rms_norm(d[0], d[1], y, eps=case["eps"])
    elif op == "softmax":
        ops.softmax(d[0], y)
    elif op == "softmax_dyn":
        ops.softmax(d[0].view(-1, case["m"]), y.view(-1, case["m"]))
    elif op == "layer_norm":
        ops.layer_norm(d[0], d[1], d[2], y, eps=case["eps"])
    elif op == "gemv":
        ops.gemv(d[0].view(1, -1), d[1], y.view(1, -1))
    elif op == "gemm":
        ops.gemm_nt(d[0], d[1], y)
        ops.poll_status()
    got = np_of(y).reshape(want.shape)
    if op in ("cast", "add", "copy"):
        util.assert_bit_exact(got, want, name)
    elif op in ("gemv", "gemm"):
        util.assert_matmul_close(got, want.astype(np.float32), name)
    else:
        util.assert_reduction_close(got, want, name, abs_floor=1e-6 if op == "layer_norm" else 0.0)


@pytest.mark.parametrize("n,m", [(1, 1), (7, 77), (64, 1000), (128, 2048), (3, 40000)])
def test_softmax_with_symbolic_reduction_length(cuda_device, n, m):
    """The attention-score softmax of the reference's model IR: fp32 [1, 32, n, m] -> fp16, both n and m
    symbolic (experiment/ModelIR/dolly-v2-3b-q0f16/before_dl.py:756-800), through one bound function."""
    import dtas_b200
    from dtas_b200 import Engine, arch
    from dtas_b200.workloads import OpSpec
    dtas_b200.set_log_level(0)
    rt = Engine(1, True, None).tune_module([OpSpec("attn_softmax", "softmax", "float32", "float16", cols=0)],
                                           arch=arch.B200(0), range_div_factor=256)
    x = seeded_normal((1, 32, n, m), 7000 + m, "float32", scale=3.0)
    y = torch.full((1, 32, n, m), 9.0, dtype=torch.float16, device=cuda_device)
    rt["attn_softmax"](x.to(cuda_device), y)
    got = np_of(y)
    util.assert_reduction_close(got, oracle.softmax(x.numpy()).reshape(got.shape), f"softmax [1,32,{n},{m}]")
    assert abs(float(got.astype(np.float64).sum()) - 32 * n) < 32 * n * 2e-3      # every row sums to one


def test_engine_search_installs_measured_table(cuda_device, tmp_path):
    """Engine.tune_module(search=True): candidates are timed on the device, the winners land in
    the library's dispatch table, survive a reload from work_dir, and results stay correct."""
    import dtas_b200
    from dtas_b200 import Engine, arch, load_module_from_file
    from dtas_b200.workloads import OpSpec
    dtas_b200.set_log_level(0)
    n, k = 1024, 1024
    spec = OpSpec("proj", "gemm", cols=n, k=k, upper=512)
    lib = _abi.lib()
    try:
        rt = Engine(1, True, str(tmp_path)).tune_module([spec], arch=arch.B200(0), range_div_factor=128, search=True)
        rows = rt.record["functions"]["proj"]["measured_table"]
        assert rows and rows[0]["m_lo"] == 1 and rows[-1]["m_hi"] == 512
        for r in rows:
            want = _abi.variant_of("gemm", r["m_hi"], n, k)
            lib.dtas_gemm_set_override(r["bn"], r["split"])
            assert _abi.variant_of("gemm", r["m_hi"], n, k) == want, "table entry is not what dispatch uses"
            lib.dtas_gemm_set_override(0, 0)
        x = seeded_normal((200, k), 1, "float16")
        w = seeded_normal((n, k), 2, "float16", scale=0.02)
        y = torch.empty((200, n), dtype=torch.float16, device=cuda_device)
        rt["proj"](x.to(cuda_device), w.to(cuda_device), y)
        ops.poll_status()
        util.assert_matmul_close(np_of(y), x.float().numpy() @ w.float().numpy().T, "gemm after search")
        lib.dtas_gemm_table_clear()
        rt2 = load_module_from_file(str(tmp_path))
        assert rt2.record["functions"]["proj"]["measured_table"] == rows
        assert _abi.variant_of("gemm", rows[0]["m_hi"], n, k) == rt.record["functions"]["proj"]["ranges"][0]["config"]["variant"]
    finally:
        lib.dtas_gemm_set_override(0, 0)
        lib.dtas_gemm_table_clear()
        _abi._install_default_tables(lib)
