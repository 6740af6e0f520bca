"""Boundary behaviour on the GPU: bounded waits that run out, split-K calls from several host threads and
on several streams.  Nothing here faults, traps or hangs a device: the wait that runs out is a wait on
a barrier that nothing arrives on, with its limit shortened to a millisecond."""
import threading

import numpy as np
import pytest
import torch

import oracle
from dtas_b200 import _abi, ops
from dtas_b200.reference import seeded_normal
from tests import util

pytestmark = pytest.mark.gpu


def _operands(m, n, k, seed, dev):
    x = seeded_normal((m, k), seed, "float16")
    w = seeded_normal((n, k), seed + 1, "float16", scale=0.02)
    want = oracle.gemm_nt(x.numpy(), w.numpy()).astype(np.float32)
    return x.to(dev), w.to(dev), want


def test_bounded_wait_runs_out_and_the_library_recovers(cuda_device):
    """A wait whose limit runs out records its code and the kernel returns; dtas_poll_status reports
    DTAS_ETIMEOUT once, clears the word, and the next calls work - including a split-K GEMM, whose
    arrival counters poll_status re-arms."""
    lib = _abi.lib()
    x, w, want = _operands(48, 512, 2048, 9100, cuda_device)
    y = torch.empty((48, 512), dtype=torch.float16, device=cuda_device)
    _abi.check(lib.dtas_gemm_set_override(64, 4))
    try:
        ops.gemm_nt(x, w, y)                                   # context, split-K scratch and counters exist
        ops.poll_status(0)
        st = torch.cuda.current_stream(0).cuda_stream
        _abi.check(lib.dtas_selftest_wait_timeout(0, st, 1_000_000))       # 1 ms
        rc = lib.dtas_poll_status(0)
        assert rc == _abi.ETIMEOUT
        assert "0x1ff" in lib.dtas_last_error().decode()
        assert lib.dtas_poll_status(0) == _abi.OK              # reported once, then clear
        y.fill_(float("nan"))
        ops.gemm_nt(x, w, y)
        ops.poll_status(0)
        util.assert_matmul_close(y.cpu().numpy(), want, "split-K GEMM after a reported timeout")
    finally:
        _abi.check(lib.dtas_gemm_set_override(0, 0))
    assert lib.dtas_selftest_wait_timeout(0, None, 10) == _abi.EINVAL       # limits outside 1 us .. 100 ms are refused


def test_split_k_calls_from_two_host_threads(cuda_device):
    """Two host threads make split-K calls at the same time, each on its own stream (so each takes a
    scratch set, one of them possibly creating it at that moment); both results match the oracle."""
    lib = _abi.lib()
    cases = [_operands(40, 768, 4096, 9200, cuda_device), _operands(64, 640, 2048, 9300, cuda_device)]
    outs = [torch.full((c[0].shape[0], c[1].shape[0]), float("nan"), dtype=torch.float16, device=cuda_device) for c in cases]
    streams = [torch.cuda.Stream(device=cuda_device) for _ in cases]
    errors = []
    start = threading.Barrier(len(cases))

    def work(i):
        try:
            x, w, _ = cases[i]
            with torch.cuda.stream(streams[i]):
                start.wait()
                for _ in range(20):
                    ops.gemm_nt(x, w, outs[i])
            streams[i].synchronize()
        except Exception as e:  # noqa: BLE001 - reported below
            errors.append(e)

    _abi.check(lib.dtas_gemm_set_override(64, 4))
    try:
        threads = [threading.Thread(target=work, args=(i,)) for i in range(len(cases))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
    finally:
        _abi.check(lib.dtas_gemm_set_override(0, 0))
    assert not errors, errors
    ops.poll_status(0)
    for i, c in enumerate(cases):
        util.assert_matmul_close(outs[i].cpu().numpy(), c[2], f"thread {i}")


def test_split_k_calls_overlap_across_streams(cuda_device):
    """Split-K GEMMs issued back to back on several streams (more streams than scratch sets, so sets
    change hands) never share partial sums: every result equals the single-stream result bit for bit."""
    lib = _abi.lib()
    n_streams = 10
    x, w, want = _operands(100, 1024, 4096, 9400, cuda_device)
    base = torch.empty((100, 1024), dtype=torch.float16, device=cuda_device)
    _abi.check(lib.dtas_gemm_set_override(128, 4))
    try:
        ops.gemm_nt(x, w, base)
        torch.cuda.synchronize()
        util.assert_matmul_close(base.cpu().numpy(), want, "single stream")
        streams = [torch.cuda.Stream(device=cuda_device) for _ in range(n_streams)]
        outs = [torch.full_like(base, float("nan")) for _ in range(n_streams)]
        for rep in range(4):
            for s, o in zip(streams, outs):
                with torch.cuda.stream(s):
                    ops.gemm_nt(x, w, o)
        torch.cuda.synchronize()
    finally:
        _abi.check(lib.dtas_gemm_set_override(0, 0))
    ops.poll_status(0)
    for i, o in enumerate(outs):
        util.assert_bit_exact(o.cpu().numpy(), base.cpu().numpy(), f"stream {i}")
