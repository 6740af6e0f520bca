"""Stream order across back-to-back launches.

The kernels are launched with programmatic stream serialization: a kernel may start its set-up
while the one before it on the stream is still running, and waits for that kernel's results
before it touches global memory.  These tests run chains of dependent calls (read-after-write,
write-after-read, shared split-K scratch) without any synchronisation in between, eagerly and as
a replayed CUDA graph, and require bit-identical results to the same chain run with a device
synchronisation after every call.
"""
import pytest
import torch

from dtas_b200 import _abi, ops
from dtas_b200.reference import seeded_normal

pytestmark = pytest.mark.gpu


class Chain:
    """cast -> rms_norm -> gemm -> gemm -> add -> softmax -> copy, repeated with buffers reused."""

    def __init__(self, m, hidden, inner, device):
        self.m, self.device = m, device
        self.x32 = [seeded_normal((m, hidden), 10 + i, "float32").to(device) for i in range(2)]
        self.wn = seeded_normal((hidden,), 3, "float16", scale=0.5).to(device)
        self.w1 = seeded_normal((inner, hidden), 4, "float16", scale=0.03).to(device)
        self.w2 = seeded_normal((hidden, inner), 5, "float16", scale=0.03).to(device)
        f16 = dict(dtype=torch.float16, device=device)
        self.h = torch.zeros((m, hidden), **f16)
        self.a = torch.zeros((m, hidden), **f16)
        self.b = torch.zeros((m, inner), **f16)
        self.c = torch.zeros((m, hidden), **f16)
        self.r = torch.zeros((m, hidden), **f16)
        self.s = torch.zeros((m, hidden), **f16)
        self.out = [torch.zeros((m, hidden), **f16) for _ in range(4)]

    def reset(self):
        for t in [self.h, self.a, self.b, self.c, self.r, self.s] + self.out:
            t.zero_()

    def run(self, sync):
        def step():
            if sync:
                torch.cuda.synchronize()

        for it in range(4):
            ops.cast(self.x32[it % 2], self.h); step()          # overwrites h that the add below read
            ops.rms_norm(self.h, self.wn, self.a); step()
            ops.gemm_nt(self.a, self.w1, self.b); step()
            ops.gemm_nt(self.b, self.w2, self.c); step()        # both GEMMs share the split-K scratch
            ops.add(self.h, self.c, self.r); step()
            ops.softmax(self.r, self.s); step()
            ops.copy(self.s, self.out[it]); step()


@pytest.mark.parametrize("m", [1, 16, 64, 300, 1100])
def test_unsynchronised_chain_matches_synchronised(cuda_device, m):
    ch = Chain(m, 1024, 2816, cuda_device)
    ch.reset()
    ch.run(sync=True)
    torch.cuda.synchronize()
    want = [o.clone() for o in ch.out]
    assert all(bool(torch.isfinite(o.float()).all()) for o in want)
    assert not torch.equal(want[0], want[1])
    for rep in range(3):
        ch.reset()
        ch.run(sync=False)
        torch.cuda.synchronize()
        ops.poll_status()
        for i, o in enumerate(ch.out):
            assert torch.equal(o, want[i]), f"m={m} rep={rep}: output {i} differs without synchronisation"


@pytest.mark.parametrize("m", [16, 300])
def test_chain_in_a_replayed_graph(cuda_device, m):
    ch = Chain(m, 1024, 2816, cuda_device)
    ch.reset()
    ch.run(sync=True)
    torch.cuda.synchronize()
    want = [o.clone() for o in ch.out]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ch.run(sync=False)          # first calls (tensor maps, scratch) happen outside the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ch.run(sync=False)
    for rep in range(3):
        ch.reset()
        graph.replay()
        torch.cuda.synchronize()
        ops.poll_status()
        for i, o in enumerate(ch.out):
            assert torch.equal(o, want[i]), f"m={m} rep={rep}: output {i} differs in graph replay"


def test_launch_mode_switch(cuda_device):
    """dtas_set_pdl returns the previous mode, rejects unknown modes, and both modes give the same bits."""
    lib = _abi.lib()
    prev = lib.dtas_set_pdl(0)
    try:
        assert prev in (0, 1)
        assert lib.dtas_set_pdl(7) == -1 and b"dtas_set_pdl" in lib.dtas_last_error()
        ch = Chain(48, 1024, 2816, cuda_device)
        ch.reset()
        ch.run(sync=False)
        torch.cuda.synchronize()
        plain = [o.clone() for o in ch.out]
        assert lib.dtas_set_pdl(1) == 0
        ch.reset()
        ch.run(sync=False)
        torch.cuda.synchronize()
        ops.poll_status()
        for a, b in zip(plain, ch.out):
            assert torch.equal(a, b)
    finally:
        lib.dtas_set_pdl(prev if prev in (0, 1) else 1)
