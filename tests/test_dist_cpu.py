"""Column / row sharding logic on CPU ranks (gloo, world_size 2): partitioning, the gather
plan, and that a gathered result equals the unsharded one bit for bit."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dtas_b200.dist import ColumnShardedLinear, row_sharded, shard_range


def test_shard_range_covers_everything():
    for total in (0, 1, 7, 8, 33, 32000, 22016):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == total
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            counts = [c for _, c in spans]
            assert max(counts) - min(counts) <= 1 and counts == sorted(counts, reverse=True)
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _cpu_matmul(x, w, out, bias=None, res1=None, res2=None, act=None):
    t = x.float() @ w.float().T
    if bias is not None:
        t = t + bias.float()
    if act == "gelu":
        t = torch.nn.functional.gelu(t)
    if res1 is not None:
        t = t + res1.float()
    if res2 is not None:
        t = t + res2.float()
    out.copy_(t.to(out.dtype))
    return out


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        m, n, k = 5, 24, 16
        x = torch.randn(m, k, generator=g).half()
        w = (torch.randn(n, k, generator=g) * 0.1).half()
        lin = ColumnShardedLinear(w, n, compute=_cpu_matmul)
        assert lin.n_local == n // world and lin.col_start == rank * (n // world)
        buf = lin.forward_gathered(x)
        assert buf.shape == (world, m, n // world)
        full = ColumnShardedLinear.as_row_major(buf)
        want = torch.empty(m, n, dtype=torch.float16)
        _cpu_matmul(x, w, want)
        ok_gemm = torch.equal(full, want)
        # fused tail: bias and activation shard with the columns, residuals are sliced per rank
        b = (torch.randn(n, generator=g) * 0.5).half()
        r1, r2 = torch.randn(m, n, generator=g).half(), torch.randn(m, n, generator=g).half()
        fused = ColumnShardedLinear(w, n, compute=_cpu_matmul, bias=b, act="gelu")
        assert fused.bias.numel() == n // world
        got = ColumnShardedLinear.as_row_major(fused.forward_gathered(x, res1=r1, res2=r2))
        want_f = torch.empty(m, n, dtype=torch.float16)
        _cpu_matmul(x, w, want_f, bias=b, res1=r1, res2=r2, act="gelu")
        ok_gemm = ok_gemm and torch.equal(got, want_f)
        # one-row (GEMV) case: the flat gather already is [N]
        y = ColumnShardedLinear(w, n, compute=_cpu_matmul).forward_gathered(x[:1])
        ok_gemv = torch.equal(y.reshape(1, n), want[:1])
        # row sharding with a remainder and with a rank that gets no rows
        a = torch.arange(7 * 4, dtype=torch.float32).reshape(7, 4)
        out = torch.zeros_like(a)
        row_sharded(lambda src, dst: dst.copy_(src * 2), rank, world, a, out)
        gathered = [torch.zeros_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        ok_rows = torch.equal(sum(gathered), a * 2)
        one = torch.ones(1, 4)
        o1 = torch.zeros(1, 4)
        shard = row_sharded(lambda src, dst: dst.copy_(src), rank, world, one, o1)
        ok_empty = shard.shape[0] == (1 if rank == 0 else 0)
        results[rank] = (ok_gemm, ok_gemv, ok_rows, ok_empty)
    finally:
        dist.destroy_process_group()


def test_two_rank_column_and_row_sharding():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        assert results[rank] == (True, True, True, True), (rank, results[rank])
