"""Column-sharded GEMM / GEMV and row-sharded elementwise ops on real GPUs (NCCL, one process
per GPU): the gathered result must equal the single-GPU result bit for bit, because sharding
along N never changes the order of any reduction.  Skipped with fewer than two GPUs."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, results):
    import torch.distributed as dist
    from dtas_b200 import ops
    from dtas_b200.dist import ColumnShardedLinear, row_sharded
    from dtas_b200.reference import seeded_normal
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        ok = {}
        for (m, n, k) in [(1, 4096, 4096), (16, 4096, 4096), (300, 2048, 1024), (1024, 4096, 4096)]:
            x = seeded_normal((m, k), 1, "float16").to(dev)
            w = seeded_normal((n, k), 2, "float16", scale=0.02).to(dev)
            lin = ColumnShardedLinear(w, n)
            full = ColumnShardedLinear.as_row_major(lin.forward_gathered(x))
            ops.poll_status(rank)
            # single-GPU reference: the same column slabs computed one after another on this GPU
            # (same kernel variant per slab as the sharded run, hence the same bits)
            want = torch.empty((m, n), dtype=torch.float16, device=dev)
            for r in range(world):
                lo, hi = r * (n // world), (r + 1) * (n // world)
                slab = torch.empty((m, hi - lo), dtype=torch.float16, device=dev)
                (ops.gemv if m == 1 else ops.gemm_nt)(x, w[lo:hi].contiguous(), slab)
                want[:, lo:hi] = slab
            ops.poll_status(rank)
            ok[(m, n, k)] = bool(torch.equal(full, want))
            # the gathered result against the fp32-accumulated CPU oracle (1e-2 relative + 1e-2 rms), and
            # against ONE single-GPU call on the whole weight, which may pick another kernel variant and K
            # order than the shards did: equal within the same bound, not necessarily bit for bit
            import numpy as np
            import oracle
            from tests import util
            ref = oracle.gemm_nt(x.cpu().numpy(), w.cpu().numpy()).astype(np.float32)
            whole = torch.empty((m, n), dtype=torch.float16, device=dev)
            (ops.gemv if m == 1 else ops.gemm_nt)(x, w, whole)
            ops.poll_status(rank)
            try:
                util.assert_matmul_close(full.cpu().numpy(), ref, f"gathered m={m} n={n} k={k}")
                util.assert_matmul_close(whole.cpu().numpy(), ref, f"single call m={m} n={n} k={k}")
                ok[("oracle", m, n, k)] = True
            except AssertionError as e:
                ok[("oracle", m, n, k)] = False
                print(e, flush=True)
        # fused tail through the sharded layer: bias + GELU + two residuals, against one single-GPU call
        for m in (1, 40):
            n, k = 2048, 1024
            x = seeded_normal((m, k), 11, "float16").to(dev)
            w = seeded_normal((n, k), 12, "float16", scale=0.02).to(dev)
            b = seeded_normal((n,), 13, "float16", scale=0.5).to(dev)
            r1 = seeded_normal((m, n), 14, "float16").to(dev)
            r2 = seeded_normal((m, n), 15, "float16").to(dev)
            lin = ColumnShardedLinear(w, n, bias=b, act="gelu")
            full = ColumnShardedLinear.as_row_major(lin.forward_gathered(x, res1=r1, res2=r2))
            want = torch.empty((m, n), dtype=torch.float16, device=dev)
            (ops.gemv if m == 1 else ops.gemm_nt)(x, w, want, bias=b, res1=r1, res2=r2, act="gelu")
            ops.poll_status(rank)
            err = (full.float() - want.float()).abs().max().item()
            ok[("fused", m)] = err <= 2e-2 * want.float().abs().max().item()
        # the gather without a collective on the data: row blocks pushed into the peers' buffers
        from dtas_b200.dist import PeerGatherBuffer
        probe = PeerGatherBuffer(world, 8, 8, torch.float16, dev)
        engines = ("kernel", "copy", "epilogue") + (("multicast",) if probe.has_multicast() else ())
        ok[("multicast mapping present", probe.has_multicast())] = True      # recorded, not required
        del probe
        for engine in engines:
            # the last shape has a ragged last column chunk per rank (1064 = 8 x 128 + 40): whole blocks
            # leave through the staged path (and, "multicast", through the switch), the rest from registers
            for (m, n, k, block) in [(1, 4096, 1024, 2048), (40, 2048, 1024, 2048), (2500, 2048, 512, 1024),
                                     (300, 2128, 512, 2048)]:
                w = seeded_normal((n, k), 22, "float16", scale=0.02).to(dev)
                b = seeded_normal((n,), 23, "float16", scale=0.5).to(dev)
                lin = ColumnShardedLinear(w, n, bias=b)
                pbuf = PeerGatherBuffer(world, m, n // world, torch.float16, dev, engine=engine)
                same = True
                for seed in (31, 32):          # the second call reuses the buffer
                    x = seeded_normal((m, k), seed, "float16").to(dev)
                    r1 = seeded_normal((m, n), seed + 10, "float16").to(dev)
                    want = lin.forward_gathered(x, res1=r1).clone()
                    got = lin.forward_pushed(x, pbuf, res1=r1, block_rows=block, min_push_bytes=0)
                    ops.poll_status(rank)
                    same = same and bool(torch.equal(got, want))
                ok[("pushed", engine, m)] = same
                if engine in ("epilogue", "multicast") and m >= 129:
                    # without residuals the GEMM itself stores to the peers (one launch, one barrier)
                    x = seeded_normal((m, k), 41, "float16").to(dev)
                    want = lin.forward_gathered(x).clone()
                    got = lin.forward_pushed(x, pbuf, min_push_bytes=0)
                    ops.poll_status(rank)
                    ok[("scattered", engine, m)] = bool(torch.equal(got, want))
                del pbuf
        a = seeded_normal((7, 11008), 3, "float16").to(dev)
        b = seeded_normal((7, 11008), 4, "float16").to(dev)
        out = torch.zeros_like(a)
        row_sharded(ops.add, rank, world, a, b, out)
        gathered = [torch.zeros_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        ok["add rows"] = bool(torch.equal(sum(gathered), (a.float() + b.float()).half()))
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharding_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    for rank in range(world):
        assert all(results[rank].values()), (rank, dict(results[rank]))
