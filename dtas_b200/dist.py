"""Multi-GPU sharding of the operator classes: one process per GPU, torch.distributed plumbing.

The reference is single-GPU.  The operators shard without any exchange on the data path:
  * GEMM / GEMV by output columns: rank r owns W[r*N/g : (r+1)*N/g, :] (loaded once) and
    computes Y[:, r*N/g : (r+1)*N/g] with the single-GPU kernel; X is replicated.  K is never
    split across GPUs, so every output element is produced by exactly the arithmetic of the
    single-GPU run and a gathered result is bit-identical to it.
  * cast / add / copy / RMSNorm / softmax by rows, remainder rows to the low ranks; a rank
    with no rows launches nothing.
A collective is needed only when the caller wants the full GEMM / GEMV output on every rank:
one all-gather (NCCL over NVLink on GPUs).  The kernel epilogue writes each rank's column slab
straight into its slot of the gather buffer, laid out [g, m, N/g]; `as_row_major` turns that
into [m, N] with one local copy when a caller needs the row-major form.
"""
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous split of `total` items, remainder on the low ranks -> (start, count)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    base, rem = divmod(int(total), world)
    count = base + (1 if rank < rem else 0)
    start = rank * base + min(rank, rem)
    return start, count


def shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's rows of a [m, H] tensor (a view; may have zero rows)."""
    start, count = shard_range(t.shape[0], rank, world)
    return t[start:start + count]


def shard_weight(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's output columns of an NT weight: rows [start, start+count) of W[N, K]."""
    start, count = shard_range(w.shape[0], rank, world)
    return w[start:start + count].contiguous()


class ColumnShardedLinear:
    """Y = X W^T with W split by output columns over the ranks of `group`.

    `compute` is the kernel entry (default: dtas_b200.ops.gemm_nt, or ops.gemv for one row);
    it is a parameter so the host-side logic can be exercised on CPU ranks.

    The fused tail shards with the columns: `bias` ([N], or this rank's [N/g] when
    already_sharded) and `act` are fixed at construction; residuals are passed per call as full
    [m, N] tensors and each rank adds its column slab of them, so
    Y = act(X W^T + bias) + res1 + res2 needs no exchange either.
    """

    def __init__(self, w_full_or_shard: torch.Tensor, n_total: int, rank: Optional[int] = None,
                 world: Optional[int] = None, group=None, compute: Optional[Callable] = None,
                 already_sharded: bool = False, bias: Optional[torch.Tensor] = None, act: Optional[str] = None):
        self.group = group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.world = dist.get_world_size(group) if world is None else world
        self.n_total = int(n_total)
        self.col_start, self.n_local = shard_range(self.n_total, self.rank, self.world)
        self.w = w_full_or_shard if already_sharded else shard_weight(w_full_or_shard, self.rank, self.world)
        if self.w.shape[0] != self.n_local:
            raise ValueError(f"weight shard has {self.w.shape[0]} rows, expected {self.n_local}")
        self.even = self.n_total % self.world == 0
        self._compute = compute
        self.act = act
        self.bias = None
        if bias is not None:
            self.bias = bias if already_sharded else bias[self.col_start:self.col_start + self.n_local].contiguous()
            if self.bias.numel() != self.n_local:
                raise ValueError(f"bias shard has {self.bias.numel()} elements, expected {self.n_local}")

    def _slab(self, res):
        """This rank's columns of a full [m, N] residual (a view: the kernels take its row stride)."""
        if res is None:
            return None
        if res.shape[-1] != self.n_total:
            raise ValueError(f"residual has {res.shape[-1]} columns, expected {self.n_total}")
        return res[..., self.col_start:self.col_start + self.n_local]

    def _kernel(self, x, w, out, res1=None, res2=None):
        tail = {}
        if self.bias is not None:
            tail["bias"] = self.bias
        if self.act is not None:
            tail["act"] = self.act
        if res1 is not None:
            tail["res1"] = self._slab(res1)
        if res2 is not None:
            tail["res2"] = self._slab(res2)
        if self._compute is not None:
            return self._compute(x, w, out, **tail)
        from . import ops
        if x.shape[0] == 1:
            tail = {k: (v.contiguous() if k.startswith("res") else v) for k, v in tail.items()}   # [1, N/g] rows
            return ops.gemv(x, w, out, **tail)
        return ops.gemm_nt(x, w, out, **tail)

    def forward_local(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, res1=None, res2=None) -> torch.Tensor:
        """This rank's column slab Y[:, col_start : col_start + n_local]; no communication."""
        m = x.shape[0]
        if out is None:
            out = torch.empty((m, self.n_local), dtype=x.dtype, device=x.device)
        self._kernel(x, self.w, out, res1, res2)
        return out

    def gather_buffer(self, m: int, dtype, device) -> torch.Tensor:
        """[g, m, N/g] buffer; slot r is where rank r's kernel writes."""
        if not self.even:
            raise ValueError("gather buffer needs N divisible by the number of ranks")
        return torch.empty((self.world, m, self.n_local), dtype=dtype, device=device)

    def forward_gathered(self, x: torch.Tensor, buf: Optional[torch.Tensor] = None, res1=None, res2=None) -> torch.Tensor:
        """Full output on every rank as [g, m, N/g]: kernel into this rank's slot, then one
        all-gather in place."""
        m = x.shape[0]
        if buf is None:
            buf = self.gather_buffer(m, x.dtype, x.device)
        self._kernel(x, self.w, buf[self.rank], res1, res2)
        if self.world > 1:
            dist.all_gather_into_tensor(buf.view(-1), buf[self.rank].reshape(-1), group=self.group)
        return buf

    def forward_pushed(self, x: torch.Tensor, pbuf: "PeerGatherBuffer", res1=None, res2=None,
                       block_rows: int = 2048, min_push_bytes: int = 8 << 20) -> torch.Tensor:
        """Full output on every rank as [g, m, N/g], without a collective on the data: the kernel
        runs over blocks of `block_rows` rows into this rank's slot, and behind every block one
        push kernel (ops.peer_push) on a second stream stores the block into the same place of
        every other rank's buffer over NVLink while the next block is computed.  A barrier across
        ranks on the launching stream ends the call (every rank's pushes have landed), and one
        opens it when the buffer has been used before (every rank has finished reading the previous
        contents; readers of the buffer must be on the launching stream, which is the only stream the
        barrier orders).  Results equal forward_gathered's bit for bit as long as a row block selects a
        kernel with the same K order as the whole m would (no split-K from 1024 rows up) and takes the
        same residual route: with residuals and m >= 2048, forward_gathered adds them in a pass of its
        own behind the GEMM (two roundings) while a row block below 2048 rows adds them in the GEMM
        epilogue (one rounding), so those results agree to one fp16 ULP, not bit for bit.

        The two barriers and the second stream cost about 80 us of host and launch time, so a
        slab below `min_push_bytes` takes forward_gathered's route (one all-gather) into the same
        buffer instead."""
        m = x.shape[0]
        if pbuf.local.shape != (self.world, m, self.n_local):
            raise ValueError(f"gather buffer is {tuple(pbuf.local.shape)}, expected {(self.world, m, self.n_local)}")
        main = torch.cuda.current_stream(x.device)
        if pbuf.used:
            pbuf.barrier()       # every rank has finished reading the previous contents (on its launching stream)
        pbuf.used = True
        if m * self.n_local * pbuf.local.element_size() < min_push_bytes:
            return self.forward_gathered(x, buf=pbuf.local, res1=res1, res2=res2)
        if pbuf.engine in ("epilogue", "multicast") and self.world > 1 and m >= 129 and res1 is None \
                and self.act is None and self._compute is None:
            # one launch: the GEMM's own epilogue stores every finished tile into the peers' buffers - with
            # one store per peer, or ("multicast") with one store that the NVLink switch fans out
            from . import ops
            mine = pbuf.local[self.rank]
            ops.gemm_nt_scatter(x, self.w, mine, [p[self.rank] for p in pbuf.peers], bias=self.bias,
                                multicast=pbuf.multicast_address(mine) if pbuf.engine == "multicast" else 0)
            pbuf.barrier()
            return pbuf.local
        blocks = max(1, m // max(1, block_rows))
        rows = -(-m // blocks)
        mine = pbuf.local[self.rank]
        for r0 in range(0, m, rows):
            r1 = min(m, r0 + rows)
            self._kernel(x[r0:r1], self.w, mine[r0:r1], None if res1 is None else res1[r0:r1],
                         None if res2 is None else res2[r0:r1])
            if self.world > 1:
                pbuf.push(self.rank, r0, r1, main)
        if self.world > 1:
            main.wait_stream(pbuf.side)
            pbuf.barrier()
        return pbuf.local

    @staticmethod
    def as_row_major(buf: torch.Tensor) -> torch.Tensor:
        """[g, m, N/g] -> [m, N] (one local copy)."""
        g, m, nl = buf.shape
        return buf.permute(1, 0, 2).reshape(m, g * nl)


class PeerGatherBuffer:
    """A [g, m, N/g] gather buffer in symmetric memory: every rank allocates the same buffer and
    maps the others' into its address space, so slot r of every copy can be written by rank r
    over NVLink (ColumnShardedLinear.forward_pushed).  Collective: every rank of `group`
    constructs it at the same point.

    engine "copy" moves a row block with one cudaMemcpyAsync per peer: copy engines, no SM, which
    is what overlaps best with a GEMM that holds every SM.  engine "kernel" uses this library's
    push kernel (ops.peer_push: the block is read once and stored to all peers in one launch); its
    stores reach about 13 GB/s per CTA and peer, so with one peer it needs most SMs to fill NVLink
    and loses to the copy engines beside a large GEMM (m = 8192, N = 22016 on two GPUs: 729 us
    against 619 us; one all-gather behind the kernel: 889 us), while with seven peers it fills
    NVLink from a few SMs and one launch replaces seven copies (eight GPUs: 670 us against 838 us;
    all-gather: 686 us; four GPUs: 657 us against 630 us; all-gather: 739 us).  "auto" takes "copy"
    up to four ranks and "kernel" above."""

    def __init__(self, world: int, m: int, n_local: int, dtype, device, group=None, engine: str = "auto"):
        import torch.distributed._symmetric_memory as symm
        if engine == "auto":
            engine = "epilogue"
        if engine not in ("kernel", "copy", "epilogue", "multicast"):
            raise ValueError("engine is 'auto', 'kernel' (this library's push kernel), 'copy' (cudaMemcpyAsync per peer), "
                             "'epilogue' (the GEMM stores to the peers itself; other cases fall back to 'copy') or "
                             "'multicast' ('epilogue' with one multimem.st per vector, fanned out by the NVLink switch)")
        group = group if group is not None else dist.group.WORLD
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = world
        self.engine = engine
        # how row blocks travel when the GEMM cannot store to the peers itself
        self.push_engine = engine if engine not in ("epilogue", "multicast") else ("copy" if world <= 4 else "kernel")
        shape = (world, m, n_local)
        self.local = symm.empty(shape, dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.local, group)
        # peers in ring order from this rank's right neighbour, so that at any moment every rank
        # is the first destination of a different source
        order = [(self.rank + d) % world for d in range(1, world)]
        self.peers = [self.handle.get_buffer(r, shape, dtype) for r in order]
        self.side = torch.cuda.Stream(device=device)
        self.token = torch.zeros(1, dtype=torch.float32, device=device)
        self.used = False
        if engine == "multicast" and not self.has_multicast():
            raise RuntimeError("PeerGatherBuffer: this allocation has no multicast mapping (no NVLink switch multicast "
                               "on this system, or it is disabled); use engine='epilogue'")

    def has_multicast(self) -> bool:
        """Whether the symmetric allocation is also mapped through an NVLink multicast object."""
        return int(getattr(self.handle, "multicast_ptr", 0) or 0) != 0

    def multicast_address(self, view: torch.Tensor) -> int:
        """Address of `view` (a view of this rank's buffer) in the multicast mapping: a store there lands
        at the same offset of every rank's buffer."""
        base = int(self.handle.buffer_ptrs[self.handle.rank])
        off = view.data_ptr() - base
        if not (0 <= off < int(self.handle.buffer_size)):
            raise ValueError("multicast_address: the view does not lie in this rank's symmetric buffer")
        return int(self.handle.multicast_ptr) + off

    def push(self, slot: int, r0: int, r1: int, after: "torch.cuda.Stream") -> None:
        """Rows [r0, r1) of this rank's slot to every peer, on the side stream, behind the work
        queued on `after` so far."""
        from . import ops
        ev = torch.cuda.Event()
        ev.record(after)
        self.side.wait_event(ev)
        src = self.local[slot, r0:r1]
        with torch.cuda.stream(self.side):
            if self.push_engine == "kernel":
                ops.peer_push(src, [p[slot, r0:r1] for p in self.peers])
            else:
                for p in self.peers:
                    p[slot, r0:r1].copy_(src, non_blocking=True)

    def barrier(self) -> None:
        """Stream-ordered barrier across the ranks (a one-element NCCL all-reduce): behind it,
        everything every rank queued before its own barrier has completed."""
        dist.all_reduce(self.token, group=self.group)


def row_sharded(fn: Callable, rank: int, world: int, *tensors_then_out):
    """Runs an elementwise / row-reduction op on this rank's rows of every [m, H] argument.
    1-D arguments (norm weights) are passed whole.  Returns the output shard (maybe empty)."""
    shards = [shard_rows(t, rank, world) if t.dim() >= 2 else t for t in tensors_then_out]
    if shards[-1].shape[0] == 0:
        return shards[-1]
    fn(*shards)
    return shards[-1]
