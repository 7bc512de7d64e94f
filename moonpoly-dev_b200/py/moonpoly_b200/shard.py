"""Column-parallel (N-sharded) Linear across the GPUs of one box.

The GEMM path shards by output columns: rank r owns rows [r*N/g, (r+1)*N/g) of the Linear weight
W[N,K] (RCC A rows), activations X[M,K] are replicated, and every rank produces Y_r[M, N/g] with no
data-path collective.  Only a layer whose full output is consumed (o_proj, down_proj in a
Llama-style block) reassembles Y.  Two ways: ONE NCCL all-gather (yields [g][M][N/g], permuted to
row-major [M, N]), or the fused path (PeerOutput): the GEMM's epilogue stores every finished tile
straight into the full [M, N] buffer of every GPU through peer-mapped pointers, and one small
flag-barrier kernel with a bounded wait tells every rank that all slabs have landed.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced split of n output features; the first n % world ranks get one more."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


# Slab bytes a rank pushes to its peers up to which the fused gather beats ncclAllGather (measured on B200 over
# NVSwitch: plain peer stores from the epilogue hide under the GEMM while they are small, but a large slab leaves
# through the epilogue warps at a fraction of the NVLink rate and stalls the accumulator drain).
FUSED_GATHER_MAX_BYTES = 8 << 20


def fused_gather_pays(rows: int, n_shard: int, world: int, itemsize: int = 2, limit: int = FUSED_GATHER_MAX_BYTES) -> bool:
    return (world - 1) * rows * n_shard * itemsize <= limit


class _DevicePointer:
    """Lets torch view memory this module allocated through the library (cuda array interface)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3}


class PeerOutput:
    """The full output Y[max_rows, n_total] (fp16) of a gathered layer: one copy per GPU, every copy mapped into
    every rank (CUDA IPC), plus a flag array per rank for the barrier.  `exchange(obj) -> list of every rank's obj`
    defaults to torch.distributed.all_gather_object on `group`."""

    def __init__(self, max_rows: int, n_total: int, rank: int, world: int, group: Optional[dist.ProcessGroup] = None,
                 exchange: Optional[Callable] = None, device: Optional[torch.device] = None):
        from . import api
        self.api, self.rank, self.world, self.n_total, self.max_rows = api, rank, world, n_total, max_rows
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.local_ptr, h_buf = api.peer_alloc(max_rows * n_total * 2)
        self.flag_ptr, h_flag = api.peer_alloc(256)
        if exchange is None:
            def exchange(obj):
                out = [None] * world
                dist.all_gather_object(out, obj, group=group)
                return out
        handles = exchange((h_buf, h_flag)) if world > 1 else [(h_buf, h_flag)]
        self.buf_ptrs, self.flag_ptrs, self._opened = [], [], []
        for r in range(world):
            if r == rank:
                self.buf_ptrs.append(self.local_ptr)
                self.flag_ptrs.append(self.flag_ptr)
            else:
                b, f = api.peer_open(handles[r][0]), api.peer_open(handles[r][1])
                self._opened += [b, f]
                self.buf_ptrs.append(b)
                self.flag_ptrs.append(f)
        # destination order of the GEMM: this GPU's copy first, then the peers
        self.dst = [self.local_ptr] + [self.buf_ptrs[r] for r in range(world) if r != rank]
        self.flag_table = torch.tensor(self.flag_ptrs, dtype=torch.int64, device=self.device)
        self.epoch = 0

    def tensor(self, rows: int) -> torch.Tensor:
        """This GPU's copy of the output, rows [0, rows), as a torch view (no copy)."""
        t = torch.as_tensor(_DevicePointer(self.local_ptr, (self.max_rows, self.n_total), "<f2"), device=self.device)
        return t[:rows]

    def linear_gather(self, x: torch.Tensor, w_shard: torch.Tensor, col_offset: int) -> None:
        if x.shape[0] > self.max_rows:
            raise ValueError(f"{x.shape[0]} rows do not fit the buffer of {self.max_rows}")
        self.api.linear_gather(x, w_shard, self.dst, self.n_total, col_offset)

    def barrier(self, timeout_us: int = 0) -> None:
        """Every rank's slab stores issued before this call are visible on this GPU once the kernel it enqueues has
        run; the wait inside is bounded (api.device_status() reports an expiry)."""
        self.epoch += 1
        self.api.peer_barrier(self.flag_table, self.world, self.rank, self.epoch, timeout_us)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            self.api.peer_close(p)
        self._opened = []
        for p in (self.local_ptr, self.flag_ptr):
            if p:
                self.api.peer_free(p)
        self.local_ptr = self.flag_ptr = 0


class ColumnParallelLinear:
    """One rank's share of a Linear layer.  `compute(x, w_shard) -> y_local` defaults to the CUDA
    library's `linear`; a different callable is for host-side tests of the sharding logic only."""

    def __init__(self, weight_shard: torch.Tensor, n_total: int, rank: int, world: int,
                 group: Optional[dist.ProcessGroup] = None,
                 compute: Optional[Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = None):
        lo, hi = shard_bounds(n_total, world, rank)
        if weight_shard.shape[0] != hi - lo:
            raise ValueError(f"rank {rank} must hold {hi - lo} weight rows, got {weight_shard.shape[0]}")
        self.w, self.n_total, self.rank, self.world, self.group = weight_shard, n_total, rank, world, group
        if compute is None:
            from . import api
            compute = api.linear
        self.compute = compute

    @classmethod
    def from_full_weight(cls, weight: torch.Tensor, rank: int, world: int, **kw) -> "ColumnParallelLinear":
        lo, hi = shard_bounds(weight.shape[0], world, rank)
        return cls(weight[lo:hi].contiguous(), weight.shape[0], rank, world, **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Local slab Y_r[M, N_r]; no communication."""
        return self.compute(x, self.w)

    def forward_gather_fused(self, x: torch.Tensor, out: PeerOutput, timeout_us: int = 0) -> torch.Tensor:
        """Full Y[M, N] on every rank without a separate collective: the GEMM stores this rank's slab into every
        GPU's copy of `out`, then the flag barrier.  Returns this GPU's copy (a view)."""
        lo, _ = shard_bounds(self.n_total, self.world, self.rank)
        out.linear_gather(x, self.w, lo)
        out.barrier(timeout_us)
        return out.tensor(x.shape[0])

    def forward_gather(self, x: torch.Tensor, out: PeerOutput, fused_max_bytes: int = None) -> torch.Tensor:
        """Full Y[M, N] on every rank by whichever way is faster for this many rows: the fused peer stores while the
        bytes this rank sends to its peers, (world - 1) * M * N_r * itemsize, stay within `fused_max_bytes`
        (default FUSED_GATHER_MAX_BYTES), ncclAllGather beyond.  Every rank sees the same M, so all ranks take the
        same branch."""
        limit = FUSED_GATHER_MAX_BYTES if fused_max_bytes is None else fused_max_bytes
        if fused_gather_pays(x.shape[0], self.w.shape[0], self.world, x.element_size(), limit):
            return self.forward_gather_fused(x, out)
        return self.gather(self.forward(x))

    def gather(self, y_local: torch.Tensor) -> torch.Tensor:
        """Full Y[M, N] on every rank (one all-gather).  Equal shards (N % world == 0, true for every
        Llama projection) use all_gather_into_tensor; ragged shards gather padded slabs."""
        if self.world == 1:
            return y_local
        M = y_local.shape[0]
        base, extra = divmod(self.n_total, self.world)
        if extra == 0:
            buf = torch.empty((self.world, M, base), dtype=y_local.dtype, device=y_local.device)
            if dist.get_backend(self.group) == "nccl":
                dist.all_gather_into_tensor(buf, y_local.contiguous(), group=self.group)
            else:   # gloo (host-side tests) has no fp16 all_gather_into_tensor
                dist.all_gather(list(buf.unbind(0)), y_local.contiguous(), group=self.group)
            return buf.permute(1, 0, 2).reshape(M, self.n_total)
        width = base + 1
        padded = torch.zeros((M, width), dtype=y_local.dtype, device=y_local.device)
        padded[:, : y_local.shape[1]] = y_local
        parts = [torch.empty_like(padded) for _ in range(self.world)]
        dist.all_gather(parts, padded, group=self.group)
        cols = []
        for r in range(self.world):
            lo, hi = shard_bounds(self.n_total, self.world, r)
            cols.append(parts[r][:, : hi - lo])
        return torch.cat(cols, dim=1)
