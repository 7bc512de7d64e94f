"""Column-parallel (N-sharded) Linear across the GPUs of one box.

The GEMM path shards by output columns: rank r owns rows [r*N/g, (r+1)*N/g) of the Linear weight
W[N,K] (RCC A rows), activations X[M,K] are replicated, and every rank produces Y_r[M, N/g] with no
data-path collective.  Only a layer whose full output is consumed (o_proj, down_proj in a
Llama-style block) reassembles Y with ONE all-gather: NCCL yields [g][M][N/g], which is permuted
to row-major [M, N].
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
