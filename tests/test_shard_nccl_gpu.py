"""Column-parallel Linear on two real GPUs: NCCL all-gather and the fused peer-store gather; skipped on a one-GPU box."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, tmp):
    import sys
    root = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
    for p in (root, os.path.join(root, "moonpoly-dev_b200", "py")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    from moonpoly_b200 import api, rng
    from moonpoly_b200.shard import ColumnParallelLinear
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        M, N, K = 48, 2048, 1024
        x = torch.from_numpy(rng.normal(41, 0, (M, K), 0.05)).cuda()
        w = torch.from_numpy(rng.normal(41, 1, (N, K), 0.02)).cuda()
        layer = ColumnParallelLinear.from_full_weight(w, rank, world)
        y = layer.gather(layer.forward(x))
        full = api.linear(x, w)
        assert torch.equal(y, full)          # same kernels on the same columns: bit-identical
        # the fused path: slabs stored straight into every GPU's copy of Y through peer-mapped pointers (plain
        # stores, no multimem), then the flag barrier
        from moonpoly_b200.shard import PeerOutput
        out = PeerOutput(256, N, rank, world)
        try:
            for rows in (48, 5, 200):
                xs = torch.from_numpy(rng.normal(42 + rows, 0, (rows, K), 0.05)).cuda()
                got = layer.forward_gather_fused(xs, out)
                torch.cuda.synchronize()
                # the NCCL-gathered result of the same shards: same kernels on the same columns, bit-identical
                assert torch.equal(got, layer.gather(layer.forward(xs))), rows
                ref = api.linear(xs, w).float()
                assert torch.all((got.float() - ref).abs() <= 1e-3 + 1e-2 * ref.abs()), rows
                dist.barrier()               # nobody overwrites the buffer while a peer still compares
            # forward_gather takes either way by the bytes a rank pushes; both give the same bits
            xs = torch.from_numpy(rng.normal(77, 0, (96, K), 0.05)).cuda()
            want = layer.gather(layer.forward(xs))
            for limit in (None, 0):          # default limit: fused for this size; 0: the collective
                got = layer.forward_gather(xs, out, fused_max_bytes=limit)
                torch.cuda.synchronize()
                assert torch.equal(got, want), limit
                dist.barrier()
        finally:
            out.close()
        assert api.device_status() == 0
        open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_column_parallel_linear_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(2))
