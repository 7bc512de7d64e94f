"""Host-side logic of the N-sharded Linear, on CPU with gloo ranks (world_size 2 and 3).

The compute callable is replaced by the CPU oracle here: the test is about partitioning and the
all-gather reassembly, not about the CUDA kernel."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from moonpoly_b200 import rng
from moonpoly_b200.shard import ColumnParallelLinear, shard_bounds


def test_shard_bounds_cover_and_balance():
    for n in (1, 7, 8, 4096, 57344, 10241):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n_total, tmp):
    import sys
    root = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
    for p in (root, os.path.join(root, "moonpoly-dev_b200", "py")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K = 5, 64
        x = rng.normal(40, 0, (M, K), 0.05)
        w = rng.normal(40, 1, (n_total, K), 0.05)

        def compute(xt, wt):
            return torch.from_numpy(oracle.linear_f16(xt.numpy(), wt.numpy(), threads=1))

        layer = ColumnParallelLinear.from_full_weight(torch.from_numpy(w), rank, world, compute=compute)
        y_local = layer.forward(torch.from_numpy(x))
        lo, hi = shard_bounds(n_total, world, rank)
        full = oracle.linear_f16(x, w, threads=1)
        assert np.array_equal(y_local.numpy(), full[:, lo:hi])
        y = layer.gather(y_local)
        assert y.shape == (M, n_total)
        assert np.array_equal(y.numpy(), full)
        with open(os.path.join(tmp, f"ok{rank}"), "w") as fh:
            fh.write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_total", [(2, 48), (2, 37), (3, 30)])
def test_column_parallel_linear_gloo(tmp_path, world, n_total):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, n_total, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_stack_token_draws_follow_the_decode_prefill_mix():
    from moonpoly_b200 import stack
    a = stack.draw_tokens(4, 2000)
    assert a == stack.draw_tokens(4, 2000) and a != stack.draw_tokens(5, 2000)
    decode = [m for m in a if m <= 256]
    prefill = [m for m in a if m >= 512]
    assert len(decode) + len(prefill) == len(a)
    assert 0.66 < len(decode) / len(a) < 0.74
    assert min(a) >= 1 and max(a) <= 8192
    n_total = sum(n * k for (_, n, k, _) in stack.PROJECTIONS)
    assert n_total == (10240 + 8192 + 57344) * 8192 + 8192 * 28672
