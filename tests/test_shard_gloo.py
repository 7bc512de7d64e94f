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


class _FakeApi:
    """Stands in for the CUDA library's peer-memory calls: pointers are numbers, handles name their owner."""

    def __init__(self, rank):
        self.rank, self.next, self.opened, self.closed, self.freed, self.calls = rank, 0, [], [], [], []

    def peer_alloc(self, nbytes):
        self.next += 1
        ptr = 1000 * (self.rank + 1) + self.next
        return ptr, f"h{self.rank}:{ptr}".encode()

    def peer_open(self, handle):
        owner, ptr = handle.decode()[1:].split(":")
        self.opened.append(int(ptr))
        return 500000 + int(ptr)                      # a different address than the owner's: a mapping

    def peer_close(self, ptr):
        self.closed.append(ptr)

    def peer_free(self, ptr):
        self.freed.append(ptr)

    def linear_gather(self, x, w, dst, ld, off):
        self.calls.append(("gather", tuple(dst), ld, off))

    def peer_barrier(self, table, world, rank, value, timeout_us):
        self.calls.append(("barrier", world, rank, value))


def test_peer_output_maps_every_rank_and_orders_destinations(monkeypatch):
    """Host logic of the fused all-gather buffers for a world of three: handle exchange, own copy first in the
    destination list, flag table in rank order, growing barrier values, clean-up."""
    from moonpoly_b200 import shard
    world = 3
    apis = [_FakeApi(r) for r in range(world)]
    handles = []
    for r in range(world):                            # what each rank would contribute to the exchange
        a = _FakeApi(r)
        handles.append((a.peer_alloc(1)[1], a.peer_alloc(1)[1]))
    outs = []
    real_tensor = torch.tensor
    for r in range(world):
        import moonpoly_b200.api as real_api
        monkeypatch.setattr(real_api, "peer_alloc", apis[r].peer_alloc)
        monkeypatch.setattr(real_api, "peer_open", apis[r].peer_open)
        monkeypatch.setattr(real_api, "peer_close", apis[r].peer_close)
        monkeypatch.setattr(real_api, "peer_free", apis[r].peer_free)
        monkeypatch.setattr(real_api, "linear_gather", apis[r].linear_gather)
        monkeypatch.setattr(real_api, "peer_barrier", apis[r].peer_barrier)
        monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
        out = shard.PeerOutput(16, 24, r, world, exchange=lambda obj: handles, device=torch.device("cpu"))
        outs.append(out)
        own = 1000 * (r + 1) + 1
        assert out.buf_ptrs[r] == own and out.dst[0] == own and len(out.dst) == world
        assert sorted(out.dst[1:]) == sorted(500000 + 1000 * (q + 1) + 1 for q in range(world) if q != r)
        assert out.flag_table.tolist() == [1000 * (q + 1) + 2 if q == r else 500000 + 1000 * (q + 1) + 2 for q in range(world)]
        layer = shard.ColumnParallelLinear(torch.zeros((8, 4)), 24, r, world, compute=lambda x, w: None)
        monkeypatch.setattr(out, "tensor", lambda rows: rows)
        layer.forward_gather_fused(torch.zeros((5, 4)), out)
        layer.forward_gather_fused(torch.zeros((5, 4)), out)
        assert [c for c in apis[r].calls if c[0] == "gather"][0][2:] == (24, 8 * r)          # ld = N, offset = r * N / g
        assert [c[3] for c in apis[r].calls if c[0] == "barrier"] == [1, 2]
        out.close()
        assert len(apis[r].closed) == 2 * (world - 1) and sorted(apis[r].freed) == [own, own + 1]
    assert real_tensor is torch.tensor


def test_forward_gather_picks_the_fused_path_by_the_bytes_a_rank_sends(monkeypatch):
    """forward_gather: fused peer stores while (world - 1) * M * N_r * itemsize stays within the limit, the collective
    beyond; the decision depends only on values every rank shares (M, shard width, world)."""
    from moonpoly_b200 import shard
    assert shard.fused_gather_pays(64, 1024, 8)                                  # a decode step of a 70B o_proj on 8 GPUs
    assert not shard.fused_gather_pays(4096, 1024, 8)                            # a prefill step: 58 MB to push
    assert shard.fused_gather_pays(4096, 1024, 8, limit=1 << 30)
    assert shard.fused_gather_pays(1, 1, 1, limit=0)                             # one rank sends nothing
    taken = []
    layer = shard.ColumnParallelLinear(torch.zeros((8, 4)), 24, 1, 3, compute=lambda x, w: "local")
    monkeypatch.setattr(layer, "forward_gather_fused", lambda x, out, timeout_us=0: taken.append("fused") or "fused")
    monkeypatch.setattr(layer, "gather", lambda y: taken.append("nccl") or "gathered")
    assert layer.forward_gather(torch.zeros((5, 4), dtype=torch.float16), None) == "fused"
    assert layer.forward_gather(torch.zeros((5, 4), dtype=torch.float16), None, fused_max_bytes=100) == "gathered"   # 2*5*8*2 = 160 B
    assert taken == ["fused", "nccl"]
