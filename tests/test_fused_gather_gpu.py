"""The column-parallel Linear fused with the all-gather of its output, on ONE GPU: the multi-destination epilogue and
the flag barrier are exercised with all "peer" buffers living on this GPU (tests/test_shard_nccl_gpu.py runs the same
path across two real GPUs)."""
import ctypes

import numpy as np
import pytest
import torch

from moonpoly_b200 import rng, shard

pytestmark = pytest.mark.gpu
DEV = "cuda"


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def close_f16(got, ref, rtol=1e-2, atol=1e-3):
    got, ref = got.astype(np.float32), ref.astype(np.float32)
    bad = np.abs(got - ref) > atol + rtol * np.abs(ref)
    assert not bad.any(), f"{bad.sum()} of {bad.size} differ; max abs {np.abs(got - ref).max()}"


@pytest.mark.parametrize("M,N,K,world", [(1, 1024, 2048, 4), (8, 2048, 1024, 2), (24, 4096, 4096, 8), (48, 1024, 8192, 2),
                                         (130, 1024, 1024, 2), (300, 2304, 512, 3), (1000, 2048, 1024, 2), (37, 520, 264, 2)])
def test_every_rank_slab_lands_in_every_copy(api, oracle, M, N, K, world):
    """`world` ranks computed one after the other on this GPU, each storing its slab into `world` copies of the full
    output (one per "GPU").  Every copy must hold the whole Y = X W^T: streaming kernels (few tokens), tensor tiles,
    split-K, ragged shards."""
    x = rng.normal(160, 0, (M, K), 0.05)
    w = rng.normal(160, 1, (N, K), 0.05)
    ref = oracle.linear_f16(x, w)
    X, W = dev(x), dev(w)
    copies = [torch.full((M, N), float("nan"), dtype=torch.float16, device=DEV) for _ in range(world)]
    for r in range(world):
        lo, hi = shard.shard_bounds(N, world, r)
        # destination order as rank r would pass it: its own copy first, then the others
        dst = [copies[r].data_ptr()] + [copies[q].data_ptr() for q in range(world) if q != r]
        api.linear_gather(X, W[lo:hi], dst, N, lo)
    torch.cuda.synchronize()
    for c in copies:
        close_f16(c.cpu().numpy(), ref)
    for c in copies[1:]:
        assert torch.equal(c, copies[0])                     # the same registers went to every copy
    # against the plain sharded Linear (same kernels on the same columns): bit-identical
    parts = [api.linear(X, W[slice(*shard.shard_bounds(N, world, r))]) for r in range(world)]
    assert torch.equal(torch.cat(parts, dim=1), copies[0])
    assert api.device_status() == 0


def test_gather_argument_checks(api):
    x = torch.zeros((4, 64), dtype=torch.float16, device=DEV)
    w = torch.zeros((8, 64), dtype=torch.float16, device=DEV)
    y = torch.zeros((4, 16), dtype=torch.float16, device=DEV)
    with pytest.raises(api.MoonpolyError):
        api.linear_gather(x, w, [y.data_ptr()], 16, 12)          # slab would cross the row end
    with pytest.raises(api.MoonpolyError):
        api.linear_gather(x, w, [y.data_ptr()] * 9, 16, 0)       # more than 8 destinations
    with pytest.raises(api.MoonpolyError):
        api.linear_gather(x.to(torch.int8), w.to(torch.int8), [y.data_ptr()], 16, 0)
    api.linear_gather(x, w, [y.data_ptr()], 16, 8)
    torch.cuda.synchronize()


def test_peer_barrier_completes_and_its_wait_is_bounded(api):
    """World of one: the barrier publishes to itself and returns.  World of two where the other rank never arrives:
    the wait gives up after its limit, records a status code the host reads, and the context stays usable."""
    flags = torch.zeros((2, 64), dtype=torch.int32, device=DEV)
    solo = torch.tensor([flags[0].data_ptr()], dtype=torch.int64, device=DEV)
    for value in (1, 2, 3):
        api.peer_barrier(solo, 1, 0, value)
    assert api.device_status() == 0
    assert int(flags[0, 0]) == 3
    pair = torch.tensor([flags[0].data_ptr(), flags[1].data_ptr()], dtype=torch.int64, device=DEV)
    api.peer_barrier(pair, 2, 0, 7, timeout_us=2000)           # nothing ever writes flags[0][1]
    with pytest.raises(api.MoonpolyError) as e:
        api.device_status()
    assert e.value.code == 7 and "108" in str(e.value)
    assert int(flags[1, 0]) == 7                                # the publication itself happened
    assert api.device_status() == 0                             # cleared; the device still works
    a = torch.ones((8, 64), dtype=torch.float16, device=DEV)
    assert torch.all(api.linear(a, a) == 64)


def test_peer_output_single_rank_round_trip(api, oracle):
    """PeerOutput with a world of one: allocation through the library, the torch view, gather + barrier, close."""
    M, N, K = 20, 512, 1024
    x = rng.normal(161, 0, (M, K), 0.05)
    w = rng.normal(161, 1, (N, K), 0.05)
    out = shard.PeerOutput(64, N, 0, 1)
    try:
        layer = shard.ColumnParallelLinear(dev(w), N, 0, 1)
        y = layer.forward_gather_fused(dev(x), out)
        torch.cuda.synchronize()
        close_f16(y.cpu().numpy(), oracle.linear_f16(x, w))
        assert y.shape == (M, N)
    finally:
        out.close()
    assert api.device_status() == 0
