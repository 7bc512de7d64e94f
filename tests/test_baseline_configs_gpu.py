"""Parity on the benchmark's own configurations, at their full sizes, through the C ABI.

The cases follow the five configurations the benchmark is quoted on:
  C2  FP16 dynamic-M sweep, M in {1..4096}, N = K = 4096, through the online selector (so the plans the
      benchmark times -- split-K tiles, 128- and 256-row tiles, streaming kernels -- are the plans checked);
  C3  FP16 decode-shaped split-K: M in {1,8,16,32} x (N,K) in {(1024,8192),(4096,14336),(1024,28672)}
      through every elite split-K pid {400,407,413,425,439} x split 1/2/4/8 (Linear mapping);
  C4  INT8 on Llama-3-8B linear shapes: int32 accumulators bit-exact and the scaled epilogue bit-exact;
  C5  Llama-3-70B projections, unsharded and sharded 2 and 8 ways along N.
The CPU oracle is slow, so large cases check a seeded sample of token rows (every output element is an
independent dot product: a row sample is an exact check of those rows), and integer-valued inputs are
checked in full against float64 BLAS, where every correct GEMM is exact.
"""
import numpy as np
import pytest
import torch

from moonpoly_b200 import rng

pytestmark = pytest.mark.gpu
DEV = "cuda"
SWEEP_M = [1, 2, 4, 8, 16, 32, 64, 127, 128, 255, 512, 1023, 2048, 4096]


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def close_f16(got, ref, rtol=1e-2, atol=1e-3):
    """FP16 tolerance of the path: |d| <= atol + rtol*|ref|."""
    got, ref = got.astype(np.float32), ref.astype(np.float32)
    assert np.isfinite(got).all()
    bad = np.abs(got - ref) > atol + rtol * np.abs(ref)
    assert not bad.any(), f"{bad.sum()} of {bad.size} differ; max abs {np.abs(got - ref).max()}"


def sample_rows(total, count, seed):
    if total <= count:
        return np.arange(total)
    picks = (rng.raw(seed, 7, count) % np.uint64(total)).astype(np.int64)
    return np.unique(np.concatenate([picks, [0, total - 1]]))


@pytest.fixture(autouse=True)
def _status(api):
    yield
    assert api.device_status() == 0


# ------------------------------------------------------------------------------------------ C2
@pytest.fixture(scope="module")
def c2_weight():
    b = rng.normal(1, rng.STREAM_B, (4096, 4096), 0.05)
    return b, dev(b)


@pytest.mark.parametrize("m", SWEEP_M)
def test_c2_fp16_sweep_full_size_vs_oracle(api, oracle, c2_weight, m):
    b, B = c2_weight
    a = rng.normal(1, rng.STREAM_A, (m, 4096), 0.05)
    c = api.gemm_rcc(dev(a), B)                                   # [n, m], the plan the benchmark times
    rows = sample_rows(m, 192, 200 + m)
    ref = oracle.gemm_f16_rcc(a[rows], b)                         # [n, len(rows)]
    close_f16(c[:, torch.from_numpy(rows).to(DEV)].cpu().numpy(), ref)


@pytest.mark.parametrize("m", SWEEP_M)
def test_c2_fp16_sweep_full_size_exact_on_integers(api, m):
    n = k = 4096
    a = rng.small_ints(31, 0, (m, k))
    b = rng.small_ints(31, 1, (n, k), lo=-1, hi=1)
    ref = (a.astype(np.float64) @ b.astype(np.float64).T).T
    assert np.abs(ref).max() < 2048                               # exactly representable in fp16
    plan = api.select_plan(api.MP_FP16, m, n, k)
    c = api.gemm_rcc(dev(a), dev(b)).cpu().numpy()
    assert np.array_equal(c, ref.astype(np.float16)), f"M={m} plan {plan}"


# ------------------------------------------------------------------------------------------ C3
C3_NK = [(1024, 8192), (4096, 14336), (1024, 28672)]


@pytest.fixture(scope="module")
def c3_weights():
    return {nk: rng.normal(2, rng.STREAM_B, nk, 0.05) for nk in C3_NK}


@pytest.mark.parametrize("nk", C3_NK)
@pytest.mark.parametrize("M", [1, 8, 16, 32])
def test_c3_fp16_decode_splitk_pids_vs_oracle(api, oracle, c3_weights, nk, M):
    N, K = nk
    w = c3_weights[nk]
    x = rng.normal(2, rng.STREAM_A, (M, K), 0.05)
    ref = oracle.linear_f16(x, w)
    X, W = dev(x), dev(w)
    close_f16(api.linear(X, W).cpu().numpy(), ref)                              # the online selector's choice
    first = {}
    for pid in (400, 407, 413, 425, 439):
        for split in (1, 2, 4, 8):
            y = api.linear_cpp_forced_pid(X, W, pid, split).cpu().numpy()
            close_f16(y, ref)
            again = api.linear_cpp_forced_pid(X, W, pid, split).cpu().numpy()
            assert np.array_equal(y, again), f"pid {pid} split {split} is not reproducible"
            first[(pid, split)] = y


# ------------------------------------------------------------------------------------------ C4
C4_NK = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]


def c4_m_values():
    ms = sorted(set(rng.log_uniform_ints(3, rng.STREAM_SHAPES, 32, 1, 8192)))
    want = [ms[0], ms[len(ms) // 5], ms[2 * len(ms) // 5], ms[3 * len(ms) // 5], ms[4 * len(ms) // 5], ms[-1]]
    near = [min(ms, key=lambda v: abs(v - t)) for t in (100, 160)]          # the tile-boundary region
    return sorted(set(want + near))


@pytest.fixture(scope="module")
def c4_weights():
    return {}


@pytest.mark.parametrize("nk", C4_NK)
def test_c4_int8_llama_shapes_bit_exact(api, oracle, nk):
    N, K = nk
    b = rng.int8_uniform(3, rng.STREAM_B, (N, K))
    sb = rng.uniform(3, rng.STREAM_B_SCALE, (N,), 0.001, 0.02)
    B, SB = dev(b), dev(sb)
    for M in c4_m_values():
        a = rng.int8_uniform(3, rng.STREAM_A, (M, K))
        sa = rng.uniform(3, rng.STREAM_A_SCALE, (M,), 0.001, 0.02)
        rows = sample_rows(M, 48, 300 + M)
        ridx = torch.from_numpy(rows).to(DEV)
        A = dev(a)
        acc = api.gemm_rcc(A, B)                                                 # int32 [N, M]
        ref_acc = oracle.gemm_i8_rcc(a[rows], b)                                 # [N, len(rows)]
        assert np.array_equal(acc[:, ridx].cpu().numpy(), ref_acc), f"accumulators differ at M={M} N={N} K={K}"
        del acc
        out = api.scaled_int8_mm(A, B.t(), dev(sa), SB)                          # fp16 [M, N]
        ref_out = oracle.scaled_mm_i8(a[rows], b, sa[rows], sb)
        got = out[ridx].cpu().numpy()
        assert np.array_equal(got.view(np.uint16), ref_out.view(np.uint16)), f"scaled output differs at M={M} N={N} K={K}"


# ------------------------------------------------------------------------------------------ C5
C5_LAYERS = {"qkv": (10240, 8192), "o_proj": (8192, 8192), "gate_up": (57344, 8192), "down": (8192, 28672)}


@pytest.mark.parametrize("name", sorted(C5_LAYERS))
@pytest.mark.parametrize("M", [37, 1500])
def test_c5_llama70b_projection_sharded_vs_unsharded(api, oracle, name, M):
    """One projection of the 70B stack: the full layer and its column-parallel shards (2 and 8 ranks, each computed
    here on one GPU, as rank r of g would) against the oracle on a sample of output channels.  The weight is drawn
    on the GPU (seed 4); the sampled rows are copied to the host for the oracle."""
    N, K = C5_LAYERS[name]
    gen = torch.Generator(device=DEV)
    gen.manual_seed(4)
    W = (torch.randn((N, K), device=DEV, generator=gen, dtype=torch.float32) * 0.02).half()
    x = rng.normal(4, rng.STREAM_A, (M, K), 1.0)
    X = dev(x)
    chans = sample_rows(N, 96, 400 + N)
    cidx = torch.from_numpy(chans).to(DEV)
    ref = oracle.linear_f16(x, W[cidx].cpu().numpy())             # [M, len(chans)]
    full = api.linear(X, W)
    # |y| ~ 0.02 * sqrt(K): the absolute floor scales with the magnitude of the outputs
    atol = 2e-3 * float(np.sqrt(K / 1024.0))
    close_f16(full[:, cidx].cpu().numpy(), ref, atol=atol)
    from moonpoly_b200 import shard
    for g in (2, 8):
        parts = []
        for r in range(g):
            lo, hi = shard.shard_bounds(N, g, r)
            parts.append(api.linear(X, W[lo:hi]))
        y = torch.cat(parts, dim=1)
        close_f16(y[:, cidx].cpu().numpy(), ref, atol=atol)
        close_f16(y.cpu().numpy(), full.cpu().numpy(), atol=atol)
