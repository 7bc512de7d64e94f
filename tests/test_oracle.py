"""CPU checks of the oracle: against the committed known answers, against the numpy restatement,
and against the properties the reference's own tests rely on."""
import os

import numpy as np
import pytest

from moonpoly_b200 import rng

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "rcc_known_answers.npz"))
SHAPES = [("s16x32x64", 16, 32, 64), ("s64x128x128", 64, 128, 128), ("s128x256x256", 128, 256, 256),
          ("twin128x384x128", 128, 384, 128)]


@pytest.mark.parametrize("name,m,n,k", SHAPES)
def test_ctest_shapes_exact_all_dtypes(oracle, name, m, n, k):
    gold = GOLD[name + "_c"]
    a = rng.small_ints(1, rng.STREAM_A, (m, k), dtype=np.float32)
    b = rng.small_ints(1, rng.STREAM_B, (n, k), dtype=np.float32)
    assert np.array_equal(oracle.gemm_f32_rcc(a, b), gold.astype(np.float32))
    assert np.array_equal(oracle.gemm_f16_rcc(a.astype(np.float16), b.astype(np.float16)), gold.astype(np.float16))
    assert np.array_equal(oracle.gemm_i8_rcc(a.astype(np.int8), b.astype(np.int8)), gold)


def test_twin_equals_plain(oracle):
    m, n, k = 128, 384, 128
    a = rng.small_ints(1, rng.STREAM_A, (m, k))
    b = rng.small_ints(1, rng.STREAM_B, (n, k))
    got = oracle.twin_gemm_f16(a, b, 256)
    assert np.array_equal(got, GOLD["twin128x384x128_c"].astype(np.float16))


def test_constant_check_all_ones(oracle):
    # moonpoly/core/moonpoly_gemm.cu:1641-1736: all-ones operands -> every output equals K
    a = np.ones((8, 4096), np.float16)
    b = np.ones((24, 4096), np.float16)
    # 4096 is representable in fp16; fp32 accumulation of ones is exact
    assert np.array_equal(oracle.gemm_f16_rcc(a, b), GOLD["ones_8x24x4096_c"].astype(np.float16))


def test_scaled_mm_known_answer(oracle):
    m, n, k = 24, 40, 64
    a = rng.int8_uniform(3, rng.STREAM_A, (m, k))
    b = rng.int8_uniform(3, rng.STREAM_B, (n, k))
    assert np.array_equal(oracle.gemm_i8_rcc(a, b).T, GOLD["scaled_24x40x64_acc"])
    out = oracle.scaled_mm_i8(a, b, GOLD["scaled_24x40x64_sa"], GOLD["scaled_24x40x64_sb"])
    assert np.array_equal(out, GOLD["scaled_24x40x64_out"])


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (3, 5, 7), (17, 9, 33), (37, 64, 100)])
def test_c_matches_numpy_restatement(oracle, m, n, k):
    a = rng.normal(5, 0, (m, k), 0.05, np.float16)
    b = rng.normal(5, 1, (n, k), 0.05, np.float16)
    c0 = rng.normal(5, 2, (n, m), 1.0, np.float16)
    for alpha, beta in ((1.0, 0.0), (0.5, 2.0)):
        got = oracle.gemm_f16_rcc(a, b, alpha, beta, c0)
        ref = oracle.np_gemm_rcc(a, b, alpha, beta, c0)
        assert np.array_equal(got, ref)
    a32 = rng.uniform(6, 0, (m, k), -1, 1)
    b32 = rng.uniform(6, 1, (n, k), -1, 1)
    assert np.array_equal(oracle.gemm_f32_rcc(a32, b32), oracle.np_gemm_rcc(a32, b32))
    a8 = rng.int8_uniform(7, 0, (m, k))
    b8 = rng.int8_uniform(7, 1, (n, k))
    c8 = (rng.int8_uniform(7, 2, (n, m)).astype(np.int32)) * 1000
    assert np.array_equal(oracle.gemm_i8_rcc(a8, b8, 2, -3, c8), oracle.np_gemm_rcc(a8, b8, 2, -3, c8))


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("scalar", [(0, 0), (1, 0), (0, 1), (1, 1)])
def test_scaled_mm_matches_numpy(oracle, bf16, with_bias, scalar):
    m, n, k = 13, 21, 48
    a = rng.int8_uniform(8, 0, (m, k))
    b = rng.int8_uniform(8, 1, (n, k))
    sa = rng.uniform(8, 2, (1 if scalar[0] else m,), 0.001, 0.02)
    sb = rng.uniform(8, 3, (1 if scalar[1] else n,), 0.001, 0.02)
    bias = None
    if with_bias:
        bias = rng.uniform(8, 5, (n,), -1, 1)
        bias = oracle.bf16_bits_from_f32(bias) if bf16 else bias.astype(np.float16)
    got = oracle.scaled_mm_i8(a, b, sa, sb, bias, bf16)
    ref = oracle.np_scaled_mm(a, b, np.broadcast_to(sa, (m,)) if sa.size == 1 else sa,
                              np.broadcast_to(sb, (n,)) if sb.size == 1 else sb, bias, bf16)
    assert np.array_equal(got, ref)


def test_linear_remap(oracle):
    # moonpolyLinear: Y[M,N] = X W^T via RCC (m = N, n = M)   (moonpoly/core/moonpoly_gemm.cu:41-44)
    M, N, K = 5, 12, 32
    x = rng.small_ints(9, 0, (M, K))
    w = rng.small_ints(9, 1, (N, K))
    y = oracle.linear_f16(x, w)
    assert np.array_equal(y.astype(np.int64), x.astype(np.int64) @ w.astype(np.int64).T)


def test_threads_do_not_change_results(oracle):
    a = rng.normal(10, 0, (33, 129), 0.05)
    b = rng.normal(10, 1, (47, 129), 0.05)
    assert np.array_equal(oracle.gemm_f16_rcc(a, b, threads=1), oracle.gemm_f16_rcc(a, b, threads=8))


def test_empty(oracle):
    assert oracle.gemm_f16_rcc(np.zeros((0, 8), np.float16), np.zeros((4, 8), np.float16)).shape == (4, 0)


def test_rng_is_stable():
    # first values of the stateless generator, fixed for all time
    assert [int(v) for v in rng.raw(0, 0, 2)] == [int(v) for v in rng.raw(0, 0, 4)[:2]]
    assert rng.raw(1, 1, 3)[2] == rng.raw(1, 1, 1, offset=2)[0]
    u = rng.uniform01(3, 4, 1000)
    assert 0.0 <= u.min() and u.max() < 1.0 and abs(u.mean() - 0.5) < 0.05
    z = rng.normal(1, 0, (20000,), 1.0, np.float32)
    assert abs(float(z.mean())) < 0.03 and abs(float(z.std()) - 1.0) < 0.03
    ms = rng.log_uniform_ints(3, rng.STREAM_SHAPES, 32, 1, 8192)
    assert len(ms) == 32 and min(ms) >= 1 and max(ms) <= 8192
