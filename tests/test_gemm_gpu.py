"""Parity of the CUDA path with the CPU oracle, through the C ABI (needs a B200)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from moonpoly_b200 import rng

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "rcc_known_answers.npz"))
DEV = "cuda"


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def close_f16(got, ref, rtol=1e-2, atol=1e-3):
    """FP16 tolerance of the path: |d| <= atol + rtol*|ref| (relative 1e-2 with an absolute floor)."""
    got = got.astype(np.float32)
    ref = ref.astype(np.float32)
    assert np.isfinite(got).all()
    bad = np.abs(got - ref) > atol + rtol * np.abs(ref)
    assert not bad.any(), f"{bad.sum()} of {bad.size} differ; max abs {np.abs(got - ref).max()}"


@pytest.fixture(autouse=True)
def _status(api):
    yield
    assert api.device_status() == 0


# ---------------------------------------------------------------------------------------- FP16
@pytest.mark.parametrize("name,m,n,k", [("s16x32x64", 16, 32, 64), ("s64x128x128", 64, 128, 128),
                                         ("s128x256x256", 128, 256, 256)])
def test_fp16_ctest_shapes_exact(api, name, m, n, k):
    # shapes and inputs of tests/cpp/fp16/test_fp16_row_col_col.cu: integer-valued, hence exact
    a = rng.small_ints(1, rng.STREAM_A, (m, k))
    b = rng.small_ints(1, rng.STREAM_B, (n, k))
    c = api.gemm_rcc(dev(a), dev(b)).cpu().numpy()
    assert np.array_equal(c, GOLD[name + "_c"].astype(np.float16))


def test_fp16_every_elite_pid_exact(api):
    m, n, k = 72, 200, 320
    a = rng.small_ints(11, 0, (m, k))
    b = rng.small_ints(11, 1, (n, k))
    ref = (a.astype(np.int64) @ b.astype(np.int64).T).T.astype(np.float16)
    A, B = dev(a), dev(b)
    for pid in api.elite_fp16_pids() + [40, 42, 43, 44, 66, 91, 286]:
        _, align = api.pid_info(api.MP_FP16, pid)
        assert k % align == 0
        c = api.gemm_rcc_pid(A, B, pid, 1).cpu().numpy()
        assert np.array_equal(c, ref), f"pid {pid}"


def test_fp16_constant_check(api):
    # all-ones operands -> every output equals K (moonpoly/core/moonpoly_gemm.cu:1641-1736)
    a = torch.ones((8, 4096), dtype=torch.float16, device=DEV)
    b = torch.ones((24, 4096), dtype=torch.float16, device=DEV)
    for pid, split in ((40, 2), (66, 2), (400, 4), (8, 1)):
        c = api.gemm_rcc_pid(a, b, pid, split)
        assert torch.all(c == 4096), (pid, split)


@pytest.mark.parametrize("m", [1, 2, 7, 16, 37, 64, 127, 128, 255, 512])
def test_fp16_sweep_vs_oracle(api, oracle, m):
    n, k = 1024, 512        # the dynamic-M sweep at a size the CPU oracle finishes in seconds
    a = rng.normal(1, rng.STREAM_A, (m, k), 0.05)
    b = rng.normal(1, rng.STREAM_B, (n, k), 0.05)
    ref = oracle.gemm_f16_rcc(a, b)
    c = api.gemm_rcc(dev(a), dev(b)).cpu().numpy()
    close_f16(c, ref)


def test_fp16_alpha_beta_and_tails(api, oracle):
    m, n, k = 133, 77, 264   # odd m and n, k = 4 K-blocks + a tail of 8
    a = rng.normal(12, 0, (m, k), 0.05)
    b = rng.normal(12, 1, (n, k), 0.05)
    c0 = rng.normal(12, 2, (n, m), 1.0)
    ref = oracle.gemm_f16_rcc(a, b, 0.5, 2.0, c0)
    for pid in (1, 8, 23, 7):
        c = api.gemm_rcc_pid(dev(a), dev(b), pid, 1, c_nm=dev(c0), alpha=0.5, beta=2.0).cpu().numpy()
        close_f16(c, ref)


def test_fp16_unaligned_k_uses_cuda_core_tiles(api, oracle):
    m, n, k = 19, 45, 67     # k*2 bytes is not a multiple of 16: TMA cannot describe the rows
    a = rng.normal(13, 0, (m, k), 0.05)
    b = rng.normal(13, 1, (n, k), 0.05)
    ref = oracle.gemm_f16_rcc(a, b)
    c = api.gemm_rcc(dev(a), dev(b)).cpu().numpy()
    close_f16(c, ref)
    with pytest.raises(api.MoonpolyError) as e:
        api.gemm_rcc_pid(dev(a), dev(b), 0, 1)       # pid 0 needs k % 8 == 0
    assert e.value.code == 3


@pytest.mark.parametrize("split_k", [1, 2, 4, 8])
@pytest.mark.parametrize("pid", [400, 407, 413, 425, 439])
def test_fp16_splitk_pids(api, oracle, pid, split_k):
    # Linear(M,N,K) through pids 400+ with run-time split-K (tests/python/test_fp16_splitk_runtime.py)
    M, N, K = 8, 1024, 1024
    x = rng.normal(2, rng.STREAM_A, (M, K), 0.1)
    w = rng.normal(2, rng.STREAM_B, (N, K), 0.1)
    ref = oracle.linear_f16(x, w)
    y = api.linear_cpp_forced_pid(dev(x), dev(w), pid, split_k).cpu().numpy()
    close_f16(y, ref, rtol=1e-2, atol=2e-3)


def test_fp16_splitk_is_deterministic_and_exact(api):
    m, n, k = 200, 136, 2048
    a = rng.small_ints(14, 0, (m, k))
    b = rng.small_ints(14, 1, (n, k), lo=-1, hi=1)
    ref = (a.astype(np.int64) @ b.astype(np.int64).T).T
    assert np.abs(ref).max() < 2048
    A, B = dev(a), dev(b)
    first = None
    for rep in range(3):
        c = api.gemm_rcc_pid(A, B, 415, 8).cpu().numpy()
        assert np.array_equal(c, ref.astype(np.float16))
        first = c if first is None else first
        assert np.array_equal(first, c)


def test_fp16_caller_workspace(api, oracle):
    M, N, K = 16, 512, 4096
    x = rng.normal(15, 0, (M, K), 0.05)
    w = rng.normal(15, 1, (N, K), 0.05)
    ref = oracle.linear_f16(x, w)
    X, W = dev(x), dev(w)
    need = api.fp16_workspace_size(X, W, 400, 4)
    assert need > 0
    ws = torch.full((need,), 0xAB, dtype=torch.uint8, device=DEV)     # garbage on purpose
    out = torch.empty((M, N), dtype=torch.float16, device=DEV)
    api.linear_fp16_pid_ws_out(X, W, out, 400, ws, 4)
    close_f16(out.cpu().numpy(), ref)
    api.linear_fp16_pid_ws_out(X, W, out, 400, ws, 4)                 # counters were left clean
    close_f16(out.cpu().numpy(), ref)
    with pytest.raises(ValueError):
        api.linear_fp16_pid_ws_out(X, W, out, 400, ws[: need // 2], 4)


def test_fp16_twin_gemm(api):
    # tests/cpp/fp16/test_fp16_pattern2_twin_gemm.cu: m=128, n=384, k=128, split_n=256
    m, n, k = 128, 384, 128
    a = rng.small_ints(1, rng.STREAM_A, (m, k))
    b = rng.small_ints(1, rng.STREAM_B, (n, k))
    c = api.twin_gemm_fp16(dev(a), dev(b), 256).cpu().numpy()
    assert np.array_equal(c, GOLD["twin128x384x128_c"].astype(np.float16))
    c = api.twin_gemm_fp16(dev(a), dev(b), 0).cpu().numpy()       # auto split: 3/4 of n, 128-aligned
    assert np.array_equal(c, GOLD["twin128x384x128_c"].astype(np.float16))
    for bad in (384, 100, 512):
        with pytest.raises(ValueError):
            api.twin_gemm_fp16(dev(a), dev(b), bad)


def test_fp16_twin_ragged_tail(api, oracle):
    m, n, k = 200, 530, 192
    a = rng.normal(16, 0, (m, k), 0.05)
    b = rng.normal(16, 1, (n, k), 0.05)
    ref = oracle.gemm_f16_rcc(a, b)
    c = api.twin_gemm_fp16(dev(a), dev(b), 512).cpu().numpy()
    close_f16(c, ref)


def test_fp16_linear_matches_rcc_remap(api, oracle):
    M, N, K = 5, 384, 256
    x = rng.normal(17, 0, (M, K), 0.05)
    w = rng.normal(17, 1, (N, K), 0.05)
    y = api.linear(dev(x), dev(w)).cpu().numpy()
    close_f16(y, oracle.linear_f16(x, w))


def test_layout_and_dtype_errors(api):
    a = torch.zeros((4, 8), dtype=torch.float16, device=DEV)
    with pytest.raises(ValueError):
        api.gemm_rcc(a.to(torch.bfloat16), a.to(torch.bfloat16))     # the RCC entry keeps the reference's dtype set
    with pytest.raises(ValueError):
        api.linear(a.to(torch.float64), a.to(torch.float64))
    L = api.lib()
    rc = L.mp_gemm(0, 4, 4, 8, a.data_ptr(), 1, a.data_ptr(), 1, a.data_ptr(), 1, 1.0, 0.0, None)
    assert rc == 2
    rc = L.mp_gemm(7, 4, 4, 8, a.data_ptr(), 0, a.data_ptr(), 1, a.data_ptr(), 1, 1.0, 0.0, None)
    assert rc == 1
    with pytest.raises(api.MoonpolyError) as e:
        api.gemm_rcc_pid(a, a, 77, 1)
    assert e.value.code == 4


def test_empty_problems(api):
    a = torch.zeros((0, 64), dtype=torch.float16, device=DEV)
    b = torch.zeros((8, 64), dtype=torch.float16, device=DEV)
    assert api.gemm_rcc(a, b).shape == (8, 0)
    # k == 0: C = beta * C
    a0 = torch.zeros((4, 0), dtype=torch.float16, device=DEV)
    b0 = torch.zeros((8, 0), dtype=torch.float16, device=DEV)
    c = torch.ones((8, 4), dtype=torch.float16, device=DEV)
    api.gemm_rcc(a0, b0, c_nm=c, alpha=1.0, beta=3.0)
    assert torch.all(c == 3)


# ---------------------------------------------------------------------------------------- FP32
def test_fp32_config_shape(api, oracle):
    # FP32 RCC 37 x 1024 x 1024, uniform[-1,1], seed 0; tolerance 1e-4 relative
    m, n, k = 37, 1024, 1024
    a = rng.uniform(0, rng.STREAM_A, (m, k), -1.0, 1.0)
    b = rng.uniform(0, rng.STREAM_B, (n, k), -1.0, 1.0)
    ref = oracle.gemm_f32_rcc(a, b)
    c = api.gemm_rcc(dev(a), dev(b)).cpu().numpy()
    assert np.all(np.abs(c - ref) <= 1e-4 * np.maximum(1.0, np.abs(ref)))


@pytest.mark.parametrize("m,n,k", [(16, 32, 64), (64, 128, 128), (33, 65, 1100)])
def test_fp32_ctest_shapes_and_forced_splitk(api, m, n, k, monkeypatch):
    # tests/cpp/fp32/test_fp32_row_col_col.cu: plain, then with MOONPOLY_FP32_PATTERN3_FORCE_SPLITK=2
    a = rng.small_ints(1, rng.STREAM_A, (m, k), dtype=np.float32)
    b = rng.small_ints(1, rng.STREAM_B, (n, k), dtype=np.float32)
    ref = (a.astype(np.int64) @ b.astype(np.int64).T).T.astype(np.float32)
    assert np.array_equal(api.gemm_rcc(dev(a), dev(b)).cpu().numpy(), ref)
    free_plan = repr(api.select_plan(api.MP_FP32, m, n, k))
    monkeypatch.setenv("MOONPOLY_FP32_PATTERN3_FORCE_SPLITK", "2")
    plan = api.select_plan(api.MP_FP32, m, n, k)
    assert plan.pattern == 3 and plan.split_k == 2 and plan.pid == -1
    assert np.array_equal(api.gemm_rcc(dev(a), dev(b)).cpu().numpy(), ref)
    monkeypatch.delenv("MOONPOLY_FP32_PATTERN3_FORCE_SPLITK")
    assert repr(api.select_plan(api.MP_FP32, m, n, k)) == free_plan     # the flag is re-read on every call


@pytest.mark.parametrize("m,n,k", [(300, 520, 1000), (129, 257, 1004), (128, 128, 16), (64, 1000, 4100), (513, 70, 2048),
                                   (200, 200, 1001)])
def test_fp32_throughput_tiles(api, oracle, m, n, k):
    """The FP32 tile kernel for 16-byte aligned rows (64 / 128 tiles, packed FMAs, double-buffered shared memory): every
    pid, ragged edges, K tails that are not a multiple of 16, forced split-K, alpha / beta; K = 1001 has unaligned rows
    and takes the plain kernel.  Within 1e-4 of the oracle on uniform inputs, exact on small integers."""
    a = rng.uniform(230, 0, (m, k), -1.0, 1.0)
    b = rng.uniform(230, 1, (n, k), -1.0, 1.0)
    c0 = rng.uniform(230, 2, (n, m), -1.0, 1.0)
    ref = oracle.gemm_f32_rcc(a, b)
    ref_ab = oracle.gemm_f32_rcc(a, b, 0.5, -1.5, c0)
    A, B = dev(a), dev(b)
    for pid in (0, 7, 15, 23, 31, 39):
        for split in (1, 3):
            c = api.gemm_rcc_pid(A, B, pid, split).cpu().numpy()
            assert np.all(np.abs(c - ref) <= 1e-4 * np.maximum(1.0, np.abs(ref))), (pid, split)
        c = api.gemm_rcc_pid(A, B, pid, 1, c_nm=dev(c0), alpha=0.5, beta=-1.5).cpu().numpy()
        assert np.all(np.abs(c - ref_ab) <= 1e-4 * np.maximum(1.0, np.abs(ref_ab))), pid
    ai = rng.small_ints(231, 0, (m, k), dtype=np.float32)
    bi = rng.small_ints(231, 1, (n, k), dtype=np.float32)
    exact = (ai.astype(np.int64) @ bi.astype(np.int64).T).T.astype(np.float32)
    for pid in (23, 31):
        assert np.array_equal(api.gemm_rcc_pid(dev(ai), dev(bi), pid, 1).cpu().numpy(), exact), pid
        assert np.array_equal(api.gemm_rcc_pid(dev(ai), dev(bi), pid, 2).cpu().numpy(), exact), pid
    assert api.device_status() == 0


@pytest.mark.parametrize("m,n,k", [(200, 300, 1001), (37, 1024, 1023), (5, 64, 3), (640, 130, 2050)])
def test_fp32_unaligned_k_padded_copies(api, oracle, m, n, k, monkeypatch):
    """FP32 rows that are not 16-byte aligned (K not a multiple of 4): the selector entry runs the aligned kernels on
    zero-padded copies; the added terms are +0, so the result equals the plain kernel's to within the tolerance of the
    oracle and is exact on small integers."""
    a = rng.uniform(232, 0, (m, k), -1.0, 1.0)
    b = rng.uniform(232, 1, (n, k), -1.0, 1.0)
    ref = oracle.gemm_f32_rcc(a, b)
    n0 = api.launch_count()
    c = api.gemm_rcc(dev(a), dev(b)).cpu().numpy()
    assert api.launch_count() - n0 >= 3
    assert np.all(np.abs(c - ref) <= 1e-4 * np.maximum(1.0, np.abs(ref)))
    monkeypatch.setenv("MOONPOLY_DISABLE_PAD", "1")
    c2 = api.gemm_rcc(dev(a), dev(b)).cpu().numpy()
    monkeypatch.delenv("MOONPOLY_DISABLE_PAD")
    assert np.all(np.abs(c2 - ref) <= 1e-4 * np.maximum(1.0, np.abs(ref)))
    ai = rng.small_ints(233, 0, (m, k), dtype=np.float32)
    bi = rng.small_ints(233, 1, (n, k), dtype=np.float32)
    exact = (ai.astype(np.int64) @ bi.astype(np.int64).T).T.astype(np.float32)
    assert np.array_equal(api.gemm_rcc(dev(ai), dev(bi)).cpu().numpy(), exact)
    assert api.device_status() == 0


def test_fp32_every_pid(api, oracle):
    m, n, k = 70, 150, 96
    a = rng.uniform(18, 0, (m, k), -1.0, 1.0)
    b = rng.uniform(18, 1, (n, k), -1.0, 1.0)
    ref = oracle.gemm_f32_rcc(a, b)
    for pid in range(40):
        c = api.gemm_rcc_pid(dev(a), dev(b), pid, 1).cpu().numpy()
        assert np.all(np.abs(c - ref) <= 1e-4 * np.maximum(1.0, np.abs(ref))), pid


# ---------------------------------------------------------------------------------------- INT8
@pytest.mark.parametrize("m,n,k", [(16, 32, 64), (64, 128, 128), (128, 256, 256), (37, 200, 4096), (1, 6144, 512)])
def test_int8_bit_exact(api, oracle, m, n, k, monkeypatch):
    a = rng.int8_uniform(3, rng.STREAM_A, (m, k))
    b = rng.int8_uniform(3, rng.STREAM_B, (n, k))
    ref = oracle.gemm_i8_rcc(a, b)
    assert np.array_equal(api.gemm_rcc(dev(a), dev(b)).cpu().numpy(), ref)
    # tests/cpp/int8/test_int8_row_col_col.cu: forced split-K 2 must stay bit-exact
    monkeypatch.setenv("MOONPOLY_INT8_PATTERN3_FORCE_SPLITK", "2")
    assert np.array_equal(api.gemm_rcc(dev(a), dev(b)).cpu().numpy(), ref)


def test_int8_every_pid_and_alpha_beta(api, oracle):
    m, n, k = 150, 70, 512
    a = rng.int8_uniform(19, 0, (m, k))
    b = rng.int8_uniform(19, 1, (n, k))
    c0 = rng.int8_uniform(19, 2, (n, m)).astype(np.int32) * 37
    ref = oracle.gemm_i8_rcc(a, b)
    ref_ab = oracle.gemm_i8_rcc(a, b, 2, -3, c0)
    for pid in range(46):
        assert np.array_equal(api.gemm_rcc_pid(dev(a), dev(b), pid, 1).cpu().numpy(), ref), pid
    got = api.gemm_rcc_pid(dev(a), dev(b), 6, 4, c_nm=dev(c0), alpha=2.0, beta=-3.0).cpu().numpy()
    assert np.array_equal(got, ref_ab)


def test_int8_unaligned_k(api, oracle):
    m, n, k = 9, 33, 100       # k % 16 != 0 -> CUDA-core tiles
    a = rng.int8_uniform(20, 0, (m, k))
    b = rng.int8_uniform(20, 1, (n, k))
    assert np.array_equal(api.gemm_rcc(dev(a), dev(b)).cpu().numpy(), oracle.gemm_i8_rcc(a, b))


def test_scaled_mm_known_answer(api):
    m, n, k = 24, 40, 64
    a = rng.int8_uniform(3, rng.STREAM_A, (m, k))
    b = rng.int8_uniform(3, rng.STREAM_B, (n, k))
    out = api.scaled_int8_mm(dev(a), dev(b).t(), dev(GOLD["scaled_24x40x64_sa"]), dev(GOLD["scaled_24x40x64_sb"]))
    assert np.array_equal(out.cpu().numpy(), GOLD["scaled_24x40x64_out"])


@pytest.mark.parametrize("M", [1, 8, 32, 47, 160, 700])
@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("mode", ["tensor", "token_channel", "tensor_channel", "token_tensor"])
@pytest.mark.parametrize("with_bias", [False, True])
def test_scaled_mm_bit_exact_vs_oracle(api, oracle, M, bf16, mode, with_bias):
    # the scale modes and dtypes of tests/python/test_int8_scaled_mm_correctness.py
    N, K = 384, 512
    a = rng.int8_uniform(3, rng.STREAM_A, (M, K))
    b = rng.int8_uniform(3, rng.STREAM_B, (N, K))
    sa = rng.uniform(3, rng.STREAM_A_SCALE, (1 if mode in ("tensor", "tensor_channel") else M,), 0.001, 0.02)
    sb = rng.uniform(3, rng.STREAM_B_SCALE, (1 if mode in ("tensor", "token_tensor") else N,), 0.001, 0.02)
    bias = None
    tb = None
    if with_bias:
        bf = rng.uniform(3, rng.STREAM_BIAS, (N,), -1.0, 1.0)
        if bf16:
            bias = oracle.bf16_bits_from_f32(bf)
            tb = dev(bias.view(np.int16)).view(torch.bfloat16)
        else:
            bias = bf.astype(np.float16)
            tb = dev(bias)
    ref = oracle.scaled_mm_i8(a, b, sa, sb, bias, bf16)
    out = api.scaled_int8_mm(dev(a), dev(b).t(), dev(sa), dev(sb), tb,
                             torch.bfloat16 if bf16 else torch.float16)
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, ref.view(np.uint16))


def test_scaled_mm_unaligned_k(api, oracle):
    M, N, K = 5, 48, 40        # K % 16 != 0: the reference falls back to a float matmul here
    a = rng.int8_uniform(21, 0, (M, K))
    b = rng.int8_uniform(21, 1, (N, K))
    sa = rng.uniform(21, 2, (M,), 0.001, 0.02)
    sb = rng.uniform(21, 3, (N,), 0.001, 0.02)
    out = api.scaled_int8_mm(dev(a), dev(b).t(), dev(sa), dev(sb)).cpu().numpy()
    assert np.array_equal(out, oracle.scaled_mm_i8(a, b, sa, sb))



@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (2, 300, 520), (5, 1000, 1024), (8, 64, 8192), (777, 3, 2048),
                                    (4096, 1, 4096)])
def test_fp16_skinny_kernel_vs_oracle(api, oracle, m, n, k):
    """pid 1100: the streaming kernel for problems with at most 8 rows on one side (both mappings)."""
    a = rng.normal(23, 0, (m, k), 0.05)
    b = rng.normal(23, 1, (n, k), 0.05)
    c0 = rng.normal(23, 2, (n, m), 1.0)
    ref = oracle.gemm_f16_rcc(a, b)
    close_f16(api.gemm_rcc_pid(dev(a), dev(b), 1100, 1).cpu().numpy(), ref)
    ref_ab = oracle.gemm_f16_rcc(a, b, 0.5, -1.5, c0)
    close_f16(api.gemm_rcc_pid(dev(a), dev(b), 1100, 1, c_nm=dev(c0), alpha=0.5, beta=-1.5).cpu().numpy(), ref_ab)
    ai = rng.small_ints(24, 0, (m, k), lo=-1, hi=1)
    bi = rng.small_ints(24, 1, (n, k))
    exact = (ai.astype(np.int64) @ bi.astype(np.int64).T).T.astype(np.float16)
    assert np.array_equal(api.gemm_rcc_pid(dev(ai), dev(bi), 1100, 1).cpu().numpy(), exact)


def test_fp16_skinny_pid_on_wide_problem_uses_tensor_tiles(api, oracle):
    a = rng.normal(25, 0, (40, 512), 0.05)
    b = rng.normal(25, 1, (200, 512), 0.05)
    close_f16(api.gemm_rcc_pid(dev(a), dev(b), 1100, 1).cpu().numpy(), oracle.gemm_f16_rcc(a, b))


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (2, 300, 520), (8, 1000, 1024), (9, 64, 8192), (16, 4096, 4096),
                                    (31, 513, 2048), (64, 1024, 4096), (777, 3, 2048), (4096, 24, 4096),
                                    (130, 57, 72)])
def test_fp16_streaming_kernel_vs_oracle(api, oracle, m, n, k):
    """pid 1101: the streaming warp-MMA kernel for problems with at most 64 rows on one side (both mappings)."""
    a = rng.normal(26, 0, (m, k), 0.05)
    b = rng.normal(26, 1, (n, k), 0.05)
    c0 = rng.normal(26, 2, (n, m), 1.0)
    ref = oracle.gemm_f16_rcc(a, b)
    close_f16(api.gemm_rcc_pid(dev(a), dev(b), 1101, 1).cpu().numpy(), ref)
    ref_ab = oracle.gemm_f16_rcc(a, b, 0.5, -1.5, c0)
    close_f16(api.gemm_rcc_pid(dev(a), dev(b), 1101, 1, c_nm=dev(c0), alpha=0.5, beta=-1.5).cpu().numpy(), ref_ab)
    ai = rng.small_ints(27, 0, (m, k), lo=-1, hi=1)
    bi = rng.small_ints(27, 1, (n, k))
    exact = (ai.astype(np.int64) @ bi.astype(np.int64).T).T.astype(np.float16)
    assert np.array_equal(api.gemm_rcc_pid(dev(ai), dev(bi), 1101, 1).cpu().numpy(), exact)


def test_fp16_streaming_pid_on_wide_problem_uses_tensor_tiles(api, oracle):
    a = rng.normal(28, 0, (100, 512), 0.05)
    b = rng.normal(28, 1, (200, 512), 0.05)
    close_f16(api.gemm_rcc_pid(dev(a), dev(b), 1101, 1).cpu().numpy(), oracle.gemm_f16_rcc(a, b))


def test_launches_are_capturable_in_a_cuda_graph(api):
    """The three kernel families (streaming, tcgen05 with split-K, tcgen05 single slice) recorded into one CUDA
    graph and replayed on fresh inputs: the library allocates nothing and synchronises nothing once warm."""
    k = 2048
    shapes = [(4, 512, None, 1), (200, 136, 415, 4), (300, 264, None, 1)]      # (m, n, pid or selector, split_k)
    A = [torch.empty((m, k), dtype=torch.float16, device="cuda") for m, _, _, _ in shapes]
    B = [torch.empty((n, k), dtype=torch.float16, device="cuda") for _, n, _, _ in shapes]
    C = [torch.empty((n, m), dtype=torch.float16, device="cuda") for m, n, _, _ in shapes]

    def fill(seed):
        refs = []
        for i, (m, n, _, _) in enumerate(shapes):
            a = rng.small_ints(seed, 2 * i, (m, k))
            b = rng.small_ints(seed, 2 * i + 1, (n, k), lo=-1, hi=1)
            A[i].copy_(dev(a))
            B[i].copy_(dev(b))
            refs.append((a.astype(np.int64) @ b.astype(np.int64).T).T.astype(np.float16))
        return refs

    def launch_all():
        for i, (_, _, pid, split_k) in enumerate(shapes):
            if pid is None:
                api.gemm_rcc(A[i], B[i], c_nm=C[i])
            else:
                api.gemm_rcc_pid(A[i], B[i], pid, split_k, c_nm=C[i])

    fill(40)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launch_all()                      # warm-up on the capture stream: scratch and plans exist afterwards
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        launch_all()
    for seed in (41, 42):
        refs = fill(seed)
        for c in C:
            c.zero_()
        g.replay()
        torch.cuda.synchronize()
        for c, ref in zip(C, refs):
            assert np.array_equal(c.cpu().numpy(), ref)
    assert api.device_status() == 0


def _exact_ref(a, b):
    # small integers: float64 BLAS is exact and fast
    return (a.astype(np.float64) @ b.astype(np.float64).T).T


@pytest.mark.parametrize("orient,bn,m,n,k", [(0, 64, 1280, 1280, 1024), (0, 64, 1275, 1270, 1096),
                                              (1, 128, 1100, 2500, 2048), (1, 256, 4096, 4096, 512),
                                              (0, 32, 700, 1000, 4096)])
def test_fp16_stream_k_head_exact_and_switchable(api, monkeypatch, orient, bn, m, n, k):
    """Tile counts that are not a multiple of the grid: the first tiles are cut along K over all CTAs and finished
    through the scratch.  Integer-valued inputs make every summation order exact, so the result must equal the
    plain schedule's (MOONPOLY_DISABLE_STREAMK=1) and the known answer, with and without alpha/beta."""
    a = rng.small_ints(50, 0, (m, k), lo=-1, hi=1)
    b = rng.small_ints(50, 1, (n, k))
    ref = _exact_ref(a, b)
    assert np.abs(ref).max() < 2048
    A, B = dev(a), dev(b)
    c0 = rng.small_ints(50, 2, (n, m)).astype(np.float16)
    try:
        got = api.gemm_rcc_tile(A, B, orient, bn).cpu().numpy()
        again = api.gemm_rcc_tile(A, B, orient, bn).cpu().numpy()
        got_ab = api.gemm_rcc_tile(A, B, orient, bn, c_nm=dev(c0).clone(), alpha=2.0, beta=-1.0).cpu().numpy()
        monkeypatch.setenv("MOONPOLY_DISABLE_STREAMK", "1")
        api.reload_env()
        plain = api.gemm_rcc_tile(A, B, orient, bn).cpu().numpy()
    finally:
        monkeypatch.delenv("MOONPOLY_DISABLE_STREAMK", raising=False)
        api.reload_env()
    assert np.array_equal(got, ref.astype(np.float16))
    assert np.array_equal(got, again)
    assert np.array_equal(got, plain)
    assert np.array_equal(got_ab, (2.0 * ref - c0.astype(np.float64)).astype(np.float16))
    assert api.device_status() == 0


def test_int8_stream_k_head_bit_exact(api):
    m, n, k = 1300, 2100, 2048
    a = rng.int8_uniform(51, 0, (m, k))
    b = rng.int8_uniform(51, 1, (n, k))
    ref = (a.astype(np.float64) @ b.astype(np.float64).T).T.astype(np.int64)
    got = api.gemm_rcc_tile(dev(a), dev(b), 1, 128).cpu().numpy()
    assert np.array_equal(got.astype(np.int64), ref)


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (7, 300, 528), (32, 1000, 1024), (64, 130, 2048), (777, 3, 2048),
                                    (4096, 24, 512)])
def test_int8_streaming_kernel_bit_exact(api, oracle, m, n, k):
    """pid 1101 with INT8 operands: exact int32 accumulators through the warp-level s8 MMA, both mappings."""
    a = rng.int8_uniform(60, 0, (m, k))
    b = rng.int8_uniform(60, 1, (n, k))
    c0 = rng.int8_uniform(60, 2, (n, m)).astype(np.int32) * 37
    ref = (a.astype(np.float64) @ b.astype(np.float64).T).T.astype(np.int64)
    got = api.gemm_rcc_pid(dev(a), dev(b), 1101, 1).cpu().numpy()
    assert np.array_equal(got.astype(np.int64), ref)
    got_ab = api.gemm_rcc_pid(dev(a), dev(b), 1101, 1, c_nm=dev(c0), alpha=2.0, beta=-3.0).cpu().numpy()
    assert np.array_equal(got_ab.astype(np.int64), 2 * ref - 3 * c0.astype(np.int64))
    if min(m, n) <= 32:
        plan = api.select_plan(api.MP_INT8, m, n, k)
        assert plan.pid == 1101
        assert np.array_equal(api.gemm_rcc(dev(a), dev(b)).cpu().numpy(), got)


@pytest.mark.parametrize("M,N", [(700, 24), (5, 48), (300, 8)])
@pytest.mark.parametrize("bf16", [False, True])
def test_scaled_mm_few_channels_bit_exact(api, oracle, M, N, bf16):
    """Few output channels: the tokens become the streamed rows and the channel index moves to the narrow side."""
    K = 1024
    a = rng.int8_uniform(61, 0, (M, K))
    b = rng.int8_uniform(61, 1, (N, K))
    sa = rng.uniform(61, 2, (M,), 0.001, 0.02)
    sb = rng.uniform(61, 3, (N,), 0.001, 0.02)
    bf = rng.uniform(61, 4, (N,), -1.0, 1.0)
    if bf16:
        bias = oracle.bf16_bits_from_f32(bf)
        tb = dev(bias.view(np.int16)).view(torch.bfloat16)
    else:
        bias = bf.astype(np.float16)
        tb = dev(bias)
    ref = oracle.scaled_mm_i8(a, b, sa, sb, bias, bf16)
    out = api.scaled_int8_mm(dev(a), dev(b).t(), dev(sa), dev(sb), tb, torch.bfloat16 if bf16 else torch.float16)
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, ref.view(np.uint16))


@pytest.mark.parametrize("orient,bn,m,n,k", [(4, 256, 600, 520, 256), (5, 256, 520, 600, 320), (4, 128, 257, 300, 1096),
                                              (5, 192, 1000, 1300, 512), (4, 64, 2500, 200, 2048)])
def test_fp16_256_row_tiles_exact(api, orient, bn, m, n, k):
    """256-row tiles (two 128-row halves share every bn-wide tile of the other operand; orient 4 / 5 of the
    tuning entry, pids 1200+): exact on integer-valued inputs, ragged edges in both dimensions, alpha/beta."""
    a = rng.small_ints(70, 0, (m, k), lo=-1, hi=1)
    b = rng.small_ints(70, 1, (n, k))
    ref = _exact_ref(a, b)
    A, B = dev(a), dev(b)
    got = api.gemm_rcc_tile(A, B, orient, bn).cpu().numpy()
    assert np.array_equal(got, ref.astype(np.float16))
    pid = 1200 + 32 * (orient - 4) + bn // 16
    assert np.array_equal(api.gemm_rcc_pid(A, B, pid, 1).cpu().numpy(), got)
    c0 = rng.small_ints(70, 2, (n, m)).astype(np.float16)
    got_ab = api.gemm_rcc_tile(A, B, orient, bn, c_nm=dev(c0).clone(), alpha=2.0, beta=-1.0).cpu().numpy()
    assert np.array_equal(got_ab, (2.0 * ref - c0.astype(np.float64)).astype(np.float16))
    assert api.device_status() == 0


def test_int8_256_row_tiles_bit_exact(api):
    m, n, k = 700, 900, 1024
    a = rng.int8_uniform(71, 0, (m, k))
    b = rng.int8_uniform(71, 1, (n, k))
    ref = (a.astype(np.float64) @ b.astype(np.float64).T).T.astype(np.int64)
    for orient in (4, 5):
        got = api.gemm_rcc_tile(dev(a), dev(b), orient, 256).cpu().numpy()
        assert np.array_equal(got.astype(np.int64), ref)



@pytest.mark.parametrize("m", [5, 100, 300, 2500])
def test_int8_gemm_follows_measured_plans_bit_exact(api, m):
    """Plain INT8 GEMM on a shape the measured scaled-matmul table covers: the selector names a library-native
    kernel (streaming, 128-row or 256-row tile) and the int32 accumulators stay exact."""
    n, k = 4096, 4096
    a = rng.int8_uniform(90, 0, (m, k))
    b = rng.int8_uniform(90, 1, (n, k))
    plan = api.select_plan(api.MP_INT8, m, n, k)
    assert plan.pid >= 1000, plan
    ref = (a.astype(np.float64) @ b.astype(np.float64).T).T.astype(np.int64)
    got = api.gemm_rcc(dev(a), dev(b)).cpu().numpy()
    assert np.array_equal(got.astype(np.int64), ref)
    assert np.array_equal(api.gemm_rcc_pid(dev(a), dev(b), plan.pid, plan.split_k).cpu().numpy(), got)


@pytest.mark.parametrize("m,n,k", [(37, 1024, 1024), (1, 300, 512), (64, 129, 2052), (700, 5, 1024), (9, 40, 8),
                                   (16, 500, 2000), (33, 2000, 1280), (40, 64, 1024), (12, 4096, 4096), (1000, 20, 2560),
                                   (17, 1001, 260), (24, 77, 516), (41, 1500, 1028), (64, 4000, 768), (25, 9, 4)])
def test_fp32_streaming_kernel(api, oracle, m, n, k):
    """Library-native pid 1101 for FP32 (one warp per row of the wide operand): within 1e-4 of the oracle on
    uniform inputs, exact on small integers, alpha/beta, both mappings; the selector names it for these shapes."""
    a = rng.uniform(95, 0, (m, k), -1.0, 1.0)
    b = rng.uniform(95, 1, (n, k), -1.0, 1.0)
    ref = oracle.gemm_f32_rcc(a, b)
    assert api.select_plan(api.MP_FP32, m, n, k).pid == 1101
    for c in (api.gemm_rcc(dev(a), dev(b)).cpu().numpy(), api.gemm_rcc_pid(dev(a), dev(b), 1101, 1).cpu().numpy()):
        assert np.all(np.abs(c - ref) <= 1e-4 * np.maximum(1.0, np.abs(ref)))
    ai = rng.small_ints(96, 0, (m, k), dtype=np.float32)
    bi = rng.small_ints(96, 1, (n, k), dtype=np.float32)
    c0 = rng.small_ints(96, 2, (n, m), dtype=np.float32)
    exact = (ai.astype(np.int64) @ bi.astype(np.int64).T).T
    assert np.array_equal(api.gemm_rcc_pid(dev(ai), dev(bi), 1101, 1).cpu().numpy(), exact.astype(np.float32))
    got = api.gemm_rcc_pid(dev(ai), dev(bi), 1101, 1, c_nm=dev(c0).clone(), alpha=2.0, beta=-1.0).cpu().numpy()
    assert np.array_equal(got, (2 * exact - c0.astype(np.int64)).astype(np.float32))


_F32_TILE_CHILD = r"""
import sys, numpy as np, torch
sys.path[:0] = [sys.argv[1], sys.argv[2]]
from moonpoly_b200 import api, rng
from oracle import oracle
for (m, n, k) in [(37, 1024, 1024), (64, 129, 2052), (9, 40, 8), (33, 2000, 1280), (1000, 20, 2560), (17, 1001, 260)]:
    a = rng.uniform(97, 0, (m, k), -1.0, 1.0)
    b = rng.uniform(97, 1, (n, k), -1.0, 1.0)
    c0 = rng.uniform(97, 2, (n, m), -1.0, 1.0)
    ref = oracle.gemm_f32_rcc(a, b, 0.5, -1.5, c0)
    got = api.gemm_rcc_pid(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), 1101, 1,
                           c_nm=torch.from_numpy(c0).cuda(), alpha=0.5, beta=-1.5).cpu().numpy()
    assert np.all(np.abs(got - ref) <= 1e-4 * np.maximum(1.0, np.abs(ref))), (m, n, k)
assert api.device_status() == 0
print("ok")
"""


@pytest.mark.parametrize("shape", ["8,1", "8,2", "16,1", "16,4", "8,8", "32,1", "32,2", "32,8"])
def test_fp32_tile_kernel_launch_shapes(shape):
    """The FP32 tile kernel with 8, 16 or 32 rows per CTA and K split over a cluster of 1, 2, 4 or 8 CTAs (the launch
    shape is read from MOONPOLY_F32_TILE once per process, hence the child process)."""
    import subprocess
    import sys
    root = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
    env = dict(os.environ, MOONPOLY_F32_TILE=shape)
    out = subprocess.run([sys.executable, "-c", _F32_TILE_CHILD, root, os.path.join(root, "moonpoly-dev_b200", "py")],
                         env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stdout + out.stderr


@pytest.mark.parametrize("m,n,k", [(438, 10, 3695), (83, 286, 3269), (1, 300, 1001), (256, 512, 130), (37, 64, 7), (700, 900, 2)])
def test_unaligned_k_runs_on_padded_copies(api, oracle, m, n, k, monkeypatch):
    """FP16 rows that miss TMA's 16-byte rule (K not a multiple of 8): the selector entries copy both operands into
    zero-padded aligned rows and run the tensor path; same results as the CUDA-core fall-back within FP16 tolerance,
    exact on small integers, alpha / beta, and a second call of another size re-uses or regrows the copy buffer."""
    a = rng.normal(220, 0, (m, k), 0.05)
    b = rng.normal(220, 1, (n, k), 0.05)
    c0 = rng.normal(220, 2, (n, m), 1.0)
    ref = oracle.gemm_f16_rcc(a, b)
    n0 = api.launch_count()
    got = api.gemm_rcc(dev(a), dev(b)).cpu().numpy()
    assert api.launch_count() - n0 >= 3                  # two copies and the GEMM
    close_f16(got, ref)
    close_f16(api.gemm_rcc(dev(a), dev(b), c_nm=dev(c0), alpha=0.5, beta=-1.5).cpu().numpy(), oracle.gemm_f16_rcc(a, b, 0.5, -1.5, c0))
    monkeypatch.setenv("MOONPOLY_DISABLE_PAD", "1")
    n0 = api.launch_count()
    close_f16(api.gemm_rcc(dev(a), dev(b)).cpu().numpy(), ref)
    assert api.launch_count() - n0 <= 2                  # the CUDA-core tiles (and their split-K pass)
    monkeypatch.delenv("MOONPOLY_DISABLE_PAD")
    ai = rng.small_ints(221, 0, (m, k), lo=-1, hi=1)
    bi = rng.small_ints(221, 1, (n, k))
    exact = (ai.astype(np.int64) @ bi.astype(np.int64).T).T.astype(np.float16)
    assert np.array_equal(api.gemm_rcc(dev(ai), dev(bi)).cpu().numpy(), exact)
    # a base address that is only element-aligned (a view one element into a buffer) takes the same route
    L = api.lib()
    out = torch.empty((n, m), dtype=torch.float16, device=DEV)
    B = dev(b)
    flat = torch.zeros((m * k + 1,), dtype=torch.float16, device=DEV)
    a_mis = flat[1:].view(m, k)
    a_mis.copy_(dev(a))
    assert a_mis.data_ptr() % 16 != 0
    rc = L.mp_gemm_rcc(api.MP_FP16, m, n, k, a_mis.data_ptr(), B.data_ptr(), out.data_ptr(), 1.0, 0.0, None)
    assert rc == 0, L.mp_last_error_string()
    torch.cuda.synchronize()
    close_f16(out.cpu().numpy(), ref)
    assert api.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(1024, 1024, 1032), (579, 1560, 3160), (5, 200, 1000), (64, 64, 24)])
def test_int8_unaligned_k_padded_copies_bit_exact(api, oracle, M, N, K):
    """INT8 with K not a multiple of 16: int32 accumulators stay exact and the scaled matmul bit-identical to the
    oracle through the padded copies."""
    a = rng.int8_uniform(222, 0, (M, K))
    b = rng.int8_uniform(222, 1, (N, K))
    assert np.array_equal(api.gemm_rcc(dev(a), dev(b)).cpu().numpy(), oracle.gemm_i8_rcc(a, b))
    sa = rng.uniform(222, 2, (M,), 0.001, 0.02)
    sb = rng.uniform(222, 3, (N,), 0.001, 0.02)
    bias = rng.uniform(222, 4, (N,), -1.0, 1.0).astype(np.float16)
    ref = oracle.scaled_mm_i8(a, b, sa, sb, bias)
    n0 = api.launch_count()
    got = api.scaled_int8_mm(dev(a), dev(b).t(), dev(sa), dev(sb), dev(bias)).cpu().numpy()
    assert api.launch_count() - n0 >= 3
    assert np.array_equal(got.view(np.uint16), ref.view(np.uint16))
    assert api.device_status() == 0


def test_scaled_mm_padded_leading_dimensions_and_ragged_k(api, oracle):
    """Rows that are padded to a 16-byte multiple while K itself is not (K = 100, lda = ldb = 112): the streaming
    kernels walk K in whole 16-byte chunks and must not be chosen; the tensor tiles zero-fill the K tail."""
    L = api.lib()
    K, ld = 100, 112
    for (M, N) in ((5, 48), (40, 200), (300, 24)):
        a = rng.int8_uniform(110, 0, (M, K))
        b = rng.int8_uniform(110, 1, (N, K))
        sa = rng.uniform(110, 2, (M,), 0.001, 0.02)
        sb = rng.uniform(110, 3, (N,), 0.001, 0.02)
        ap = np.full((M, ld), 77, np.int8); ap[:, :K] = a          # the padding holds garbage on purpose
        bp = np.full((N, ld), -55, np.int8); bp[:, :K] = b
        A, B, SA, SB = dev(ap), dev(bp), dev(sa), dev(sb)
        out = torch.empty((M, N), dtype=torch.float16, device=DEV)
        rc = L.mp_scaled_mm_i8(M, N, K, A.data_ptr(), ld, B.data_ptr(), ld, SA.data_ptr(), 0, SB.data_ptr(), 0, None,
                               out.data_ptr(), N, 0, None)
        assert rc == 0, L.mp_last_error_string()
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), oracle.scaled_mm_i8(a, b, sa, sb)), (M, N)


def test_library_scratch_regrows_behind_a_large_counter_area(api):
    """A forced split-K call with 2592 tiles gives the library's own scratch a 162 KB counter area (the default is
    64 KB) in front of 82 MB of partial sums.  The next call has few tiles but needs 82 MB + 32 KB of partial sums:
    that fits behind a 64 KB counter area, not behind the one the buffer really has, so the buffer must grow.
    Integer-valued inputs: results are exact whatever the summation order."""
    k = 1024
    a1 = rng.small_ints(120, 0, (2304, k), lo=-1, hi=1)            # 18 x 144 tiles of 128 x 16
    b1 = rng.small_ints(120, 1, (2304, k))
    got = api.gemm_rcc_tile(dev(a1), dev(b1), 0, 16, split_k=2).cpu().numpy()
    assert np.array_equal(got, _exact_ref(a1, b1).astype(np.float16))
    a2 = rng.small_ints(121, 0, (640, k), lo=-1, hi=1)             # 5 x 25 tiles of 128 x 224, 6 slices
    b2 = rng.small_ints(121, 1, (5600, k))
    got = api.gemm_rcc_tile(dev(a2), dev(b2), 0, 224, split_k=6).cpu().numpy()
    assert np.array_equal(got, _exact_ref(a2, b2).astype(np.float16))
    again = api.gemm_rcc_tile(dev(a1), dev(b1), 0, 16, split_k=2).cpu().numpy()
    assert np.array_equal(again, _exact_ref(a1, b1).astype(np.float16))
    assert api.device_status() == 0


@pytest.mark.parametrize("pid,m,n", [(1101, 130, 65), (1101, 65, 130), (1100, 130, 65), (1101, 200, 300)])
def test_reported_workspace_is_enough_for_the_streaming_pids_fallback(api, oracle, pid, m, n):
    k, split = 2048, 2
    a = rng.normal(122, 0, (m, k), 0.05)
    b = rng.normal(122, 1, (n, k), 0.05)
    need = api.workspace_size(api.MP_FP16, pid, m, n, k, split)
    assert need > 0
    ws = torch.full((need,), 0xCD, dtype=torch.uint8, device=DEV)
    c = api.gemm_rcc_pid(dev(a), dev(b), pid, split, workspace=ws).cpu().numpy()
    close_f16(c, oracle.gemm_f16_rcc(a, b))


# ------------------------------------------------------------------ split-K inside a thread-block cluster
def _with_and_without_cluster(api, monkeypatch, fn):
    """Runs fn() with the cluster split-K path (MOONPOLY_ENABLE_CLUSTER_SPLITK=1) and with the default path (partials
    through the global scratch)."""
    try:
        monkeypatch.setenv("MOONPOLY_ENABLE_CLUSTER_SPLITK", "1")
        api.reload_env()
        with_cluster = fn()
    finally:
        monkeypatch.delenv("MOONPOLY_ENABLE_CLUSTER_SPLITK", raising=False)
        api.reload_env()
    without = fn()
    return with_cluster, without


@pytest.mark.parametrize("orient,bn,split,m,n,k", [
    (1, 128, 4, 128, 4096, 4096),      # the sweep's M = 128 plan: 32 tiles x 4 slices, one CTA each
    (1, 64, 4, 64, 4096, 4096), (0, 128, 2, 4096, 255, 4096), (1, 256, 2, 250, 2000, 2048),
    (0, 16, 8, 1024, 8, 8192),         # decode shape through a 128 x 16 tile, 8 slices
    (0, 32, 8, 1000, 30, 8200), (1, 48, 4, 40, 1100, 2072), (0, 96, 2, 300, 90, 520), (0, 208, 4, 130, 200, 2048)])
def test_fp16_cluster_splitk_bit_identical_to_scratch_path(api, oracle, monkeypatch, orient, bn, split, m, n, k):
    """The K slices of a tile run as one thread-block cluster and exchange partial sums through distributed shared
    memory.  Every column is still summed in slice order, so the result must equal the scratch path's bit for bit
    (N(0,1)*0.05 inputs: any change of summation order would show), and agree with the oracle."""
    a = rng.normal(130, 0, (m, k), 0.05)
    b = rng.normal(130, 1, (n, k), 0.05)
    c0 = rng.normal(130, 2, (n, m), 1.0)
    A, B = dev(a), dev(b)
    got, plain = _with_and_without_cluster(api, monkeypatch, lambda: api.gemm_rcc_tile(A, B, orient, bn, split_k=split).cpu().numpy())
    assert np.array_equal(got, plain)
    rows = min(m, 256)                                   # every output is an independent dot product: check the first rows
    close_f16(got[:, :rows], oracle.gemm_f16_rcc(a[:rows], b))
    got_ab, plain_ab = _with_and_without_cluster(
        api, monkeypatch,
        lambda: api.gemm_rcc_tile(A, B, orient, bn, split_k=split, c_nm=dev(c0).clone(), alpha=0.5, beta=-1.5).cpu().numpy())
    assert np.array_equal(got_ab, plain_ab)
    assert api.device_status() == 0


@pytest.mark.parametrize("split", [2, 4, 8])
def test_int8_cluster_splitk_exact(api, oracle, monkeypatch, split):
    m, n, k = 150, 700, 4096
    a = rng.int8_uniform(131, 0, (m, k))
    b = rng.int8_uniform(131, 1, (n, k))
    A, B = dev(a), dev(b)
    got, plain = _with_and_without_cluster(api, monkeypatch, lambda: api.gemm_rcc_tile(A, B, 1, 128, split_k=split).cpu().numpy())
    assert np.array_equal(got, plain)
    assert np.array_equal(got, oracle.gemm_i8_rcc(a, b))
    # the scaled epilogue on the same launch shape
    sa = rng.uniform(131, 2, (m,), 0.001, 0.02)
    sb = rng.uniform(131, 3, (n,), 0.001, 0.02)
    bias = rng.uniform(131, 4, (n,), -1.0, 1.0).astype(np.float16)
    L = api.lib()
    SA, SB, BI = dev(sa), dev(sb), dev(bias)

    def scaled():
        out = torch.empty((m, n), dtype=torch.float16, device=DEV)
        rc = L.mp_scaled_mm_i8_tile(1, 128, split, m, n, k, A.data_ptr(), k, B.data_ptr(), k, SA.data_ptr(), 0, SB.data_ptr(), 0,
                                    BI.data_ptr(), out.data_ptr(), n, 0, None)
        assert rc == 0, L.mp_last_error_string()
        torch.cuda.synchronize()
        return out.cpu().numpy()
    s_got, s_plain = _with_and_without_cluster(api, monkeypatch, scaled)
    assert np.array_equal(s_got.view(np.uint16), s_plain.view(np.uint16))
    assert np.array_equal(s_got.view(np.uint16), oracle.scaled_mm_i8(a, b, sa, sb, bias).view(np.uint16))
    assert api.device_status() == 0


# ------------------------------------------------------------------ 256-row tiles with K slices
@pytest.mark.parametrize("orient,bn,split,m,n,k", [(4, 256, 4, 512, 4096, 4096), (5, 256, 2, 1000, 1023, 4096),
                                                    (4, 128, 8, 257, 300, 2120), (5, 192, 3, 600, 700, 1096),
                                                    (4, 64, 2, 2500, 200, 2048), (4, 256, 8, 255, 4096, 4096)])
def test_fp16_256_row_tiles_with_k_slices(api, oracle, orient, bn, split, m, n, k):
    """256-row tiles whose K is cut into slices: both 128-row halves of every slice are parked in the scratch and
    summed in slice order.  Exact on integer-valued inputs (ragged edges, alpha / beta), reproducible and within
    tolerance of the oracle on N(0,1)*0.05 inputs; pids 1200+ honour the run-time split factor."""
    a = rng.small_ints(150, 0, (m, k), lo=-1, hi=1)
    b = rng.small_ints(150, 1, (n, k))
    ref = _exact_ref(a, b)
    assert np.abs(ref).max() < 2048
    A, B = dev(a), dev(b)
    got = api.gemm_rcc_tile(A, B, orient, bn, split_k=split).cpu().numpy()
    assert np.array_equal(got, ref.astype(np.float16))
    pid = 1200 + 32 * (orient - 4) + bn // 16
    assert np.array_equal(api.gemm_rcc_pid(A, B, pid, split).cpu().numpy(), got)
    need = api.workspace_size(api.MP_FP16, pid, m, n, k, split)
    ws = torch.full((need,), 0x5A, dtype=torch.uint8, device=DEV)
    assert np.array_equal(api.gemm_rcc_pid(A, B, pid, split, workspace=ws).cpu().numpy(), got)
    c0 = rng.small_ints(150, 2, (n, m)).astype(np.float16)
    got_ab = api.gemm_rcc_tile(A, B, orient, bn, split_k=split, c_nm=dev(c0).clone(), alpha=2.0, beta=-1.0).cpu().numpy()
    assert np.array_equal(got_ab, (2.0 * ref - c0.astype(np.float64)).astype(np.float16))
    an = rng.normal(151, 0, (m, k), 0.05)
    bn_ = rng.normal(151, 1, (n, k), 0.05)
    rows = sorted(set([0, m - 1] + list(range(0, m, max(1, m // 64)))))
    gn = api.gemm_rcc_tile(dev(an), dev(bn_), orient, bn, split_k=split).cpu().numpy()
    close_f16(gn[:, rows], oracle.gemm_f16_rcc(an[rows], bn_))
    assert np.array_equal(gn, api.gemm_rcc_tile(dev(an), dev(bn_), orient, bn, split_k=split).cpu().numpy())
    assert api.device_status() == 0


def test_256_row_tiles_stream_k_head_and_int8_slices(api, monkeypatch):
    # 10 x 20 tiles of 256 x 256 on 148 CTAs: the 52 left-over tiles go first, cut along K over all CTAs
    m, n, k = 2560, 5120, 512
    a = rng.small_ints(152, 0, (m, k), lo=-1, hi=1)
    b = rng.small_ints(152, 1, (n, k))
    ref = _exact_ref(a, b).astype(np.float16)
    A, B = dev(a), dev(b)
    try:
        got = api.gemm_rcc_tile(A, B, 4, 256).cpu().numpy()
        monkeypatch.setenv("MOONPOLY_DISABLE_STREAMK", "1")
        api.reload_env()
        plain = api.gemm_rcc_tile(A, B, 4, 256).cpu().numpy()
    finally:
        monkeypatch.delenv("MOONPOLY_DISABLE_STREAMK", raising=False)
        api.reload_env()
    assert np.array_equal(got, ref) and np.array_equal(plain, ref)
    a8 = rng.int8_uniform(153, 0, (700, 2048))
    b8 = rng.int8_uniform(153, 1, (900, 2048))
    ref8 = (a8.astype(np.float64) @ b8.astype(np.float64).T).T.astype(np.int64)
    for orient, split in ((4, 2), (5, 4)):
        got8 = api.gemm_rcc_tile(dev(a8), dev(b8), orient, 256, split_k=split).cpu().numpy()
        assert np.array_equal(got8.astype(np.int64), ref8)
    assert api.device_status() == 0


# ------------------------------------------------------------------ BF16 and fused bias (Linear)
@pytest.mark.parametrize("M,N,K", [(1, 1024, 2048), (7, 4096, 4096), (24, 512, 8192), (64, 1000, 1024), (130, 384, 520),
                                   (300, 2304, 1024), (1000, 520, 2048), (5, 48, 40), (2100, 4096, 512)])
@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("with_bias", [False, True])
def test_linear_bias_fp16_bf16_vs_oracle(api, oracle, M, N, K, bf16, with_bias):
    """Linear with the bias fused into the epilogue, fp16 and bf16: streaming kernels, tensor tiles with and without
    split-K, 256-row tiles, and the CUDA-core tiles for K that TMA cannot describe (K = 40).  Against the oracle within
    the path's tolerance, and bit-identical to the two-step linear + bias the reference's callers do."""
    x32 = rng.normal(170, 0, (M, K), 0.05, dtype=np.float32)
    w32 = rng.normal(170, 1, (N, K), 0.05, dtype=np.float32)
    b32 = rng.uniform(170, 5, (N,), -1.0, 1.0)
    if bf16:
        xb, wb, bb = (oracle.bf16_bits_from_f32(v) for v in (x32, w32, b32))
        X, W, B = (dev(v.view(np.int16)).view(torch.bfloat16) for v in (xb, wb, bb))
        ref = oracle.f32_from_bf16_bits(oracle.linear_bias(xb, wb, bb if with_bias else None, bf16=True))
        rtol, atol = 2e-2, 8e-3            # bf16 keeps 8 bits of mantissa
    else:
        xh, wh, bh = x32.astype(np.float16), w32.astype(np.float16), b32.astype(np.float16)
        X, W, B = dev(xh), dev(wh), dev(bh)
        ref = oracle.linear_bias(xh, wh, bh if with_bias else None).astype(np.float32)
        rtol, atol = 1e-2, 1e-3
    y = api.linear_bias(X, W, B if with_bias else None)
    got = y.float().cpu().numpy()
    bad = np.abs(got - ref) > atol + rtol * np.abs(ref)
    assert not bad.any(), f"{bad.sum()} of {bad.size} differ; max abs {np.abs(got - ref).max()}"
    two_step = api.linear(X, W)
    if with_bias:
        two_step = two_step + B            # torch adds in fp32 and rounds once to the tensor dtype: the same operation
    assert torch.equal(y, two_step)
    assert api.device_status() == 0


def test_bf16_linear_exact_on_integers(api):
    M, N, K = 70, 300, 1024
    x = rng.small_ints(171, 0, (M, K), lo=-1, hi=1, dtype=np.float32)
    w = rng.small_ints(171, 1, (N, K), dtype=np.float32)
    ref = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(ref).max() <= 256                # exactly representable in bf16
    y = api.linear(dev(x).to(torch.bfloat16), dev(w).to(torch.bfloat16))
    assert y.dtype == torch.bfloat16
    assert np.array_equal(y.float().cpu().numpy(), ref.astype(np.float32))


# ------------------------------------------------------------------ token split of the streaming kernel
@pytest.mark.parametrize("m,n,k,parts", [(16, 4096, 4096, 2), (32, 4096, 4096, 2), (32, 4096, 4096, 4), (64, 2048, 4096, 4),
                                          (64, 1024, 2048, 8), (17, 1000, 1024, 2), (17, 1000, 1024, 4), (40, 513, 2056, 2),
                                          (4096, 24, 4096, 2), (700, 33, 2048, 4), (9, 64, 8192, 2), (8, 300, 512, 4)])
def test_fp16_streaming_kernel_token_split(api, oracle, m, n, k, parts):
    """Every block of streamed rows is shared by `parts` neighbouring CTAs, each against its own rows of the narrow
    operand: the same dot products, so the result equals the unsplit kernel's bit for bit; both mappings, ragged
    parts, parts that would be empty are dropped, alpha / beta."""
    a = rng.normal(200, 0, (m, k), 0.05)
    b = rng.normal(200, 1, (n, k), 0.05)
    c0 = rng.normal(200, 2, (n, m), 1.0)
    A, B = dev(a), dev(b)
    plain = api.gemm_rcc_tile(A, B, 3, 16, kc=-1, split_k=1).cpu().numpy()
    split = api.gemm_rcc_tile(A, B, 3, 16, kc=-1, split_k=parts).cpu().numpy()
    assert np.array_equal(split, plain)
    close_f16(split, oracle.gemm_f16_rcc(a, b))
    ref_ab = oracle.gemm_f16_rcc(a, b, 0.5, -1.5, c0)
    close_f16(api.gemm_rcc_tile(A, B, 3, 16, kc=-1, split_k=parts, c_nm=dev(c0), alpha=0.5, beta=-1.5).cpu().numpy(), ref_ab)
    assert api.device_status() == 0


@pytest.mark.parametrize("m,n,k", [(1, 1024, 8192), (8, 1024, 28672), (24, 1000, 4096), (64, 2048, 8192), (1280, 12, 8192),
                                   (40, 37, 2048), (5, 3000, 4104)])
@pytest.mark.parametrize("kparts", [2, 4, 8])
def test_fp16_streaming_kernel_k_split(api, oracle, m, n, k, kparts):
    """K cut over a cluster of 2, 4 or 8 CTAs, partial blocks added in rank order through distributed shared memory:
    within FP16 tolerance of the oracle (the summation order differs from the whole-K kernel), identical from run to
    run, exact on small integers, both mappings, with and without a token split, alpha / beta."""
    a = rng.normal(210, 0, (m, k), 0.05)
    b = rng.normal(210, 1, (n, k), 0.05)
    c0 = rng.normal(210, 2, (n, m), 1.0)
    A, B = dev(a), dev(b)
    ref = oracle.gemm_f16_rcc(a, b)
    first = api.gemm_rcc_tile(A, B, 3, 16, kc=-kparts, split_k=1).cpu().numpy()
    close_f16(first, ref)
    assert np.array_equal(api.gemm_rcc_tile(A, B, 3, 16, kc=-kparts, split_k=1).cpu().numpy(), first)
    if min(m, n) > 8:
        both = api.gemm_rcc_tile(A, B, 3, 16, kc=-kparts, split_k=2).cpu().numpy()
        assert np.array_equal(both, first)          # the token split changes no dot product
    ref_ab = oracle.gemm_f16_rcc(a, b, 0.5, -1.5, c0)
    close_f16(api.gemm_rcc_tile(A, B, 3, 16, kc=-kparts, split_k=1, c_nm=dev(c0), alpha=0.5, beta=-1.5).cpu().numpy(), ref_ab)
    ai = rng.small_ints(211, 0, (m, k), lo=-1, hi=1)
    bi = rng.small_ints(211, 1, (n, k))
    exact = (ai.astype(np.int64) @ bi.astype(np.int64).T).T.astype(np.float16)
    assert np.array_equal(api.gemm_rcc_tile(dev(ai), dev(bi), 3, 16, kc=-kparts, split_k=1).cpu().numpy(), exact)
    assert api.device_status() == 0


def test_streaming_kernel_k_split_rule_and_int8(api, oracle, monkeypatch):
    """The library's own rule (few rows: K parts until there are two CTAs per SM) on the shapes it is for, checked
    through the public entry; INT8 accumulators stay bit-exact and the scaled epilogue bit-identical to the oracle under
    every forced number of K parts."""
    for (M, N, K) in [(1, 1024, 8192), (16, 1024, 28672), (32, 2048, 8192), (8, 1280, 8192)]:
        x = rng.normal(212, 0, (M, K), 0.05)
        w = rng.normal(212, 1, (N, K), 0.05)
        got = api.gemm_rcc_pid(dev(w), dev(x), 1101, 1).cpu().numpy()          # Linear mapping: m = N rows of W
        close_f16(got, oracle.gemm_f16_rcc(w, x))
    M, N, K = 24, 1024, 8192
    a = rng.int8_uniform(213, 0, (M, K))
    b = rng.int8_uniform(213, 1, (N, K))
    sa = rng.uniform(213, 2, (M,), 0.001, 0.02)
    sb = rng.uniform(213, 3, (N,), 0.001, 0.02)
    ref = oracle.scaled_mm_i8(a, b, sa, sb, None)
    L = api.lib()
    A, B, SA, SB = dev(a), dev(b), dev(sa), dev(sb)
    for parts in ("0", "1", "2", "4", "8"):
        monkeypatch.setenv("MOONPOLY_STREAM_KSPLIT", parts)
        api.reload_env()
        out = torch.empty((M, N), dtype=torch.float16, device=DEV)
        rc = L.mp_scaled_mm_i8_tile(3, 16, 1, M, N, K, A.data_ptr(), K, B.data_ptr(), K, SA.data_ptr(), 0, SB.data_ptr(), 0,
                                    None, out.data_ptr(), N, 0, None)
        assert rc == 0, L.mp_last_error_string()
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy().view(np.uint16), ref.view(np.uint16)), parts
        assert np.array_equal(api.gemm_rcc_pid(A, B, 1101, 1).cpu().numpy(), oracle.gemm_i8_rcc(a, b)), parts
    monkeypatch.delenv("MOONPOLY_STREAM_KSPLIT")
    api.reload_env()
    assert api.device_status() == 0


def test_int8_scaled_streaming_kernel_token_split(api, oracle, monkeypatch):
    M, N, K = 40, 600, 4096
    a = rng.int8_uniform(201, 0, (M, K))
    b = rng.int8_uniform(201, 1, (N, K))
    sa = rng.uniform(201, 2, (M,), 0.001, 0.02)
    sb = rng.uniform(201, 3, (N,), 0.001, 0.02)
    bias = rng.uniform(201, 4, (N,), -1.0, 1.0).astype(np.float16)
    ref = oracle.scaled_mm_i8(a, b, sa, sb, bias)
    L = api.lib()
    A, B, SA, SB, BI = dev(a), dev(b), dev(sa), dev(sb), dev(bias)
    for parts in ("1", "2", "4"):
        monkeypatch.setenv("MOONPOLY_STREAM_TSPLIT", parts)
        api.reload_env()
        out = torch.empty((M, N), dtype=torch.float16, device=DEV)
        rc = L.mp_scaled_mm_i8_tile(3, 16, 1, M, N, K, A.data_ptr(), K, B.data_ptr(), K, SA.data_ptr(), 0, SB.data_ptr(), 0,
                                    BI.data_ptr(), out.data_ptr(), N, 0, None)
        assert rc == 0, L.mp_last_error_string()
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy().view(np.uint16), ref.view(np.uint16)), parts
        acc = api.gemm_rcc_pid(A, B, 1101, 1).cpu().numpy()
        assert np.array_equal(acc, oracle.gemm_i8_rcc(a, b)), parts
    monkeypatch.delenv("MOONPOLY_STREAM_TSPLIT")
    api.reload_env()
    assert api.device_status() == 0


def test_scratch_never_grows_inside_a_stream_capture(api, oracle):
    """A stream that is being captured must not see an allocation: a split-K call whose scratch does not exist yet is
    refused with the workspace error (the capture stays valid), an unaligned-K call keeps the plain tiles instead of
    allocating padded copies, and the same calls made once before the capture are captured and replay correctly."""
    L = api.lib()
    m, n, k = 2048, 512, 8192            # 8 slices of 2048 x 512 partial sums: 33 MB of scratch, more than any stream holds
    a = rng.normal(240, 0, (m, k), 0.05)
    b = rng.normal(240, 1, (n, k), 0.05)
    au = rng.normal(241, 0, (130, 1001), 0.05)
    bu = rng.normal(241, 1, (70, 1001), 0.05)
    A, B, AU, BU = dev(a), dev(b), dev(au), dev(bu)
    C = torch.empty((n, m), dtype=torch.float16, device=DEV)
    CU = torch.empty((70, 130), dtype=torch.float16, device=DEV)
    side = torch.cuda.Stream()
    st = ctypes.c_void_p(side.cuda_stream)

    def split_call():
        return L.mp_gemm_rcc_pid(api.MP_FP16, 400, 8, m, n, k, A.data_ptr(), B.data_ptr(), C.data_ptr(), 1.0, 0.0, None, 0, st)

    def unaligned_call():
        return L.mp_gemm_rcc(api.MP_FP16, 130, 70, 1001, AU.data_ptr(), BU.data_ptr(), CU.data_ptr(), 1.0, 0.0, st)

    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        rc_split = split_call()               # this stream has no scratch yet: refused, nothing allocated
        n0 = api.launch_count()
        rc_un = unaligned_call()              # no padded copies: one plain-tile launch
        launches_un = api.launch_count() - n0
    assert rc_split == 5 and b"captur" in L.mp_last_error_string()          # MP_ERR_WORKSPACE
    assert rc_un == 0 and launches_un <= 2
    g.replay()
    torch.cuda.synchronize()
    close_f16(CU.cpu().numpy(), oracle.gemm_f16_rcc(au, bu))
    # warmed up outside a capture, both are captured as they run
    with torch.cuda.stream(side):
        assert split_call() == 0 and unaligned_call() == 0
    torch.cuda.synchronize()
    C.zero_(); CU.zero_()
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2, stream=side):
        assert split_call() == 0
        n0 = api.launch_count()
        assert unaligned_call() == 0
        assert api.launch_count() - n0 >= 3   # the padded copies and the GEMM
    g2.replay()
    torch.cuda.synchronize()
    close_f16(C.cpu().numpy(), oracle.gemm_f16_rcc(a, b))
    close_f16(CU.cpu().numpy(), oracle.gemm_f16_rcc(au, bu))
    assert api.device_status() == 0
