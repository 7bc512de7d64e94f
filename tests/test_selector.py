"""Host logic of the selector, pid tables and cost model (no GPU needed)."""
import ctypes
import os
import subprocess
import time

import pytest


def test_pid_tables_follow_the_reference_contract(api):
    # alignment contract of the primary FP16 pids (moonpoly/core/fp16/fp16_rcc_cost.cu:32-36)
    ref_align = [8, 8, 8, 8, 8, 8, 8, 2, 8, 2, 1, 2, 2, 2, 8, 8, 8, 8, 8, 8,
                 8, 4, 8, 8, 4, 8, 4, 4, 8, 1, 8, 8, 2, 1, 8, 2, 2, 8, 1, 8, 8]
    for pid, al in enumerate(ref_align):
        tile, got = api.pid_info(api.MP_FP16, pid)
        assert got == al, pid
        pm, pn, pk = tile
        assert pk == 64 and 128 in (pm, pn) and min(pm, pn) % 16 == 0 and max(pm, pn) <= 256
    # split-K pids reuse the primary tiles: 407 -> pid 8's tile, 439 -> pid 7's (splitk_candidates.json)
    assert api.pid_info(api.MP_FP16, 407)[0] == api.pid_info(api.MP_FP16, 8)[0]
    assert api.pid_info(api.MP_FP16, 439)[0] == api.pid_info(api.MP_FP16, 7)[0]
    assert api.pid_info(api.MP_FP16, 413) == (api.pid_info(api.MP_FP16, 13)[0], 2)
    for pid in range(400, 440):
        api.pid_info(api.MP_FP16, pid)
    # the explicit-neighbourhood ranges 90..205 and 216..321 all have a kernel (generated/fp16/rcc/candidates.cu:62-65)
    for pid in (90, 150, 205, 216, 321):
        assert api.pid_info(api.MP_FP16, pid)[0][0] == 16
    assert api.pid_info(api.MP_FP16, 114)[1] == 4 and api.pid_info(api.MP_FP16, 91)[1] == 8
    # pids without a kernel fail cleanly
    for pid in (41, 77, 89, 206, 215, 322, 399, 440, -1):
        with pytest.raises(api.MoonpolyError) as e:
            api.pid_info(api.MP_FP16, pid)
        assert e.value.code == 4
    assert all(api.pid_info(api.MP_INT8, p)[0][2] == 128 for p in range(46))
    assert all(api.pid_info(api.MP_FP32, p)[1] == 1 for p in range(40))
    for dt, bad in ((api.MP_INT8, 46), (api.MP_FP32, 40)):
        with pytest.raises(api.MoonpolyError):
            api.pid_info(dt, bad)


def test_plan_is_argmin_of_cost_under_alignment(api, monkeypatch):
    # the cost-model path proper: measured plans off (MOONPOLY_ENABLE_GENERATED_SELECTOR, re-read per call)
    monkeypatch.setenv("MOONPOLY_ENABLE_GENERATED_SELECTOR", "0")
    for (m, n, k) in [(1, 4096, 4096), (4096, 4096, 4096), (512, 11008, 4096), (37, 1000, 520), (8, 1024, 8190)]:
        plan = api.select_plan(api.MP_FP16, m, n, k)
        if plan.pattern == 1:
            best = min((api.cost_ms(api.MP_FP16, pid, 1, m, n, k), pid) for pid in range(40)
                       if k % api.pid_info(api.MP_FP16, pid)[1] == 0)
            assert plan.pid == best[1] and abs(plan.estimated_ms - best[0]) < 1e-6
        elif plan.pattern == 3:
            assert plan.split_k in (2, 4, 8) and k >= 2048 and (k + plan.split_k - 1) // plan.split_k >= 512
            assert plan.pid in (4, 6, 7, 12, 13, 15, 19, 20, 23, 24, 25, 29, 31, 32, 33, 37, 39)
            single = min(api.cost_ms(api.MP_FP16, pid, 1, m, n, k) for pid in range(40)
                         if k % api.pid_info(api.MP_FP16, pid)[1] == 0)
            assert plan.estimated_ms < single * 0.97 + 1e-9          # MOONPOLY_PATTERN3_MARGIN
        # k = 8190 is only divisible by 2 and 1: the alignment contract must hold for the choice
        if plan.pid >= 0:
            assert k % api.pid_info(api.MP_FP16, plan.pid)[1] == 0


def test_measured_plan_table(api, monkeypatch):
    """Bucketed measured plans short-circuit the cost model (MOONPOLY_LLM_DECODE_SELECTOR_STRICT=1 by
    default, as the reference's decode selector does) and name library-native tiles (pid >= 1000)."""
    for (m, n, k) in [(1, 4096, 4096), (3, 4096, 4096), (4096, 5, 4096), (600, 4096, 4096), (599, 4096, 4096)]:
        plan = api.select_plan(api.MP_FP16, m, n, k)
        assert 1000 <= plan.pid < 1064 or 1200 <= plan.pid < 1264 or plan.pid in (1100, 1101), (m, n, k, plan)
        tile, align = api.pid_info(api.MP_FP16, plan.pid)
        assert align == 8 and (128 in tile[:2] or 256 in tile[:2] or plan.pid in (1100, 1101))
        assert plan.estimated_ms > 0
    # aligned and unaligned m land in different rows of the same bucket
    a = api.select_plan(api.MP_FP16, 1024, 4096, 4096)
    b = api.select_plan(api.MP_FP16, 1023, 4096, 4096)
    assert (a.pid, a.split_k) != (b.pid, b.split_k) or a.estimated_ms != b.estimated_ms
    # a shape outside the table goes through the cost model ...
    assert api.select_plan(api.MP_FP16, 2048, 2048, 2048).pid < 1000
    # ... whose choice is refined, tile kept: rows of A on the TMEM lanes when m leaves the rows of C unaligned,
    # 256-row tiles once a wide tile fills half the GPU that way
    base = api.select_plan(api.MP_FP16, 2048, 2048, 2048)
    odd = api.select_plan(api.MP_FP16, 2047, 2048, 2048)
    assert 1000 <= odd.pid < 1032 and api.pid_info(api.MP_FP16, odd.pid)[0][1] == 128            # orient 0: m on the 128 side
    assert sorted(api.pid_info(api.MP_FP16, odd.pid)[0][:2]) == sorted(api.pid_info(api.MP_FP16, base.pid)[0][:2])
    big = api.select_plan(api.MP_FP16, 4096, 4096, 4104)
    assert 1200 <= big.pid < 1264 and 256 in api.pid_info(api.MP_FP16, big.pid)[0][:2]
    assert 1200 <= api.select_plan(api.MP_FP16, 2297, 5120, 5120).pid < 1232                        # both: orient 0, 256 rows
    # switching the table off is honoured on the next call
    monkeypatch.setenv("MOONPOLY_ENABLE_GENERATED_SELECTOR", "0")
    assert api.select_plan(api.MP_FP16, 1, 4096, 4096).pid < 1000
    monkeypatch.delenv("MOONPOLY_ENABLE_GENERATED_SELECTOR")
    # non-strict: the measured plan competes with the cost model instead of short-circuiting it
    monkeypatch.setenv("MOONPOLY_LLM_DECODE_SELECTOR_STRICT", "0")
    p = api.select_plan(api.MP_FP16, 1, 4096, 4096)
    assert p.estimated_ms <= api.select_plan(api.MP_FP16, 1, 4096, 4096).estimated_ms


def test_env_flags(api, monkeypatch):
    monkeypatch.setenv("MOONPOLY_ENABLE_GENERATED_SELECTOR", "0")
    m, n, k = 8, 4096, 8192
    assert api.select_plan(api.MP_FP16, m, n, k).pattern == 3
    monkeypatch.setenv("MOONPOLY_ENABLE_PATTERN3", "0")          # re-read on every call
    assert api.select_plan(api.MP_FP16, m, n, k).pattern == 1
    monkeypatch.setenv("MOONPOLY_ENABLE_PATTERN3", "off")
    assert api.select_plan(api.MP_FP16, m, n, k).pattern == 1
    monkeypatch.delenv("MOONPOLY_ENABLE_PATTERN3")
    assert api.select_plan(api.MP_FP16, m, n, k).pattern == 3
    # numeric flags are cached until mp_reload_env()
    monkeypatch.setenv("MOONPOLY_PATTERN3_MIN_K", "100000")
    assert api.select_plan(api.MP_FP16, m, n, k).pattern == 3
    api.reload_env()
    assert api.select_plan(api.MP_FP16, m, n, k).pattern == 1
    monkeypatch.delenv("MOONPOLY_PATTERN3_MIN_K")
    api.reload_env()
    assert api.select_plan(api.MP_FP16, m, n, k).pattern == 3
    # forced split for INT8 / FP32 (tests/cpp/int8/test_int8_row_col_col.cu:70-77)
    monkeypatch.setenv("MOONPOLY_INT8_PATTERN3_FORCE_SPLITK", "2")
    p = api.select_plan(api.MP_INT8, 64, 128, 128)
    assert (p.pattern, p.pid, p.split_k) == (3, -1, 2)
    monkeypatch.delenv("MOONPOLY_INT8_PATTERN3_FORCE_SPLITK")
    assert api.select_plan(api.MP_INT8, 64, 128, 128).pattern == 1


def test_pattern2_gate(api, monkeypatch):
    monkeypatch.setenv("MOONPOLY_ENABLE_GENERATED_SELECTOR", "0")
    # tail of n % 128 within 25 % of a tile opens the twin plan; it must still win by the margin
    m, k = 4096, 4096
    monkeypatch.setenv("MOONPOLY_PATTERN2_MARGIN", "10.0")       # let it win whenever the gate opens
    api.reload_env()
    try:
        p = api.select_plan(api.MP_FP16, m, 4096 + 16, k)
        assert p.pattern == 2 and p.split_n == 4096 and p.pid == -1
        assert api.select_plan(api.MP_FP16, m, 4096 + 100, k).pattern != 2     # tail ratio 0.78 > 0.25
        assert api.select_plan(api.MP_FP16, m, 4096, k).pattern != 2           # regular n: closed by default
        assert api.select_plan(api.MP_FP16, m, 256 + 16, k).pattern != 2       # n < MOONPOLY_PATTERN2_MIN_N
        assert api.select_plan(api.MP_FP16, m, 4096 + 16, 4100).pattern != 2   # k % 8 != 0
        monkeypatch.setenv("MOONPOLY_ENABLE_PATTERN2", "0")
        assert api.select_plan(api.MP_FP16, m, 4096 + 16, k).pattern != 2
    finally:
        monkeypatch.delenv("MOONPOLY_PATTERN2_MARGIN")
        monkeypatch.delenv("MOONPOLY_ENABLE_PATTERN2", raising=False)
        api.reload_env()


def test_bad_arguments(api):
    L = api.lib()
    p = api.Plan()
    assert L.mp_select_plan(9, 1, 1, 1, ctypes.byref(p)) == 1
    assert L.mp_select_plan(0, 0, 1, 1, ctypes.byref(p)) == 1
    assert b"Unsupported data type" in L.mp_last_error_string() or L.mp_last_error_string()
    out = (ctypes.c_int * 4)()
    assert L.mp_scaled_mm_config(6, ctypes.byref(out)) == 1
    for cfg in range(6):
        tm, tn, tk, al = api.get_int8_scaled_mm_kernel_config(cfg)
        assert tk == 128 and al == 16 and 128 in (tm, tn)


def test_selection_overhead_budget(api, tmp_path):
    """<= 5 us per shape on the host at first sight of a shape, <= 2 us memoised: timed in C around mp_select_plan
    (tests/host_timing/select_timing.c), best of 24 passes so a busy host does not fail the test."""
    here = os.path.dirname(os.path.abspath(__file__))
    exe = str(tmp_path / "select_timing")
    lib_dir = os.path.dirname(api.LIB_PATH)
    subprocess.check_call(["gcc", "-O2", os.path.join(here, "host_timing", "select_timing.c"), "-o", exe,
                           "-I", os.path.join(here, "..", "include"), "-L", lib_dir, "-lmoonpoly_gemm",
                           f"-Wl,-rpath,{lib_dir}"])
    out = subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split()
    cold, warm = float(out[1]) * 1e-9, float(out[3]) * 1e-9
    print(f"selection: first sight {cold * 1e6:.2f} us, memoised {warm * 1e6:.2f} us")
    assert cold < 5e-6
    assert warm < 2e-6


def test_measured_tables_name_runnable_kernels(api):
    """Every bucket of the measured tables resolves to a kernel the library has, for FP16 (both mappings of the tuned
    layers, aligned and unaligned token counts) and for INT8 on the scaled-matmul layers."""
    fp16_layers = [(4096, 4096), (6144, 4096), (28672, 4096), (4096, 14336), (10240, 8192), (8192, 8192), (57344, 8192),
                   (8192, 28672), (1024, 8192), (1024, 28672), (5120, 8192), (1280, 8192), (7168, 8192), (2048, 28672)]
    tokens = [1, 2, 3, 7, 16, 31, 33, 64, 65, 100, 128, 129, 200, 255, 256, 300, 511, 512, 700, 1000, 1024, 1500, 2047, 2048,
              3000, 4095, 4096, 6000, 8192, 12000]
    for (N, K) in fp16_layers:
        for M in tokens:
            for (m, n) in ((N, M), (M, N)):             # Linear mapping and direct mapping
                plan = api.select_plan(api.MP_FP16, m, n, K)
                tile, align = api.pid_info(api.MP_FP16, plan.pid if plan.pid >= 0 else 0)
                assert K % align == 0 and plan.split_k >= 1 and plan.estimated_ms > 0, (m, n, K, plan)
                if plan.pid in (1100, 1101):
                    assert min(m, n) <= 64, (m, n, K, plan)
                if 1200 <= plan.pid < 1264:
                    assert plan.split_k == 1 and 256 in tile[:2], (m, n, K, plan)
    for (N, K) in [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]:
        for M in tokens:
            plan = api.select_plan(api.MP_INT8, M, N, K)
            assert plan.pid >= 1000, (M, N, K, plan)
            api.pid_info(api.MP_INT8, plan.pid)
            if plan.pid == 1101:
                assert M <= 64
            cfg = api.predict_int8_scaled_mm_kernel(M, N, K)
            assert 0 <= cfg < 6
