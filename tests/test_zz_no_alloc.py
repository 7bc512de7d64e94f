"""The allocation-free forced-pid entry point (collected last on purpose).

Some hosts of this library may not allocate GPU memory once they are running: a serving process
that has handed the whole device to its weights and KV cache, or a plug-in inside a runtime that
owns the memory budget.  For them mp_gemm_rcc_pid_static_scratch keeps the split-K scratch in a
fixed 8 MiB array inside the library instead of a buffer grown with cudaMalloc.  This test calls
it through the C ABI twice in a row and requires bit-identical output to mp_gemm_rcc_pid (the
split-K sum has a fixed order, so equality is exact), checks that the amount of free device memory
does not change across the calls, then that an oversized problem is refused with a clear message
and leaves C untouched.
"""
import ctypes

import numpy as np
import pytest
import torch

from moonpoly_b200 import rng

pytestmark = pytest.mark.gpu


def _call(fn, *args):
    return fn(*args)


def test_static_scratch_matches_regular_entry_twice(api):
    L = api.lib()
    dev = "cuda"
    m, n, k, pid, split = 24, 1024, 4096, 400, 4
    a = torch.from_numpy(rng.normal(31, 0, (m, k), 0.05)).to(dev)
    b = torch.from_numpy(rng.normal(31, 1, (n, k), 0.05)).to(dev)
    ref = torch.empty((n, m), dtype=torch.float16, device=dev)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.mp_gemm_rcc_pid(api.MP_FP16, pid, split, m, n, k, a.data_ptr(), b.data_ptr(), ref.data_ptr(), 1.0, 0.0,
                           None, 0, st)
    assert rc == 0, L.mp_last_error_string()
    need = api.workspace_size(api.MP_FP16, pid, m, n, k, split)
    assert 0 < need <= 8 << 20
    outs = [torch.full((n, m), float("nan"), dtype=torch.float16, device=dev) for _ in range(3)]
    free_before = None
    for attempt in range(3):
        if attempt == 1:
            # the first call looked up the array's address; from here on device memory must not move at all
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
        out = outs[attempt]
        rc = L.mp_gemm_rcc_pid_static_scratch(api.MP_FP16, pid, split, m, n, k, a.data_ptr(), b.data_ptr(),
                                              out.data_ptr(), 1.0, 0.0, st)
        assert rc == 0, L.mp_last_error_string()
        torch.cuda.synchronize()
        assert torch.equal(out, ref), f"call {attempt + 1} differs from mp_gemm_rcc_pid"
    assert torch.cuda.mem_get_info()[0] == free_before, "free device memory changed across allocation-free calls"
    # split_k = 1 on a tile count that is not a multiple of the SM count: the stream-K head completes its first
    # tiles through the same array
    ms, ns, ks = 1280, 1280, 1024
    a_s = torch.from_numpy(rng.small_ints(32, 0, (ms, ks), lo=-1, hi=1)).to(dev)
    b_s = torch.from_numpy(rng.small_ints(32, 1, (ns, ks))).to(dev)
    ref_s, out_s = (torch.empty((ns, ms), dtype=torch.float16, device=dev) for _ in range(2))
    assert L.mp_gemm_rcc_pid(api.MP_FP16, 1004, 1, ms, ns, ks, a_s.data_ptr(), b_s.data_ptr(), ref_s.data_ptr(), 1.0, 0.0,
                             None, 0, st) == 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    assert L.mp_gemm_rcc_pid_static_scratch(api.MP_FP16, 1004, 1, ms, ns, ks, a_s.data_ptr(), b_s.data_ptr(),
                                            out_s.data_ptr(), 1.0, 0.0, st) == 0, L.mp_last_error_string()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.equal(out_s, ref_s)
    # a different shape right after, on the same array (it still holds the previous call's partials)
    m2, n2 = 8, 512
    a2, b2 = a[:m2].contiguous(), b[:n2].contiguous()
    ref2 = torch.empty((n2, m2), dtype=torch.float16, device=dev)
    out2 = torch.empty_like(ref2)
    assert L.mp_gemm_rcc_pid(api.MP_FP16, 413, 8, m2, n2, k, a2.data_ptr(), b2.data_ptr(), ref2.data_ptr(), 1.0, 0.0,
                             None, 0, st) == 0
    assert L.mp_gemm_rcc_pid_static_scratch(api.MP_FP16, 413, 8, m2, n2, k, a2.data_ptr(), b2.data_ptr(),
                                            out2.data_ptr(), 1.0, 0.0, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(out2, ref2)
    assert api.device_status() == 0


def test_static_scratch_refuses_oversized_problem(api):
    L = api.lib()
    dev = "cuda"
    m, n, k, pid, split = 2048, 2048, 4096, 401, 8        # needs far more than 8 MiB of partials
    assert api.workspace_size(api.MP_FP16, pid, m, n, k, split) > 8 << 20
    a = torch.zeros((m, k), dtype=torch.float16, device=dev)
    b = torch.zeros((n, k), dtype=torch.float16, device=dev)
    c = torch.full((n, m), 7.0, dtype=torch.float16, device=dev)
    rc = L.mp_gemm_rcc_pid_static_scratch(api.MP_FP16, pid, split, m, n, k, a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                          1.0, 0.0, None)
    assert rc == 5
    msg = L.mp_last_error_string().decode()
    assert "8388608" in msg and "scratch" in msg
    torch.cuda.synchronize()
    assert torch.all(c == 7.0)
