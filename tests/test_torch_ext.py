"""The torch extension `moonpoly` / `moonpoly_ops`, exercised the way the reference's Python tests do
(tests/python/test_fp16_splitk_runtime.py, test_fp16_streamk_graph.py,
test_int8_scaled_mm_correctness.py, test_moonpoly_linear.py)."""
import os
import sys

import numpy as np
import pytest
import torch

from moonpoly_b200 import rng

EXT_DIR = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "moonpoly-dev_b200", "torch_ext"))


@pytest.fixture(scope="module")
def moonpoly():
    if EXT_DIR not in sys.path:
        sys.path.insert(0, EXT_DIR)
    import moonpoly as ext          # torch must be imported first, as with the reference
    return ext


def test_schemas_and_meta_kernels(moonpoly):
    ops = torch.ops.moonpoly_ops
    x = torch.empty((5, 64), dtype=torch.float16, device="meta")
    w = torch.empty((24, 64), dtype=torch.float16, device="meta")
    ws = torch.empty((0,), dtype=torch.uint8, device="meta")
    assert ops.linear(x, w).shape == (5, 24)
    assert ops.linear_cpp_selector(x, w).shape == (5, 24)
    assert ops.linear_bias(x, w, None).shape == (5, 24)            # beyond the reference's op set
    assert ops.fp16_workspace_size(x, w, 40) == 0
    assert ops.linear_fp16_pid_ws(x, w, 40, ws).shape == (5, 24)
    out = torch.empty((5, 24), dtype=torch.float16, device="meta")
    assert ops.linear_fp16_pid_ws_out(x, w, out, 40, ws, 2) is None
    assert moonpoly.get_int8_scaled_mm_kernel_config(0)[3] == 16
    assert 0 <= moonpoly.predict_int8_scaled_mm_kernel(16, 4096, 4096) < 6


@pytest.mark.gpu
@pytest.mark.parametrize("split_k", [1, 2, 4])
def test_forced_pid_split_k_runtime(moonpoly, split_k):
    # tests/python/test_fp16_splitk_runtime.py: pid 400, shape (8,1024,1024), randn*0.1, tol 5e-2
    torch.manual_seed(0)
    a = (torch.randn(8, 1024, device="cuda") * 0.1).half()
    b = (torch.randn(1024, 1024, device="cuda") * 0.1).half()
    out = moonpoly.linear_cpp_forced_pid(a, b, 400, split_k)
    ref = a @ b.t()
    assert torch.isfinite(out).all()
    torch.testing.assert_close(out, ref, rtol=5e-2, atol=5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("pid,split", [(40, 2), (400, 4), (413, 8), (1, 1)])
def test_workspace_ops_eager_and_graph(moonpoly, pid, split):
    # tests/python/test_fp16_streamk_graph.py: caller-owned workspace, eager and under graph capture
    ops = torch.ops.moonpoly_ops
    torch.manual_seed(1)
    M, N, K = 16, 1024, 2048
    x = (torch.randn(M, K, device="cuda") * 0.05).half()
    w = (torch.randn(N, K, device="cuda") * 0.05).half()
    ref = torch.nn.functional.linear(x, w)
    need = ops.fp16_workspace_size(x, w, pid, split)
    ws = torch.zeros((max(need, 1),), dtype=torch.uint8, device="cuda")
    out = torch.empty((M, N), dtype=torch.float16, device="cuda")
    ops.linear_fp16_pid_ws_out(x, w, out, pid, ws, split)
    torch.testing.assert_close(out, ref, rtol=5e-2, atol=5e-2)
    eager = out.clone()

    g = torch.cuda.CUDAGraph()
    out.zero_()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        ops.linear_fp16_pid_ws_out(x, w, out, pid, ws, split)      # warm-up on the capture stream
    torch.cuda.current_stream().wait_stream(s)
    with torch.cuda.graph(g):
        ops.linear_fp16_pid_ws_out(x, w, out, pid, ws, split)
    for _ in range(3):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)

    # RCC flavour: b_col [k,n] strides (1,k), c_col [m,n] strides (1,m)
    a = w                                # [m=N, k]
    b_col = x.t()                        # logical [k, n=M], strides (1, k)
    c_col = torch.empty((M, N), dtype=torch.float16, device="cuda").t()   # logical [m=N, n=M], strides (1, N)
    need2 = ops.fp16_rcc_workspace_size(a, b_col, pid, split)
    assert need2 == need
    ops.fp16_rcc_pid_ws_out(a, b_col, c_col, pid, ws, split)
    assert torch.equal(c_col.t(), eager)

    if need > 0:
        with pytest.raises(Exception):
            ops.linear_fp16_pid_ws_out(x, w, out, pid, ws[: need // 2], split)


@pytest.mark.gpu
def test_linear_and_fallbacks(moonpoly):
    torch.manual_seed(2)
    for (M, N, K) in [(1, 512, 256), (32, 5120, 640), (7, 100, 72)]:
        x = (torch.randn(M, K, device="cuda") * 0.05).half()
        w = (torch.randn(N, K, device="cuda") * 0.05).half()
        ref = torch.nn.functional.linear(x.float(), w.float())
        for fn in (moonpoly.linear, moonpoly.linear_cpp_selector, torch.ops.moonpoly_ops.linear):
            torch.testing.assert_close(fn(x, w).float(), ref, rtol=1e-2, atol=1e-3)
    # non-contiguous input to the forced-pid entry falls back to linear (moonpoly_gemm.cu:188-196)
    xt = (torch.randn(64, 9, device="cuda") * 0.05).half().t()
    w = (torch.randn(40, 64, device="cuda") * 0.05).half()
    torch.testing.assert_close(moonpoly.linear_cpp_forced_pid(xt, w, 400, 2).float(),
                               torch.nn.functional.linear(xt.float(), w.float()), rtol=1e-2, atol=1e-3)
    with pytest.raises(Exception):
        moonpoly.linear(x.bfloat16(), w.bfloat16())
    # fp32 and int8 through the same op
    xf = torch.randn(9, 96, device="cuda")
    wf = torch.randn(33, 96, device="cuda")
    torch.testing.assert_close(moonpoly.linear(xf, wf), torch.nn.functional.linear(xf, wf), rtol=1e-4, atol=1e-4)
    xi = torch.randint(-127, 128, (9, 96), dtype=torch.int8, device="cuda")
    wi = torch.randint(-127, 128, (33, 96), dtype=torch.int8, device="cuda")
    assert torch.equal(moonpoly.linear(xi, wi), (xi.double() @ wi.double().t()).to(torch.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (33, 6144, 4096), (257, 1024, 512)])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("mode", ["per_tensor", "per_token_channel"])
@pytest.mark.parametrize("with_bias", [False, True])
def test_scaled_int8_mm_vs_float_reference(moonpoly, M, N, K, out_dtype, mode, with_bias):
    # tests/python/test_int8_scaled_mm_correctness.py:107-132,253-259: float32 reference
    # (a*sa) @ (b*sb) + bias; pass if max_abs below the dtype threshold or max_rel < 0.01
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda", generator=g)
    w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda", generator=g)
    if mode == "per_tensor":
        sa = torch.full((1,), 0.01, device="cuda")
        sb = torch.full((1,), 0.005, device="cuda")
    else:
        sa = torch.rand((M, 1), device="cuda", generator=g) * 0.019 + 0.001
        sb = torch.rand((1, N), device="cuda", generator=g) * 0.019 + 0.001
    bias = (torch.randn((N,), device="cuda", generator=g)).to(out_dtype) if with_bias else None
    out = moonpoly.scaled_int8_mm(a, w.t(), sa, sb, bias, out_dtype)
    assert out.dtype == out_dtype and out.shape == (M, N)
    ref = (a.float() * sa.reshape(-1, 1)) @ (w.float().t() * sb.reshape(1, -1))
    if bias is not None:
        ref = ref + bias.float()
    # two roundings to the output type (product, then the bias sum): a few ulp of the output dtype
    # (the product is rounded before the bias is added, so a cancelling bias keeps the product's ulp)
    rtol, atol = (4e-3, 1e-2) if out_dtype == torch.float16 else (3e-2, 6e-2)
    torch.testing.assert_close(out.float(), ref, rtol=rtol, atol=atol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_linear_bias_op_matches_two_step(moonpoly, dtype):
    torch.manual_seed(3)
    x = (torch.randn(33, 1024, device="cuda") * 0.05).to(dtype)
    w = (torch.randn(520, 1024, device="cuda") * 0.05).to(dtype)
    b = torch.randn(520, device="cuda").to(dtype)
    fused = torch.ops.moonpoly_ops.linear_bias(x, w, b)
    plain = torch.ops.moonpoly_ops.linear_bias(x, w, None)
    assert torch.equal(fused, plain + b)
    assert torch.equal(moonpoly.linear_bias(x, w, b), fused)
    if dtype == torch.float16:
        assert torch.equal(plain, torch.ops.moonpoly_ops.linear(x, w))
    torch.testing.assert_close(fused.float(), x.float() @ w.float().t() + b.float(), rtol=2e-2, atol=2e-2)
