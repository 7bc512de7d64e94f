"""The serving-engine Linear path over the `moonpoly_ops` operators, end to end (moonpoly_b200/vllm_linear.py): every
branch the reference's vLLM patch tries, in its order, under its environment switches -- C++ selector, pid whitelist
with a decode-selector table, split-K pid with the pooled workspace, plain linear -- with inputs of rank 3, a bias,
workspace reuse across shapes, fall-through on failure, and torch.compile over the operators' Meta kernels."""
import os
import sys

import numpy as np
import pytest
import torch

from moonpoly_b200 import rng, vllm_linear

pytestmark = pytest.mark.gpu
EXT_DIR = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "moonpoly-dev_b200", "torch_ext"))
DEV = "cuda"
SWITCHES = ["VLLM_USE_MOONPOLY_LINEAR", "VLLM_USE_MOONPOLY_CPP_SELECTOR", "VLLM_USE_MOONPOLY_PID_WHITELIST",
            "VLLM_USE_MOONPOLY_STREAMK", "VLLM_MOONPOLY_STREAMK_PID", "VLLM_MOONPOLY_STREAMK_SPLITK",
            "VLLM_MOONPOLY_STREAMK_MAX_M", "VLLM_MOONPOLY_STREAMK_ALLOW_N"]


@pytest.fixture(scope="module")
def ext():
    if EXT_DIR not in sys.path:
        sys.path.insert(0, EXT_DIR)
    import moonpoly as module          # registers torch.ops.moonpoly_ops
    return module


@pytest.fixture(autouse=True)
def _clean(monkeypatch):
    for name in SWITCHES:
        monkeypatch.delenv(name, raising=False)
    vllm_linear.reset_stats()
    vllm_linear.load_decode_selector({})
    yield


class Layer(torch.nn.Module):
    def __init__(self, w):
        super().__init__()
        self.weight = torch.nn.Parameter(w, requires_grad=False)


def tensors(seed, lead, n, k):
    x = rng.normal(seed, 0, tuple(lead) + (k,), 0.05)
    w = rng.normal(seed, 1, (n, k), 0.05)
    b = rng.uniform(seed, 5, (n,), -1.0, 1.0).astype(np.float16)
    return x, w, b


def check(out, x, w, b, oracle):
    ref = oracle.linear_bias(x.reshape(-1, x.shape[-1]), w, b).astype(np.float32).reshape(x.shape[:-1] + (w.shape[0],))
    got = out.float().cpu().numpy()
    assert out.shape == ref.shape
    bad = np.abs(got - ref) > 1e-3 + 1e-2 * np.abs(ref)
    assert not bad.any(), f"{bad.sum()} of {bad.size} differ; max abs {np.abs(got - ref).max()}"


def test_switch_off_declines_and_falls_back(ext, oracle):
    x, w, b = tensors(180, (3, 5), 256, 128)
    layer = Layer(torch.from_numpy(w).to(DEV))
    assert vllm_linear.apply_moonpoly_linear(layer.weight, torch.from_numpy(x).to(DEV)) is None
    out = vllm_linear.apply(layer, torch.from_numpy(x).to(DEV), torch.from_numpy(b).to(DEV))       # the caller's own GEMM
    check(out, x, w, b, oracle)
    assert sum(vllm_linear.STATS.values()) == 0


def test_plain_linear_rank3_input_and_bias(ext, oracle, monkeypatch):
    monkeypatch.setenv("VLLM_USE_MOONPOLY_LINEAR", "1")
    x, w, b = tensors(181, (4, 7), 1024, 512)
    layer = Layer(torch.from_numpy(w).to(DEV))
    out = vllm_linear.apply(layer, torch.from_numpy(x).to(DEV), torch.from_numpy(b).to(DEV))
    check(out, x, w, b, oracle)
    assert vllm_linear.STATS["linear"] == 1 and vllm_linear.STATS["streamk_skipped"] == 1
    # non-contiguous input, no bias; bf16 is declined exactly as the reference's path declines it
    xt = torch.from_numpy(x).to(DEV).transpose(0, 1)
    out = vllm_linear.apply(layer, xt)
    check(out, np.ascontiguousarray(x.transpose(1, 0, 2)), w, None, oracle)
    assert vllm_linear.apply_moonpoly_linear(layer.weight.to(torch.bfloat16), xt.to(torch.bfloat16)) is None
    assert vllm_linear.STATS["declined"] == 1


def test_cpp_selector_branch(ext, oracle, monkeypatch):
    monkeypatch.setenv("VLLM_USE_MOONPOLY_LINEAR", "1")
    monkeypatch.setenv("VLLM_USE_MOONPOLY_CPP_SELECTOR", "1")
    x, w, b = tensors(182, (9,), 2048, 1024)
    out = vllm_linear.apply(Layer(torch.from_numpy(w).to(DEV)), torch.from_numpy(x).to(DEV), torch.from_numpy(b).to(DEV))
    check(out, x, w, b, oracle)
    assert vllm_linear.STATS["cpp_selector"] == 1 and vllm_linear.STATS["linear"] == 0


def test_pid_whitelist_branch_and_workspace_pool(ext, oracle, monkeypatch):
    """(M, N, K) -> (pid, split_k) rows as the reference's merged decode selector holds them (explicit-neighbourhood
    pids with a run-time split factor); unmapped shapes and failing rows fall through."""
    monkeypatch.setenv("VLLM_USE_MOONPOLY_LINEAR", "1")
    monkeypatch.setenv("VLLM_USE_MOONPOLY_PID_WHITELIST", "1")
    monkeypatch.setenv("VLLM_USE_MOONPOLY_STREAMK", "0")
    vllm_linear.load_decode_selector({(8, 5120, 5120): (91, 2), (1, 5120, 13824): (99, 2), (4, 1024, 2048): (400, 4),
                                      (2, 1024, 2048): (77, 2)})                 # pid 77 has no kernel
    pool_before = dict(vllm_linear._WS_POOL)
    for lead, n, k in (((8,), 5120, 5120), ((1, 1), 5120, 13824), ((2, 2), 1024, 2048)):
        x, w, b = tensors(183 + n + k, lead, n, k)
        out = vllm_linear.apply(Layer(torch.from_numpy(w).to(DEV)), torch.from_numpy(x).to(DEV), torch.from_numpy(b).to(DEV))
        check(out, x, w, b, oracle)
    assert vllm_linear.STATS["whitelist_hit"] == 3 and vllm_linear.STATS["whitelist_attempt"] == 3
    x, w, b = tensors(184, (2,), 1024, 2048)
    out = vllm_linear.apply(Layer(torch.from_numpy(w).to(DEV)), torch.from_numpy(x).to(DEV), None)      # row names pid 77
    check(out, x, w, None, oracle)
    assert vllm_linear.STATS["whitelist_fallback"] == 1 and vllm_linear.STATS["linear"] == 1
    x, w, b = tensors(185, (3,), 512, 256)
    vllm_linear.apply(Layer(torch.from_numpy(w).to(DEV)), torch.from_numpy(x).to(DEV), None)
    assert vllm_linear.STATS["whitelist_unmapped"] == 1
    # one buffer per (device, stream), grown to the largest request, reused by every shape
    key = (torch.cuda.current_device(), int(torch.cuda.current_stream().cuda_stream))
    assert key in vllm_linear._WS_POOL and len(vllm_linear._WS_POOL) <= len(pool_before) + 1
    big = vllm_linear.workspace(torch.device(DEV, torch.cuda.current_device()), 1)
    assert big.data_ptr() == vllm_linear._WS_POOL[key].data_ptr()


def test_streamk_branch_gates_and_runs(ext, oracle, monkeypatch):
    monkeypatch.setenv("VLLM_USE_MOONPOLY_LINEAR", "1")
    for pid, split in ((40, 2), (400, 4)):
        monkeypatch.setenv("VLLM_MOONPOLY_STREAMK_PID", str(pid))
        monkeypatch.setenv("VLLM_MOONPOLY_STREAMK_SPLITK", str(split))
        x, w, b = tensors(186 + pid, (8,), 5120, 5120)
        out = vllm_linear.apply(Layer(torch.from_numpy(w).to(DEV)), torch.from_numpy(x).to(DEV), torch.from_numpy(b).to(DEV))
        check(out, x, w, b, oracle)
    assert vllm_linear.STATS["streamk_success"] == 2 and vllm_linear.STATS["linear"] == 0
    assert not vllm_linear.streamk_shape_allowed(16, 5120, 5120)
    assert not vllm_linear.streamk_shape_allowed(8, 4096, 5120)
    monkeypatch.setenv("VLLM_MOONPOLY_STREAMK_ALLOW_N", "8192,10240")
    assert not vllm_linear.streamk_shape_allowed(8, 5120, 5120) and vllm_linear.streamk_shape_allowed(8, 8192, 5120)
    monkeypatch.setenv("VLLM_MOONPOLY_STREAMK_MAX_M", "4")
    assert not vllm_linear.streamk_shape_allowed(8, 8192, 5120)


def test_operators_under_torch_compile(ext, oracle, monkeypatch):
    """The operators trace through their Meta kernels: one graph, no breaks, and the compiled module computes what
    the eager one does."""
    ops = torch.ops.moonpoly_ops

    class Block(torch.nn.Module):
        def __init__(self, w1, w2, ws):
            super().__init__()
            self.w1, self.w2, self.ws = w1, w2, ws

        def forward(self, x, bias):
            h = ops.linear(x, self.w1) + bias
            out = torch.empty((h.shape[0], self.w2.shape[0]), dtype=h.dtype, device=h.device)
            ops.linear_fp16_pid_ws_out(h, self.w2, out, 400, self.ws, 2)
            return ops.linear_cpp_selector(out, self.w1[:, : out.shape[1]].contiguous())

    x, w1, b = tensors(190, (12,), 1024, 1024)
    w2 = rng.normal(190, 2, (1024, 1024), 0.05)
    W1, W2 = torch.from_numpy(w1).to(DEV), torch.from_numpy(w2).to(DEV)
    X, B = torch.from_numpy(x).to(DEV), torch.from_numpy(b).to(DEV)
    ws = torch.zeros((int(ops.fp16_workspace_size(X, W2, 400, 2)) + 16,), dtype=torch.uint8, device=DEV)
    block = Block(W1, W2, ws)
    eager = block(X, B)
    compiled = torch.compile(block, fullgraph=True)
    got = compiled(X, B)
    torch.cuda.synchronize()
    assert torch.equal(got, eager)
    # the whole serving path (environment reads, counters, try / except) compiled without the one-graph demand
    monkeypatch.setenv("VLLM_USE_MOONPOLY_LINEAR", "1")
    layer = Layer(W1)
    fn = torch.compile(lambda t, bb: vllm_linear.apply(layer, t, bb))
    out = fn(X.reshape(3, 4, -1), B)
    check(out, x.reshape(3, 4, -1), w1, b, oracle)


def test_install_routes_an_engines_linear_method(ext, oracle, monkeypatch):
    """install() on a stand-in for a serving engine's linear module: the engine's UnquantizedLinearMethod.apply goes
    through the operators when the switch is on and through the engine's own GEMM when it is off."""
    import types
    calls = []

    class UnquantizedLinearMethod:
        def apply(self, layer, x, bias=None):
            calls.append("engine")
            return torch.nn.functional.linear(x, layer.weight, bias)

    module = types.SimpleNamespace(UnquantizedLinearMethod=UnquantizedLinearMethod)
    assert vllm_linear.install(module) and vllm_linear.install(module)          # idempotent
    x, w, b = tensors(191, (2, 3), 512, 256)
    layer = Layer(torch.from_numpy(w).to(DEV))
    method = module.UnquantizedLinearMethod()
    out = method.apply(layer, torch.from_numpy(x).to(DEV), torch.from_numpy(b).to(DEV))
    check(out, x, w, b, oracle)
    assert calls == ["engine"]
    monkeypatch.setenv("VLLM_USE_MOONPOLY_LINEAR", "1")
    out = method.apply(layer, torch.from_numpy(x).to(DEV), torch.from_numpy(b).to(DEV))
    check(out, x, w, b, oracle)
    assert calls == ["engine"] and vllm_linear.STATS["linear"] == 1
