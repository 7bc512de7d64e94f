"""Three-way parity on identical seeded inputs: the REFERENCE'S OWN kernels, the CPU oracle and this library.

oracle/build_ref_kernels.sh compiles the reference's CUTLASS kernels, selectors and cost models from
the reference tree (moonpoly/core/**, moonpoly/generated/fp16/rcc/candidates.cu) into the checker
binary oracle/_ref/mp_ref_runner.  Here that binary runs on the GPU next to the product:

* integer-valued inputs (the value range of the reference's CTest programmes): reference, oracle and
  product must agree bit for bit, for every dtype;
* N(0,1)*0.05 FP16 and U[-1,1] FP32 inputs: the reference's rounded outputs pin the oracle's restated
  arithmetic (fp32 accumulation, one rounding to the output type) within the path's tolerance, and
  the product is held to the same tolerance against the reference itself;
* INT8: exact int32 accumulators, three ways.

pids 40 and 66 are left out: the reference's own notes record that they return NaN.
"""
import os
import subprocess

import numpy as np
import pytest
import torch

from moonpoly_b200 import rng

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
RUNNER = os.path.join(ROOT, "oracle", "_ref", "mp_ref_runner")
DEV = "cuda"


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


class RefBatch:
    """Collects cases, runs them in one process of the reference runner, returns the outputs."""

    def __init__(self, tmp_path):
        self.dir = str(tmp_path)
        self.lines, self.meta = [], []

    def add(self, op, a, b, pid=0, split=1, alpha=1.0, beta=0.0, c0=None):
        i = len(self.lines)
        m, k = a.shape
        n = b.shape[0]
        fin, fout = os.path.join(self.dir, f"in{i}.bin"), os.path.join(self.dir, f"out{i}.bin")
        with open(fin, "wb") as fh:
            fh.write(np.ascontiguousarray(a).tobytes())
            fh.write(np.ascontiguousarray(b).tobytes())
            if beta != 0.0:
                fh.write(np.ascontiguousarray(c0).tobytes())
        self.lines.append(f"{op} {m} {n} {k} {pid} {split} {alpha} {beta} {fin} {fout}")
        out_dtype = np.float16 if op.startswith("fp16") else (np.int32 if op.startswith("int8") else np.float32)
        self.meta.append((fout, out_dtype, n, m))
        return i

    def run(self):
        manifest = os.path.join(self.dir, "manifest.txt")
        with open(manifest, "w") as fh:
            fh.write("\n".join(self.lines) + "\n")
        res = subprocess.run([RUNNER, manifest], capture_output=True, text=True, timeout=900)
        done = res.stdout.count("ok ")
        assert res.returncode == 0 and done == len(self.lines), (
            f"the reference runner finished {done} of {len(self.lines)} cases (rc {res.returncode}): "
            f"{res.stdout[-400:]} {res.stderr[-400:]}")
        return [np.fromfile(f, dtype=dt).reshape(n, m) for f, dt, n, m in self.meta]


@pytest.fixture(scope="module", autouse=True)
def _need_runner():
    if not os.path.exists(RUNNER):
        pytest.skip("oracle/_ref/mp_ref_runner not built (needs the reference tree at build time)")


def within(got, ref, rtol, atol):
    got, ref = got.astype(np.float64), ref.astype(np.float64)
    bad = np.abs(got - ref) > atol + rtol * np.abs(ref)
    return not bad.any(), f"{bad.sum()} of {bad.size} differ; max abs {np.abs(got - ref).max():.4g}"


FP16_PIDS = [0, 3, 8, 15, 16, 23, 31, 39]


def test_fp16_pids_three_way(api, oracle, tmp_path):
    """FP16 primary pids on integer-valued and on N(0,1)*0.05 inputs."""
    m, n, k = 136, 264, 512
    ai, bi = rng.small_ints(101, 0, (m, k)), rng.small_ints(101, 1, (n, k))
    an, bn = rng.normal(102, 0, (m, k), 0.05), rng.normal(102, 1, (n, k), 0.05)
    c0 = rng.normal(102, 2, (n, m), 1.0)
    batch = RefBatch(tmp_path)
    for pid in FP16_PIDS:
        batch.add("fp16_pid", ai, bi, pid=pid)
        batch.add("fp16_pid", an, bn, pid=pid)
    batch.add("fp16_pid", an, bn, pid=8, alpha=0.5, beta=2.0, c0=c0)
    outs = batch.run()
    exact = oracle.gemm_f16_rcc(ai, bi)
    orc = oracle.gemm_f16_rcc(an, bn)
    for j, pid in enumerate(FP16_PIDS):
        ref_i, ref_n = outs[2 * j], outs[2 * j + 1]
        assert np.array_equal(ref_i, exact), f"reference pid {pid} vs oracle on integer inputs"
        assert np.array_equal(api.gemm_rcc_pid(dev(ai), dev(bi), pid, 1).cpu().numpy(), ref_i), f"product pid {pid}"
        ok, msg = within(orc, ref_n, 1e-2, 1e-3)
        assert ok, f"oracle vs reference pid {pid}: {msg}"
        ok, msg = within(api.gemm_rcc_pid(dev(an), dev(bn), pid, 1).cpu().numpy(), ref_n, 1e-2, 1e-3)
        assert ok, f"product vs reference pid {pid}: {msg}"
    ref_ab = outs[-1]
    ok, msg = within(oracle.gemm_f16_rcc(an, bn, 0.5, 2.0, c0), ref_ab, 1e-2, 1e-3)
    assert ok, "oracle alpha/beta vs reference: " + msg
    got = api.gemm_rcc_pid(dev(an), dev(bn), 8, 1, c_nm=dev(c0), alpha=0.5, beta=2.0).cpu().numpy()
    ok, msg = within(got, ref_ab, 1e-2, 1e-3)
    assert ok, "product alpha/beta vs reference: " + msg


def test_fp16_oracle_rounding_pinned_by_reference(oracle, tmp_path):
    """How closely the oracle's rounded FP16 outputs follow the reference's kernels: the two accumulate in fp32 in a
    different order, so a small share of outputs may land on the neighbouring fp16 value, never further."""
    m, n, k = 64, 512, 4096
    a, b = rng.normal(103, 0, (m, k), 0.05), rng.normal(103, 1, (n, k), 0.05)
    batch = RefBatch(tmp_path)
    batch.add("fp16_pid", a, b, pid=8)
    ref = batch.run()[0]
    orc = oracle.gemm_f16_rcc(a, b)
    # fp32 accumulation noise of a 4096-term sum of this size is a few 1e-6: outputs may differ by that, or by one
    # fp16 step where a sum lands near a rounding boundary -- never by more
    r32, o32 = ref.astype(np.float32), orc.astype(np.float32)
    step = np.spacing(np.maximum(np.abs(ref), np.abs(orc)).astype(np.float16)).astype(np.float32)
    diff = np.abs(r32 - o32)
    assert np.all(diff <= step + 5e-6), f"max excess {(diff - step).max():.3g}"
    assert (diff == 0).mean() > 0.97, f"only {(diff == 0).mean():.4f} of the outputs are identical"


def test_fp16_online_selector_three_way(api, oracle, tmp_path):
    """run_fp16_gemm (the reference's online selector picks the kernel) on sweep shapes at N = K = 4096."""
    n = k = 4096
    b = rng.normal(1, rng.STREAM_B, (n, k), 0.05)
    batch = RefBatch(tmp_path)
    ms = [1, 16, 127, 512]
    a = {m: rng.normal(1, rng.STREAM_A, (m, k), 0.05) for m in ms}
    for m in ms:
        batch.add("fp16_auto", a[m], b)
    outs = batch.run()
    B = dev(b)
    for m, ref in zip(ms, outs):
        ok, msg = within(oracle.gemm_f16_rcc(a[m], b), ref, 1e-2, 1e-3)
        assert ok, f"oracle vs reference M={m}: {msg}"
        ok, msg = within(api.gemm_rcc(dev(a[m]), B).cpu().numpy(), ref, 1e-2, 1e-3)
        assert ok, f"product vs reference M={m}: {msg}"


def test_fp16_splitk_pid_400_three_way(api, oracle, tmp_path):
    """Linear (8, 1024, 1024) through pid 400 with split 1 / 2 / 4 (tests/python/test_fp16_splitk_runtime.py)."""
    M, N, K = 8, 1024, 1024
    x, w = rng.normal(2, rng.STREAM_A, (M, K), 0.1), rng.normal(2, rng.STREAM_B, (N, K), 0.1)
    batch = RefBatch(tmp_path)
    for s in (1, 2, 4):
        batch.add("fp16_pid", w, x, pid=400, split=s)          # Linear -> RCC: m = N, A = W, B = X
    outs = batch.run()
    orc = oracle.linear_f16(x, w)
    for s, ref in zip((1, 2, 4), outs):
        ref_y = ref.reshape(M, N)                                # C stored [n = M][m = N] is Y[M, N]
        ok, msg = within(orc, ref_y, 1e-2, 2e-3)
        assert ok, f"oracle vs reference split {s}: {msg}"
        got = api.linear_cpp_forced_pid(dev(x), dev(w), 400, s).cpu().numpy()
        ok, msg = within(got, ref_y, 1e-2, 2e-3)
        assert ok, f"product vs reference split {s}: {msg}"


def test_fp16_twin_gemm_three_way(api, oracle, tmp_path):
    m, n, k = 128, 384, 128
    a, b = rng.small_ints(1, rng.STREAM_A, (m, k)), rng.small_ints(1, rng.STREAM_B, (n, k))
    batch = RefBatch(tmp_path)
    batch.add("fp16_twin", a, b, split=256)
    ref = batch.run()[0]
    assert np.array_equal(ref, oracle.twin_gemm_f16(a, b, 256))
    assert np.array_equal(api.twin_gemm_fp16(dev(a), dev(b), 256).cpu().numpy(), ref)


def test_int8_three_way_bit_exact(api, oracle, tmp_path):
    batch = RefBatch(tmp_path)
    cases = []
    # m % 4 == 0 throughout: the reference's INT8 kernels store C with 16-byte vectors along m and fault with
    # "misaligned address" on column-major C whose leading dimension m is not a multiple of 4
    for (m, n, k) in ((64, 128, 128), (36, 200, 4096), (152, 72, 512)):
        a, b = rng.int8_uniform(3, rng.STREAM_A, (m, k)), rng.int8_uniform(3, rng.STREAM_B, (n, k))
        cases.append(("auto", 0, a, b))
        batch.add("int8_auto", a, b)
    a, b = rng.int8_uniform(104, 0, (152, 512)), rng.int8_uniform(104, 1, (72, 512))
    for pid in (0, 6, 17, 30, 45):
        cases.append(("pid", pid, a, b))
        batch.add("int8_pid", a, b, pid=pid)
    outs = batch.run()
    for (kind, pid, a, b), ref in zip(cases, outs):
        assert np.array_equal(ref, oracle.gemm_i8_rcc(a, b)), f"reference {kind} {pid} vs oracle"
        got = api.gemm_rcc(dev(a), dev(b)) if kind == "auto" else api.gemm_rcc_pid(dev(a), dev(b), pid, 1)
        assert np.array_equal(got.cpu().numpy(), ref), f"product {kind} {pid} vs reference"


def test_fp32_three_way(api, oracle, tmp_path):
    """The FP32 configuration shape (37 x 1024 x 1024, U[-1,1], seed 0) and a sample of pids."""
    a, b = rng.uniform(0, rng.STREAM_A, (37, 1024), -1.0, 1.0), rng.uniform(0, rng.STREAM_B, (1024, 1024), -1.0, 1.0)
    a2, b2 = rng.uniform(18, 0, (70, 96), -1.0, 1.0), rng.uniform(18, 1, (150, 96), -1.0, 1.0)
    ai, bi = rng.small_ints(1, 0, (33, 1100), dtype=np.float32), rng.small_ints(1, 1, (65, 1100), dtype=np.float32)
    batch = RefBatch(tmp_path)
    batch.add("fp32_auto", a, b)
    batch.add("fp32_auto", ai, bi)
    pids = (0, 7, 19, 23, 39)
    for pid in pids:
        batch.add("fp32_pid", a2, b2, pid=pid)
    outs = batch.run()

    def close32(x, y):
        return np.all(np.abs(x - y) <= 1e-4 * np.maximum(1.0, np.abs(y)))
    assert close32(oracle.gemm_f32_rcc(a, b), outs[0]), "oracle vs reference on the configuration shape"
    assert close32(api.gemm_rcc(dev(a), dev(b)).cpu().numpy(), outs[0]), "product vs reference on the configuration shape"
    assert np.array_equal(outs[1], oracle.gemm_f32_rcc(ai, bi))
    assert np.array_equal(api.gemm_rcc(dev(ai), dev(bi)).cpu().numpy(), outs[1])
    orc2 = oracle.gemm_f32_rcc(a2, b2)
    for pid, ref in zip(pids, outs[2:]):
        assert close32(orc2, ref), f"oracle vs reference pid {pid}"
        assert close32(api.gemm_rcc_pid(dev(a2), dev(b2), pid, 1).cpu().numpy(), ref), f"product vs reference pid {pid}"
