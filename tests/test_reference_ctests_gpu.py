"""Runs the reference's own four CTest programmes against this library.

oracle/build_ref.sh compiles tests/cpp/{fp16,fp32,int8}/*.cu of the reference, in place, against
moonpoly-dev_b200/host/moonpoly.cuh and libmoonpoly_gemm.so (CTest names moonpoly.fp16_rcc,
moonpoly.fp16_pattern2, moonpoly.fp32_rcc, moonpoly.int8_rcc).  Each programme compares the
library with cuBLAS on the GPU under the reference's own tolerances and prints PASS.
"""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
REF_BIN = os.path.join(ROOT, "oracle", "_ref")

PROGRAMMES = {
    "moonpoly.fp16_rcc": "test_fp16_row_col_col",
    "moonpoly.fp16_pattern2": "test_fp16_pattern2_twin_gemm",
    "moonpoly.fp32_rcc": "test_fp32_row_col_col",
    "moonpoly.int8_rcc": "test_int8_row_col_col",
}


@pytest.mark.parametrize("ctest_name", sorted(PROGRAMMES))
def test_reference_ctest_programme(ctest_name):
    exe = os.path.join(REF_BIN, PROGRAMMES[ctest_name])
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref not built (needs the reference tree at build time)")
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.pathsep.join(
        [os.path.join(ROOT, "moonpoly-dev_b200"), "/usr/local/cuda/lib64", env.get("LD_LIBRARY_PATH", "")])
    res = subprocess.run([exe], capture_output=True, text=True, timeout=120, env=env)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "PASS" in res.stdout


def test_reference_fp16_ctest_on_bench_shapes():
    """The FP16 programme accepts a shape on its command line: run it on sweep shapes too."""
    exe = os.path.join(REF_BIN, "test_fp16_row_col_col")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref not built")
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.pathsep.join(
        [os.path.join(ROOT, "moonpoly-dev_b200"), "/usr/local/cuda/lib64", env.get("LD_LIBRARY_PATH", "")])
    for m, n, k in ((1, 4096, 4096), (127, 4096, 4096), (512, 1024, 4096)):
        res = subprocess.run([exe, str(m), str(n), str(k)], capture_output=True, text=True, timeout=300, env=env)
        assert res.returncode == 0 and "PASS" in res.stdout, (m, n, k, res.stdout[-500:], res.stderr[-500:])
