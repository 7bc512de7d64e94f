"""The CMake project exposes the reference's target and CTest names (configure + `ctest -N` only; nothing is compiled)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
SOURCES = ["fp16/test_fp16_row_col_col.cu", "fp16/test_fp16_pattern2_twin_gemm.cu", "fp32/test_fp32_row_col_col.cu",
           "int8/test_int8_row_col_col.cu"]


@pytest.mark.skipif(shutil.which("cmake") is None or shutil.which("nvcc") is None, reason="needs cmake and nvcc")
def test_cmake_lists_target_and_the_four_ctest_names(tmp_path):
    # a stand-in tree with the reference's test file names: configuring needs the files to exist, not their content
    ref = tmp_path / "ref"
    for s in SOURCES:
        p = ref / "tests" / "cpp" / s
        p.parent.mkdir(parents=True, exist_ok=True)
        p.write_text("int main() { return 0; }\n")
    build = tmp_path / "build"
    res = subprocess.run(["cmake", "-S", os.path.join(ROOT, "moonpoly-dev_b200"), "-B", str(build),
                          f"-DMOONPOLY_REFERENCE_DIR={ref}", f"-DMOONPOLY_CUTLASS_DIR={tmp_path}"],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    listing = subprocess.run(["ctest", "--test-dir", str(build), "-N"], capture_output=True, text=True, timeout=60).stdout
    for name in ("moonpoly.fp16_rcc", "moonpoly.fp16_pattern2", "moonpoly.fp32_rcc", "moonpoly.int8_rcc"):
        assert name in listing, listing
    assert "Total Tests: 4" in listing
    targets = subprocess.run(["cmake", "--build", str(build), "--target", "help"], capture_output=True, text=True,
                             timeout=60).stdout
    assert "moonpoly_gemm" in targets
