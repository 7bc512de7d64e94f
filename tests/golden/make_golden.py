"""Generates tests/golden/rcc_known_answers.npz.

The reference keeps no stored vectors for this path; its CTest programmes fill the operands with
integer-valued entries in [-2, 2] (TensorFillRandomUniform(view, 1, 2, -2, 0),
tests/cpp/fp16/test_fp16_row_col_col.cu:62-65) and compare with cuBLAS at run time.  For such
inputs every product and partial sum is an exactly representable integer, so the result any
correct implementation (the reference's included) must produce is fixed by arithmetic alone.
This script computes those answers in int64 with numpy -- independently of oracle/mp_oracle.c --
for the shapes of the four CTest programmes, plus the all-ones "constant check"
(moonpoly/core/moonpoly_gemm.cu:1641-1736: every output equals K).

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "moonpoly-dev_b200", "py"))
from moonpoly_b200 import rng  # noqa: E402

# (name, m, n, k) -- tests/cpp/fp16/test_fp16_row_col_col.cu:102-106,
# tests/cpp/fp16/test_fp16_pattern2_twin_gemm.cu (m=128, n=384, k=128, split_n=256)
SHAPES = [("s16x32x64", 16, 32, 64), ("s64x128x128", 64, 128, 128), ("s128x256x256", 128, 256, 256),
          ("twin128x384x128", 128, 384, 128)]


def main():
    out = {}
    for name, m, n, k in SHAPES:
        a = rng.small_ints(1, rng.STREAM_A, (m, k), dtype=np.int64)
        b = rng.small_ints(1, rng.STREAM_B, (n, k), dtype=np.int64)
        c = (a @ b.T).T                      # [n, m] == column-major [m, n]
        assert np.abs(c).max() < 2048        # exactly representable in fp16
        out[name + "_c"] = c.astype(np.int32)
    # constant check: all ones -> K
    out["ones_8x24x4096_c"] = np.full((24, 8), 4096, np.int32)
    # scaled int8 matmul with power-of-two scales: every rounding step is exact
    m, n, k = 24, 40, 64
    a = rng.int8_uniform(3, rng.STREAM_A, (m, k)).astype(np.int64)
    b = rng.int8_uniform(3, rng.STREAM_B, (n, k)).astype(np.int64)
    acc = a @ b.T
    sa = np.ldexp(1.0, -(np.arange(m) % 3) - 8)
    sb = np.ldexp(1.0, -(np.arange(n) % 2) - 9)
    out["scaled_24x40x64_acc"] = acc.astype(np.int32)
    out["scaled_24x40x64_out"] = (acc * sa[:, None] * sb[None, :]).astype(np.float16)
    out["scaled_24x40x64_sa"] = sa.astype(np.float32)
    out["scaled_24x40x64_sb"] = sb.astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "rcc_known_answers.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
