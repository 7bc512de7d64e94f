#!/usr/bin/env bash
# Compiles the REFERENCE'S OWN four CTest programmes, from the sources where they lie in the
# read-only reference tree, against this repository's moonpoly.cuh + libmoonpoly_gemm.so.
# They are checkers (each compares the library with cuBLAS on the GPU and prints PASS): test
# infrastructure, never part of the product.  Outputs go to oracle/_ref/ only.
#   tests/cpp/fp16/test_fp16_row_col_col.cu        -> CTest moonpoly.fp16_rcc
#   tests/cpp/fp16/test_fp16_pattern2_twin_gemm.cu -> CTest moonpoly.fp16_pattern2
#   tests/cpp/fp32/test_fp32_row_col_col.cu        -> CTest moonpoly.fp32_rcc
#   tests/cpp/int8/test_int8_row_col_col.cu        -> CTest moonpoly.int8_rcc
# The programmes use CUTLASS *utility* headers (host tensors, random fill) and cuBLAS as their
# oracle; both come from the image (a CUTLASS header tree under site-packages, cuBLAS under the
# CUDA toolkit).  Nothing from the reference is copied into the repository.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ROOT="$(dirname "$HERE")"
REF="${REFERENCE_DIR:-/root/reference}"
CUTLASS="${CUTLASS_DIR:-$(python -c 'import tilelang,os;print(os.path.join(os.path.dirname(tilelang.__file__),"3rdparty","cutlass"))' 2>/dev/null || true)}"
if [ ! -d "$REF/tests/cpp" ] || [ ! -d "$CUTLASS/include" ]; then
  echo "build_ref: reference tree or CUTLASS utility headers not found; nothing built" >&2
  exit 0
fi
OUT="$HERE/_ref"
mkdir -p "$OUT"
PKG="$ROOT/moonpoly-dev_b200"
for t in fp16/test_fp16_row_col_col fp16/test_fp16_pattern2_twin_gemm fp32/test_fp32_row_col_col int8/test_int8_row_col_col; do
  name="$(basename "$t")"
  if [ "$OUT/$name" -nt "$REF/tests/cpp/$t.cu" ] && [ "$OUT/$name" -nt "$PKG/host/moonpoly.cuh" ]; then continue; fi
  nvcc -std=c++17 -O2 -gencode arch=compute_100a,code=sm_100a --expt-relaxed-constexpr -w \
       -I "$PKG/host" -I "$CUTLASS/include" -I "$CUTLASS/tools/util/include" \
       "$REF/tests/cpp/$t.cu" -o "$OUT/$name" \
       -L "$PKG" -lmoonpoly_gemm -lcublas -Xlinker -rpath,'$ORIGIN/../../moonpoly-dev_b200'
  echo "built $OUT/$name"
done
