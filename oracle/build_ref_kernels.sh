#!/usr/bin/env bash
# Compiles the REFERENCE'S OWN GEMM kernels (its CUTLASS instantiations for FP16 / INT8 / FP32 RCC,
# the selectors and the cost models) from the sources where they lie in the read-only reference
# tree, plus this repository's small command-line driver oracle/ref_runner.cu, into
#     oracle/_ref/mp_ref_runner
# a checker binary that reads operands from a file, runs the reference on the GPU and writes the
# result back.  It pins the CPU oracle and the product: tests/test_reference_kernels_gpu.py feeds
# identical seeded inputs to the reference, to oracle/mp_oracle.c and to libmoonpoly_gemm.so.
# Test infrastructure only; nothing of it is linked into, or called by, the product.
#
# Third-party input: the reference's device arithmetic is NVIDIA CUTLASS 4.1 plus the reference's
# own patch integrations/cutlass/cutlass_4_1_pattern2_twin_gemm.patch.  The header tree found in
# the image (CUTLASS 4.1.0, vendored by a Python package) is copied to a scratch directory and
# patched there.  No reference source and no CUTLASS file enters the repository; objects live
# under the scratch directory and only the linked binary is written to oracle/_ref/.
#
#   REFERENCE_DIR   reference checkout
#   CUTLASS_DIR     CUTLASS 4.1 tree with include/ and tools/util/include/
#   MP_REF_SCRATCH  scratch directory            (default ${TMPDIR:-/tmp}/mp_ref_build)
#   MP_REF_JOBS     parallel nvcc jobs           (default 4)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${REFERENCE_DIR:-/root/reference}"
CUTLASS="${CUTLASS_DIR:-$(python -c 'import tilelang,os;print(os.path.join(os.path.dirname(tilelang.__file__),"3rdparty","cutlass"))' 2>/dev/null || true)}"
SCRATCH="${MP_REF_SCRATCH:-${TMPDIR:-/tmp}/mp_ref_build}"
JOBS="${MP_REF_JOBS:-4}"
OUT="$HERE/_ref"
BIN="$OUT/mp_ref_runner"
PATCH="$REF/integrations/cutlass/cutlass_4_1_pattern2_twin_gemm.patch"

if [ ! -d "$REF/moonpoly/core" ] || [ ! -d "$CUTLASS/include" ] || [ ! -f "$PATCH" ]; then
  echo "build_ref_kernels: reference tree, its CUTLASS patch or the CUTLASS headers not found; nothing built" >&2
  exit 0
fi

SRCS=(
  moonpoly/core/fp16/fp16_rcc.cu
  moonpoly/core/fp16/fp16_rcc_cost.cu
  moonpoly/core/fp16/fp16_dispatch.cu
  moonpoly/generated/fp16/rcc/candidates.cu
  moonpoly/core/int8/i8_rcc.cu
  moonpoly/core/int8/i8_rcc_cost.cu
  moonpoly/core/int8/i8_dispatch.cu
  moonpoly/core/fp32/fp32_rcc.cu
  moonpoly/core/fp32/fp32_rcc_cost.cu
  moonpoly/core/fp32/fp32_dispatch.cu
  moonpoly/core/moonpoly_gemm.cu
)

newest_src=0
for s in "${SRCS[@]}"; do
  t=$(stat -c %Y "$REF/$s"); [ "$t" -gt "$newest_src" ] && newest_src=$t
done
t=$(stat -c %Y "$HERE/ref_runner.cu"); [ "$t" -gt "$newest_src" ] && newest_src=$t
if [ -x "$BIN" ] && [ "$(stat -c %Y "$BIN")" -ge "$newest_src" ]; then
  echo "build_ref_kernels: $BIN is up to date"
  exit 0
fi

mkdir -p "$OUT" "$SCRATCH/obj"
if [ ! -f "$SCRATCH/cutlass/.patched" ]; then
  rm -rf "$SCRATCH/cutlass"
  mkdir -p "$SCRATCH/cutlass/tools/util"
  cp -r "$CUTLASS/include" "$SCRATCH/cutlass/include"
  cp -r "$CUTLASS/tools/util/include" "$SCRATCH/cutlass/tools/util/include"
  (cd "$SCRATCH/cutlass" && patch -p3 --forward --silent --batch < "$PATCH")
  touch "$SCRATCH/cutlass/.patched"
fi

# The reference's kernels are mma.sync / SIMT CUTLASS kernels written for sm_80; they compile
# unchanged for sm_100 (no arch-specific "a" features are involved).
NVCCFLAGS=(-std=c++17 -O3 --expt-relaxed-constexpr -w -Xcompiler -fPIC
           -gencode arch=compute_100,code=sm_100
           -I "$REF/moonpoly/include" -I "$REF/moonpoly/generated/fp16/rcc"
           -I "$SCRATCH/cutlass/include" -I "$SCRATCH/cutlass/tools/util/include")

pids=()
objs=()
running=0
for s in "${SRCS[@]}"; do
  o="$SCRATCH/obj/$(echo "$s" | tr '/' '_' | sed 's/\.cu$/.o/')"
  objs+=("$o")
  if [ -f "$o" ] && [ "$(stat -c %Y "$o")" -ge "$(stat -c %Y "$REF/$s")" ]; then continue; fi
  ( nvcc "${NVCCFLAGS[@]}" -c "$REF/$s" -o "$o.tmp" && mv "$o.tmp" "$o" ) &
  pids+=($!)
  running=$((running + 1))
  if [ "$running" -ge "$JOBS" ]; then wait -n; running=$((running - 1)); fi
done
for p in "${pids[@]:-}"; do [ -n "$p" ] && wait "$p"; done
for o in "${objs[@]}"; do [ -f "$o" ] || { echo "build_ref_kernels: $o failed to build" >&2; exit 1; }; done

nvcc "${NVCCFLAGS[@]}" "$HERE/ref_runner.cu" "${objs[@]}" -o "$BIN" -cudart static
echo "built $BIN"
