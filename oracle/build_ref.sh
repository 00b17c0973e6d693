#!/usr/bin/env bash
# Builds the reference's own CUDA sources for the quantized-linear path into oracle/_ref/libref.so,
# compiled for sm_100a from where they lie (nothing is copied into this repository).
#
# The resulting library is TEST INFRASTRUCTURE: the GPU parity tests load it beside the product
# library and compare outputs; the product never links or loads it.
#
# Units (paths inside the reference project), flags as the reference's build.rs passes them
# (build.rs:119-126; no fast-math for these units):
#   csrc/kernels.cu  csrc/h3.cu  csrc/sd.cu  csrc/vendor/w6a8_requant.cu  csrc/vendor/cutlass_gemm_int8.cu
# csrc/gemm.cu is not built (it pulls cuBLASLt and conv templates); its two int8 wrappers only forward to
# launch_cutlass_int8_dequant[_residual] (gemm.cu:123-140), which the tests call directly.
#
# Usage: oracle/build_ref.sh [REFERENCE_ROOT]     (or the REFERENCE_ROOT variable, or a checkout named "reference" beside
# this repository; skipped when the tree is absent)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-${REFERENCE_ROOT:-$(dirname "$(dirname "$HERE")")/reference}}"
OUT="$HERE/_ref"
if [ ! -d "$REF/csrc" ]; then echo "build_ref: no reference tree at $REF; nothing built"; exit 0; fi
CUTLASS_INC="$(python - <<'PY'
import site, os
for sp in site.getsitepackages():
    p = os.path.join(sp, "flashinfer", "data", "cutlass")
    if os.path.exists(os.path.join(p, "include", "cutlass", "cutlass.h")):
        print(p); break
PY
)"
if [ -z "$CUTLASS_INC" ]; then echo "build_ref: CUTLASS headers not found"; exit 1; fi
mkdir -p "$OUT"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
FLAGS=(-O3 -std=c++17 --expt-relaxed-constexpr --expt-extended-lambda -DNDEBUG -DCOMFY_HAVE_CUTLASS
  -U__CUDA_NO_HALF_OPERATORS__ -U__CUDA_NO_HALF_CONVERSIONS__ -U__CUDA_NO_HALF2_OPERATORS__
  -U__CUDA_NO_BFLOAT16_CONVERSIONS__ -gencode=arch=compute_100a,code=sm_100a
  -I"$REF/csrc" -I"$REF/csrc/vendor" -I"$CUTLASS_INC/include" -I"$CUTLASS_INC/tools/util/include"
  -Xcompiler=-fPIC -w)
pids=()
for u in kernels h3 sd vendor/w6a8_requant vendor/cutlass_gemm_int8; do
  o="$OUT/$(basename "$u").o"
  if [ "$o" -nt "$REF/csrc/$u.cu" ]; then continue; fi
  ( "$NVCC" -c "$REF/csrc/$u.cu" -o "$o" "${FLAGS[@]}" && echo "built $u" ) &
  pids+=($!)
done
for p in "${pids[@]:-}"; do [ -n "$p" ] && wait "$p"; done
"$NVCC" -shared -o "$OUT/libref.so" "$OUT"/kernels.o "$OUT"/h3.o "$OUT"/sd.o "$OUT"/w6a8_requant.o \
  "$OUT"/cutlass_gemm_int8.o -gencode=arch=compute_100a,code=sm_100a -Xlinker -Bsymbolic -lcudart
echo "build_ref: $OUT/libref.so"
