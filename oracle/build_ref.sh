#!/usr/bin/env bash
# Test infrastructure, not product code.
#
# Compiles the reference project's own CUDA kernel sources, unmodified and from
# where they lie (the checkout named by REF_ROOT), into
# oracle/_ref/librisa_ref.so together with ref_shim.cpp (exception-catching
# C wrappers around the reference's extern "C" launchers, csrc/launchers.h:8-64).
# Flags follow the reference's csrc/CMakeLists.txt:30-44 because --use_fast_math
# is part of its numeric contract.  Nothing is copied into this repository; the
# output directory is git-ignored.  attention_dispatch.cu alone takes ~15 min.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF_ROOT="${REF_ROOT:-/root/reference}"
OUT="$HERE/_ref"
SRC="$REF_ROOT/csrc"
[ -d "$SRC/kernels" ] || { echo "reference sources not found at $SRC" >&2; exit 3; }
mkdir -p "$OUT/obj"
FLAGS=(-std=c++20 -O3 --use_fast_math -DNDEBUG
  -U__CUDA_NO_HALF_OPERATORS__ -U__CUDA_NO_HALF_CONVERSIONS__
  -U__CUDA_NO_BFLOAT16_OPERATORS__ -U__CUDA_NO_BFLOAT16_CONVERSIONS__
  -U__CUDA_NO_BFLOAT162_OPERATORS__ -U__CUDA_NO_BFLOAT162_CONVERSIONS__
  --expt-relaxed-constexpr --expt-extended-lambda
  -gencode arch=compute_100,code=sm_100 -Xcompiler -fPIC
  -I"$SRC" -I"$SRC/kernels")
UNITS=(quantize_v quantize_qk quantize_gather lse_correction key_mask_tiles sparse_selection attention_dispatch)
for u in "${UNITS[@]}"; do
  if [ ! -f "$OUT/obj/$u.o" ] || [ "$SRC/kernels/$u.cu" -nt "$OUT/obj/$u.o" ]; then
    echo "[build_ref] nvcc $u.cu"
    nvcc "${FLAGS[@]}" --threads "${REF_NVCC_THREADS:-8}" -c "$SRC/kernels/$u.cu" -o "$OUT/obj/$u.o"
  fi
done
echo "[build_ref] shim + link"
nvcc -std=c++20 -O2 -Xcompiler -fPIC -I"$SRC" -I"$SRC/kernels" -c "$HERE/ref_shim.cpp" -x cu -o "$OUT/obj/ref_shim.o"
OBJS=(); for u in "${UNITS[@]}"; do OBJS+=("$OUT/obj/$u.o"); done
nvcc -shared -o "$OUT/librisa_ref.so" "${OBJS[@]}" "$OUT/obj/ref_shim.o" -lcudart
echo "[build_ref] wrote $OUT/librisa_ref.so"
