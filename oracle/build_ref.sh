#!/usr/bin/env bash
# Builds oracle/_ref/libflb_ref.so: the reference's own attention kernels (compiled from the
# reference checkout where it lies — nothing is copied into this repository) plus the runner in
# ref_runner.cu, for sm_100a.  The reference's CMake build is not used (it pins sm_75 and a
# CUDA 11.7 path); its two kernel translation units compile as they are with nvcc 12.9.
# usage: build_ref.sh <reference-root>
set -euo pipefail
REF="${1:?usage: build_ref.sh <reference-root>}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
OUT="$HERE/_ref"
mkdir -p "$OUT"
NVCC="${NVCC:-$(command -v nvcc || echo /usr/local/cuda/bin/nvcc)}"
"$NVCC" -std=c++17 -O3 -DNDEBUG -w -gencode arch=compute_100a,code=sm_100a \
    -Xcompiler -fPIC -shared -cudart shared \
    -I "$REF/fasterLlama" -I "$REF/fasterLlama/cuda" \
    "$REF/fasterLlama/cuda/decoder_kernels.cu" "$REF/fasterLlama/cuda/decoding_kernels.cu" "$HERE/ref_runner.cu" \
    -lcublas -lcurand -o "$OUT/libflb_ref.so"
echo "built $OUT/libflb_ref.so"
