#!/usr/bin/env bash
# Builds the reference's CUDA library, unmodified, with the reference's own rule (`make cuda-only`,
# Makefile:50-70 of Leeaandrob/neurogrid) into baseline/_ref/libgpu_engine.so.
#
#   baseline/build_reference.sh [REFERENCE_CHECKOUT]        (default: /root/reference)
#
# The sources are copied to a temporary folder (the checkout may be read-only) and not changed.
# The only departures are build flags given on the make command line: `-arch=sm_100` in place of
# `-arch=native` (the library is compiled on a machine without a GPU), and an rpath so that the
# library finds the CUDA toolkit's cuBLAS without LD_LIBRARY_PATH.  The reference has no Python
# package (no setup.py / pyproject.toml), so there is nothing for pip to install; its Go program
# needs a Go toolchain, which this image lacks; its LFM2 compute path is this library alone.
set -euo pipefail
REF="${1:-/root/reference}"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
CUDA_PATH="${CUDA_PATH:-/usr/local/cuda}"
TMP="$(mktemp -d)"
trap 'rm -rf "$TMP"' EXIT
mkdir -p "$TMP/src" "$OUT"
cp -r "$REF/gpu" "$TMP/src/gpu"
cp "$REF/Makefile" "$TMP/src/Makefile"
make -C "$TMP/src" -j"$(nproc)" cuda-only \
    NVCC_FLAGS="-arch=sm_100 -O3 --use_fast_math -std=c++17 -Xcompiler -fPIC -I$CUDA_PATH/include" \
    LDFLAGS="-L$CUDA_PATH/lib64 -lcudart -lcublas -lcublasLt -Xlinker -rpath=$CUDA_PATH/lib64"
cp "$TMP/src/build/libgpu_engine.so" "$OUT/libgpu_engine.so"
( cd "$REF" && { git rev-parse HEAD 2>/dev/null || echo "no git metadata"; } ) > "$OUT/SOURCE_REVISION"
echo "built $OUT/libgpu_engine.so"
