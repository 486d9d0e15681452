#!/bin/bash
# Builds the kernels-only reference arm: the reference's own CUDA GEMM / GEMV / repack translation units, unmodified, plus
# the link shim beside this script, into baseline/_ref/libllaminar_ref_kernels.so.
#   usage: baseline/build_ref_kernels.sh /path/to/reference
set -e
REF=${1:-/root/reference}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=$HERE/_ref
TMP=${TMPDIR:-/tmp}/llaminar_ref_build
mkdir -p "$OUT" "$TMP"
R=$REF/src/v2
FL="-std=c++20 -O3 -I$R -I$REF/src -gencode arch=compute_100,code=sm_100 --expt-relaxed-constexpr -Xcompiler -fPIC -w"
pids=()
for f in kernels/cuda/gemm/CUDANativeVNNIPrefillKernels.cu kernels/cuda/gemm/CUDANativeVNNIGemvTuned.cu \
         kernels/cuda/repack/CUDAVnniRepackKernels.cu kernels/cuda/gemm/CUDANativeVNNIIQTables.cu; do
  o=$TMP/$(basename $f .cu).o
  if [ ! -f "$o" ]; then nvcc $FL -c $R/$f -o $o & pids+=($!); fi
done
g++ -std=c++20 -O2 -fPIC -I$R -I$REF/src -I/usr/local/cuda/include -c $HERE/ref_shim.cpp -o $TMP/ref_shim.o
for p in "${pids[@]}"; do wait $p; done
nvcc -shared -o $OUT/libllaminar_ref_kernels.so $TMP/*.o -lcudart
echo built $OUT/libllaminar_ref_kernels.so
