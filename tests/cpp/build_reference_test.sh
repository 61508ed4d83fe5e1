#!/bin/sh
# Compiles the reference's own typed tests (test/gemm/test_float_accum.cpp and
# test/gemm/test_same_prec.cpp of a adelj88/rocm_wmma_gemm checkout, unmodified, from where they
# lie) against this repository's
# front end: only include paths change - include/ supplies rocm_wmma_gemm/kernel_loader.hpp,
# tests/cpp/compat/ supplies stand-ins for <hip/hip_runtime.h> and <gtest/gtest.h>.
#   usage: build_reference_test.sh <path to the reference checkout>
set -e
ref="$1"
[ -f "$ref/test/gemm/test_float_accum.cpp" ] || { echo "no reference checkout at '$ref'"; exit 3; }
here="$(cd "$(dirname "$0")" && pwd)"
root="$(dirname "$(dirname "$here")")"
pkg="$root/rocm_wmma_gemm_b200"
cuda="${CUDA_HOME:-/usr/local/cuda}"
for t in float_accum same_prec; do
    g++ -O2 -std=c++20 -I"$here/compat" -I"$root/include" -I"$cuda/include" -I"$ref" -I"$ref/test" \
        "$ref/test/gemm/test_$t.cpp" -o "$here/test_reference_$t" \
        -L"$cuda/lib64" -lcudart -ldl -lpthread -lm
    echo "$here/test_reference_$t"
done
