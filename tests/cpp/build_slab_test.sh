#!/bin/sh
# Builds tests/cpp/test_slab_driver against the in-tree library and the oracle's C restatement.
set -e
here="$(cd "$(dirname "$0")" && pwd)"
root="$(dirname "$(dirname "$here")")"
pkg="$root/rocm_wmma_gemm_b200"
cuda="${CUDA_HOME:-/usr/local/cuda}"
gcc -O2 -ffp-contract=off -std=c11 -c "$root/oracle/cpu_gemm.c" -o "$here/cpu_gemm.o"
g++ -O2 -std=c++17 -I"$root/include" -I"$cuda/include" "$here/test_slab_driver.cpp" "$here/cpu_gemm.o" -o "$here/test_slab_driver" \
    -L"$pkg" -lrocm_wmma_gemm_sm100a -Wl,-rpath,"$pkg" -L"$cuda/lib64" -lcudart -ldl -lpthread -lm
echo "$here/test_slab_driver"
