#!/bin/sh
# Builds the `tuner` binary beside this script against the in-tree library.
set -e
here="$(cd "$(dirname "$0")" && pwd)"
pkg="$(dirname "$here")"
root="$(dirname "$pkg")"
cuda="${CUDA_HOME:-/usr/local/cuda}"
g++ -O2 -std=c++17 -I"$root/include" -I"$cuda/include" "$here/tuner.cpp" -o "$here/tuner" \
    -L"$pkg" -lrocm_wmma_gemm_sm100a -Wl,-rpath,"$pkg" -L"$cuda/lib64" -lcudart
echo "$here/tuner"
