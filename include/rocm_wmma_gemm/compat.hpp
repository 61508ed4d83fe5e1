// Source-compatibility names for host programs written against the reference's HIP headers:
// the reference's API spells its element types `half` / `__hip_bfloat16` and its stream type
// `hipStream_t` (rocm_wmma_gemm/include/rocm_wmma_gemm/gemm.hpp:50-73 of
// adelj88/rocm_wmma_gemm).  On CUDA they are __half, __nv_bfloat16 and cudaStream_t.
// Define ROCM_WMMA_GEMM_NO_COMPAT_NAMES to keep these names out of the global namespace.
#ifndef ROCM_WMMA_GEMM_COMPAT_HPP
#define ROCM_WMMA_GEMM_COMPAT_HPP

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#ifndef ROCM_WMMA_GEMM_NO_COMPAT_NAMES
using half           = __half;
using __hip_bfloat16 = __nv_bfloat16;
using hipStream_t    = cudaStream_t;
#endif

#endif // ROCM_WMMA_GEMM_COMPAT_HPP
