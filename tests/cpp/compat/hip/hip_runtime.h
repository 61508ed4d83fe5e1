// Stand-in for <hip/hip_runtime.h> so that host programs written against the reference's HIP
// API (its tests and benchmarks: test/gemm/*.cpp, common/hip_utils.hpp of
// adelj88/rocm_wmma_gemm) compile against the CUDA runtime with only include-path changes.
// Only the runtime calls those programs make are mapped.  Test infrastructure.
#ifndef B200_COMPAT_HIP_RUNTIME_H
#define B200_COMPAT_HIP_RUNTIME_H

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

using half           = __half;
using __hip_bfloat16 = __nv_bfloat16;

using hipError_t  = cudaError_t;
using hipStream_t = cudaStream_t;
using hipEvent_t  = cudaEvent_t;
constexpr hipError_t hipSuccess = cudaSuccess;

enum hipMemcpyKind_compat {
    hipMemcpyHostToDevice   = cudaMemcpyHostToDevice,
    hipMemcpyDeviceToHost   = cudaMemcpyDeviceToHost,
    hipMemcpyDeviceToDevice = cudaMemcpyDeviceToDevice
};

inline const char* hipGetErrorString(hipError_t e) { return cudaGetErrorString(e); }
inline hipError_t  hipStreamCreate(hipStream_t* s) { return cudaStreamCreate(s); }
inline hipError_t  hipStreamDestroy(hipStream_t s) { return cudaStreamDestroy(s); }
inline hipError_t  hipStreamSynchronize(hipStream_t s) { return cudaStreamSynchronize(s); }
template <class T>
inline hipError_t hipMalloc(T** p, size_t bytes) { return cudaMalloc(reinterpret_cast<void**>(p), bytes); }
inline hipError_t hipFree(void* p) { return cudaFree(p); }
inline hipError_t hipMemcpy(void* dst, const void* src, size_t bytes, hipMemcpyKind_compat kind)
{
    return cudaMemcpy(dst, src, bytes, static_cast<cudaMemcpyKind>(kind));
}
inline hipError_t hipMemset(void* p, int v, size_t bytes) { return cudaMemset(p, v, bytes); }
inline hipError_t hipDeviceSynchronize() { return cudaDeviceSynchronize(); }
inline hipError_t hipPeekAtLastError() { return cudaPeekAtLastError(); }
inline hipError_t hipGetLastError() { return cudaGetLastError(); }
inline hipError_t hipEventCreate(hipEvent_t* e) { return cudaEventCreate(e); }
inline hipError_t hipEventDestroy(hipEvent_t e) { return cudaEventDestroy(e); }
inline hipError_t hipEventRecord(hipEvent_t e, hipStream_t s) { return cudaEventRecord(e, s); }
inline hipError_t hipEventSynchronize(hipEvent_t e) { return cudaEventSynchronize(e); }
inline hipError_t hipEventElapsedTime(float* ms, hipEvent_t a, hipEvent_t b) { return cudaEventElapsedTime(ms, a, b); }

#endif // B200_COMPAT_HIP_RUNTIME_H
