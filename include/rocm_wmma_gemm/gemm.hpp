// Templated C++ entry point of the GEMM library: C = A * B for
//   (T, U) in {(half, half), (float, half), (__hip_bfloat16, __hip_bfloat16), (float, __hip_bfloat16)}
// and any row-/column-major combination of C, A and B.  Same template parameter order
// (layout_C, layout_A, layout_B), same argument order and same stream-by-reference as the
// reference's rocm_wmma_gemm/include/rocm_wmma_gemm/gemm.hpp:50-73; the reference exports
// explicit instantiations from its shared object (src/gemm.cpp:56-198), here the templates
// are header-inline forwards to the C ABI of include/b200_gemm.h, so a program links
// librocm_wmma_gemm_sm100a.so and nothing else.
//
// A is M x K, B is K x N, C is M x N, all dense-packed; batched matrices are `batch_count`
// consecutive matrices (strides M*K, K*N, M*N).  The call is asynchronous on `stream`.
// A failing call throws std::runtime_error (the reference throws from its launcher when a
// kernel is missing, kernel_launcher.hpp:119-125); the message is b200_gemm_last_error().
#ifndef ROCM_WMMA_GEMM_GEMM_HPP
#define ROCM_WMMA_GEMM_GEMM_HPP

#include <b200_gemm.h>
#include <rocm_wmma_gemm/kernel/common.hpp>

#include <cstddef>
#include <stdexcept>
#include <string>
#include <type_traits>

namespace rocm_wmma_gemm
{

// Tuned parameters of one problem; counterpart of the reference's generated `gemm_params`
// (config/generate_config.py:94-103) with the sm_100a key set.
struct gemm_params
{
    int tile_m;
    int tile_n;
    int stages;
    int cluster;
    int split_k;
    int raster;
};

namespace detail
{

template<class T, class U>
constexpr int type_index()
{
    if constexpr(std::is_same_v<T, half> && std::is_same_v<U, half>) return B200_GEMM_F16_F16;
    else if constexpr(std::is_same_v<T, float> && std::is_same_v<U, half>) return B200_GEMM_F32_F16;
    else if constexpr(std::is_same_v<T, __hip_bfloat16> && std::is_same_v<U, __hip_bfloat16>)
        return B200_GEMM_BF16_BF16;
    else if constexpr(std::is_same_v<T, float> && std::is_same_v<U, __hip_bfloat16>)
        return B200_GEMM_F32_BF16;
    else
    {
        static_assert(sizeof(T) == 0, "Unsupported type pair for rocm_wmma_gemm::gemm");
        return -1;
    }
}

// Index of the compiled configuration the tuned table selects; argument order of the
// reference's detail::find_best_config (m, n, k, type_group, layout_a, layout_b, layout_c).
inline size_t find_best_config(size_t   m,
                               size_t   n,
                               size_t   k,
                               size_t   type_group,
                               m_layout layout_a,
                               m_layout layout_b,
                               m_layout layout_c)
{
    const int idx = b200_gemm_select_config(m,
                                            n,
                                            k,
                                            type_group ? B200_GEMM_F32_F16 : B200_GEMM_F16_F16,
                                            static_cast<int>(layout_c),
                                            static_cast<int>(layout_a),
                                            static_cast<int>(layout_b),
                                            nullptr);
    if(idx < 0) throw std::runtime_error(b200_gemm_last_error());
    return static_cast<size_t>(idx);
}

} // namespace detail

inline gemm_params get_gemm_params(size_t   m,
                                   size_t   n,
                                   size_t   k,
                                   m_layout layout_c,
                                   m_layout layout_a,
                                   m_layout layout_b,
                                   size_t   type_group = 0)
{
    b200_gemm_config c{};
    const int        idx = b200_gemm_select_config(m,
                                            n,
                                            k,
                                            type_group ? B200_GEMM_F32_F16 : B200_GEMM_F16_F16,
                                            static_cast<int>(layout_c),
                                            static_cast<int>(layout_a),
                                            static_cast<int>(layout_b),
                                            &c);
    if(idx < 0) throw std::runtime_error(b200_gemm_last_error());
    return gemm_params{c.tile_m, c.tile_n, c.stages, c.cluster, c.split_k, c.raster};
}

template<m_layout layout_C, m_layout layout_A, m_layout layout_B, class T, class U>
void gemm(T* C, U* A, U* B, size_t M, size_t N, size_t K, size_t batch_count, hipStream_t& stream)
{
    const int st = b200_gemm_ex(detail::type_index<T, U>(),
                                C,
                                A,
                                B,
                                M,
                                N,
                                K,
                                batch_count,
                                static_cast<int>(layout_C),
                                static_cast<int>(layout_A),
                                static_cast<int>(layout_B),
                                &stream,
                                nullptr);
    if(st != B200_GEMM_OK)
        throw std::runtime_error(std::string("rocm_wmma_gemm::gemm: ") + b200_gemm_last_error());
}

template<m_layout layout_C, m_layout layout_A, m_layout layout_B, class T, class U>
void gemm(T* C, U* A, U* B, size_t M, size_t N, size_t K, hipStream_t& stream)
{
    gemm<layout_C, layout_A, layout_B>(C, A, B, M, N, K, 1, stream);
}

} // namespace rocm_wmma_gemm

#endif // ROCM_WMMA_GEMM_GEMM_HPP
