// Layout enum and constants shared by the host front end.  Counterpart of the reference's
// rocm_wmma_gemm/include/rocm_wmma_gemm/kernel/common.hpp:38-86; the enumerator values are
// part of the C ABI (0 = row-major, 1 = column-major).
#ifndef ROCM_WMMA_GEMM_KERNEL_COMMON_HPP
#define ROCM_WMMA_GEMM_KERNEL_COMMON_HPP

#include <rocm_wmma_gemm/compat.hpp>

namespace rocm_wmma_gemm
{

enum class m_layout
{
    row_major = 0, ///< elements of a row are contiguous
    col_major = 1  ///< elements of a column are contiguous
};

enum class m_input
{
    matrix_a,
    matrix_b
};

// Granularity of the tensor-core instruction on this architecture: one tcgen05.mma covers
// K = 16 half-precision elements and 32-lane warps read the accumulators.
static constexpr int wmma_tile = 16;
static constexpr int warp_size = 32;

} // namespace rocm_wmma_gemm

#endif // ROCM_WMMA_GEMM_KERNEL_COMMON_HPP
