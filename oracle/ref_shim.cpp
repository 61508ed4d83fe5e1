// TEST INFRASTRUCTURE — NOT PRODUCT CODE.
//
// Compiles the reference's own CPU check path — test/test.hpp (init_matrix, hgemm_cpu,
// calculate_cosine_similarity) and common/matrix.hpp — UNMODIFIED, from where it lies in the
// reference checkout (passed with -I), and exports it through a small C ABI so the C
// restatement in cpu_gemm.c can be pinned against it and the benchmark can time it.
// No reference source is copied: this file only supplies the five names the header expects
// from HIP / gtest and thin wrappers that move raw buffers in and out of its `matrix` class.
//
// The reference's half types map to CUDA's host-usable ones (same IEEE formats, same
// round-to-nearest-even conversions): half -> __half, __hip_bfloat16 -> __nv_bfloat16.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <random>
#include <sstream>
#include <thread>
#include <vector>

using half           = __half;
using __hip_bfloat16 = __nv_bfloat16;

// verify_results() streams into the result of ASSERT_GT; give it a sink.
struct ref_assert_sink {
    template <class T>
    ref_assert_sink& operator<<(const T&) { return *this; }
};
#define ASSERT_GT(a, b) ref_assert_sink()

#include <test.hpp> // the reference's test/test.hpp (pulls in common/matrix.hpp)

namespace {

template <class T, m_layout L>
void fill_from(matrix<T, L>& m, const void* src) { std::memcpy(m.data(), src, m.size() * sizeof(T)); }

template <class T, m_layout L>
void copy_to(const matrix<T, L>& m, void* dst) { std::memcpy(dst, m.data(), m.size() * sizeof(T)); }

template <class TOut, class TIn, m_layout LC, m_layout LA, m_layout LB>
void gemm_one(void* C, const void* A, const void* B, size_t M, size_t N, size_t K)
{
    matrix<TIn, LA>  a(M, K);
    matrix<TIn, LB>  b(K, N);
    matrix<TOut, LC> c(M, N);
    fill_from(a, A);
    fill_from(b, B);
    hgemm_cpu(c, a, b);
    copy_to(c, C);
}

template <class TOut, class TIn>
void gemm_layouts(void* C, const void* A, const void* B, size_t M, size_t N, size_t K, int lc, int la, int lb)
{
    constexpr m_layout R = m_layout::row_major, Cm = m_layout::col_major;
    switch (lc << 2 | la << 1 | lb) {
        case 0: gemm_one<TOut, TIn, R, R, R>(C, A, B, M, N, K); break;
        case 1: gemm_one<TOut, TIn, R, R, Cm>(C, A, B, M, N, K); break;
        case 2: gemm_one<TOut, TIn, R, Cm, R>(C, A, B, M, N, K); break;
        case 3: gemm_one<TOut, TIn, R, Cm, Cm>(C, A, B, M, N, K); break;
        case 4: gemm_one<TOut, TIn, Cm, R, R>(C, A, B, M, N, K); break;
        case 5: gemm_one<TOut, TIn, Cm, R, Cm>(C, A, B, M, N, K); break;
        case 6: gemm_one<TOut, TIn, Cm, Cm, R>(C, A, B, M, N, K); break;
        case 7: gemm_one<TOut, TIn, Cm, Cm, Cm>(C, A, B, M, N, K); break;
        default: break;
    }
}

void gemm_types(int types, void* C, const void* A, const void* B, size_t M, size_t N, size_t K, int lc, int la, int lb)
{
    switch (types) {
        case 0: gemm_layouts<half, half>(C, A, B, M, N, K, lc, la, lb); break;
        case 1: gemm_layouts<float, half>(C, A, B, M, N, K, lc, la, lb); break;
        case 2: gemm_layouts<__hip_bfloat16, __hip_bfloat16>(C, A, B, M, N, K, lc, la, lb); break;
        case 3: gemm_layouts<float, __hip_bfloat16>(C, A, B, M, N, K, lc, la, lb); break;
        default: break;
    }
}

template <class T>
void init_one(void* data, size_t rows, size_t cols, int layout)
{
    if (layout == 0) {
        matrix<T, m_layout::row_major> m(rows, cols);
        init_matrix(m);
        copy_to(m, data);
    } else {
        matrix<T, m_layout::col_major> m(rows, cols);
        init_matrix(m);
        copy_to(m, data);
    }
}

template <class T>
float cosine_one(const void* g, const void* c, size_t M, size_t N, int layout)
{
    if (layout == 0) {
        matrix<T, m_layout::row_major> a(M, N), b(M, N);
        fill_from(a, g);
        fill_from(b, c);
        return calculate_cosine_similarity(a, b);
    }
    matrix<T, m_layout::col_major> a(M, N), b(M, N);
    fill_from(a, g);
    fill_from(b, c);
    return calculate_cosine_similarity(a, b);
}

} // namespace

// hgemm_cpu on rows [row_begin, row_end) of C, the rows split over `threads` host threads.
// B is placed in ONE `matrix` object shared by all threads; each thread gathers its own row
// panel of A and calls the reference's hgemm_cpu on (C panel, A panel, B).  `C_rows` receives
// the panels as a (row_end - row_begin) x N matrix in layout lc.  Used to time the
// reference's CPU path on all host cores.
namespace {

template <class TOut, class TIn, m_layout LC, m_layout LA, m_layout LB>
void rows_mt(void* C_rows, const void* A, const void* B, size_t M, size_t N, size_t K, size_t row_begin,
             size_t row_end, int threads)
{
    const size_t rows = row_end - row_begin;
    matrix<TIn, LB> b(K, N);
    fill_from(b, B);
    const matrix<TIn, LB>&   bref = b;
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) {
        const size_t r0 = rows * t / threads, r1 = rows * (t + 1) / threads;
        if (r1 == r0) continue;
        pool.emplace_back([=, &bref]() {
            const size_t     pr = r1 - r0;
            matrix<TIn, LA>  a(pr, K);
            matrix<TOut, LC> c(pr, N);
            const TIn*       src = static_cast<const TIn*>(A);
            for (size_t i = 0; i < pr; ++i)
                for (size_t k = 0; k < K; ++k) {
                    const size_t gi = row_begin + r0 + i;
                    a(i, k)         = src[LA == m_layout::row_major ? gi * K + k : k * M + gi];
                }
            hgemm_cpu(c, a, bref);
            TOut* dst = static_cast<TOut*>(C_rows);
            for (size_t i = 0; i < pr; ++i)
                for (size_t j = 0; j < N; ++j)
                    dst[LC == m_layout::row_major ? (r0 + i) * N + j : j * rows + (r0 + i)] = c(i, j);
        });
    }
    for (auto& th : pool) th.join();
}

template <class TOut, class TIn>
void rows_mt_layouts(void* C, const void* A, const void* B, size_t M, size_t N, size_t K, int lc, int la, int lb,
                     size_t r0, size_t r1, int threads)
{
    constexpr m_layout R = m_layout::row_major, Cm = m_layout::col_major;
    switch (lc << 2 | la << 1 | lb) {
        case 0: rows_mt<TOut, TIn, R, R, R>(C, A, B, M, N, K, r0, r1, threads); break;
        case 1: rows_mt<TOut, TIn, R, R, Cm>(C, A, B, M, N, K, r0, r1, threads); break;
        case 2: rows_mt<TOut, TIn, R, Cm, R>(C, A, B, M, N, K, r0, r1, threads); break;
        case 3: rows_mt<TOut, TIn, R, Cm, Cm>(C, A, B, M, N, K, r0, r1, threads); break;
        case 4: rows_mt<TOut, TIn, Cm, R, R>(C, A, B, M, N, K, r0, r1, threads); break;
        case 5: rows_mt<TOut, TIn, Cm, R, Cm>(C, A, B, M, N, K, r0, r1, threads); break;
        case 6: rows_mt<TOut, TIn, Cm, Cm, R>(C, A, B, M, N, K, r0, r1, threads); break;
        case 7: rows_mt<TOut, TIn, Cm, Cm, Cm>(C, A, B, M, N, K, r0, r1, threads); break;
        default: break;
    }
}

} // namespace

extern "C" {

// init_matrix of test/test.hpp on a rows x cols matrix of f16 (bf16 == 0) or bf16 elements.
void ref_init_matrix(void* data, size_t rows, size_t cols, int layout, int bf16)
{
    if (bf16) init_one<__hip_bfloat16>(data, rows, cols, layout);
    else init_one<half>(data, rows, cols, layout);
}

// hgemm_cpu of test/test.hpp.  types: 0 f16<-f16, 1 f32<-f16, 2 bf16<-bf16, 3 f32<-bf16.
void ref_hgemm(int types, void* C, const void* A, const void* B, size_t M, size_t N, size_t K, int lc, int la, int lb)
{
    gemm_types(types, C, A, B, M, N, K, lc, la, lb);
}

void ref_hgemm_rows_mt(int types, void* C_rows, const void* A, const void* B, size_t M, size_t N, size_t K, int lc,
                       int la, int lb, size_t row_begin, size_t row_end, int threads)
{
    if (row_end <= row_begin) return;
    threads = std::max(1, std::min<int>(threads, (int)(row_end - row_begin)));
    switch (types) {
        case 0: rows_mt_layouts<half, half>(C_rows, A, B, M, N, K, lc, la, lb, row_begin, row_end, threads); break;
        case 1: rows_mt_layouts<float, half>(C_rows, A, B, M, N, K, lc, la, lb, row_begin, row_end, threads); break;
        case 2:
            rows_mt_layouts<__hip_bfloat16, __hip_bfloat16>(C_rows, A, B, M, N, K, lc, la, lb, row_begin, row_end, threads);
            break;
        case 3: rows_mt_layouts<float, __hip_bfloat16>(C_rows, A, B, M, N, K, lc, la, lb, row_begin, row_end, threads); break;
        default: break;
    }
}

// calculate_cosine_similarity of test/test.hpp.  kind: 0 f16, 1 f32, 2 bf16.
float ref_cosine_similarity(const void* gpu, const void* cpu, size_t M, size_t N, int layout, int kind)
{
    if (kind == 1) return cosine_one<float>(gpu, cpu, M, N, layout);
    if (kind == 2) return cosine_one<__hip_bfloat16>(gpu, cpu, M, N, layout);
    return cosine_one<half>(gpu, cpu, M, N, layout);
}

unsigned ref_hardware_threads(void) { return std::thread::hardware_concurrency(); }

} // extern "C"
