// C++ front-end test: drives the library the way the reference's typed tests do
// (test/gemm/test_float_accum.cpp:80-142, test/gemm/test_same_prec.cpp) — host matrices from
// the seeded generator, device copies, `loader().gemm<C, A, B>(...)` on a stream, CPU GEMM,
// compare — once through the dlopen()ing `rocm_wmma_gemm::loader` and once through the
// header-inline `rocm_wmma_gemm::gemm<>`.  The CPU side is the oracle's C restatement
// (oracle/cpu_gemm.c), linked into this test only.
//
// Exit code 0 = all checks passed; prints one line per failed case.
#include <rocm_wmma_gemm/gemm.hpp>
#include <rocm_wmma_gemm/kernel_loader.hpp>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

extern "C" {
void  oracle_init_matrix(uint16_t* data, size_t rows, size_t cols, int layout, int bf16);
int   oracle_hgemm(int types, void* C, const uint16_t* A, const uint16_t* B, size_t M, size_t N, size_t K, int lc,
                   int la, int lb, int threads);
float oracle_cosine_similarity(const void* gpu, const void* cpu, size_t M, size_t N, int layout, int kind);
float oracle_f16_to_f32(uint16_t h);
float oracle_bf16_to_f32(uint16_t h);
}

using rocm_wmma_gemm::m_layout;

#define CUDA_OK(x)                                                                \
    do {                                                                          \
        cudaError_t e_ = (x);                                                     \
        if (e_ != cudaSuccess) {                                                  \
            std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));         \
            std::exit(2);                                                         \
        }                                                                         \
    } while (0)

static rocm_wmma_gemm::loader& wmma_loader()
{
    static rocm_wmma_gemm::loader l;
    return l;
}

static int g_failed = 0, g_cases = 0;

template <class T>
struct type_info;
template <>
struct type_info<half> {
    static constexpr int kind = 0;
};
template <>
struct type_info<float> {
    static constexpr int kind = 1;
};
template <>
struct type_info<__hip_bfloat16> {
    static constexpr int kind = 2;
};

template <class T, class U, m_layout LC, m_layout LA, m_layout LB>
void verify(size_t M, size_t N, size_t K, bool use_loader, hipStream_t& stream)
{
    constexpr int  types = rocm_wmma_gemm::detail::type_index<T, U>();
    constexpr bool bf16  = std::is_same_v<U, __hip_bfloat16>;
    constexpr int  lc = static_cast<int>(LC), la = static_cast<int>(LA), lb = static_cast<int>(LB);
    std::vector<uint16_t> hA(M * K), hB(K * N);
    oracle_init_matrix(hA.data(), M, K, la, bf16);
    oracle_init_matrix(hB.data(), K, N, lb, bf16);
    std::vector<T> hC(M * N), hRef(M * N);

    U *dA, *dB;
    T* dC;
    CUDA_OK(cudaMalloc((void**)&dA, hA.size() * 2));
    CUDA_OK(cudaMalloc((void**)&dB, hB.size() * 2));
    CUDA_OK(cudaMalloc((void**)&dC, hC.size() * sizeof(T)));
    CUDA_OK(cudaMemcpy(dA, hA.data(), hA.size() * 2, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dB, hB.data(), hB.size() * 2, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemset(dC, 0xFF, hC.size() * sizeof(T)));

    if (use_loader) wmma_loader().gemm<LC, LA, LB>(dC, dA, dB, M, N, K, stream);
    else rocm_wmma_gemm::gemm<LC, LA, LB>(dC, dA, dB, M, N, K, stream);
    CUDA_OK(cudaPeekAtLastError());
    CUDA_OK(cudaDeviceSynchronize());
    CUDA_OK(cudaMemcpy(hC.data(), dC, hC.size() * sizeof(T), cudaMemcpyDeviceToHost));

    oracle_hgemm(types, hRef.data(), hA.data(), hB.data(), M, N, K, lc, la, lb, 8);

    bool ok = true;
    if constexpr (std::is_same_v<T, float>) {
        // the reference's own bar: every element within 1e-4 (test_float_accum.cpp:128-136)
        for (size_t i = 0; i < hC.size() && ok; ++i) ok = std::fabs(hC[i] - hRef[i]) <= 1e-4f;
    } else {
        // the reference's own bar: cosine similarity (test/test.hpp:199-215)
        const float cs = oracle_cosine_similarity(hC.data(), hRef.data(), M, N, lc, type_info<T>::kind);
        ok             = cs > (bf16 ? 0.97f : 0.995f);
        // and, tighter: every element within 2 output ulps of the CPU value
        const uint16_t* g = reinterpret_cast<const uint16_t*>(hC.data());
        const uint16_t* r = reinterpret_cast<const uint16_t*>(hRef.data());
        for (size_t i = 0; i < hC.size() && ok; ++i) {
            const float gv = bf16 ? oracle_bf16_to_f32(g[i]) : oracle_f16_to_f32(g[i]);
            const float rv = bf16 ? oracle_bf16_to_f32(r[i]) : oracle_f16_to_f32(r[i]);
            const float eps = bf16 ? 0.0078125f : 0.0009765625f;
            ok              = std::fabs(gv - rv) <= 2.f * eps * std::fabs(rv) + eps * 0.34f * std::sqrt((float)K);
        }
    }
    ++g_cases;
    if (!ok) {
        ++g_failed;
        std::printf("FAILED types=%d C=%d A=%d B=%d %zux%zux%zu via %s\n", types, lc, la, lb, M, N, K,
                    use_loader ? "loader" : "gemm<>");
    }
    cudaFree(dA);
    cudaFree(dB);
    cudaFree(dC);
}

template <class T, class U, m_layout LC, m_layout LA, m_layout LB>
void shapes(hipStream_t& stream)
{
    // a subset of the reference's 13 shapes, aligned and unaligned to the tile
    const size_t s[][3] = {{128, 128, 128}, {256, 128, 128}, {320, 320, 320}, {512, 320, 512}, {256, 1024, 256}};
    for (auto& d : s) {
        verify<T, U, LC, LA, LB>(d[0], d[1], d[2], true, stream);
        verify<T, U, LC, LA, LB>(d[0], d[1], d[2], false, stream);
    }
}

template <class T, class U>
void layouts(hipStream_t& stream)
{
    constexpr m_layout R = m_layout::row_major, C = m_layout::col_major;
    shapes<T, U, R, R, R>(stream);
    shapes<T, U, R, R, C>(stream);
    shapes<T, U, R, C, R>(stream);
    shapes<T, U, R, C, C>(stream);
    shapes<T, U, C, R, R>(stream);
    shapes<T, U, C, R, C>(stream);
    shapes<T, U, C, C, R>(stream);
    shapes<T, U, C, C, C>(stream);
}

int main()
{
    hipStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));
    layouts<half, half>(stream);
    layouts<float, half>(stream);
    layouts<__hip_bfloat16, __hip_bfloat16>(stream);
    layouts<float, __hip_bfloat16>(stream);

    // batched overload
    {
        const size_t          M = 128, N = 256, K = 192, batch = 3;
        std::vector<uint16_t> hA(M * K * batch), hB(K * N * batch);
        for (size_t b = 0; b < batch; ++b) {
            oracle_init_matrix(hA.data() + b * M * K, M, K, 0, 0);
            oracle_init_matrix(hB.data() + b * K * N, K, N, 1, 0);
            hA[b * M * K] = static_cast<uint16_t>(0x3C00 + b); // make the batches differ
        }
        half * dA, *dB;
        float* dC;
        CUDA_OK(cudaMalloc((void**)&dA, hA.size() * 2));
        CUDA_OK(cudaMalloc((void**)&dB, hB.size() * 2));
        CUDA_OK(cudaMalloc((void**)&dC, M * N * batch * 4));
        CUDA_OK(cudaMemcpy(dA, hA.data(), hA.size() * 2, cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(dB, hB.data(), hB.size() * 2, cudaMemcpyHostToDevice));
        wmma_loader().gemm<m_layout::row_major, m_layout::row_major, m_layout::col_major>(dC, dA, dB, M, N, K, batch, stream);
        CUDA_OK(cudaDeviceSynchronize());
        std::vector<float> hC(M * N * batch), ref(M * N);
        CUDA_OK(cudaMemcpy(hC.data(), dC, hC.size() * 4, cudaMemcpyDeviceToHost));
        for (size_t b = 0; b < batch; ++b) {
            oracle_hgemm(1, ref.data(), hA.data() + b * M * K, hB.data() + b * K * N, M, N, K, 0, 0, 1, 4);
            bool ok = true;
            for (size_t i = 0; i < M * N && ok; ++i) ok = std::fabs(hC[b * M * N + i] - ref[i]) <= 1e-4f;
            ++g_cases;
            if (!ok) {
                ++g_failed;
                std::printf("FAILED batched b=%zu\n", b);
            }
        }
    }

    // error behaviour of the C++ template: a bad size throws
    {
        bool  threw = false;
        float dummy;
        try {
            rocm_wmma_gemm::gemm<m_layout::row_major, m_layout::row_major, m_layout::row_major>(
                &dummy, (half*)nullptr, (half*)nullptr, 8, 8, 8, stream);
        } catch (const std::runtime_error&) {
            threw = true;
        }
        ++g_cases;
        if (!threw) {
            ++g_failed;
            std::printf("FAILED: NULL operand did not throw\n");
        }
        const rocm_wmma_gemm::gemm_params p = rocm_wmma_gemm::get_gemm_params(8192, 8192, 8192, m_layout::row_major,
                                                                             m_layout::row_major, m_layout::col_major);
        ++g_cases;
        if (p.tile_m != 128 * p.cluster) {
            ++g_failed;
            std::printf("FAILED: get_gemm_params returned an inconsistent config\n");
        }
    }
    std::printf("%d cases, %d failed\n", g_cases, g_failed);
    return g_failed ? 1 : 0;
}
