// tuner — times ONE launch configuration of the B200 GEMM from the command line.
//
//   tuner M N K tile_m tile_n stages cluster split_k raster layout_a layout_b layout_c [arch] [type]
//
// Counterpart of the reference's rocm_wmma_gemm/config/tuner.cpp:458-508 (which compiles one
// kernel instantiation with hipRTC and times it): here every variant is precompiled, so the
// binary only selects one through b200_gemm_ex.  Inputs are seeded normal(0, 1) values, not
// the reference tuner's five-value cyclic fill (tuner.cpp:107-122): on a power-capped B200
// the clock a large GEMM settles at depends on how many operand bits toggle, and a
// low-entropy fill ranks tile shapes differently from real data.  Prints one parseable line
//     dynamic_kernel/manual_time <ms> ms  <TFLOP/s> TFLOP/s
// and exits non-zero when the configuration is invalid or the launch fails.
//
// Build: g++ -O2 -std=c++17 -I<repo>/include tuner.cpp -o tuner -L<pkg> -lrocm_wmma_gemm_sm100a
//        -L/usr/local/cuda/lib64 -lcudart   (rocm_wmma_gemm_b200/config/build_tuner.sh)
#include <b200_gemm.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#define CHECK(x)                                                                      \
    do {                                                                              \
        cudaError_t e_ = (x);                                                         \
        if (e_ != cudaSuccess) {                                                      \
            std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));             \
            return 2;                                                                 \
        }                                                                             \
    } while (0)

template <class T>
static std::vector<T> random_normal(size_t n, unsigned seed)
{
    std::mt19937                    gen(seed);
    std::normal_distribution<float> dist(0.f, 1.f);
    // 4096 draws repeated with a stride co-prime to every tile extent: as random as the
    // kernel can tell, and filling gigabytes stays cheap
    std::vector<float> pool(4099);
    for (float& x : pool) x = dist(gen);
    std::vector<T> out(n);
    for (size_t i = 0; i < n; ++i) out[i] = T(pool[i % pool.size()]);
    return out;
}

int main(int argc, char** argv)
{
    if (argc < 13) {
        std::fprintf(stderr,
                     "usage: %s M N K tile_m tile_n stages cluster split_k raster layout_a layout_b layout_c [arch] [type]\n"
                     "  layouts: 0 = row_major, 1 = col_major; type: f16_f16 | f32_f16 | bf16_bf16 | f32_bf16\n",
                     argv[0]);
        return 1;
    }
    const size_t     M = std::strtoull(argv[1], nullptr, 10), N = std::strtoull(argv[2], nullptr, 10),
                 K = std::strtoull(argv[3], nullptr, 10);
    b200_gemm_config cfg{std::atoi(argv[4]), std::atoi(argv[5]), std::atoi(argv[6]),
                         std::atoi(argv[7]), std::atoi(argv[8]), std::atoi(argv[9])};
    const int         la = std::atoi(argv[10]), lb = std::atoi(argv[11]), lc = std::atoi(argv[12]);
    const std::string type = argc > 14 ? argv[14] : "f16_f16";
    int               types;
    if (type == "f16_f16") types = B200_GEMM_F16_F16;
    else if (type == "f32_f16") types = B200_GEMM_F32_F16;
    else if (type == "bf16_bf16") types = B200_GEMM_BF16_BF16;
    else if (type == "f32_bf16") types = B200_GEMM_F32_BF16;
    else {
        std::fprintf(stderr, "unknown type %s\n", type.c_str());
        return 1;
    }
    const bool   bf16   = types >= 2;
    const size_t out_sz = (types == 1 || types == 3) ? 4 : 2;

    void *dA, *dB, *dC;
    CHECK(cudaMalloc(&dA, M * K * 2));
    CHECK(cudaMalloc(&dB, K * N * 2));
    CHECK(cudaMalloc(&dC, M * N * out_sz));
    if (bf16) {
        auto a = random_normal<__nv_bfloat16>(M * K, 1234), b = random_normal<__nv_bfloat16>(K * N, 4321);
        CHECK(cudaMemcpy(dA, a.data(), M * K * 2, cudaMemcpyHostToDevice));
        CHECK(cudaMemcpy(dB, b.data(), K * N * 2, cudaMemcpyHostToDevice));
    } else {
        auto a = random_normal<__half>(M * K, 1234), b = random_normal<__half>(K * N, 4321);
        CHECK(cudaMemcpy(dA, a.data(), M * K * 2, cudaMemcpyHostToDevice));
        CHECK(cudaMemcpy(dB, b.data(), K * N * 2, cudaMemcpyHostToDevice));
    }
    cudaStream_t stream;
    CHECK(cudaStreamCreate(&stream));
    cudaEvent_t e0, e1;
    CHECK(cudaEventCreate(&e0));
    CHECK(cudaEventCreate(&e1));

    auto run = [&]() { return b200_gemm_ex(types, dC, dA, dB, M, N, K, 1, lc, la, lb, &stream, &cfg); };
    for (int i = 0; i < 3; ++i) {
        if (int st = run()) {
            std::fprintf(stderr, "b200_gemm_ex failed (%d): %s\n", st, b200_gemm_last_error());
            return 3;
        }
    }
    CHECK(cudaStreamSynchronize(stream));
    std::vector<float> ms;
    for (int rep = 0; rep < 10; ++rep) {
        CHECK(cudaEventRecord(e0, stream));
        if (run()) return 3;
        CHECK(cudaEventRecord(e1, stream));
        CHECK(cudaEventSynchronize(e1));
        float t = 0.f;
        CHECK(cudaEventElapsedTime(&t, e0, e1));
        ms.push_back(t);
    }
    unsigned int word = 0;
    if (b200_gemm_device_status(&word) != B200_GEMM_OK) {
        std::fprintf(stderr, "device status 0x%x: %s\n", word, b200_gemm_last_error());
        return 4;
    }
    std::sort(ms.begin(), ms.end());
    const double med = ms[ms.size() / 2];
    std::printf("dynamic_kernel/manual_time %.5f ms  %.1f TFLOP/s  (min %.5f max %.5f, %zux%zux%zu %s)\n", med,
                2.0 * M * N * K / (med * 1e-3) / 1e12, ms.front(), ms.back(), M, N, K, type.c_str());
    cudaFree(dA);
    cudaFree(dB);
    cudaFree(dC);
    return 0;
}
