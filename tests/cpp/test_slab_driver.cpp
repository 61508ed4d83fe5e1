// The multi-GPU column-slab driver from plain C++ (no Python, no MPI): one host thread per GPU
// of this process acts as a rank.  Each rank creates its communicator from an id shared in
// memory, computes its slab of C = A * B with the gather fused into the GEMM
// (b200_gemm_slab_gather: every tile stored into every GPU's copy of C; inside one process the
// copies are plain cudaMalloc pointers with peer access enabled), and - as the second route -
// with the ordinary slab call followed by the NCCL all-gather (b200_gemm_slab_allgather).  Every
// rank then compares its full C with the CPU reference GEMM (the oracle's C restatement, linked
// into this test only).  Exit code 0 = every rank agreed; 77 = fewer than two GPUs.
#include <b200_gemm.h>
#include <cuda_runtime_api.h>

#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

extern "C" {
void  oracle_init_matrix(uint16_t* data, size_t rows, size_t cols, int layout, int bf16);
int   oracle_hgemm(int types, void* C, const uint16_t* A, const uint16_t* B, size_t M, size_t N, size_t K, int lc,
                   int la, int lb, int threads);
}

#define CUDA_OK(x)                                                        \
    do {                                                                  \
        cudaError_t e_ = (x);                                             \
        if (e_ != cudaSuccess) {                                          \
            std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); \
            std::exit(2);                                                 \
        }                                                                 \
    } while (0)
#define GEMM_OK(x)                                                              \
    do {                                                                        \
        int s_ = (x);                                                           \
        if (s_ != B200_GEMM_OK) {                                               \
            std::fprintf(stderr, "%s: status %d: %s\n", #x, s_, b200_gemm_last_error()); \
            std::exit(3);                                                       \
        }                                                                       \
    } while (0)

namespace {

struct Barrier { // all ranks of this process
    explicit Barrier(int n) : n_(n) {}
    void wait()
    {
        const int gen = gen_.load();
        if (count_.fetch_add(1) + 1 == n_) {
            count_.store(0);
            gen_.fetch_add(1);
        } else {
            while (gen_.load() == gen) std::this_thread::yield();
        }
    }
    int              n_;
    std::atomic<int> count_{0}, gen_{0};
};

constexpr size_t M = 512, N = 2048, K = 384; // f32 <- bf16, A row / B col / C row
constexpr int    TYPES = B200_GEMM_F32_BF16, LC = 0, LA = 0, LB = 1;

} // namespace

int main()
{
    int devices = 0;
    CUDA_OK(cudaGetDeviceCount(&devices));
    if (devices < 2) {
        std::printf("needs two GPUs, found %d\n", devices);
        return 77;
    }
    const int world = devices >= 4 ? 4 : 2;
    std::vector<uint16_t> hA(M * K), hB(K * N);
    oracle_init_matrix(hA.data(), M, K, LA, 1);
    oracle_init_matrix(hB.data(), K, N, LB, 1);
    std::vector<float> ref(M * N);
    oracle_hgemm(TYPES, ref.data(), hA.data(), hB.data(), M, N, K, LC, LA, LB, 8);

    char id[B200_GEMM_COMM_ID_BYTES];
    GEMM_OK(b200_gemm_comm_id(id));
    std::vector<void*>       full(world, nullptr); // every rank's copy of C, visible to all threads
    std::vector<int>         bad(world, 0);
    Barrier                  barrier(world);
    std::vector<std::thread> ranks;
    for (int r = 0; r < world; ++r) {
        ranks.emplace_back([&, r] {
            CUDA_OK(cudaSetDevice(r));
            for (int p = 0; p < world; ++p)
                if (p != r) {
                    cudaError_t e = cudaDeviceEnablePeerAccess(p, 0);
                    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) CUDA_OK(e);
                    (void)cudaGetLastError();
                }
            cudaStream_t stream;
            CUDA_OK(cudaStreamCreate(&stream));
            size_t n0 = 0, nc = 0;
            GEMM_OK(b200_gemm_slab(N, world, r, 256, &n0, &nc));
            void *dA, *dB, *dSlab, *dStage, *dFull2;
            CUDA_OK(cudaMalloc(&dA, M * K * 2));
            CUDA_OK(cudaMalloc(&dB, K * nc * 2));
            CUDA_OK(cudaMalloc(&dSlab, M * nc * 4));
            CUDA_OK(cudaMalloc(&dStage, M * N * 4));
            CUDA_OK(cudaMalloc(&dFull2, M * N * 4));
            CUDA_OK(cudaMalloc(&full[r], M * N * 4));
            CUDA_OK(cudaMemset(full[r], 0xFF, M * N * 4));
            CUDA_OK(cudaMemcpy(dA, hA.data(), M * K * 2, cudaMemcpyHostToDevice));
            // column-major B: the slab is the contiguous block of columns [n0, n0 + nc)
            CUDA_OK(cudaMemcpy(dB, hB.data() + n0 * K, K * nc * 2, cudaMemcpyHostToDevice));
            b200_gemm_comm* comm = nullptr;
            GEMM_OK(b200_gemm_comm_create(id, world, r, &comm));
            barrier.wait(); // every rank's buffer exists

            // route 1: GEMM + gather in one kernel, then a barrier on the stream
            GEMM_OK(b200_gemm_slab_gather(TYPES, full.data(), dA, dB, M, N, K, LC, LA, LB, world, r, 256, &stream, nullptr));
            GEMM_OK(b200_gemm_comm_barrier(comm, &stream));
            CUDA_OK(cudaStreamSynchronize(stream));
            // route 2: the ordinary slab call, then the NCCL all-gather (+ re-layout for row-major C)
            GEMM_OK(b200_gemm_f32_bf16(dSlab, dA, dB, M, nc, K, 1, LC, LA, LB, &stream));
            GEMM_OK(b200_gemm_slab_allgather(comm, TYPES, dFull2, dSlab, dStage, M, N, LC, 256, &stream));
            CUDA_OK(cudaStreamSynchronize(stream));
            GEMM_OK(b200_gemm_device_status(nullptr));

            std::vector<float> got(M * N), got2(M * N);
            CUDA_OK(cudaMemcpy(got.data(), full[r], M * N * 4, cudaMemcpyDeviceToHost));
            CUDA_OK(cudaMemcpy(got2.data(), dFull2, M * N * 4, cudaMemcpyDeviceToHost));
            for (size_t i = 0; i < M * N; ++i) {
                if (!(std::fabs(got[i] - ref[i]) <= 1e-4f)) ++bad[r];   // the reference test's own tolerance
                if (!(std::fabs(got2[i] - ref[i]) <= 1e-4f)) ++bad[r];
            }
            barrier.wait(); // nobody frees a buffer a peer may still be writing
            GEMM_OK(b200_gemm_comm_destroy(comm));
            for (void* p : {dA, dB, dSlab, dStage, dFull2, full[r]}) cudaFree(p);
            cudaStreamDestroy(stream);
        });
    }
    for (auto& t : ranks) t.join();
    int failed = 0;
    for (int r = 0; r < world; ++r) {
        if (bad[r]) std::printf("rank %d: %d elements differ from the CPU reference\n", r, bad[r]);
        failed += bad[r] != 0;
    }
    std::printf("%d ranks, %d failed\n", world, failed);
    return failed ? 1 : 0;
}
