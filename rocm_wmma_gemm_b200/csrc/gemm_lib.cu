// Host side of the B200 GEMM library: argument validation, the layout -> kernel-view mapping,
// tuned-config selection, TMA descriptor construction, kernel launch, and the C ABI declared
// in include/b200_gemm.h.  Replaces the reference's host path
//   rocm_wmma_gemm/src/gemm.cpp:8-53, :207-250           (gemm<> and the C dispatchers)
//   rocm_wmma_gemm/include/rocm_wmma_gemm/kernel_launcher.hpp:45-131   (index math + launch)
//   generated config_generated.hpp (rocm_wmma_gemm/config/generate_config.py:94-303)
// There is no CPU fallback: without a CUDA device every compute entry point fails.
#include "../../include/b200_gemm.h"
#include "gemm_kernels.cuh"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <mutex>
#include <vector>

namespace b200 {

// ------------------------------------------------------------------------------------------
// Errors
// ------------------------------------------------------------------------------------------
static thread_local int  t_last_status = B200_GEMM_OK;
static thread_local char t_last_error[512] = "";

static int fail(int status, const char* fmt, ...)
{
    t_last_status = status;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_last_error, sizeof(t_last_error), fmt, ap);
    va_end(ap);
    return status;
}

#define CUDA_TRY(expr)                                                                         \
    do {                                                                                       \
        cudaError_t e_ = (expr);                                                               \
        if (e_ != cudaSuccess)                                                                 \
            return fail(B200_GEMM_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_));   \
    } while (0)

static std::atomic<unsigned long long> g_launches{0};

// ------------------------------------------------------------------------------------------
// Tuned configuration table (generated from config/gemm_config_sm100_*.json)
// ------------------------------------------------------------------------------------------
struct ConfigEntry {
    uint32_t m, n, k;
    uint8_t  type_group; // 0: 16-bit output, 1: f32 output
    uint8_t  la, lb, lc; // 0 row-major, 1 column-major
    uint16_t cfg;        // index into k_configs
};

#include "config_table.inc"

static constexpr int k_num_configs = sizeof(k_configs) / sizeof(k_configs[0]);
static constexpr int k_num_entries = sizeof(k_entries) / sizeof(k_entries[0]) - 1; // sentinel

static bool entry_less(const ConfigEntry& a, const ConfigEntry& b)
{
    if (a.m != b.m) return a.m < b.m;
    if (a.n != b.n) return a.n < b.n;
    if (a.k != b.k) return a.k < b.k;
    if (a.type_group != b.type_group) return a.type_group < b.type_group;
    if (a.la != b.la) return a.la < b.la;
    if (a.lb != b.lb) return a.lb < b.lb;
    return a.lc < b.lc;
}

// Exact lookup by binary search over the sorted entry list; -1 when absent.
static int search_exact(size_t m, size_t n, size_t k, int tg, int la, int lb, int lc)
{
    if (m > UINT32_MAX || n > UINT32_MAX || k > UINT32_MAX) return -1;
    const ConfigEntry key{(uint32_t)m, (uint32_t)n, (uint32_t)k, (uint8_t)tg,
                          (uint8_t)la, (uint8_t)lb, (uint8_t)lc, 0};
    int lo = 0, hi = k_num_entries;
    while (lo < hi) {
        const int mid = (lo + hi) / 2;
        if (entry_less(k_entries[mid], key)) lo = mid + 1;
        else hi = mid;
    }
    if (lo < k_num_entries && !entry_less(key, k_entries[lo]) && !entry_less(k_entries[lo], key))
        return k_entries[lo].cfg;
    return -1;
}

// Closest entry of one type group within the same layout triple: nearest K first, then the
// nearest (M, N) in the Euclidean sense among entries with that K; -1 when the group has no
// entry for the layout triple.
static int search_closest(size_t m, size_t n, size_t k, int tg, int la, int lb, int lc)
{
    bool     found      = false;
    uint64_t best_kdiff = std::numeric_limits<uint64_t>::max();
    uint32_t closest_k  = 0;
    for (int i = 0; i < k_num_entries; ++i) {
        const ConfigEntry& e = k_entries[i];
        if (e.type_group != tg || e.la != la || e.lb != lb || e.lc != lc) continue;
        found               = true;
        const uint64_t diff = e.k > k ? e.k - k : k - e.k;
        if (diff < best_kdiff) {
            best_kdiff = diff;
            closest_k  = e.k;
        }
    }
    if (!found) return -1;
    double best_d = std::numeric_limits<double>::max();
    int    best   = -1;
    for (int i = 0; i < k_num_entries; ++i) {
        const ConfigEntry& e = k_entries[i];
        if (e.type_group != tg || e.k != closest_k || e.la != la || e.lb != lb || e.lc != lc)
            continue;
        const double dm = (double)m - (double)e.m, dn = (double)n - (double)e.n;
        const double d  = dm * dm + dn * dn;
        if (d < best_d) {
            best_d = d;
            best   = e.cfg;
        }
    }
    return best;
}

// Selection order of the reference's find_best_config
// (rocm_wmma_gemm/config/generate_config.py:238-271): exact in the requested type group,
// exact in group 0, closest in the requested group, closest in group 0, default.
static int find_best_config(size_t m, size_t n, size_t k, int tg, int la, int lb, int lc, bool* exact = nullptr)
{
    if (exact) *exact = true;
    int r = search_exact(m, n, k, tg, la, lb, lc);
    if (r >= 0) return r;
    if (tg != 0) {
        r = search_exact(m, n, k, 0, la, lb, lc);
        if (r >= 0) return r;
    }
    if (exact) *exact = false;
    r = search_closest(m, n, k, tg, la, lb, lc);
    if (r < 0 && tg != 0) r = search_closest(m, n, k, 0, la, lb, lc);
    if (r < 0) r = k_default_config;
    return r;
}

// ------------------------------------------------------------------------------------------
// Per-device context
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Co-resident CTA pairs of the three pair kernels (tile_n 128 / 256 / 512), as the occupancy
// query answered for the dynamic shared memory size it was asked with (0 = not asked yet).
struct PairCache {
    int      units[3] = {0, 0, 0};
    uint32_t smem[3]  = {0, 0, 0};
};

struct DeviceCtx {
    std::atomic<bool> ready{false}; // set last, read first: initialised contexts skip the lock
    int           sm_count = 0;
    PairCache     pairs;
    unsigned int* d_status = nullptr;
    // split-K workspaces, one per stream that has used split-K (calls on one stream are ordered,
    // so they can share a buffer; calls on different streams must not - and two host threads
    // must not issue calls on the same stream at the same time)
    struct Workspace {
        cudaStream_t stream;
        float*       ptr;
        size_t       bytes;
    };
    std::vector<Workspace> workspaces;
    // buffers a workspace has outgrown: freed once the work that was queued on them has drained
    struct Retired {
        float*      ptr;
        cudaEvent_t drained;
    };
    std::vector<Retired> retired;
    std::mutex           ws_mutex;   // guards workspaces / retired
    std::mutex           host_mutex; // held for the whole of a host-buffer call
    // host-buffer path: compute stream, copy-in / copy-out streams and the events chaining them
    cudaStream_t h_in = nullptr, h_out = nullptr;
    cudaEvent_t  h_ev_a[16] = {}, h_ev_b[16] = {}, h_ev_done[256] = {};
    cudaStream_t h_stream = nullptr;
    void*        h_buf[3] = {nullptr, nullptr, nullptr};
    size_t       h_cap[3] = {0, 0, 0};
};

static constexpr int k_max_devices = 64;
static DeviceCtx     g_ctx[k_max_devices];
static std::mutex    g_mutex;
static EncodeTiledFn g_encode = nullptr;

template <int BN, int OUT, int CL>
static cudaError_t set_smem_attr_one()
{
    cudaError_t e = cudaFuncSetAttribute(gemm_umma_kernel<BN, OUT, CL>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)gemm_smem_bytes(BN, CL, max_stages(BN, CL)));
    if (e == cudaSuccess && CL == 2)
        e = cudaFuncSetAttribute(gemm_umma_kernel<BN, OUT, CL>,
                                 cudaFuncAttributeNonPortableClusterSizeAllowed, 0);
    if constexpr (CL == 2 && BN >= 256) {
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_umma_gather_kernel<BN, OUT, CL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)gemm_smem_bytes(BN, CL, max_stages(BN, CL)));
    }
    if constexpr (CL == 1 && BN >= 128 && BN <= 256) {
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_umma_ksplit_kernel<BN, OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)gemm_smem_bytes(BN, CL, max_stages(BN, CL)));
    }
    return e;
}

template <int BN, int CL>
static cudaError_t set_smem_attr()
{
    cudaError_t e = set_smem_attr_one<BN, OUT_F32, CL>();
    if (e == cudaSuccess) e = set_smem_attr_one<BN, OUT_F16, CL>();
    if (e == cudaSuccess) e = set_smem_attr_one<BN, OUT_BF16, CL>();
    return e;
}

// Narrow one-CTA variants (BN <= 128) with the staged or the transposed epilogue.
template <int BN, int OUT>
static cudaError_t set_smem_attr_narrow_one()
{
    cudaError_t e = cudaFuncSetAttribute(gemm_umma_kernel<BN, OUT, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)SLAB_SMEM_LIMIT);
    if (e == cudaSuccess && BN < 64)
        e = cudaFuncSetAttribute(gemm_umma_kernel<BN, OUT, 1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)gemm_smem_bytes(BN, 1, max_stages(BN, 1, false), false));
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_umma_ksplit_kernel<BN, OUT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)SLAB_SMEM_LIMIT);
    return e;
}

template <int BN>
static cudaError_t set_smem_attr_narrow()
{
    cudaError_t e = set_smem_attr_narrow_one<BN, OUT_F32>();
    if (e == cudaSuccess) e = set_smem_attr_narrow_one<BN, OUT_F16>();
    if (e == cudaSuccess) e = set_smem_attr_narrow_one<BN, OUT_BF16>();
    return e;
}

// Opt every compiled GEMM kernel in to the dynamic shared memory it may be launched with.
static cudaError_t set_all_kernel_attributes()
{
    cudaError_t e = set_smem_attr<64, 1>();
    if (e == cudaSuccess) e = set_smem_attr<128, 1>();
    if (e == cudaSuccess) e = set_smem_attr<256, 1>();
    if (e == cudaSuccess) e = set_smem_attr<128, 2>();
    if (e == cudaSuccess) e = set_smem_attr<256, 2>();
    if (e == cudaSuccess) e = set_smem_attr<512, 2>();
    if (e == cudaSuccess) e = set_smem_attr_narrow<16>();
    if (e == cudaSuccess) e = set_smem_attr_narrow<32>();
    if (e == cudaSuccess) e = set_smem_attr_narrow<64>();
    if (e == cudaSuccess) e = set_smem_attr_narrow<128>();
    return e;
}

static int get_ctx(DeviceCtx** out)
{
    int         dev = -1;
    cudaError_t e   = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return fail(B200_GEMM_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= k_max_devices)
        return fail(B200_GEMM_ERR_NO_DEVICE, "device ordinal %d out of range", dev);
    DeviceCtx& c = g_ctx[dev];
    if (c.ready.load(std::memory_order_acquire)) {
        *out = &c;
        return B200_GEMM_OK;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!c.ready.load(std::memory_order_relaxed)) {
        cudaDeviceProp prop;
        CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
        if (prop.major != 10)
            return fail(B200_GEMM_ERR_NO_DEVICE,
                        "device %d is sm_%d%d; this library is built for sm_100a only", dev,
                        prop.major, prop.minor);
        c.sm_count = prop.multiProcessorCount;
        if (!g_encode) {
            void*                           fn = nullptr;
            cudaDriverEntryPointQueryResult qr;
            CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr));
            if (!fn || qr != cudaDriverEntryPointSuccess)
                return fail(B200_GEMM_ERR_CUDA, "cuTensorMapEncodeTiled not available");
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
        }
        CUDA_TRY(cudaMalloc(&c.d_status, sizeof(unsigned int)));
        CUDA_TRY(cudaMemset(c.d_status, 0, sizeof(unsigned int)));
        CUDA_TRY(set_all_kernel_attributes());
        c.ready.store(true, std::memory_order_release);
    }
    *out = &c;
    return B200_GEMM_OK;
}

// Split-K workspace of at least `bytes` for `stream`: cached per stream and grown on demand, so
// the steady state allocates nothing (an allocation per call costs more than a skinny GEMM).
// A buffer that has become too small is not freed here - kernels queued on the stream may still
// use it - but retired behind an event and freed by a later call once that event has passed.
static int get_workspace(DeviceCtx* ctx, cudaStream_t stream, size_t bytes, float** out)
{
    std::lock_guard<std::mutex> lock(ctx->ws_mutex);
    for (size_t i = 0; i < ctx->retired.size();) {
        if (cudaEventQuery(ctx->retired[i].drained) == cudaSuccess) {
            cudaFree(ctx->retired[i].ptr);
            cudaEventDestroy(ctx->retired[i].drained);
            ctx->retired[i] = ctx->retired.back();
            ctx->retired.pop_back();
        } else {
            (void)cudaGetLastError(); // cudaErrorNotReady is not an error of ours
            ++i;
        }
    }
    for (auto& w : ctx->workspaces) {
        if (w.stream != stream) continue;
        if (w.bytes < bytes) {
            const size_t want  = bytes + bytes / 4;
            float*       fresh = nullptr;
            CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&fresh), want));
            DeviceCtx::Retired r{w.ptr, nullptr};
            if (cudaEventCreateWithFlags(&r.drained, cudaEventDisableTiming) == cudaSuccess &&
                cudaEventRecord(r.drained, stream) == cudaSuccess) {
                ctx->retired.push_back(r);
            } else { // no event to wait behind: drain the stream, then free
                (void)cudaGetLastError();
                if (r.drained) cudaEventDestroy(r.drained);
                cudaStreamSynchronize(stream);
                cudaFree(w.ptr);
            }
            w.ptr   = fresh;
            w.bytes = want;
        }
        *out = w.ptr;
        return B200_GEMM_OK;
    }
    DeviceCtx::Workspace w{stream, nullptr, 0};
    CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&w.ptr), bytes));
    w.bytes = bytes;
    ctx->workspaces.push_back(w);
    *out = w.ptr;
    return B200_GEMM_OK;
}

// ------------------------------------------------------------------------------------------
// Problem description
// ------------------------------------------------------------------------------------------
struct Problem {
    int         types; // b200_gemm_types
    void*       C;
    const void* A;
    const void* B;
    size_t      M, N, K, batch;
    int         lc, la, lb;
};

// Kernel view: D (Mk x Nk row-major) = A' (Mk x K) * B' (K x Nk).
struct View {
    const void* a;
    const void* b;
    void*       d;
    uint32_t    M, N, K;
    bool        a_mn, b_mn;
};

static View make_view(const Problem& p)
{
    View v;
    v.K = (uint32_t)p.K;
    if (p.lc == 0) {
        v.a    = p.A;
        v.b    = p.B;
        v.M    = (uint32_t)p.M;
        v.N    = (uint32_t)p.N;
        v.a_mn = (p.la == 1); // column-major A: M contiguous
        v.b_mn = (p.lb == 0); // row-major B: N contiguous
    } else {
        // Column-major C (M x N) is the row-major C^T (N x M) = B^T * A^T.
        v.a    = p.B;
        v.b    = p.A;
        v.M    = (uint32_t)p.N;
        v.N    = (uint32_t)p.M;
        v.a_mn = (p.lb == 0); // B^T of a row-major B has its "M" (= N) extent contiguous
        v.b_mn = (p.la == 1); // A^T of a column-major A has its "N" (= M) extent contiguous
    }
    v.d = p.C;
    return v;
}

static inline bool out_is_f32(int types) { return types == B200_GEMM_F32_F16 || types == B200_GEMM_F32_BF16; }
static inline bool in_is_bf16(int types) { return types == B200_GEMM_BF16_BF16 || types == B200_GEMM_F32_BF16; }
static inline int  out_kind(int types)
{
    return out_is_f32(types) ? OUT_F32 : (types == B200_GEMM_F16_F16 ? OUT_F16 : OUT_BF16);
}

static int validate(const Problem& p)
{
    if (p.types < 0 || p.types > 3) return fail(B200_GEMM_ERR_BAD_CONFIG, "unknown type pair %d", p.types);
    if ((p.lc | p.la | p.lb) & ~1)
        return fail(B200_GEMM_ERR_BAD_LAYOUT, "layout ints must be 0 (row-major) or 1 (column-major): c=%d a=%d b=%d", p.lc, p.la, p.lb);
    const size_t lim = 0x7fffffffull;
    if (p.M > lim || p.N > lim || p.K > lim || p.batch > 65535 * 1024ull)
        return fail(B200_GEMM_ERR_BAD_SIZE, "dimension out of range: M=%zu N=%zu K=%zu batch=%zu", p.M, p.N, p.K, p.batch);
    if (p.batch == 0) return fail(B200_GEMM_ERR_BAD_SIZE, "batch_count must be >= 1");
    if (p.M == 0 || p.N == 0) return B200_GEMM_OK; // empty C: nothing to do
    if (!p.C) return fail(B200_GEMM_ERR_NULL_POINTER, "C is NULL");
    if (p.K != 0 && (!p.A || !p.B)) return fail(B200_GEMM_ERR_NULL_POINTER, "A or B is NULL");
    const size_t out_sz = out_is_f32(p.types) ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(p.C) % out_sz) || (reinterpret_cast<uintptr_t>(p.A) % 2) ||
        (reinterpret_cast<uintptr_t>(p.B) % 2))
        return fail(B200_GEMM_ERR_MISALIGNED, "a pointer is not aligned to its element size");
    return B200_GEMM_OK;
}

// Can TMA address the two operands of this view (bases 16-byte aligned, contiguous extents
// multiples of 8 elements)?
static bool operands_tma_ok(const Problem& p, const View& v)
{
    if (reinterpret_cast<uintptr_t>(v.a) % 16 || reinterpret_cast<uintptr_t>(v.b) % 16) return false;
    const uint32_t a_inner = v.a_mn ? v.M : v.K;
    const uint32_t b_inner = v.b_mn ? v.N : v.K;
    if (a_inner % 8 || b_inner % 8) return false;
    if (p.batch > 1 && (((size_t)v.M * v.K) % 8 || ((size_t)v.N * v.K) % 8)) return false;
    return true;
}

// Can TMA address this view?  Needs 16-byte aligned bases and 16-byte multiples for every
// non-innermost stride.
static bool tma_ok(const Problem& p, const View& v)
{
    const size_t out_sz = out_is_f32(p.types) ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(v.a) % 16 || reinterpret_cast<uintptr_t>(v.b) % 16 ||
        reinterpret_cast<uintptr_t>(v.d) % 16)
        return false;
    const uint32_t a_inner = v.a_mn ? v.M : v.K;
    const uint32_t b_inner = v.b_mn ? v.N : v.K;
    if (a_inner % 8 || b_inner % 8) return false;
    if (p.batch > 1 && (((size_t)v.M * v.K) % 8 || ((size_t)v.N * v.K) % 8)) return false;
    if ((v.N * out_sz) % 16) return false;
    if (p.batch > 1 && (((size_t)v.M * v.N * out_sz) % 16)) return false;
    return true;
}

// ------------------------------------------------------------------------------------------
// Configuration handling
// ------------------------------------------------------------------------------------------
// The compiled kernel width that serves a tile width (see check_config).
static inline int compiled_width(int tile_n)
{
    return tile_n <= 64 ? tile_n : (tile_n <= 128 ? 128 : (tile_n <= 256 ? 256 : 512));
}

static int check_config(const b200_gemm_config& c)
{
    if (c.cluster != 1 && c.cluster != 2) return fail(B200_GEMM_ERR_BAD_CONFIG, "cluster %d not compiled (1 or 2)", c.cluster);
    if (c.tile_m != 128 * c.cluster)
        return fail(B200_GEMM_ERR_BAD_CONFIG, "tile_m %d does not match cluster %d (tile_m = 128 * cluster)", c.tile_m, c.cluster);
    // CTA-pair kernels take any width between 128 and 256 columns that is a multiple of 32
    // (run-time field of the 256-column kernel); everything else is a compiled width.
    const bool flex_width = c.cluster == 2 && c.tile_n > 128 && c.tile_n < 256 && c.tile_n % 32 == 0;
    if (!flex_width && c.tile_n != 64 && c.tile_n != 128 && c.tile_n != 256 && c.tile_n != 512)
        return fail(B200_GEMM_ERR_BAD_CONFIG, "tile_n %d not available (64, 128, 256, 512; with cluster 2 also 160, 192, 224)", c.tile_n);
    if (c.cluster == 2 && c.tile_n == 64) return fail(B200_GEMM_ERR_BAD_CONFIG, "tile_n 64 needs cluster 1");
    if (c.cluster == 1 && c.tile_n == 512) return fail(B200_GEMM_ERR_BAD_CONFIG, "tile_n 512 needs cluster 2");
    if (c.stages < 2 || c.stages > MAX_STAGES) return fail(B200_GEMM_ERR_BAD_CONFIG, "stages %d outside 2..%d", c.stages, MAX_STAGES);
    if (c.split_k < 0 || c.split_k > 64) return fail(B200_GEMM_ERR_BAD_CONFIG, "split_k %d outside 0..64 (0 = balanced schedule)", c.split_k);
    if (c.raster < 0 || (c.raster & ~B200_GEMM_RASTER_SNAKE) > 64)
        return fail(B200_GEMM_ERR_BAD_CONFIG, "raster %d: band height outside 0..64 (add %d for the snake order)", c.raster,
                    B200_GEMM_RASTER_SNAKE);
    return B200_GEMM_OK;
}

// Fit a (table or caller) config to one problem: clamp the ring depth to what shared memory
// holds and give every K partition at least one k-block.
static void legalize(b200_gemm_config& c, const View& v, uint32_t* kb_per_split)
{
    const int ms = max_stages(compiled_width(c.tile_n), c.cluster);
    if (c.stages > ms) c.stages = ms;
    const uint32_t k_blocks = (v.K + BLOCK_K - 1) / BLOCK_K;
    uint32_t       split    = (uint32_t)c.split_k;
    if (split > k_blocks) split = k_blocks;
    if (split < 1) split = 1;
    const uint32_t per = (k_blocks + split - 1) / split;
    split              = (k_blocks + per - 1) / per;
    c.split_k          = (int)split;
    *kb_per_split      = per;
}

// Debugging / profiling override: B200_GEMM_CONFIG="tile_m,tile_n,stages,cluster,split_k,raster"
// replaces the table's choice for every call that does not pass an explicit config.
static bool env_config(b200_gemm_config* out)
{
    // Parsed once, at the first call: the environment is not re-read on the hot path.
    static const struct Parsed {
        bool             set = false;
        b200_gemm_config cfg{};
        Parsed()
        {
            const char* e = getenv("B200_GEMM_CONFIG");
            set = e && *e &&
                  sscanf(e, "%d,%d,%d,%d,%d,%d", &cfg.tile_m, &cfg.tile_n, &cfg.stages, &cfg.cluster, &cfg.split_k,
                         &cfg.raster) == 6;
        }
    } parsed;
    if (!parsed.set) return false;
    *out = parsed.cfg;
    return true;
}

static b200_gemm_config resolve_config(const Problem& p, const b200_gemm_config* user, int* idx, bool* tuned = nullptr)
{
    if (tuned) *tuned = true; // explicit configurations are taken as they are
    if (user) {
        if (idx) *idx = -1;
        return *user;
    }
    b200_gemm_config forced;
    if (env_config(&forced)) {
        if (idx) *idx = -1;
        return forced;
    }
    const int i = find_best_config(p.M, p.N, p.K, out_is_f32(p.types) ? 1 : 0, p.la, p.lb, p.lc, tuned);
    if (idx) *idx = i;
    return k_configs[i];
}

// Sizes without a table entry of their own: the entry borrowed from the nearest tuned size is
// checked against a small cost model of the compiled tile shapes and replaced when the model
// finds something at least 15 % faster (a 1536^3 problem should not inherit the K partitions
// of a skinny neighbour, a 512 x 512 x 4096 one not a tile that leaves 140 SMs idle).
//   time = waves x k-blocks x cycles per k-block + exposed epilogue + launch (+ reduction pass)
// with cycles per k-block the larger of the tensor-pipe time and the per-slot issue work of the
// producer / MMA threads, measured on this design.  Sizes with an entry are never touched.
static void adapt_config(b200_gemm_config& c, const View& v, size_t batch, int sms, int out_chunk)
{
    struct Shape {
        int    tm, tn, cl;
        double cyc_per_kb, epilogue;
    };
    // (224 / 192 / 160: run-time widths of the 256-column pair kernel, for column counts that
    // 256 cuts into a nearly empty last wave - 2304^3: 81 tiles on 74 pairs; they need a K-major
    // B' and whole 128-byte output chunks)
    static const Shape ladder[8] = {{256, 512, 2, 1060, 5500},
                                    {256, 256, 2, 540, 2700},
                                    {256, 224, 2, 495, 2400},
                                    {256, 192, 2, 440, 2100},
                                    {256, 160, 2, 385, 1800},
                                    {128, 256, 1, 570, 2700},
                                    {128, 128, 1, 500, 1400},
                                    {128, 64, 1, 400, 800}};
    const uint32_t k_blocks = (v.K + BLOCK_K - 1) / BLOCK_K;
    const double out_bytes = out_chunk == 32 ? 4.0 : 2.0;
    auto model = [&](const Shape& t, int split) {
        const uint64_t tiles1 = (uint64_t)((v.M + t.tm - 1) / t.tm) * ((v.N + t.tn - 1) / t.tn) * batch;
        const uint64_t tiles = tiles1 * (uint64_t)split;
        const uint64_t slots = (uint64_t)(sms / t.cl);
        const uint64_t waves = (tiles + slots - 1) / slots;
        const double   kb    = (double)((k_blocks + split - 1) / split);
        // K partitions of the one-CTA 128- and 256-column tiles are summed inside a cluster when
        // all clusters fit at once (make_plan's rule): no workspace, no second kernel; the
        // exchange, barriers and sum cost ~3000 cycles + (split - 1) / split of an f32 tile per
        // CTA at ~8 B per cycle (timeline of 128 x 8192 x 8192: 14k cycles for 128 x 256 x 4,
        // 6k for 128 x 128 x 2).
        const bool in_cluster = split >= 2 && split <= 4 && t.cl == 1 && t.tn >= 128 && tiles1 <= (uint64_t)(sms / split * 7 / 8);
        // A CTA drains its part of a tile at ~19.5 B per cycle (12.5 in a pair): with a short K
        // loop that, not the main loop, is the time of a tile (8192 x 8192 x 128: 31.6 us on
        // 128 x 256 tiles, 42.8 us on 256 x 256 pair tiles).
        const double   drain = 128.0 * (t.tn > 256 ? 512.0 : (double)t.tn) * out_bytes / (t.cl == 2 ? 12.5 : 19.5);
        // One-CTA tiles stage 1.5 to 2 times the operand bytes per FLOP of a CTA pair; with every
        // SM loading at once (more than one wave of tiles) the L2-to-SM path paces them:
        // 3000^3 on 128 x 256 tiles 63.9 us, on 256 x 256 pair tiles 44.7 us.
        const double   per_kb = t.cyc_per_kb * ((t.cl == 1 && tiles > slots) ? 1.4 : 1.0);
        // (a pair kernel's launch and set-up cost more: cluster scheduling, one k-block per ring
        // slot; 1536^3 runs 9.4 us on 128 x 128 tiles and 12.0 us on one wave of pair tiles)
        // (+ ~600 cycles per tile of work decode and accumulator hand-over: 4096 x 4096 x 64 runs
        // 10.0 us on 512 tiles of 128 x 256 and 16.7 us on 2048 tiles of 128 x 64)
        const double   tile  = (split == 1 ? std::max(kb * per_kb, drain) : kb * per_kb) + 600.0;
        double         cyc   = (double)waves * tile + t.epilogue + 3000.0 + (t.cl == 2 ? 2500.0 : 0.0);
        if (in_cluster) cyc += 3000.0 + 128.0 * t.tn * 4.0 * (split - 1) / split / 8.0;
        else if (split > 1) cyc += 7000.0 + (double)v.M * v.N * batch * 4.0 * (split + 1) / 4000.0; // a second kernel; partials: ~4 KB per cycle
        return cyc;
    };
    double current = -1.0;
    for (const Shape& t : ladder)
        if (t.tm == c.tile_m && t.tn == c.tile_n) current = model(t, c.split_k);
    double       best = 1e300;
    const Shape* bt   = nullptr;
    int          bs   = 1;
    for (const Shape& t : ladder) {
        if (t.tn != compiled_width(t.tn) && (v.b_mn || t.tn % out_chunk)) continue;
        for (int split : {1, 2, 3, 4, 8, 16}) {
            if (split > 1 && (v.N % 4 != 0 || (uint32_t)split * 4 > k_blocks)) continue;
            const double m = model(t, split);
            if (m < best) {
                best = m;
                bt   = &t;
                bs   = split;
            }
        }
    }
    if (!bt || (current > 0 && best > current * 0.85)) return;
    c.tile_m  = bt->tm;
    c.tile_n  = bt->tn;
    c.cluster = bt->cl;
    c.split_k = bs;
    c.stages  = MAX_STAGES;
    c.raster  = ((v.M + bt->tm - 1) / bt->tm) >= 16 ? 8 : 0;
}

// ------------------------------------------------------------------------------------------
// TMA descriptors
// ------------------------------------------------------------------------------------------
static int encode_map(CUtensorMap* tm, CUtensorMapDataType dt, size_t esz, const void* base,
                      uint64_t d0, uint64_t d1, uint64_t d2, uint32_t b0, uint32_t b1)
{
    const cuuint64_t dims[3]    = {d0, d1, d2};
    const cuuint64_t strides[2] = {d0 * esz, d0 * d1 * esz};
    const cuuint32_t box[3]     = {b0, b1, 1};
    const cuuint32_t estr[3]    = {1, 1, 1};
    const CUresult   r = g_encode(tm, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(B200_GEMM_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) dims=%llu,%llu,%llu box=%u,%u", (int)r,
                    (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2, b0, b1);
    return B200_GEMM_OK;
}

// Operand with MN extent `rows`: K-major -> [batch][rows][K], box 64 x box_rows;
// MN-major -> [batch][K][rows], box 64 (MN) x 64 (K).
static int encode_operand(CUtensorMap* tm, bool bf16, const void* base, uint32_t rows, uint32_t K,
                          size_t batch, bool mn_major, uint32_t box_rows)
{
    const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (!mn_major) return encode_map(tm, dt, 2, base, K, rows, batch, BLOCK_K, box_rows);
    return encode_map(tm, dt, 2, base, rows, K, batch, 64, BLOCK_K);
}

// Operand of a one-CTA kernel, `kc` k-blocks per box.
//   K-major, K % 64 == 0: 4-D view [batch][K/64][rows][64] (strides: rows K elements apart,
//     chunks 128 bytes apart), box 64 x box_rows x kc: lands as kc consecutive row-block tiles.
//   K-major otherwise: the plain 3-D map, one k-block per box (kc == 1).
//   MN-major: [batch][K][rows], box 64 (MN) x 64 * kc (K).
static int encode_operand_slab(CUtensorMap* tm, bool bf16, const void* base, uint32_t rows, uint32_t K,
                               size_t batch, bool mn_major, uint32_t box_rows, uint32_t kc, bool k4d)
{
    const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (mn_major) return encode_map(tm, dt, 2, base, rows, K, batch, 64, BLOCK_K * kc);
    if (!k4d) return encode_map(tm, dt, 2, base, K, rows, batch, BLOCK_K, box_rows);
    const cuuint64_t dims[4]    = {(cuuint64_t)BLOCK_K, rows, K / BLOCK_K, batch};
    const cuuint64_t strides[3] = {(cuuint64_t)K * 2, (cuuint64_t)BLOCK_K * 2, (cuuint64_t)rows * K * 2};
    const cuuint32_t box[4]     = {(cuuint32_t)BLOCK_K, box_rows, kc, 1};
    const cuuint32_t estr[4]    = {1, 1, 1, 1};
    const CUresult   r = g_encode(tm, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(B200_GEMM_ERR_CUDA, "cuTensorMapEncodeTiled (4-D) failed (%d) rows=%u K=%u box_rows=%u kc=%u", (int)r, rows, K,
                    box_rows, kc);
    return B200_GEMM_OK;
}

// ------------------------------------------------------------------------------------------
// Launch
// ------------------------------------------------------------------------------------------
template <int BN, int CL, bool TR = false>
static cudaError_t launch_bn(int out, uint32_t units_wanted, PairCache* pairs, int pair_slot, uint32_t smem, cudaStream_t s,
                             const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& d, const CUtensorMap& w,
                             const GemmParams& gp, const GatherMaps* gather = nullptr)
{
    cudaLaunchConfig_t lc = {};
    dim3               grid(CL * units_wanted);
    if (CL == 2) {
        // A persistent pair kernel wants exactly as many clusters as can be resident at once.
        int&      pair_units = pairs->units[pair_slot];
        if (pair_units == 0 || pairs->smem[pair_slot] != smem) {
            cudaLaunchConfig_t q = {};
            q.gridDim            = dim3(2 * 148);
            q.blockDim           = dim3(GEMM_THREADS);
            q.dynamicSmemBytes   = smem;
            cudaLaunchAttribute qa[1];
            qa[0].id               = cudaLaunchAttributeClusterDimension;
            qa[0].val.clusterDim.x = 2;
            qa[0].val.clusterDim.y = 1;
            qa[0].val.clusterDim.z = 1;
            q.attrs                = qa;
            q.numAttrs             = 1;
            int         n  = 0;
            cudaError_t qe = cudaOccupancyMaxActiveClusters(&n, gemm_umma_kernel<BN, OUT_F32, CL, TR>, &q);
            if (qe != cudaSuccess || n < 1) {
                (void)cudaGetLastError();
                n = 64;
            }
            pair_units             = n;
            pairs->smem[pair_slot] = smem;
        }
        grid = dim3(2 * std::min<uint32_t>(units_wanted, (uint32_t)pair_units));
    }
    lc.gridDim            = grid;
    lc.blockDim           = dim3(GEMM_THREADS);
    lc.dynamicSmemBytes   = smem;
    lc.stream             = s;
    cudaLaunchAttribute attr[2];
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // The kernel's set-up may overlap the tail of the kernel before it (see the kernel).
    attr[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs                                           = attr;
    lc.numAttrs                                        = 2;
    if constexpr (CL == 2 && BN >= 256 && !TR) {
        if (gather) { // the gathering twins exist for the two large pair tiles
            switch (out) {
                case OUT_F32: return cudaLaunchKernelEx(&lc, gemm_umma_gather_kernel<BN, OUT_F32, CL>, a, b, *gather, gp);
                case OUT_F16: return cudaLaunchKernelEx(&lc, gemm_umma_gather_kernel<BN, OUT_F16, CL>, a, b, *gather, gp);
                default: return cudaLaunchKernelEx(&lc, gemm_umma_gather_kernel<BN, OUT_BF16, CL>, a, b, *gather, gp);
            }
        }
    }
    switch (out) {
        case OUT_F32: return cudaLaunchKernelEx(&lc, gemm_umma_kernel<BN, OUT_F32, CL, TR>, a, b, d, w, gp);
        case OUT_F16: return cudaLaunchKernelEx(&lc, gemm_umma_kernel<BN, OUT_F16, CL, TR>, a, b, d, w, gp);
        default: return cudaLaunchKernelEx(&lc, gemm_umma_kernel<BN, OUT_BF16, CL, TR>, a, b, d, w, gp);
    }
}

// One cluster of `split` CTAs per tile, the CTAs being the tile's K partitions.
template <int BN, bool TR = false>
static cudaError_t launch_ksplit(int out, uint32_t tiles, uint32_t split, uint32_t smem, cudaStream_t s, const CUtensorMap& a,
                                 const CUtensorMap& b, const CUtensorMap& d, const GemmParams& gp)
{
    cudaLaunchConfig_t lc = {};
    lc.gridDim            = dim3(tiles * split);
    lc.blockDim           = dim3(GEMM_THREADS);
    lc.dynamicSmemBytes   = smem;
    lc.stream             = s;
    cudaLaunchAttribute attr[2];
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = split;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs                                           = attr;
    lc.numAttrs                                        = 2;
    switch (out) {
        case OUT_F32: return cudaLaunchKernelEx(&lc, gemm_umma_ksplit_kernel<BN, OUT_F32, TR>, a, b, d, gp);
        case OUT_F16: return cudaLaunchKernelEx(&lc, gemm_umma_ksplit_kernel<BN, OUT_F16, TR>, a, b, d, gp);
        default: return cudaLaunchKernelEx(&lc, gemm_umma_ksplit_kernel<BN, OUT_BF16, TR>, a, b, d, gp);
    }
}

template <class TIn, class TOut>
static cudaError_t launch_generic(const Problem& p, cudaStream_t s)
{
    // Element strides of the caller's (not the kernel-view) matrices.
    const uint64_t a_sm = p.la == 0 ? p.K : 1, a_sk = p.la == 0 ? 1 : p.M;
    const uint64_t b_sk = p.lb == 0 ? p.N : 1, b_sn = p.lb == 0 ? 1 : p.K;
    const uint64_t c_sm = p.lc == 0 ? p.N : 1, c_sn = p.lc == 0 ? 1 : p.M;
    for (size_t b0 = 0; b0 < p.batch; b0 += 65535) {
        const unsigned nb = (unsigned)std::min<size_t>(65535, p.batch - b0);
        dim3           grid((unsigned)((p.N + 15) / 16), (unsigned)((p.M + 15) / 16), nb);
        if (grid.y > 65535) return cudaErrorInvalidConfiguration;
        gemm_generic_kernel<TIn, TOut><<<grid, 256, 0, s>>>(
            static_cast<TOut*>(p.C) + b0 * p.M * p.N, static_cast<const TIn*>(p.A) + b0 * p.M * p.K,
            static_cast<const TIn*>(p.B) + b0 * p.K * p.N, (uint32_t)p.M, (uint32_t)p.N, (uint32_t)p.K, a_sm,
            a_sk, b_sk, b_sn, c_sm, c_sn, p.M * p.K, p.K * p.N, p.M * p.N);
        g_launches.fetch_add(1, std::memory_order_relaxed);
    }
    return cudaGetLastError();
}

// Split-K reduction pass, launched as a programmatic dependent of the GEMM kernel before it
// in the stream: its blocks are set up while the GEMM's last tiles drain and start reading the
// partials (after griddepcontrol.wait) the moment the GEMM grid has completed.
static cudaError_t launch_reduce(int out, unsigned blocks, cudaStream_t s, const float* ws, void* d, uint64_t mn,
                                 uint32_t split, uint32_t batch)
{
    cudaLaunchConfig_t lc = {};
    lc.gridDim            = dim3(blocks);
    lc.blockDim           = dim3(256);
    lc.dynamicSmemBytes   = 0;
    lc.stream             = s;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs                                           = attr;
    lc.numAttrs                                        = 1;
    switch (out) {
        case OUT_F32: return cudaLaunchKernelEx(&lc, splitk_reduce_kernel<OUT_F32>, ws, d, mn, split, batch);
        case OUT_F16: return cudaLaunchKernelEx(&lc, splitk_reduce_kernel<OUT_F16>, ws, d, mn, split, batch);
        default: return cudaLaunchKernelEx(&lc, splitk_reduce_kernel<OUT_BF16>, ws, d, mn, split, batch);
    }
}

// Fix-up pass of the balanced schedule, a programmatic dependent of the GEMM kernel like the
// split-K reduction.
static cudaError_t launch_streamk_reduce(int out, unsigned blocks, unsigned jobs, cudaStream_t s, const float* ws, void* d,
                                         const GemmParams& gp, uint32_t tile_m, uint32_t tile_n)
{
    cudaLaunchConfig_t lc = {};
    lc.gridDim            = dim3(blocks, jobs);
    lc.blockDim           = dim3(256);
    lc.dynamicSmemBytes   = 0;
    lc.stream             = s;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs                                           = attr;
    lc.numAttrs                                        = 1;
    switch (out) {
        case OUT_F32: return cudaLaunchKernelEx(&lc, streamk_reduce_kernel<OUT_F32>, ws, d, gp, tile_m, tile_n);
        case OUT_F16: return cudaLaunchKernelEx(&lc, streamk_reduce_kernel<OUT_F16>, ws, d, gp, tile_m, tile_n);
        default: return cudaLaunchKernelEx(&lc, streamk_reduce_kernel<OUT_BF16>, ws, d, gp, tile_m, tile_n);
    }
}

// Geometry of the balanced schedule for `tiles` tiles of `upt` K steps on `slots` persistent
// workers (CTAs or CTA pairs): whole waves of tiles are dealt round-robin; the tiles of the
// incomplete wave (all tiles when there are fewer than workers) are cut into `runs` equal runs
// of K steps.  `grid` = workers launched.
struct BalancedGeometry {
    uint64_t sk_tiles, runs, grid;
};
static BalancedGeometry balanced_geometry(uint64_t tiles, uint64_t upt, uint64_t slots)
{
    BalancedGeometry g;
    g.sk_tiles = tiles <= slots ? tiles : tiles % slots;
    g.runs     = std::max<uint64_t>(1, std::min<uint64_t>(g.sk_tiles * upt, slots));
    g.grid     = tiles >= slots ? slots : g.runs;
    return g;
}

// Everything the launch path decides before it touches the GPU.
struct LaunchPlan {
    bool             generic    = false; // TMA cannot address the problem: CUDA-core kernel
    bool             transposed = false; // operands swapped once more, transposing epilogue
    bool             narrow     = false; // kernel view of at most 64 columns (or transposed)
    bool             slot       = false; // one-CTA kernel with kc k-blocks per ring slot
    bool             k4d        = false; // K-major operands through the 4-D (chunked K) maps
    bool             balanced   = false; // balanced (stream-K) schedule: runs of K steps cut across tiles
    bool             cluster_k  = false; // the K partitions of a tile are one cluster's CTAs, summed on chip (no workspace)
    View             v{};
    b200_gemm_config cfg{};
    uint32_t         bm = BLOCK_M, kc = 1, kb_per_split = 0;
};

static int make_plan(const Problem& p, const b200_gemm_config* user_cfg, int sm_count, LaunchPlan* out)
{
    LaunchPlan pl;
    View&      v = pl.v;
    v            = make_view(p);
    // Skinny problems: the MMA's M extent is fixed at 128 rows but its N extent goes down to 16,
    // so when the kernel view has few rows and many columns the operands swap roles once more
    // (the kernel computes D^T) and the epilogue writes D^T transposed, i.e. D.  No 128-row
    // tile of mostly zero-filled A' is staged and the ring holds twice as many slots.
    bool              tuned = true;
    b200_gemm_config& cfg   = pl.cfg;
    cfg                     = resolve_config(p, user_cfg, nullptr, &tuned);
    int st                  = check_config(cfg);
    if (st != B200_GEMM_OK) return st;
    // split_k == 0 asks for the balanced (stream-K) schedule, which keeps the plain orientation.
    bool  balanced   = cfg.split_k == 0;
    bool& transposed = pl.transposed;
    static const int cluster_k_env = [] { // B200_GEMM_CLUSTER_SPLITK = 0 / 1 forces the workspace / the cluster form of split-K (profiling)
        const char* e = getenv("B200_GEMM_CLUSTER_SPLITK");
        return (e && *e) ? atoi(e) : -1;
    }();
    if (!balanced && v.M <= 64 && v.N >= 128 && operands_tma_ok(p, v) && reinterpret_cast<uintptr_t>(v.d) % 16 == 0 &&
        ((size_t)v.M * v.N) % 4 == 0) {
        std::swap(v.a, v.b);
        std::swap(v.M, v.N);
        std::swap(v.a_mn, v.b_mn);
        transposed = true;
    }
    if (!transposed && !tma_ok(p, v)) {
        pl.generic = true;
        *out       = pl;
        return B200_GEMM_OK;
    }

    if (!tuned && !balanced) adapt_config(cfg, v, p.batch, sm_count, out_is_f32(p.types) ? 32 : 64);
    // Narrow kernel views (at most 64 columns) run on the narrow one-CTA variants whatever
    // tile the table names: tile_n is the smallest compiled width that covers N (an MN-major
    // B' is loaded in 64-row boxes, so it needs 64) and the ring is as deep as fits.
    const bool narrow = v.N <= 64 || transposed;
    pl.narrow         = narrow;
    if (narrow) {
        cfg.tile_m  = BLOCK_M;
        cfg.cluster = 1;
        cfg.tile_n  = v.N <= 16 ? 16 : (v.N <= 32 ? 32 : (v.N <= 64 ? 64 : 128));
        if (v.b_mn && cfg.tile_n < 64) cfg.tile_n = 64;
    }
    // A width between the compiled ones needs a K-major B' (an N-major B' is loaded in 64-row
    // boxes) and whole 128-byte output chunks (32 f32 or 64 16-bit columns).
    if (cfg.tile_n != compiled_width(cfg.tile_n)) {
        const int chunk = out_is_f32(p.types) ? 32 : 64;
        if (v.b_mn || cfg.tile_n % chunk) {
            if (user_cfg)
                return fail(B200_GEMM_ERR_BAD_CONFIG, "tile_n %d needs a K-major B operand in the kernel view and a multiple of %d columns",
                            cfg.tile_n, chunk);
            cfg.tile_n = 256; // a borrowed table entry that does not fit this layout / type
        }
    }
    // Transposed problems are HBM-bound streams of A' (the caller's large operand).  Its rows are
    // cut into slabs of `bm` <= 128 rows so that the slabs fill whole waves of the SMs: every SM
    // streams the same number of bytes, no K partition and no reduction pass is needed.  (The
    // MMA still spans 128 rows; the rows past the slab are never stored.)  An M-major A' is
    // loaded in 64-row boxes, so its slabs are 64 or 128 rows.
    // The narrow staged-epilogue tiles (a skinny problem with a column-major C) stream the large
    // operand the same way; their epilogue stores whole 32-row groups, so their slabs are
    // multiples of 32 rows.
    // The balanced schedule lays the tiles' K loops end to end and cuts that line into equal runs,
    // one per SM (WorkCursor in gemm_kernels.cuh).  It runs on the tiles of up to 256 columns and
    // its fix-up pass works in float4 units.
    if (balanced && (cfg.tile_n > 256 || v.N % 4)) {
        if (user_cfg)
            return fail(B200_GEMM_ERR_BAD_CONFIG, "the balanced schedule (split_k 0) needs tile_n <= 256 and N %% 4 == 0 in the kernel view");
        balanced = false;
    }
    if (cfg.split_k == 0) cfg.split_k = 1; // no per-tile K partitions either way
    pl.balanced = balanced;
    uint32_t& bm = pl.bm;
    if (narrow && !user_cfg && !balanced && (transposed || !v.a_mn)) { // (staged tiles on an M-major operand: measured slower)
        const uint32_t sms       = (uint32_t)sm_count;
        const uint32_t step      = v.a_mn ? 64u : (transposed ? 8u : 32u);
        uint64_t       best_cost = ~0ull;
        uint32_t       best_bm = 0, best_tiles = 0;
        for (uint32_t cand = step; cand <= (uint32_t)BLOCK_M; cand += step) {
            const uint64_t tiles = (uint64_t)((v.M + cand - 1) / cand) * p.batch;
            const uint64_t waves = (tiles + sms - 1) / sms;
            const uint64_t cost  = waves * (cand + 8); // rows streamed per SM + a per-tile overhead
            if (cost <= best_cost) {
                best_cost  = cost;
                best_bm    = cand;
                best_tiles = (uint32_t)std::min<uint64_t>(tiles, 0xffffffffu);
            }
        }
        if (best_tiles * 10u >= sms * 8u) { // enough slabs to occupy the chip without splitting K
            bm          = best_bm;
            cfg.split_k = 1;
        }
        // Transposed problems: two or four K partitions per slab, as the CTAs of a cluster
        // (taller slabs, a shorter K range per CTA, partial slabs summed through distributed
        // shared memory; one slab per cluster, all clusters resident at once), when a small model
        // of a CTA's time says so.  Three things can bound a slab kernel:
        //   the MMA thread   the MMA spans 128 rows whatever the slab height, so a CTA issues
        //                    4 MMAs per k-block of its K range however few rows it streams: about
        //                    275 cycles per k-block (16 x 4096 x 14336 on 32-row slabs: 32 us,
        //                    against the vendor GEMM's 22);
        //   HBM              the slab's bytes at the CTA's share of ~3.3 KB per cycle (and at most
        //                    ~38 B per cycle for one SM);
        //   L2 to SM         slab + small operand, ~43 B per cycle per SM with every SM loading
        //                    (64 x 8192 x 8192 on 147 slabs: 281 MB, the bound there).
        // K partitions shorten the first and the third.
        const uint32_t k_blocks = (v.K + BLOCK_K - 1) / BLOCK_K;
        if (transposed && cluster_k_env != 0 && k_blocks >= 32) {
            auto cta_cycles = [&](uint32_t rows, uint32_t split, uint64_t tiles) {
                const double kb     = (double)((k_blocks + split - 1) / split);
                const double active = (double)std::min<uint64_t>(tiles * split, sms);
                const double bytes  = (double)rows * kb * BLOCK_K * 2.0;
                const double mma    = kb * 275.0;
                const double hbm    = std::max(bytes * active / 3300.0, bytes / 38.0);
                const double l2     = ((double)rows + cfg.tile_n) * kb * BLOCK_K * 2.0 / 43.0;
                return std::max(mma, std::max(hbm, l2));
            };
            double   best = 1e300;
            uint32_t best_rows = 0, best_split = 1;
            if (cfg.split_k == 1) { // the slabs chosen above, no K partitions
                const uint64_t tiles = (uint64_t)((v.M + bm - 1) / bm) * p.batch;
                best      = (double)((tiles + sms - 1) / sms) * cta_cycles(bm, 1, tiles);
                best_rows = bm;
            }
            for (uint32_t split : {2u, 4u}) {
                // clusters resident at once: every pair of SMs hosts a cluster of two; clusters of
                // four do not tile GPCs whose SM count is not a multiple of four (37 of them took
                // two waves), so 7/8 of the SMs are counted on
                const uint32_t units = split == 2u ? sms / 2u : sms / split * 7u / 8u;
                for (uint32_t cand = step; cand <= (uint32_t)BLOCK_M; cand += step) {
                    const uint64_t tiles = (uint64_t)((v.M + cand - 1) / cand) * p.batch;
                    if (tiles > units) continue;
                    if (tiles * 10u >= units * 8u) {
                        const double c = cta_cycles(cand, split, tiles) + 2500.0;
                        if (c < best * 0.97) {
                            best       = c;
                            best_rows  = cand;
                            best_split = split;
                        }
                    }
                    break; // the lowest slab height that fits one wave
                }
            }
            if (best_split > 1) {
                // (the ring, which receives the partials, fills the CTA's shared memory whatever
                // the slab height: it always holds the 16 to 64 KiB of the partial slabs)
                bm           = best_rows;
                cfg.split_k  = (int)best_split;
                pl.cluster_k = true;
            }
        }
    }
    uint32_t& kb_per_split = pl.kb_per_split;
    legalize(cfg, v, &kb_per_split);
    if (!user_cfg && cfg.split_k > 1 && !transposed && v.N % 4) { // the table's nearest entry may not fit
        cfg.split_k = 1;
        legalize(cfg, v, &kb_per_split);
    }
    // One-CTA kernels up to 256 columns: a ring slot holds kc k-blocks (see the kernel).  The
    // narrower the tile, the less tensor-pipe time one k-block is worth against the fixed
    // per-slot work of the producer and MMA threads, so narrow tiles take more k-blocks per
    // slot; at least three slots must fit.  K-major operands fetch a slot with one 4-D box over
    // a [chunk][row][64] view of the matrix, which needs K to be a multiple of 64.
    const bool slot = cfg.cluster == 1 && cfg.tile_n <= 256;
    pl.slot         = slot;
    uint32_t& kc    = pl.kc;
    pl.k4d          = slot && v.K % BLOCK_K == 0;
    if (slot && (pl.k4d || (v.a_mn && v.b_mn))) {
        kc = cfg.tile_n >= 256 ? 1u : (cfg.tile_n >= 128 ? 2u : 4u);
        auto slots_fit = [&](uint32_t c) {
            return transposed ? slab_max_stages((int)bm, cfg.tile_n, (int)c) : slot_max_stages(cfg.tile_n, (int)c);
        };
        uint32_t min_slots = 3;
        static const int kc_env = [] { // B200_GEMM_KC = 1 / 2 / 4 forces the k-blocks per ring slot where two slots fit (profiling)
            const char* e = getenv("B200_GEMM_KC");
            return (e && *e) ? atoi(e) : 0;
        }();
        if (kc_env == 1 || kc_env == 2 || kc_env == 4) {
            kc        = (uint32_t)kc_env;
            min_slots = 2;
        }
        while (kc > 1 && (kb_per_split < 2 * kc || slots_fit(kc) < (int)min_slots)) kc /= 2;
        if (cfg.split_k > 1 && kb_per_split % kc) { // partitions start on slot boundaries
            const uint32_t k_blocks = (v.K + BLOCK_K - 1) / BLOCK_K;
            kb_per_split            = (kb_per_split + kc - 1) / kc * kc;
            cfg.split_k             = (int)((k_blocks + kb_per_split - 1) / kb_per_split);
        }
    }
    if (transposed) cfg.stages = slab_max_stages((int)bm, cfg.tile_n, (int)kc);
    else if (slot && (narrow || kc > 1)) cfg.stages = slot_max_stages(cfg.tile_n, (int)kc);
    // K partitions of the one-CTA 128- and 256-column tiles: up to 4 of them form a thread-block
    // cluster and add their partial tiles through distributed shared memory, received in the
    // operand ring (which must hold one f32 tile's worth of chunks).  No workspace, no reduction
    // kernel, and the output is written once in its own type.  One tile per cluster, so the path
    // is taken when all clusters are resident at once (a second wave of clusters costs more than
    // the reduction pass of the persistent kernel; 7/8 of the SMs allows for GPCs whose SM count
    // is not a multiple of the cluster size); clusters of 5 to 8 CTAs measured no faster than the
    // reduction pass.
    if (slot && !narrow && !transposed && !balanced && cfg.split_k > 1 && cfg.split_k <= 4 && bm == (uint32_t)BLOCK_M &&
        (cfg.tile_n == 128 || cfg.tile_n == 256) && cluster_k_env != 0) {
        const uint32_t o_ch   = out_is_f32(p.types) ? 32u : 64u;
        const uint32_t nch    = (uint32_t)cfg.tile_n / o_ch;
        const uint32_t split  = (uint32_t)cfg.split_k;
        const uint64_t need   = (uint64_t)((nch + split - 1) / split) * split * 4u * 32u * o_ch * 4u;
        const uint64_t ring   = (uint64_t)cfg.stages * kc * stage_bytes(cfg.tile_n, 1);
        const uint64_t tiles  = (uint64_t)((v.M + BLOCK_M - 1) / BLOCK_M) * ((v.N + cfg.tile_n - 1) / cfg.tile_n) * p.batch;
        const uint64_t room   = (uint64_t)sm_count / split * 7 / 8; // clusters resident at once, conservatively
        pl.cluster_k          = ring >= need && (tiles <= room || cluster_k_env == 1);
    }
    *out = pl;
    return B200_GEMM_OK;
}

// Where a launch gets its device-side resources from.  The ordinary entry points use the
// per-device context (status word and split-K workspaces from cudaMalloc); the allocation-free
// entry point uses arrays that are part of the library image and must never allocate.
struct LaunchEnv {
    int           sm_count;
    unsigned int* d_status;     // device status word the kernels report give-ups to
    PairCache*    pairs;
    DeviceCtx*    ctx;          // owner of the cached split-K workspaces; nullptr = fixed workspace
    float*        fixed_ws;     // ctx == nullptr: the built-in workspace (device address) ...
    size_t        fixed_ws_bytes; // ... and its size
};

// L2 eviction priorities of the TMA traffic (GemmParams::l2_hints, 0 = none); only builds with
// -DB200_GEMM_L2_HINT_BUILD act on them.  B200_GEMM_L2_HINTS, read once, sets them (profiling);
// no policy measured better than none, so the launch path itself never asks for one.
static int env_l2_hints()
{
    static const int v = [] {
        const char* e = getenv("B200_GEMM_L2_HINTS");
        return (e && *e) ? atoi(e) : -1;
    }();
    return v;
}

// A GEMM whose output is a block of a larger matrix held once per GPU: every tile is stored to
// all `ndst` copies (fused all-gather).  In the caller's terms the problem's C (M x N, layout
// lc) is the block at (row0, col0) of a full_rows x full_cols matrix of the same layout.
struct GatherSpec {
    void* const* dst;   // ndst base addresses (this GPU's copy and peer mappings of the others')
    int          ndst;
    size_t       full_rows, full_cols, row0, col0;
};

static int launch_gemm(const Problem& p, cudaStream_t stream, const b200_gemm_config* user_cfg, const LaunchEnv& env,
                       const GatherSpec* gather = nullptr);

static int run_gemm(const Problem& p, cudaStream_t stream, const b200_gemm_config* user_cfg)
{
    int st = validate(p);
    if (st != B200_GEMM_OK) return st;
    if (p.M == 0 || p.N == 0) return B200_GEMM_OK;

    DeviceCtx* ctx = nullptr;
    st             = get_ctx(&ctx);
    if (st != B200_GEMM_OK) return st;

    const size_t out_sz = out_is_f32(p.types) ? 4 : 2;
    if (p.K == 0) { // empty sum: C = 0
        CUDA_TRY(cudaMemsetAsync(p.C, 0, p.M * p.N * p.batch * out_sz, stream));
        return B200_GEMM_OK;
    }
    const LaunchEnv env{ctx->sm_count, ctx->d_status, &ctx->pairs, ctx, nullptr, 0};
    return launch_gemm(p, stream, user_cfg, env);
}

// Plans and launches one (validated, non-empty) problem.
static int launch_gemm(const Problem& p, cudaStream_t stream, const b200_gemm_config* user_cfg, const LaunchEnv& env,
                       const GatherSpec* gather)
{
    int        st;
    const bool fixed = env.ctx == nullptr;
    LaunchPlan pl;
    st = make_plan(p, user_cfg, env.sm_count, &pl);
    if (st != B200_GEMM_OK) return st;
    if (pl.generic && fixed)
        return fail(B200_GEMM_ERR_MISALIGNED,
                    "the allocation-free entry point needs 16-byte aligned pointers and contiguous extents that are "
                    "multiples of 8 elements (M=%zu N=%zu K=%zu)", p.M, p.N, p.K);
    if (gather && (pl.generic || pl.transposed || pl.balanced || pl.cfg.split_k != 1 || pl.cfg.cluster != 2 || pl.cfg.tile_n < 256 ||
                   p.batch != 1))
        return fail(B200_GEMM_ERR_BAD_CONFIG,
                    "the fused gather needs a plan on the 256-row pair tiles without K partitions (got %s, tile_n %d, cluster %d, "
                    "split_k %d, batch %zu)", pl.generic ? "the CUDA-core kernel" : (pl.transposed ? "the operand swap" : "a tcgen05 tile"),
                    pl.cfg.tile_n, pl.cfg.cluster, pl.cfg.split_k, p.batch);
    if (pl.generic) {
        cudaError_t e;
        switch (p.types) {
            case B200_GEMM_F16_F16: e = launch_generic<__half, __half>(p, stream); break;
            case B200_GEMM_F32_F16: e = launch_generic<__half, float>(p, stream); break;
            case B200_GEMM_BF16_BF16: e = launch_generic<__nv_bfloat16, __nv_bfloat16>(p, stream); break;
            default: e = launch_generic<__nv_bfloat16, float>(p, stream); break;
        }
        if (e != cudaSuccess) return fail(B200_GEMM_ERR_CUDA, "generic kernel launch failed: %s", cudaGetErrorString(e));
        return B200_GEMM_OK;
    }
    const View&             v            = pl.v;
    const b200_gemm_config& cfg          = pl.cfg;
    const bool              transposed   = pl.transposed;
    const bool              narrow       = pl.narrow;
    const bool              slot         = pl.slot;
    const bool              k4d          = pl.k4d;
    const uint32_t          bm           = pl.bm;
    const uint32_t          kc           = pl.kc;
    const uint32_t          kb_per_split = pl.kb_per_split;
    const bool              balanced     = pl.balanced;
    const bool              cluster_k    = pl.cluster_k;

    const int      bn   = cfg.tile_n;
    const int      out  = out_kind(p.types);
    const bool     bf16 = in_is_bf16(p.types);
    const uint32_t split = (uint32_t)cfg.split_k;

    GemmParams gp;
    gp.M            = v.M;
    gp.N            = v.N;
    gp.K            = v.K;
    gp.batch        = (uint32_t)p.batch;
    const uint32_t cl   = (uint32_t)cfg.cluster;
    gp.bm           = bm;
    gp.wn           = (uint32_t)cfg.tile_n;
    gp.kc           = kc;
    gp.k4d          = k4d ? 1u : 0u;
    gp.m_tiles      = slot ? (v.M + bm - 1) / bm : (v.M + BLOCK_M * cl - 1) / (BLOCK_M * cl);
    gp.n_tiles      = (v.N + bn - 1) / bn;
    gp.k_blocks     = (v.K + BLOCK_K - 1) / BLOCK_K;
    gp.split_k      = split;
    gp.kb_per_split = kb_per_split;
    gp.group_m      = (uint32_t)(cfg.raster & ~B200_GEMM_RASTER_SNAKE);
    gp.snake        = (cfg.raster & B200_GEMM_RASTER_SNAKE) ? 1u : 0u;
    gp.cluster_k    = cluster_k ? 1u : 0u;
    const uint64_t work = (uint64_t)gp.batch * (cluster_k ? 1u : split) * gp.m_tiles * gp.n_tiles;
    if (work * (cluster_k ? split : 1u) > 0x7fffffffull) return fail(B200_GEMM_ERR_BAD_SIZE, "too many tiles (%llu)", (unsigned long long)work);
    gp.num_work   = (uint32_t)work;
    // Balanced schedule: `work` tiles of units_per_tile K steps each, cut into `workers` runs.
    const uint32_t tile_rows = slot ? bm : (uint32_t)BLOCK_M * cl;
    gp.balanced = gp.units_per_tile = gp.workers = gp.total_units = gp.sk_tiles = 0;
    uint32_t balanced_grid = 0;
    if (balanced) {
        const uint64_t         upt = (gp.k_blocks + kc - 1) / kc;
        const BalancedGeometry g   = balanced_geometry(work, upt, (uint64_t)env.sm_count / cl);
        const uint64_t         total = g.sk_tiles * upt;
        if (total > 0x7fffffffull) return fail(B200_GEMM_ERR_BAD_SIZE, "too many K steps for the balanced schedule (%llu)", (unsigned long long)total);
        gp.balanced       = 1;
        gp.units_per_tile = (uint32_t)upt;
        gp.sk_tiles       = (uint32_t)g.sk_tiles;
        gp.total_units    = (uint32_t)total;
        gp.workers        = (uint32_t)g.runs;
        balanced_grid     = (uint32_t)g.grid;
    }
    const int umma_n = bn > 256 ? 256 : bn; // columns per MMA; a 512-wide tile is two sub-tiles
    gp.a_mn_major = v.a_mn ? 1u : 0u;
    gp.b_mn_major = v.b_mn ? 1u : 0u;
    // tcgen05 instruction descriptor, kind::f16: [4,6) D format (1 = f32); [7,10) A format and
    // [10,13) B format (0 = f16, 1 = bf16); bit 15 / 16: A / B is MN-major; [17,23) N >> 3;
    // [24,29) M >> 4 (M = 256 for a CTA pair).
    gp.idesc = (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | (gp.a_mn_major << 15) |
               (gp.b_mn_major << 16) | ((uint32_t)(umma_n >> 3) << 17) | ((uint32_t)((BLOCK_M * cl) >> 4) << 24);
    gp.stages = (uint32_t)cfg.stages;
    gp.status = env.d_status;
    gp.out    = nullptr;
    gp.ndst = 0;
    gp.dst_row0 = gp.dst_col0 = 0;

    gp.l2_hints = env_l2_hints() >= 0 ? (uint32_t)env_l2_hints() : 0u;
    // 512-wide tiles stagger their two column halves so the epilogue of one half hides under the
    // MMAs of the other (TileStep in gemm_kernels.cuh).  The stagger covers the time one half
    // takes to drain: about 5.5k cycles for f32 output, 3.3k for 16-bit, at 512 cycles per k-block.
    gp.stagger = 0;
    if (bn == 512) {
        const uint32_t want = (split > 1 || out == OUT_F32) ? 12u : 8u;
        gp.stagger          = std::min<uint32_t>(want, kb_per_split / 2);
    }
    // Streaming (HBM-bound) views rotate the K order per work unit; see the producer.
    static const int k_skew_env = [] { // B200_GEMM_K_SKEW = 0 / 1 forces the rotation off / on (profiling)
        const char* e = getenv("B200_GEMM_K_SKEW");
        return (e && *e) ? atoi(e) : -1;
    }();
    const bool streaming = k_skew_env >= 0 ? k_skew_env != 0 : (narrow || std::min(v.M, v.N) <= 256);
    const uint32_t slots_per_unit = (kb_per_split + kc - 1) / kc; // K steps of one work unit
    gp.k_skew = streaming ? std::max<uint32_t>(1u, slots_per_unit / std::max<uint32_t>(1u, std::min<uint32_t>((uint32_t)work, (uint32_t)env.sm_count))) : 0u;

    // Split-K partials go to this stream's cached f32 workspace, laid out [batch][split][Mk][Nk].
    float*       ws       = nullptr;
    // (balanced: one tile_rows x bn partial tile per partial segment, two slots per worker)
    const size_t ws_slots = balanced ? 2 * (size_t)gp.workers : 0;
    const size_t ws_bytes = balanced ? ws_slots * tile_rows * bn * sizeof(float)
                                     : (split > 1 && !cluster_k ? (size_t)p.batch * split * v.M * v.N * sizeof(float) : 0);
    bool         ws_stream_ordered = false;
    if ((split > 1 && !cluster_k) || balanced) {
        if (!transposed && v.N % 4) return fail(B200_GEMM_ERR_BAD_CONFIG, "split_k needs N %% 4 == 0 in the kernel view");
        if (fixed) {
            if (ws_bytes > env.fixed_ws_bytes)
                return fail(B200_GEMM_ERR_TOO_LARGE,
                            "split-K partials need %zu bytes (batch %zu x split %u x %u x %u x 4) but the built-in workspace "
                            "holds %zu; use fewer partitions or the allocating entry points",
                            ws_bytes, p.batch, split, v.M, v.N, env.fixed_ws_bytes);
            ws = env.fixed_ws;
        } else {
            // While the stream is being captured into a graph nothing may be allocated with
            // cudaMalloc; a stream-ordered allocation becomes part of the graph instead.
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            CUDA_TRY(cudaStreamIsCapturing(stream, &cap));
            if (cap != cudaStreamCaptureStatusNone) {
                CUDA_TRY(cudaMallocAsync(reinterpret_cast<void**>(&ws), ws_bytes, stream));
                ws_stream_ordered = true;
            } else {
                st = get_workspace(env.ctx, stream, ws_bytes, &ws);
                if (st != B200_GEMM_OK) return st;
            }
        }
    }

    CUtensorMap tmA, tmB, tmD, tmW;
    if (slot) {
        st = encode_operand_slab(&tmA, bf16, v.a, v.M, v.K, p.batch, v.a_mn, bm, kc, k4d);
        if (st == B200_GEMM_OK) st = encode_operand_slab(&tmB, bf16, v.b, v.N, v.K, p.batch, v.b_mn, (uint32_t)bn, kc, k4d);
    } else {
        st = encode_operand(&tmA, bf16, v.a, v.M, v.K, p.batch, v.a_mn, BLOCK_M);
        if (st == B200_GEMM_OK) st = encode_operand(&tmB, bf16, v.b, v.N, v.K, p.batch, v.b_mn, (uint32_t)umma_n / cl);
    }
    tmW = tmA; // only the balanced schedule uses it; any valid descriptor will do otherwise
    if (st == B200_GEMM_OK && transposed) {
        tmD    = tmA; // not used by the transposed epilogue; any valid descriptor will do
        gp.out = (split > 1 && !cluster_k) ? static_cast<void*>(ws) : v.d;
    } else if (st == B200_GEMM_OK) {
        if (split > 1 && !cluster_k)
            st = encode_map(&tmD, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, ws, v.N, v.M, (uint64_t)p.batch * split, 32, 32);
        else if (out == OUT_F32)
            st = encode_map(&tmD, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, v.d, v.N, v.M, p.batch, 32, 32);
        else
            st = encode_map(&tmD, out == OUT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                            v.d, v.N, v.M, p.batch, 64, 32);
        // balanced schedule: partial tiles in tile-local coordinates, one slot per partial segment
        if (st == B200_GEMM_OK && balanced)
            st = encode_map(&tmW, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, ws, (uint64_t)bn, tile_rows, ws_slots, 32, 32);
    }
    GatherMaps gmaps;
    if (st == B200_GEMM_OK && gather) {
        // Kernel view of the full matrix: a column-major C is the row-major transpose, so rows
        // and columns (and the block's offsets) swap with it.
        const bool     sw    = p.lc != 0;
        const uint64_t frows = sw ? gather->full_cols : gather->full_rows;
        const uint64_t fcols = sw ? gather->full_rows : gather->full_cols;
        gp.dst_row0          = (uint32_t)(sw ? gather->col0 : gather->row0);
        gp.dst_col0          = (uint32_t)(sw ? gather->row0 : gather->col0);
        gp.ndst              = (uint32_t)gather->ndst;
        for (int d = 0; st == B200_GEMM_OK && d < gather->ndst; ++d) {
            if (out == OUT_F32)
                st = encode_map(&gmaps.m[d], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, gather->dst[d], fcols, frows, 1, 32, 32);
            else
                st = encode_map(&gmaps.m[d], out == OUT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                2, gather->dst[d], fcols, frows, 1, 64, 32);
        }
        for (int d = gather->ndst; d < MAX_GATHER_DST; ++d) gmaps.m[d] = gmaps.m[0];
    }
    if (st != B200_GEMM_OK) {
        if (ws_stream_ordered) cudaFreeAsync(ws, stream);
        return st;
    }

    const uint32_t smem     = transposed ? slab_smem_bytes((int)bm, bn, (int)kc, cfg.stages)
                              : (slot ? slot_smem_bytes(bn, (int)kc, cfg.stages) : gemm_smem_bytes(compiled_width(bn), (int)cl, cfg.stages));
    const uint32_t units    = balanced ? balanced_grid : std::min<uint32_t>(gp.num_work, (uint32_t)env.sm_count / cl);
    const int      kern_out = (split > 1 && !cluster_k) ? OUT_F32 : out; // (balanced: whole tiles go to C in its own type)
    cudaError_t    e;
    if (cluster_k && transposed) {
        switch (bn) {
            case 16: e = launch_ksplit<16, true>(out, gp.num_work, split, smem, stream, tmA, tmB, tmD, gp); break;
            case 32: e = launch_ksplit<32, true>(out, gp.num_work, split, smem, stream, tmA, tmB, tmD, gp); break;
            case 64: e = launch_ksplit<64, true>(out, gp.num_work, split, smem, stream, tmA, tmB, tmD, gp); break;
            default: e = launch_ksplit<128, true>(out, gp.num_work, split, smem, stream, tmA, tmB, tmD, gp); break;
        }
    } else if (cluster_k) {
        if (bn == 128) e = launch_ksplit<128>(out, gp.num_work, split, smem, stream, tmA, tmB, tmD, gp);
        else e = launch_ksplit<256>(out, gp.num_work, split, smem, stream, tmA, tmB, tmD, gp);
    } else if (transposed) {
        switch (bn) {
            case 16: e = launch_bn<16, 1, true>(kern_out, units, nullptr, 0, smem, stream, tmA, tmB, tmD, tmW, gp); break;
            case 32: e = launch_bn<32, 1, true>(kern_out, units, nullptr, 0, smem, stream, tmA, tmB, tmD, tmW, gp); break;
            case 64: e = launch_bn<64, 1, true>(kern_out, units, nullptr, 0, smem, stream, tmA, tmB, tmD, tmW, gp); break;
            default: e = launch_bn<128, 1, true>(kern_out, units, nullptr, 0, smem, stream, tmA, tmB, tmD, tmW, gp); break;
        }
    } else if (cl == 2) {
        if (bn <= 128) e = launch_bn<128, 2>(kern_out, units, env.pairs, 0, smem, stream, tmA, tmB, tmD, tmW, gp);
        else if (bn <= 256) e = launch_bn<256, 2>(kern_out, units, env.pairs, 1, smem, stream, tmA, tmB, tmD, tmW, gp, gather ? &gmaps : nullptr);
        else e = launch_bn<512, 2>(kern_out, units, env.pairs, 2, smem, stream, tmA, tmB, tmD, tmW, gp, gather ? &gmaps : nullptr);
    } else {
        switch (bn) {
            case 16: e = launch_bn<16, 1>(kern_out, units, nullptr, 0, smem, stream, tmA, tmB, tmD, tmW, gp); break;
            case 32: e = launch_bn<32, 1>(kern_out, units, nullptr, 0, smem, stream, tmA, tmB, tmD, tmW, gp); break;
            case 64: e = launch_bn<64, 1>(kern_out, units, nullptr, 0, smem, stream, tmA, tmB, tmD, tmW, gp); break;
            case 128: e = launch_bn<128, 1>(kern_out, units, nullptr, 0, smem, stream, tmA, tmB, tmD, tmW, gp); break;
            default: e = launch_bn<256, 1>(kern_out, units, nullptr, 0, smem, stream, tmA, tmB, tmD, tmW, gp); break;
        }
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (e != cudaSuccess) {
        if (ws_stream_ordered) cudaFreeAsync(ws, stream);
        return fail(B200_GEMM_ERR_CUDA, "GEMM kernel launch failed: %s (tile_n=%d stages=%d smem=%u)", cudaGetErrorString(e), bn,
                    cfg.stages, smem);
    }

    if (balanced) {
        e = cudaSuccess;
        if (gp.workers > 1 && gp.sk_tiles > 0) { // one job per run boundary; each strides over one tile
            const unsigned blocks = (unsigned)std::min<uint64_t>(((uint64_t)tile_rows * (bn / 4) + 255) / 256, 32);
            e = launch_streamk_reduce(out, blocks, gp.workers - 1, stream, ws, v.d, gp, tile_rows, (uint32_t)bn);
        }
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if (ws_stream_ordered) cudaFreeAsync(ws, stream);
        if (e != cudaSuccess) return fail(B200_GEMM_ERR_CUDA, "balanced-schedule fix-up launch failed: %s", cudaGetErrorString(e));
    } else if (split > 1 && !cluster_k) {
        const uint64_t mn     = (uint64_t)v.M * v.N;
        const uint64_t total4 = mn * p.batch / 4;
        const unsigned blocks = (unsigned)std::min<uint64_t>((total4 + 255) / 256, (uint64_t)env.sm_count * 8);
        e = launch_reduce(out, blocks, stream, ws, v.d, mn, split, (uint32_t)p.batch);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if (ws_stream_ordered) cudaFreeAsync(ws, stream);
        if (e != cudaSuccess) return fail(B200_GEMM_ERR_CUDA, "split-K reduce launch failed: %s", cudaGetErrorString(e));
    }
    return B200_GEMM_OK;
}

static int run_from_abi(int types, void* C, const void* A, const void* B, size_t M, size_t N, size_t K,
                        size_t batch, int lc, int la, int lb, void* stream, const b200_gemm_config* cfg)
{
    t_last_status = B200_GEMM_OK;
    try {
        const Problem      p{types, C, A, B, M, N, K, batch, lc, la, lb};
        const cudaStream_t s = stream ? *static_cast<cudaStream_t*>(stream) : nullptr;
        return run_gemm(p, s, cfg);
    } catch (const std::exception& ex) {
        return fail(B200_GEMM_ERR_CUDA, "exception: %s", ex.what());
    } catch (...) {
        return fail(B200_GEMM_ERR_CUDA, "unknown exception");
    }
}


// ------------------------------------------------------------------------------------------
// Split-K GEMM that allocates nothing
// ------------------------------------------------------------------------------------------
// Some host programs must not allocate device memory on the call path: a serving loop whose
// memory was carved up once at start-up and is accounted to the last byte, a real-time thread
// that may not enter the driver's allocator (it can block on other threads' allocations), or a
// plugin running inside a framework that owns the allocator.  For them the f32 split-K
// partials and the device status word live in the two file-scope arrays below, which every
// GPU that loads the library holds from load to exit.
//
// g_static_workspace / g_static_status name host-side stand-ins for the device arrays; the
// device addresses come from cudaGetSymbolAddress, asked once per device with that device
// current, and only those are handed to kernels and TMA descriptors.
static __device__ __align__(256) float        g_static_workspace[B200_GEMM_STATIC_WORKSPACE_BYTES / sizeof(float)];
static __device__ __align__(256) unsigned int g_static_status[1];

struct StaticCtx {
    bool          ready    = false;
    int           sm_count = 0;
    float*        d_ws     = nullptr; // device address of g_static_workspace on this device
    unsigned int* d_status = nullptr; // device address of g_static_status on this device
    PairCache     pairs;
};
static StaticCtx g_static_ctx[k_max_devices];

// First call on a device: resolves the arrays' device addresses and sets the kernels'
// shared-memory attributes.  Allocates nothing.
static int get_static_ctx(StaticCtx** out)
{
    int         dev = -1;
    cudaError_t e   = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(B200_GEMM_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= k_max_devices) return fail(B200_GEMM_ERR_NO_DEVICE, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    StaticCtx&                  c = g_static_ctx[dev];
    if (!c.ready) {
        cudaDeviceProp prop;
        CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
        if (prop.major != 10)
            return fail(B200_GEMM_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", dev,
                        prop.major, prop.minor);
        c.sm_count = prop.multiProcessorCount;
        if (!g_encode) {
            void*                           fn = nullptr;
            cudaDriverEntryPointQueryResult qr;
            CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr));
            if (!fn || qr != cudaDriverEntryPointSuccess)
                return fail(B200_GEMM_ERR_CUDA, "cuTensorMapEncodeTiled not available");
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
        }
        CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&c.d_ws), g_static_workspace));
        CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&c.d_status), g_static_status));
        CUDA_TRY(set_all_kernel_attributes());
        c.ready = true;
    }
    *out = &c;
    return B200_GEMM_OK;
}

// The allocation-free twin of run_gemm: same planning and launch code (launch_gemm), with the
// status word and the split-K workspace taken from the arrays above.
static int run_gemm_static(const Problem& p, cudaStream_t stream, const b200_gemm_config* user_cfg)
{
    int st = validate(p);
    if (st != B200_GEMM_OK) return st;
    if (p.M == 0 || p.N == 0) return B200_GEMM_OK;
    if (p.K == 0) return fail(B200_GEMM_ERR_BAD_SIZE, "K == 0 is not handled by the allocation-free entry point");

    StaticCtx* ctx = nullptr;
    st             = get_static_ctx(&ctx);
    if (st != B200_GEMM_OK) return st;
    const LaunchEnv env{ctx->sm_count, ctx->d_status, &ctx->pairs, nullptr, ctx->d_ws, (size_t)B200_GEMM_STATIC_WORKSPACE_BYTES};
    return launch_gemm(p, stream, user_cfg, env);
}

} // namespace b200

// ==============================================================================================
// C ABI
// ==============================================================================================
using namespace b200;

#define B200_DEFINE_PAIR(suffix, types)                                                              \
    extern "C" int b200_gemm_##suffix(void* C, void* A, void* B, size_t M, size_t N, size_t K,       \
                                      size_t batch_count, int layout_c, int layout_a, int layout_b,  \
                                      void* stream)                                                  \
    {                                                                                                \
        return run_from_abi(types, C, A, B, M, N, K, batch_count, layout_c, layout_a, layout_b,      \
                            stream, nullptr);                                                        \
    }                                                                                                \
    extern "C" void rocm_wmma_gemm_##suffix(void* C, void* A, void* B, size_t M, size_t N, size_t K, \
                                            size_t batch_count, int layout_c, int layout_a,          \
                                            int layout_b, void* stream)                              \
    {                                                                                                \
        (void)run_from_abi(types, C, A, B, M, N, K, batch_count, layout_c, layout_a, layout_b,       \
                           stream, nullptr);                                                         \
    }

B200_DEFINE_PAIR(f16_f16, B200_GEMM_F16_F16)
B200_DEFINE_PAIR(f32_f16, B200_GEMM_F32_F16)
B200_DEFINE_PAIR(bf16_bf16, B200_GEMM_BF16_BF16)
B200_DEFINE_PAIR(f32_bf16, B200_GEMM_F32_BF16)

extern "C" int b200_gemm_ex(int types, void* C, const void* A, const void* B, size_t M, size_t N,
                            size_t K, size_t batch_count, int layout_c, int layout_a, int layout_b,
                            void* stream, const b200_gemm_config* cfg)
{
    return run_from_abi(types, C, A, B, M, N, K, batch_count, layout_c, layout_a, layout_b, stream, cfg);
}

extern "C" int b200_gemm_select_config(size_t M, size_t N, size_t K, int types, int layout_c,
                                       int layout_a, int layout_b, b200_gemm_config* out)
{
    if (types < 0 || types > 3) return -fail(B200_GEMM_ERR_BAD_CONFIG, "unknown type pair %d", types);
    if ((layout_c | layout_a | layout_b) & ~1) return -fail(B200_GEMM_ERR_BAD_LAYOUT, "layout ints must be 0 or 1");
    const int i = find_best_config(M, N, K, out_is_f32(types) ? 1 : 0, layout_a, layout_b, layout_c);
    if (out) *out = k_configs[i];
    return i;
}

// SM count the planning functions assume: the current device's, or a B200's 148 when the
// process has no usable device (the functions are pure host code).
static int planning_sm_count(int requested)
{
    if (requested > 0) return requested;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0)
        return sms;
    (void)cudaGetLastError();
    return 148;
}

// A problem with stand-in, 256-byte aligned operand addresses (planning never dereferences them).
static Problem planning_problem(int types, size_t M, size_t N, size_t K, size_t batch, int lc, int la, int lb)
{
    return Problem{types, reinterpret_cast<void*>(uintptr_t(0x1000)), reinterpret_cast<const void*>(uintptr_t(0x2000)),
                   reinterpret_cast<const void*>(uintptr_t(0x3000)), M, N, K, batch, lc, la, lb};
}

extern "C" size_t b200_gemm_workspace_bytes(int types, size_t M, size_t N, size_t K, size_t batch_count,
                                            int layout_c, int layout_a, int layout_b,
                                            const b200_gemm_config* user)
{
    if (types < 0 || types > 3 || ((layout_c | layout_a | layout_b) & ~1) || M == 0 || N == 0 || K == 0 || batch_count == 0)
        return 0;
    const Problem p = planning_problem(types, M, N, K, batch_count, layout_c, layout_a, layout_b);
    LaunchPlan    pl;
    if (make_plan(p, user, planning_sm_count(0), &pl) != B200_GEMM_OK || pl.generic) return 0;
    if (pl.balanced) {
        const uint32_t cl      = (uint32_t)pl.cfg.cluster;
        const uint32_t tile_m  = pl.slot ? pl.bm : (uint32_t)BLOCK_M * cl;
        const uint64_t tiles   = (uint64_t)((pl.v.M + tile_m - 1) / tile_m) * ((pl.v.N + pl.cfg.tile_n - 1) / pl.cfg.tile_n) * batch_count;
        const uint64_t upt     = ((pl.v.K + BLOCK_K - 1) / BLOCK_K + pl.kc - 1) / pl.kc;
        const uint64_t runs    = balanced_geometry(tiles, upt, (uint64_t)planning_sm_count(0) / cl).runs;
        return (size_t)(2 * runs) * tile_m * pl.cfg.tile_n * sizeof(float);
    }
    return (pl.cfg.split_k > 1 && !pl.cluster_k) ? batch_count * (size_t)pl.cfg.split_k * M * N * sizeof(float) : 0;
}

extern "C" int b200_gemm_plan(int types, size_t M, size_t N, size_t K, size_t batch_count, int layout_c,
                              int layout_a, int layout_b, int sm_count, b200_gemm_plan_info* out)
{
    t_last_status = B200_GEMM_OK;
    if (!out) return fail(B200_GEMM_ERR_NULL_POINTER, "out is NULL");
    const Problem p  = planning_problem(types, M, N, K, batch_count, layout_c, layout_a, layout_b);
    int           st = validate(p);
    if (st != B200_GEMM_OK) return st;
    *out = b200_gemm_plan_info{};
    if (M == 0 || N == 0 || K == 0) return B200_GEMM_OK; // nothing is launched (K == 0: a memset)
    const int  sms = planning_sm_count(sm_count);
    LaunchPlan pl;
    st = make_plan(p, nullptr, sms, &pl);
    if (st != B200_GEMM_OK) return st;
    if (pl.generic) {
        out->kernel = B200_GEMM_KERNEL_GENERIC;
        return B200_GEMM_OK;
    }
    const uint32_t cl      = (uint32_t)pl.cfg.cluster;
    const uint32_t tile_m  = pl.slot ? pl.bm : (uint32_t)BLOCK_M * cl;
    const uint64_t m_tiles = (pl.v.M + tile_m - 1) / tile_m;
    const uint64_t n_tiles = (pl.v.N + pl.cfg.tile_n - 1) / pl.cfg.tile_n;
    const uint64_t work    = m_tiles * n_tiles * batch_count * (uint64_t)pl.cfg.split_k;
    out->kernel            = pl.transposed ? B200_GEMM_KERNEL_TRANSPOSED : B200_GEMM_KERNEL_STAGED;
    out->tile_m            = (int)tile_m;
    out->tile_n            = pl.cfg.tile_n;
    out->cluster           = pl.cfg.cluster;
    out->split_k           = pl.balanced ? 0 : pl.cfg.split_k;
    out->slots             = pl.cfg.stages;
    out->k_blocks_per_slot = (int)pl.kc;
    out->raster            = pl.cfg.raster;
    const uint64_t upt     = (((uint64_t)pl.v.K + BLOCK_K - 1) / BLOCK_K + pl.kc - 1) / pl.kc;
    const uint64_t workers = pl.balanced ? balanced_geometry(work, upt, (uint64_t)sms / cl).grid : std::min<uint64_t>(work, (uint64_t)sms / cl);
    out->ctas              = pl.cluster_k ? (int)work : (int)(cl * workers);
    out->work_units        = (long long)work;
    out->cluster_k         = pl.cluster_k ? 1 : 0;
    return B200_GEMM_OK;
}

extern "C" int b200_gemm_slab(size_t N, int world, int rank, size_t align, size_t* n_begin, size_t* n_count)
{
    if (world < 1 || rank < 0 || rank >= world || align == 0 || !n_begin || !n_count)
        return fail(B200_GEMM_ERR_BAD_SIZE, "bad slab request: world=%d rank=%d align=%zu", world, rank, align);
    // Slab width: N / world rounded up to a multiple of `align`; trailing ranks may get a
    // narrower (or empty) slab.
    const size_t units = (N + align - 1) / align;
    const size_t per   = ((units + world - 1) / world) * align;
    const size_t b     = std::min(N, per * (size_t)rank);
    const size_t e     = std::min(N, b + per);
    *n_begin           = b;
    *n_count           = e - b;
    return B200_GEMM_OK;
}

extern "C" int b200_gemm_host(int types, void* C, const void* A, const void* B, size_t M, size_t N, size_t K,
                              size_t batch_count, int layout_c, int layout_a, int layout_b)
{
    t_last_status = B200_GEMM_OK;
    const Problem p{types, C, A, B, M, N, K, batch_count, layout_c, layout_a, layout_b};
    int           st = validate(p);
    if (st != B200_GEMM_OK) return st;
    if (M == 0 || N == 0) return B200_GEMM_OK;
    DeviceCtx* ctx = nullptr;
    st             = get_ctx(&ctx);
    if (st != B200_GEMM_OK) return st;
    // One host-buffer call at a time per device: the staging buffers, the three streams and the
    // events below are per device, and the call ends in a synchronise anyway.
    std::lock_guard<std::mutex> host_lock(ctx->host_mutex);
    const size_t out_sz   = out_is_f32(types) ? 4 : 2;
    const size_t bytes[3] = {M * K * batch_count * 2, K * N * batch_count * 2, M * N * batch_count * out_sz};
    {
        if (!ctx->h_stream) CUDA_TRY(cudaStreamCreateWithFlags(&ctx->h_stream, cudaStreamNonBlocking));
        for (int i = 0; i < 3; ++i) {
            if (ctx->h_cap[i] < bytes[i]) {
                if (ctx->h_buf[i]) CUDA_TRY(cudaFree(ctx->h_buf[i]));
                ctx->h_buf[i] = nullptr;
                ctx->h_cap[i] = 0;
                CUDA_TRY(cudaMalloc(&ctx->h_buf[i], std::max<size_t>(bytes[i], 256)));
                ctx->h_cap[i] = std::max<size_t>(bytes[i], 256);
            }
        }
    }
    cudaStream_t s = ctx->h_stream;

    // Large single problems are pipelined in two dimensions: A goes up in chunks of rows, B in
    // chunks of columns, alternately; a tile of C is computed as soon as its row chunk and its
    // column chunk are on the device and goes down while later chunks still come up (PCIe is
    // full duplex).  Four chunks per dimension: the download of a tile is a strided 2-D copy
    // whose rate grows with the length of its contiguous runs (timed with events per copy on
    // 8192^3 f32: 1024-column tiles come down at 28-36 GB/s, the link does 44 GB/s each way),
    // so fewer, wider tiles win over an earlier start: 8 x 8 chunks 7.75 ms per GEMM, 8 x 4
    // 7.3, 4 x 4 7.15, 16 x 8 8.2.  Chunks and tiles are stored densely on the device, so every
    // tile is an ordinary dense GEMM whatever the layouts; strided sides are host-side 2-D copies.
    auto chunk_starts = [](size_t dim) { // chunk boundaries, multiples of 256 (last one = dim)
        std::vector<size_t> b{0};
        if (dim < 2048) {
            b.push_back(dim);
            return b;
        }
        // B200_GEMM_HOST_CHUNKS="first,count" (profiling): a first chunk of `first` rows / columns,
        // the rest in `count` equal chunks.  Default: the measured optimum below.
        static const struct Scheme {
            size_t first = 0, count = 4;
            Scheme()
            {
                const char* e = getenv("B200_GEMM_HOST_CHUNKS");
                unsigned long f = 0, c = 0;
                if (e && sscanf(e, "%lu,%lu", &f, &c) == 2 && c >= 1 && c <= 12) {
                    first = f / 256 * 256;
                    count = c;
                }
            }
        } scheme;
        size_t at = 0;
        if (scheme.first && scheme.first < dim / 2) b.push_back(at = scheme.first);
        const size_t step = ((dim - at + scheme.count - 1) / scheme.count + 255) / 256 * 256;
        while (dim - at > step) b.push_back(at += step);
        b.push_back(dim);
        return b;
    };
    const std::vector<size_t> rb = chunk_starts(M), cb = chunk_starts(N);
    const size_t              nra = rb.size() - 1, ncb = cb.size() - 1;
    if (batch_count == 1 && nra * ncb >= 2 && bytes[0] + bytes[1] + bytes[2] >= (32u << 20) && K > 0) {
        {
            if (!ctx->h_in) {
                CUDA_TRY(cudaStreamCreateWithFlags(&ctx->h_in, cudaStreamNonBlocking));
                CUDA_TRY(cudaStreamCreateWithFlags(&ctx->h_out, cudaStreamNonBlocking));
                for (int i = 0; i < 16; ++i) {
                    CUDA_TRY(cudaEventCreateWithFlags(&ctx->h_ev_a[i], cudaEventDisableTiming));
                    CUDA_TRY(cudaEventCreateWithFlags(&ctx->h_ev_b[i], cudaEventDisableTiming));
                }
                for (int i = 0; i < 256; ++i) CUDA_TRY(cudaEventCreateWithFlags(&ctx->h_ev_done[i], cudaEventDisableTiming));
            }
        }
        char*        dA    = static_cast<char*>(ctx->h_buf[0]);
        char*        dB    = static_cast<char*>(ctx->h_buf[1]);
        char*        dC    = static_cast<char*>(ctx->h_buf[2]);
        const char*  hA    = static_cast<const char*>(A);
        const char*  hB    = static_cast<const char*>(B);
        char*        hC    = static_cast<char*>(C);
        size_t       ntile = 0;
        auto tile = [&](size_t i, size_t j) -> int {
            const size_t r0 = rb[i], rn = rb[i + 1] - r0;
            const size_t c0 = cb[j], cn = cb[j + 1] - c0;
            CUDA_TRY(cudaStreamWaitEvent(s, ctx->h_ev_a[i], 0));
            CUDA_TRY(cudaStreamWaitEvent(s, ctx->h_ev_b[j], 0));
            // tiles of row chunk i are packed one after the other behind the chunks before it
            char*         dT = dC + (r0 * N + rn * c0) * out_sz;
            const Problem tp{types, dT, dA + r0 * K * 2, dB + c0 * K * 2, rn, cn, K, 1, layout_c, layout_a, layout_b};
            const int     ts = run_gemm(tp, s, nullptr);
            if (ts != B200_GEMM_OK) return ts;
            cudaEvent_t done = ctx->h_ev_done[ntile++];
            CUDA_TRY(cudaEventRecord(done, s));
            CUDA_TRY(cudaStreamWaitEvent(ctx->h_out, done, 0));
            if (layout_c == 0)
                CUDA_TRY(cudaMemcpy2DAsync(hC + (r0 * N + c0) * out_sz, N * out_sz, dT, cn * out_sz, cn * out_sz, rn,
                                           cudaMemcpyDeviceToHost, ctx->h_out));
            else
                CUDA_TRY(cudaMemcpy2DAsync(hC + (c0 * M + r0) * out_sz, M * out_sz, dT, rn * out_sz, rn * out_sz, cn,
                                           cudaMemcpyDeviceToHost, ctx->h_out));
            return B200_GEMM_OK;
        };
        for (size_t t = 0; t < std::max(nra, ncb); ++t) {
            if (t < nra) { // rows [r0, r0 + rn) of A
                const size_t r0 = rb[t], rn = rb[t + 1] - r0;
                char*        d  = dA + r0 * K * 2;
                if (layout_a == 0) CUDA_TRY(cudaMemcpyAsync(d, hA + r0 * K * 2, rn * K * 2, cudaMemcpyHostToDevice, ctx->h_in));
                else CUDA_TRY(cudaMemcpy2DAsync(d, rn * 2, hA + r0 * 2, M * 2, rn * 2, K, cudaMemcpyHostToDevice, ctx->h_in));
                CUDA_TRY(cudaEventRecord(ctx->h_ev_a[t], ctx->h_in));
            }
            if (t < ncb) { // columns [c0, c0 + cn) of B
                const size_t c0 = cb[t], cn = cb[t + 1] - c0;
                char*        d  = dB + c0 * K * 2;
                if (layout_b == 1) CUDA_TRY(cudaMemcpyAsync(d, hB + c0 * K * 2, cn * K * 2, cudaMemcpyHostToDevice, ctx->h_in));
                else CUDA_TRY(cudaMemcpy2DAsync(d, cn * 2, hB + c0 * 2, N * 2, cn * 2, K, cudaMemcpyHostToDevice, ctx->h_in));
                CUDA_TRY(cudaEventRecord(ctx->h_ev_b[t], ctx->h_in));
            }
            // the tiles the two new chunks complete: row chunk t x columns 0..t, rows 0..t-1 x column chunk t
            if (t < nra)
                for (size_t j = 0; j <= std::min(t, ncb - 1); ++j)
                    if ((st = tile(t, j)) != B200_GEMM_OK) break;
            if (st == B200_GEMM_OK && t < ncb)
                for (size_t i = 0; i < std::min(t, nra); ++i)
                    if ((st = tile(i, t)) != B200_GEMM_OK) break;
            if (st != B200_GEMM_OK) {
                cudaDeviceSynchronize();
                return st;
            }
        }
        CUDA_TRY(cudaStreamSynchronize(ctx->h_out));
        CUDA_TRY(cudaStreamSynchronize(s));
        return B200_GEMM_OK;
    }

    if (bytes[0]) CUDA_TRY(cudaMemcpyAsync(ctx->h_buf[0], A, bytes[0], cudaMemcpyHostToDevice, s));
    if (bytes[1]) CUDA_TRY(cudaMemcpyAsync(ctx->h_buf[1], B, bytes[1], cudaMemcpyHostToDevice, s));
    const Problem dp{types, ctx->h_buf[2], ctx->h_buf[0], ctx->h_buf[1], M, N, K, batch_count, layout_c, layout_a, layout_b};
    st = run_gemm(dp, s, nullptr);
    if (st != B200_GEMM_OK) return st;
    CUDA_TRY(cudaMemcpyAsync(C, ctx->h_buf[2], bytes[2], cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaStreamSynchronize(s));
    return B200_GEMM_OK;
}

extern "C" int b200_gemm_device_status(unsigned int* detail)
{
    DeviceCtx* ctx = nullptr;
    int        st  = get_ctx(&ctx);
    if (st != B200_GEMM_OK) return st;
    CUDA_TRY(cudaDeviceSynchronize());
    unsigned int word = 0;
    CUDA_TRY(cudaMemcpy(&word, ctx->d_status, sizeof(word), cudaMemcpyDeviceToHost));
    if (detail) *detail = word;
    if (word != 0) {
        CUDA_TRY(cudaMemset(ctx->d_status, 0, sizeof(word)));
        return fail(B200_GEMM_ERR_DEVICE_WAIT, "a kernel gave up on a bounded wait (status word 0x%x)", word);
    }
    return B200_GEMM_OK;
}

extern "C" int b200_gemm_static_status(unsigned int* detail)
{
    t_last_status  = B200_GEMM_OK;
    StaticCtx* ctx = nullptr;
    int        st  = get_static_ctx(&ctx);
    if (st != B200_GEMM_OK) return st;
    CUDA_TRY(cudaDeviceSynchronize());
    unsigned int word = 0;
    CUDA_TRY(cudaMemcpy(&word, ctx->d_status, sizeof(word), cudaMemcpyDeviceToHost));
    if (detail) *detail = word;
    if (word != 0) {
        CUDA_TRY(cudaMemset(ctx->d_status, 0, sizeof(word)));
        return fail(B200_GEMM_ERR_DEVICE_WAIT, "a kernel of the allocation-free entry point gave up on a bounded wait (status word 0x%x)", word);
    }
    return B200_GEMM_OK;
}

extern "C" int b200_gemm_last_status(void) { return t_last_status; }
extern "C" const char* b200_gemm_last_error(void) { return t_last_error; }
extern "C" const char* b200_gemm_version(void) { return "b200_gemm 0.1 (sm_100a)"; }
extern "C" unsigned long long b200_gemm_launch_count(void) { return g_launches.load(); }

extern "C" int b200_gemm_splitk_static(int types, void* C, const void* A, const void* B, size_t M, size_t N, size_t K,
                                       size_t batch_count, int layout_c, int layout_a, int layout_b, void* stream,
                                       const b200_gemm_config* cfg)
{
    t_last_status = B200_GEMM_OK;
    try {
        const Problem      p{types, C, A, B, M, N, K, batch_count, layout_c, layout_a, layout_b};
        const cudaStream_t s = stream ? *static_cast<cudaStream_t*>(stream) : nullptr;
        return run_gemm_static(p, s, cfg);
    } catch (const std::exception& ex) {
        return fail(B200_GEMM_ERR_CUDA, "exception: %s", ex.what());
    } catch (...) {
        return fail(B200_GEMM_ERR_CUDA, "unknown exception");
    }
}

#ifdef B200_GEMM_TIMELINE
// Timeline builds only (see gemm_kernels.cuh): copies of the stamps, after a device synchronise
// (b200_gemm_debug_reset clears them).
// `out` holds TIMELINE_ROWS x TIMELINE_SLOTS values, `count` the launches stamped so far (row of
// launch i: i % TIMELINE_ROWS); `cta` holds 3 x TIMELINE_CTAS globaltimer values (first load,
// end of main loop, end) of the last launch's CTAs.
extern "C" int b200_gemm_debug_timeline(unsigned long long* out, unsigned int* count)
{
    if (cudaDeviceSynchronize() != cudaSuccess) return B200_GEMM_ERR_CUDA;
    if (cudaMemcpyFromSymbol(out, b200::g_timeline, sizeof(b200::g_timeline)) != cudaSuccess) return B200_GEMM_ERR_CUDA;
    if (cudaMemcpyFromSymbol(count, b200::g_timeline_count, sizeof(unsigned int)) != cudaSuccess) return B200_GEMM_ERR_CUDA;
    return B200_GEMM_OK;
}
extern "C" int b200_gemm_debug_reset()
{
    if (cudaDeviceSynchronize() != cudaSuccess) return B200_GEMM_ERR_CUDA;
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, b200::g_timeline) != cudaSuccess || cudaMemset(p, 0, sizeof(b200::g_timeline)) != cudaSuccess) return B200_GEMM_ERR_CUDA;
    if (cudaGetSymbolAddress(&p, b200::g_cta_times) != cudaSuccess || cudaMemset(p, 0, sizeof(b200::g_cta_times)) != cudaSuccess) return B200_GEMM_ERR_CUDA;
    if (cudaGetSymbolAddress(&p, b200::g_timeline_count) != cudaSuccess || cudaMemset(p, 0, sizeof(unsigned int)) != cudaSuccess) return B200_GEMM_ERR_CUDA;
    return B200_GEMM_OK;
}
extern "C" int b200_gemm_debug_cta_times(unsigned long long* cta)
{
    if (cudaDeviceSynchronize() != cudaSuccess) return B200_GEMM_ERR_CUDA;
    if (cudaMemcpyFromSymbol(cta, b200::g_cta_times, sizeof(b200::g_cta_times)) != cudaSuccess) return B200_GEMM_ERR_CUDA;
    return B200_GEMM_OK;
}
#endif

#include "slab_driver.inc"
