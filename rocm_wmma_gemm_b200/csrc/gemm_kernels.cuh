// Device kernels of the B200 GEMM library.
//
//   gemm_umma_kernel   persistent, warp-specialised tcgen05 GEMM; one CTA per 128 x BN tile or a
//                      CTA pair per 256 x BN tile
//   splitk_reduce_kernel   deterministic sum of split-K partials + conversion to the output type
//   gemm_generic_kernel    CUDA-core GEMM for shapes whose leading dimensions TMA cannot address
//
// "Kernel view" of a problem: D (Mk x Nk, row-major) = A' (Mk x K) * B' (K x Nk) where each
// operand is either K-major (K contiguous) or MN-major (its M or N extent contiguous).  The
// host maps the reference's eight layout combinations onto this view; a column-major C is
// the row-major C^T = B^T * A^T, i.e. the operands swap roles
// (reference semantics: rocm_wmma_gemm/include/rocm_wmma_gemm/gemm.hpp:50-73).
#pragma once

#include "ptx_sm100.cuh"

#include <type_traits>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200 {

// ---------------------------------------------------------------------------------------------
// Launch timeline (builds with -DB200_GEMM_TIMELINE only; the macros are empty otherwise).
// CTA 0 of every GEMM launch stamps clock64() at fixed points of its three roles into one row
// of g_timeline (64 rows, used round-robin; slots 0 and 15 hold globaltimer values instead),
// and every CTA stamps globaltimer at its first load, at the end of its main loop and at its
// end into g_cta_times: where a launch spends its time between the dependency wait and the
// last store, and how evenly the CTAs of a grid finish.  Read back by b200_gemm_debug_timeline /
// b200_gemm_debug_cta_times (gemm_lib.cu) and printed by rocm_wmma_gemm_b200/timeline.py.
//   0 entry (globaltimer)  1 entry  2 set-up done  3 dependency wait done (producer)
//   4 first TMA load issued  5 last TMA load issued  6 first ring slot full (MMA thread)
//   7 last accumulator committed  8 MMAs drained  9 accumulator seen by the epilogue
//   10 first store issued  11 last store issued  12 staging buffers read  13 tail barrier
//   14 TMEM freed  15 producer ready to wait (globaltimer)
//   cluster K partitions: 16 before / 17 after the first cluster barrier  18 partials sent
//   19 after the second barrier  20 sums stored  21 staging buffers read
// ---------------------------------------------------------------------------------------------
#ifdef B200_GEMM_TIMELINE
constexpr int TIMELINE_ROWS = 64, TIMELINE_SLOTS = 24, TIMELINE_CTAS = 1024;
__device__ unsigned long long g_timeline[TIMELINE_ROWS * TIMELINE_SLOTS];
__device__ unsigned int       g_timeline_count;
__device__ unsigned long long g_cta_times[3 * TIMELINE_CTAS];
#define B200_TL(slot)                                                   \
    do {                                                                \
        if (blockIdx.x == 0) g_timeline[tl_base + (slot)] = clock64(); \
    } while (0)
#define B200_TLG(slot)                                                                 \
    do {                                                                               \
        if (blockIdx.x == 0) g_timeline[tl_base + (slot)] = ptx::global_timer_ns();   \
    } while (0)
#define B200_TL_CTA(row)                                                                                         \
    do {                                                                                                         \
        if (blockIdx.x < TIMELINE_CTAS) g_cta_times[(row) * TIMELINE_CTAS + blockIdx.x] = ptx::global_timer_ns(); \
    } while (0)
#else
#define B200_TL(slot) do { } while (0)
#define B200_TLG(slot) do { } while (0)
#define B200_TL_CTA(row) do { } while (0)
#endif

// Output element kinds of the epilogue.
enum : int { OUT_F32 = 0, OUT_F16 = 1, OUT_BF16 = 2 };

// Bits of the device status word (set when a bounded wait expires).
enum : unsigned int {
    ST_PRODUCER_WAIT = 1u,  // TMA producer waiting for a free ring slot
    ST_MMA_WAIT_FULL = 2u,  // MMA issuer waiting for a filled ring slot
    ST_MMA_WAIT_ACC  = 4u,  // MMA issuer waiting for a drained accumulator
    ST_EPI_WAIT      = 8u,  // epilogue waiting for a finished accumulator
    ST_DRAIN_WAIT    = 16u, // tail waiting for outstanding MMAs / loads
    ST_PEER_WAIT     = 32u  // CTA-pair handshake
};

struct GemmParams {
    uint32_t M, N, K;      // kernel-view extents
    uint32_t batch;        // batch count
    uint32_t m_tiles;      // ceil(M / (128 * cluster))
    uint32_t n_tiles;      // ceil(N / BN)
    uint32_t k_blocks;     // ceil(K / 64)
    uint32_t split_k;      // K partitions (>= 1); every partition owns >= 1 k-block
    uint32_t kb_per_split; // k-blocks per partition
    uint32_t group_m;      // raster band height in tiles (0 = sweep columns)
    uint32_t num_work;     // batch * split_k * m_tiles * n_tiles
    uint32_t a_mn_major;   // 0: A' K-major, 1: A' M-major
    uint32_t b_mn_major;   // 0: B' K-major, 1: B' N-major
    uint32_t idesc;        // tcgen05 instruction descriptor
    uint32_t stages;       // ring depth actually used (<= MAX_STAGES)
    unsigned int* status;  // device status word
    void*    out;          // transposed epilogue only: base of the (Nk x Mk, row-major) output
    uint32_t k_skew;       // work unit w starts its K loop (w * k_skew) k-blocks in (0 = in order)
    uint32_t stagger;      // 512-wide tiles: k-blocks by which the two column halves are staggered
    uint32_t bm;           // one-CTA kernels: rows of A' per tile (128; 8 .. 128 with the transposed epilogue)
    uint32_t wn;           // CTA-pair kernels up to 256 columns: columns per tile actually used (<= BN)
    uint32_t kc;           // one-CTA kernels: k-blocks per ring slot (1, 2 or 4)
    uint32_t k4d;          // one-CTA kernels: K-major operands use the 4-D (chunked K) maps
    uint32_t snake;        // raster: odd bands (odd columns of a column sweep) run backwards
    uint32_t l2_hints;     // L2 eviction priorities: bits [0,2) A', [2,4) B', [4,6) D (L2_HINT_*)
    uint32_t balanced;     // 1: balanced (stream-K) schedule, see WorkCursor
    uint32_t units_per_tile; // balanced: K steps (ring slots of kc k-blocks) per tile
    uint32_t workers;      // balanced: runs the cut tiles' K loops are divided into (<= persistent CTAs / CTA pairs)
    uint32_t total_units;  // balanced: sk_tiles x units_per_tile
    uint32_t sk_tiles;     // balanced: tiles [0, sk_tiles) are cut into runs; tiles [sk_tiles, num_work) are dealt whole
    uint32_t ndst;         // gathering kernels: number of destination matrices every tile is stored to
    uint32_t dst_row0;     // gathering kernels: row and column of D(0, 0) within each destination
    uint32_t dst_col0;
    uint32_t cluster_k;    // 1: the split_k K partitions of a tile are the CTAs of one cluster, summed through
                           //    distributed shared memory (work items are tiles; the cluster rank is the partition)
};

// Destinations of a gathering kernel: one tensor map per copy of the full output matrix (this
// GPU's own and its peers'), all of the same shape.
constexpr int MAX_GATHER_DST = 8;
struct GatherMaps {
    CUtensorMap m[MAX_GATHER_DST];
};

// L2 eviction priority of one operand's TMA traffic (GemmParams::l2_hints).
enum : uint32_t { L2_HINT_NONE = 0u, L2_HINT_EVICT_FIRST = 1u, L2_HINT_EVICT_LAST = 2u };

constexpr int      BLOCK_M        = 128;
constexpr int      BLOCK_K        = 64; // 64 x 2 B = one 128-byte swizzle row
constexpr int      UMMA_K         = 16;
constexpr int      MAX_STAGES     = 12; // ring depth of the staged-epilogue kernels
constexpr int      MAX_SLAB_STAGES = 24; // ring depth of the transposed-epilogue (slab) kernels
constexpr int      GEMM_THREADS   = 192; // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr uint32_t A_TILE_BYTES   = BLOCK_M * BLOCK_K * 2;
constexpr uint32_t EPI_BUF_BYTES  = 32 * 128; // one warp's 32 rows x 128 B
constexpr uint32_t EPI_BYTES      = 4 * 2 * EPI_BUF_BYTES;
constexpr uint64_t WAIT_LIMIT_NS  = 2000000000ull; // 2 s per bounded wait

// Bytes of one ring slot in one CTA: A' 128 x 64 plus B' (bn / cluster) x 64.
__host__ __device__ constexpr uint32_t stage_bytes(int bn, int cluster)
{
    return A_TILE_BYTES + static_cast<uint32_t>(bn / cluster) * BLOCK_K * 2;
}

// Dynamic shared memory a launch needs (1 KiB slack for manual 1024-byte alignment).  The
// transposed epilogue stores straight from registers and needs no staging.
__host__ __device__ constexpr uint32_t gemm_smem_bytes(int bn, int cluster, int stages, bool transposed = false)
{
    return static_cast<uint32_t>(stages) * stage_bytes(bn, cluster) + (transposed ? 0u : EPI_BYTES) + 1024;
}

// Transposed-epilogue kernels stage `bm` <= 128 rows of A' per slot (a "slab"): the MMA still
// reads 128 rows, so the ring is followed by the slack the last slot's read runs into.
constexpr uint32_t SLAB_SMEM_LIMIT = 232448u - 1024u; // 227 KiB minus the static barriers
// A slot holds `kc` consecutive k-blocks of both operands (one TMA instruction per operand
// fetches all of them: the per-slot barrier and issue work is amortised over kc k-blocks).
__host__ __device__ constexpr uint32_t slab_stage_bytes(int bm, int bn, int kc)
{
    return static_cast<uint32_t>(kc) * static_cast<uint32_t>(bm + bn) * BLOCK_K * 2;
}
// The MMA reads 128 rows of A' whatever the slab height, i.e. up to 16 KiB (K-major) or kc x 8 KiB
// (a 64-row M-major slab) past the last slot: the ring is followed by that much slack.
__host__ __device__ constexpr uint32_t slab_slack_bytes(int kc)
{
    return kc * 8192u > 16384u ? kc * 8192u : 16384u;
}
__host__ __device__ constexpr uint32_t slab_smem_bytes(int bm, int bn, int kc, int stages)
{
    return static_cast<uint32_t>(stages) * slab_stage_bytes(bm, bn, kc) + slab_slack_bytes(kc) + 1024;
}
__host__ __device__ constexpr int slab_max_stages(int bm, int bn, int kc)
{
    int s = static_cast<int>((SLAB_SMEM_LIMIT - 1024u - slab_slack_bytes(kc)) / slab_stage_bytes(bm, bn, kc));
    return s > MAX_SLAB_STAGES ? MAX_SLAB_STAGES : s;
}

// One-CTA kernels with the staged epilogue and kc k-blocks per slot.
__host__ __device__ constexpr uint32_t slot_smem_bytes(int bn, int kc, int stages)
{
    return static_cast<uint32_t>(stages) * kc * stage_bytes(bn, 1) + EPI_BYTES + 1024;
}
__host__ __device__ constexpr int slot_max_stages(int bn, int kc)
{
    int s = static_cast<int>((232448u - 512u - EPI_BYTES - 1024u) / (kc * stage_bytes(bn, 1)));
    return s > MAX_STAGES ? MAX_STAGES : s;
}

// Deepest ring that fits the 227 KiB a CTA may use (static barriers included).
__host__ __device__ constexpr int max_stages(int bn, int cluster, bool transposed = false)
{
    int s = static_cast<int>((232448u - 512u - (transposed ? 0u : EPI_BYTES) - 1024u) / stage_bytes(bn, cluster));
    return s > MAX_STAGES ? MAX_STAGES : s;
}

// Waits for the phase with the given parity; gives up after WAIT_LIMIT_NS or as soon as
// another role of this CTA has given up.  Returns false on give-up.  CLUSTER_SCOPE selects an
// acquire at cluster scope (the arrivals come from the peer CTA's threads).
template <bool CLUSTER_SCOPE = false>
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity,
                                             volatile uint32_t* s_abort, unsigned int* status,
                                             unsigned int code)
{
    auto try_wait = [&]() {
        if constexpr (CLUSTER_SCOPE) return ptx::mbar_try_wait_cluster(bar, parity);
        else return ptx::mbar_try_wait(bar, parity);
    };
    // The common case is a short wait: try_wait itself blocks for a while, so the timer (a slow
    // read) and the abort flag are only looked at every 128 failed attempts, and the deadline
    // starts at the first look.
    if constexpr (!CLUSTER_SCOPE) {
        if (ptx::mbar_test_wait(bar, parity)) return true; // already complete: no blocking wait
    }
    uint64_t t0    = 0;
    uint32_t spins = 0;
    while (true) {
        if (try_wait()) return true;
        if ((++spins & 127u) == 0u) {
            if (*s_abort != 0u) return false;
            const uint64_t now = ptx::global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > WAIT_LIMIT_NS) {
                *s_abort = 1u;
                atomicOr(status, code);
                return false;
            }
        }
    }
}

struct WorkCoord {
    uint32_t m0, n0;   // first row / column of the tile
    uint32_t z_in;     // batch index (third TMA coordinate of A' and B')
    uint32_t z_out;    // third TMA coordinate of D: batch * split_k + split
    uint32_t kb0, kb1; // k-block range
    uint32_t partial;  // balanced schedule: the segment is only part of its tile's K loop (f32 partial to the workspace)
};

// Tile index -> (tile-row, tile-column) under the problem's raster.
// Raster (the reference's tile_mapper, kernel/mapping.hpp:108-287): tiles are walked in bands
// of group_m tile-rows, tile-rows fastest, so that the tiles in flight share a panel of A'
// and a few panels of B' in L2.  With `snake` every other band runs its columns backwards
// (and every other column its rows): the first tiles of a band reuse the B' panels the last
// tiles of the band before it have just read.
__device__ __forceinline__ void tile_coords(const GemmParams& p, uint32_t t, uint32_t& m_idx, uint32_t& n_idx)
{
    if (p.group_m == 0u) {
        m_idx = t % p.m_tiles;
        n_idx = t / p.m_tiles;
        if (p.snake && (n_idx & 1u)) m_idx = p.m_tiles - 1u - m_idx;
    } else {
        const uint32_t per_group = p.group_m * p.n_tiles;
        const uint32_t g         = t / per_group;
        const uint32_t first_m   = g * p.group_m;
        const uint32_t gsize     = min(p.group_m, p.m_tiles - first_m);
        const uint32_t in_g      = t - g * per_group;
        uint32_t       m_in      = in_g % gsize;
        n_idx                    = in_g / gsize;
        if (p.snake) {
            if (n_idx & 1u) m_in = gsize - 1u - m_in;
            if (g & 1u) n_idx = p.n_tiles - 1u - n_idx;
        }
        m_idx = first_m + m_in;
    }
}

__device__ __forceinline__ WorkCoord decode_work(const GemmParams& p, uint32_t w, int bn, int bm, uint32_t krank)
{
    const uint32_t tiles = p.m_tiles * p.n_tiles;
    const uint32_t t     = w % tiles;
    const uint32_t r     = w / tiles;
    const uint32_t split = p.cluster_k ? krank : r % p.split_k;
    const uint32_t b     = p.cluster_k ? r : r / p.split_k;
    uint32_t       m_idx, n_idx;
    tile_coords(p, t, m_idx, n_idx);
    WorkCoord c;
    c.m0    = m_idx * static_cast<uint32_t>(bm);
    c.n0    = n_idx * static_cast<uint32_t>(bn);
    c.z_in  = b;
    c.z_out = p.cluster_k ? b : b * p.split_k + split;
    c.kb0   = split * p.kb_per_split;
    c.kb1   = min(p.k_blocks, c.kb0 + p.kb_per_split);
    c.partial = 0u;
    return c;
}

// ---------------------------------------------------------------------------------------------
// Work of one persistent worker (a CTA, or a CTA pair).
//
// Plain schedule: work items unit, unit + units, ... of the num_work (batch x K partition x
// tile) items.
//
// Balanced schedule (stream-K; the reference's roadmap names it, README.md:202).  Whole waves
// of tiles need no balancing, so only the tiles of the incomplete wave - sk_tiles = tiles mod
// workers, or all of them when there are fewer tiles than workers - are cut: their K loops are
// laid end to end - tile 0's K steps, then tile 1's, ... - and that line of total_units steps
// is cut into `workers` equal runs, one per worker, wherever the cuts fall.  A worker first
// walks its run segment by segment (a segment = the part of one tile's K loop inside the run)
// and then takes whole tiles sk_tiles + worker, sk_tiles + worker + grid, ... like the plain
// schedule: every SM gets the same number of K steps whatever the tile count, and the cut
// tiles' partials are written early in the kernel, not at its end.  A segment that covers a
// tile's whole K loop stores the tile to C like the plain schedule does.  A partial segment
// leaves an f32 partial tile in the workspace: a run has at most two of them, its first (it
// starts inside a tile: slot 2 * worker) and its last (it ends inside a tile: slot
// 2 * worker + 1); the fix-up pass (streamk_reduce_kernel) adds a split tile's partials in
// K order and writes C.  No CTA waits for another.
// ---------------------------------------------------------------------------------------------
struct WorkCursor {
    uint32_t next;  // plain: next work item; balanced: next K step of the run
    uint32_t end;   // balanced: end of the run
    uint32_t krank; // cluster K partitions: this CTA's partition (its rank in the cluster)
    uint32_t dp;    // balanced: next whole tile of this worker
};

__device__ __forceinline__ uint32_t run_start(const GemmParams& p, uint32_t worker)
{
    return static_cast<uint32_t>(static_cast<uint64_t>(worker) * p.total_units / p.workers);
}

__device__ __forceinline__ WorkCursor work_begin(const GemmParams& p, uint32_t unit, uint32_t krank = 0u)
{
    WorkCursor cur;
    cur.krank = krank;
    cur.dp = 0u;
    if (p.balanced) {
        const bool has_run = unit < p.workers;
        cur.next = has_run ? run_start(p, unit) : 0u;
        cur.end  = has_run ? run_start(p, unit + 1u) : 0u;
        cur.dp   = p.sk_tiles + unit;
    } else {
        cur.next = unit;
        cur.end  = p.num_work;
    }
    return cur;
}

// Next piece of work of this worker; false when there is none left.
__device__ __forceinline__ bool work_next(const GemmParams& p, WorkCursor& cur, uint32_t unit, uint32_t units,
                                          int bn, int bm, WorkCoord& c)
{
    if (!p.balanced) {
        if (cur.next >= cur.end) return false;
        c = decode_work(p, cur.next, bn, bm, cur.krank);
        cur.next += units;
        return true;
    }
    if (cur.next >= cur.end) { // the run is done: whole tiles, round-robin over the grid
        if (cur.dp >= p.num_work) return false;
        const uint32_t tiles = p.m_tiles * p.n_tiles;
        uint32_t       m_idx, n_idx;
        tile_coords(p, cur.dp % tiles, m_idx, n_idx);
        c.m0      = m_idx * static_cast<uint32_t>(bm);
        c.n0      = n_idx * static_cast<uint32_t>(bn);
        c.z_in    = cur.dp / tiles;
        c.z_out   = c.z_in;
        c.partial = 0u;
        c.kb0     = 0u;
        c.kb1     = p.k_blocks;
        cur.dp += units;
        return true;
    }
    const uint32_t tile  = cur.next / p.units_per_tile;          // over batch x tiles
    const uint32_t first = cur.next - tile * p.units_per_tile;   // first K step of the segment within the tile
    const uint32_t last  = min(p.units_per_tile, first + (cur.end - cur.next));
    const uint32_t tiles = p.m_tiles * p.n_tiles;
    uint32_t       m_idx, n_idx;
    tile_coords(p, tile % tiles, m_idx, n_idx);
    c.m0    = m_idx * static_cast<uint32_t>(bm);
    c.n0    = n_idx * static_cast<uint32_t>(bn);
    c.z_in    = tile / tiles;
    c.partial = (first != 0u || last != p.units_per_tile) ? 1u : 0u;
    // whole tile: third coordinate of C (the batch index); partial: the workspace slot
    c.z_out   = c.partial ? 2u * unit + (first != 0u ? 0u : 1u) : c.z_in;
    c.kb0     = first * p.kc;
    c.kb1     = min(p.k_blocks, last * p.kc);
    cur.next += last - first;
    return true;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c),
                 "r"(d)
                 : "memory");
}

// TMA load whose completion bytes go to `bar`: this CTA's barrier (CL = 1) or a
// shared::cluster address naming the pair leader's barrier (CL = 2).
template <int CL>
__device__ __forceinline__ void tma_load(uint32_t dst, const CUtensorMap* tm, uint32_t bar,
                                         int32_t c0, int32_t c1, int32_t c2, uint64_t policy)
{
    if constexpr (CL == 2) ptx::tma_load_3d_pair(dst, tm, bar, c0, c1, c2, policy);
    else ptx::tma_load_3d(dst, tm, bar, c0, c1, c2, policy);
}

// tcgen05.commit arriving on `bar` of this CTA (CL = 1) or of both CTAs of the pair (CL = 2).
template <int CL>
__device__ __forceinline__ void umma_arrive(uint32_t bar)
{
    if constexpr (CL == 2) ptx::umma_commit_pair(bar, 0x3);
    else ptx::umma_commit(bar);
}

// Schedule of a 512-wide tile (two 256-column halves that share the staged A' tile).
// With a stagger of X k-blocks a work unit of nkb k-blocks runs nkb + X steps:
//   steps [0, X)          half 0 alone on k-blocks 0 .. X-1
//   steps [X, nkb)        both halves on k-block s (one A' tile feeds two MMAs)
//   steps [nkb, nkb + X)  half 1 alone on k-blocks 0 .. X-1 (its K order is rotated by X)
// Half 0 is complete X steps before half 1, so its accumulator drains while half 1 finishes,
// and half 1 drains under the next tile's half-0-only steps: the tensor pipe does not wait for
// the epilogue although one tile fills all 512 TMEM columns.  Cost: A' k-blocks 0 .. X-1 are
// staged twice.
struct TileStep {
    uint32_t kb_rel; // k-block relative to the work unit's first
    uint32_t mask;   // bit h set: column half h takes part
};

__device__ __forceinline__ TileStep tile_step(uint32_t s, uint32_t nkb, uint32_t stagger)
{
    TileStep t;
    if (s < stagger) {
        t.kb_rel = s;
        t.mask   = 1u;
    } else if (s < nkb) {
        t.kb_rel = s;
        t.mask   = 3u;
    } else {
        t.kb_rel = s - nkb;
        t.mask   = 2u;
    }
    return t;
}

template <int OUT>
__device__ __forceinline__ uint32_t pack2(uint32_t lo_bits, uint32_t hi_bits)
{
    const float lo = __uint_as_float(lo_bits);
    const float hi = __uint_as_float(hi_bits);
    if constexpr (OUT == OUT_F16) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    } else {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
}

// ---------------------------------------------------------------------------------------------
// Persistent tcgen05 GEMM.  CL = 1: one CTA per 128 x BN output tile.  CL = 2: a cluster of two
// CTAs (a "pair", ranks 0 and 1) per 256 x BN tile; each CTA loads its own 128 rows of A' and
// its own BN/2 columns of B', rank 0 issues one cta_group::2 MMA per K = 16 slice that reads
// both CTAs' shared memory and writes both CTAs' TMEM (each holds its 128 rows x BN columns).
// The pair halves the B' bytes each SM has to stage per FLOP.
//
//   warp 0 (one elected lane)  TMA producer: fills a `stages`-deep ring of slots (128-byte
//                      swizzle): {A' 128x64, B' (BN/CL)x64} per slot, or - one-CTA kernels up to
//                      256 columns - kc k-blocks of {A' bm x 64, B' BN x 64}, one TMA instruction
//                      per operand.  Slot s has a `full` barrier (bytes landed; for a pair it
//                      lives in rank 0 and counts both CTAs' bytes) and an `empty` barrier
//                      (MMAs that read the slot have retired).
//   warp 1 (one elected lane)  MMA issuer (rank 0 only for a pair): 4 x tcgen05.mma per
//                      k-block into one of the TMEM accumulators (BN f32 columns each);
//                      tcgen05.commit releases the slot and, after the last k-block, publishes
//                      the accumulator.  (The two single threads are chosen with elect.sync:
//                      the compiler then issues TMA / MMA / commit from uniform registers.)
//   warps 2..5         epilogue: tcgen05.ld 32 lanes x 32 columns, convert, swizzled store to a
//                      per-warp staging buffer, TMA store of 32 rows x 128 B; the accumulator
//                      is handed back as soon as its last column chunk is in registers, so the
//                      epilogue of tile i overlaps the main loop of tile i + 1.  TR = true:
//                      the transposing epilogue of skinny problems (direct coalesced stores).
//
// Edges: TMA zero-fills out-of-range loads (M, N and K tails) and clips stores.
// No TMA load here uses cluster multicast.
// ---------------------------------------------------------------------------------------------
template <int BN, int OUT, int CL, bool TR, bool GATHER, bool KS = false>
__device__ __forceinline__ void gemm_umma_body(const CUtensorMap& tmA, const CUtensorMap& tmB,
                                               const CUtensorMap* tmDs, const CUtensorMap& tmW, const GemmParams& p)
{
    const CUtensorMap& tmD = tmDs[0];
    static_assert(BN == 16 || BN == 32 || BN == 64 || BN == 128 || BN == 256 || BN == 512,
                  "BN must be 16, 32, 64, 128, 256 or 512");
    static_assert(CL == 1 || CL == 2, "cluster size must be 1 or 2");
    static_assert(!TR || CL == 1, "the transposed epilogue is a one-CTA variant");
    static_assert(!KS || (CL == 1 && !GATHER && ((!TR && BN >= 128 && BN <= 256) || (TR && BN <= 128))),
                  "cluster K partitions: one-CTA staged tiles of 128 or 256 columns, transposed slabs of up to 128");
    // One MMA covers at most 256 columns: a 512-wide tile is two sub-tiles that share the A'
    // operand of every K slice (A' is staged once for 512 columns of output).
    constexpr int      UMMA_N       = BN > 256 ? 256 : BN;
    constexpr int      NSUB         = BN / UMMA_N;
    constexpr int      SUB_ROWS     = UMMA_N / CL;          // B' rows per sub-tile in this CTA
    constexpr int      BN_CTA       = NSUB * SUB_ROWS;      // B' rows this CTA stages
    constexpr uint32_t SUB_BYTES    = SUB_ROWS * BLOCK_K * 2;
    constexpr uint32_t B_TILE_BYTES = BN_CTA * BLOCK_K * 2;
    constexpr uint32_t STAGE_BYTES  = A_TILE_BYTES + B_TILE_BYTES;
    // TMEM holds 512 f32 columns: two accumulators (epilogue of tile i overlaps the main loop
    // of tile i + 1) up to BN = 256, a single one for BN = 512.
    constexpr uint32_t NUM_ACC      = BN > 256 ? 1 : 2;
    constexpr uint32_t ACC_COLS     = BN < 64 ? 64 : BN; // the epilogue reads up to 64 columns at a time
    constexpr uint32_t TMEM_COLS    = NUM_ACC * ACC_COLS; // power of two >= 32
    constexpr int      OUT_BYTES    = (OUT == OUT_F32) ? 4 : 2;
    constexpr int      CH           = 128 / OUT_BYTES; // output columns per 128-byte chunk
    constexpr int      NCHUNK       = BN < CH ? 1 : BN / CH; // a narrow tile is one (clipped) chunk
    static_assert(SUB_ROWS >= 16, "each CTA stages at least 16 rows of B' per sub-tile");
    // (an MN-major B' is loaded in 64-row boxes: the host only picks BN >= 64 * CL for it)

#ifdef B200_GEMM_TIMELINE
    __shared__ uint32_t s_tl_base;
    if (blockIdx.x == 0 && threadIdx.x == 0) s_tl_base = (atomicAdd(&g_timeline_count, 1u) % TIMELINE_ROWS) * TIMELINE_SLOTS;
    uint32_t tl_base = 0;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        tl_base = s_tl_base;
        B200_TLG(0);
        B200_TL(1);
    }
#endif
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_full[TR ? MAX_SLAB_STAGES : MAX_STAGES];
    __shared__ __align__(8) uint64_t s_empty[TR ? MAX_SLAB_STAGES : MAX_STAGES];
    __shared__ __align__(8) uint64_t s_tfull[2];
    __shared__ __align__(8) uint64_t s_tempty[2];
    __shared__ __align__(8) uint64_t s_drain;
    __shared__ uint32_t              s_tmem_base;
    __shared__ volatile uint32_t     s_abort;

    const uint32_t tid    = threadIdx.x;
    const uint32_t warp   = tid >> 5;
    const uint32_t lane   = tid & 31u;
    const uint32_t stages = p.stages;
    const uint32_t rank   = (CL == 2) ? ptx::cluster_ctarank() : 0u; // CTA rank in the pair
    // KS: the cluster is the worker, its rank the K partition (p.split_k CTAs per cluster).
    const uint32_t krank  = KS ? ptx::cluster_ctarank() : 0u;
    const uint32_t unit   = KS ? blockIdx.x / p.split_k : blockIdx.x / CL; // persistent worker index
    const uint32_t units  = KS ? gridDim.x / p.split_k : gridDim.x / CL;
    WorkCoord      ks_c{};        // KS: the one tile of this cluster (epilogue warps)
    bool           ks_ok = false; // KS: accumulator complete

    // Bytes of A' per ring slot and slot pitch: compile-time for the staged epilogue; the
    // transposed variant stages p.bm (a multiple of 8, <= 128) rows of A' per slot.
    // One-CTA kernels up to 256 columns use "slots" of kc k-blocks:
    // [A' k-block 0 .. kc-1][B' k-block 0 .. kc-1], each operand fetched by one TMA instruction
    // (the per-slot barrier and issue work of the two single-thread roles is amortised over kc
    // k-blocks; with narrow tiles that work, not the tensor pipe, bounds the K loop).  A' has
    // p.bm rows per k-block: 128, or a shorter slab with the transposed epilogue.
    constexpr bool SLOT    = (CL == 1) && (NSUB == 1);
    const uint32_t kc      = SLOT ? p.kc : 1u;
    const uint32_t a_bytes = SLOT ? p.bm * (BLOCK_K * 2u) : A_TILE_BYTES;
    const uint32_t pitch   = SLOT ? kc * (a_bytes + B_TILE_BYTES) : STAGE_BYTES;
    const uint32_t tile_m  = SLOT ? p.bm : static_cast<uint32_t>(BLOCK_M * CL);
    // CTA-pair kernels up to 256 columns take the tile width at run time (any multiple of the
    // epilogue's 128-byte chunk up to BN): the MMA's N extent is a field of the instruction
    // descriptor and the B' box height a field of the tensor map, so one compiled kernel serves
    // widths that cut N into whole waves of tiles.  Ring slots and TMEM stay sized for BN.
    constexpr bool FLEX     = (CL == 2) && (NSUB == 1);
    const uint32_t wn       = FLEX ? p.wn : static_cast<uint32_t>(BN);
    const uint32_t sub_rows = FLEX ? wn / CL : static_cast<uint32_t>(SUB_ROWS);
    const uint32_t sub_bytes = FLEX ? sub_rows * (BLOCK_K * 2u) : SUB_BYTES;

    const uint32_t ring = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u; // ring of operand tiles
    const uint32_t epi  = ring + stages * pitch;                      // epilogue staging (unused when TR)

    if (warp == 0) {
        // Barrier set-up spread over the lanes of warp 0 (one thread doing all of it serially is
        // a third of a microsecond of every launch; small problems notice).
        if (lane == 0) {
            ptx::prefetch_tensormap(&tmA);
            ptx::prefetch_tensormap(&tmB);
            if constexpr (GATHER) {
                for (uint32_t d = 0; d < p.ndst; ++d) ptx::prefetch_tensormap(&tmDs[d]);
            } else {
                ptx::prefetch_tensormap(&tmD);
            }
            ptx::mbar_init(ptx::smem_u32(&s_drain), 1);
            s_abort = 0u;
        }
        if (lane < stages) {
            ptx::mbar_init(ptx::smem_u32(&s_full[lane]), 1);
            ptx::mbar_init(ptx::smem_u32(&s_empty[lane]), 1);
        }
        if (lane >= 30u) {
            ptx::mbar_init(ptx::smem_u32(&s_tfull[lane - 30u]), 1);
            ptx::mbar_init(ptx::smem_u32(&s_tempty[lane - 30u]), 4 * CL);
        }
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc<CL>(ptx::smem_u32(&s_tmem_base), TMEM_COLS);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if constexpr (CL == 2) { // the peer's barriers must exist before anything arrives on them
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
    ptx::tc_fence_after();
#ifdef B200_GEMM_TIMELINE
    tl_base = s_tl_base;
    if (threadIdx.x == 0) B200_TL(2);
#endif
    const uint32_t tmem_base = s_tmem_base;
    // Programmatic dependent launch, both directions.  This grid may have been scheduled while
    // the kernel before it in the stream was still draining: everything above touched only this
    // CTA's shared memory and TMEM.  Each thread that touches global memory waits for the kernel
    // before this one right before its first access (the producer before its first TMA load, the
    // epilogue threads before their first store), so the work decode, the address arithmetic and
    // the first barrier operations of every role run while that kernel drains - about a
    // microsecond of every launch otherwise.  The MMA thread touches no global memory.  The
    // kernel after this one (a reduction pass, or the next GEMM) may be scheduled as SMs free
    // up; it waits for this grid to complete before it reads or writes anything.
    ptx::grid_dep_launch();
    bool dep_waited = false;
    auto dep_wait = [&]() {
        if (!dep_waited) {
            ptx::grid_dep_wait();
            dep_waited = true;
        }
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (ptx::elect_one()) {
            uint32_t stage = 0, phase = 0, issued = 0;
            bool     ok = true;
            const uint64_t pol_a = ptx::make_l2_policy(p.l2_hints & 3u);
            const uint64_t pol_b = ptx::make_l2_policy((p.l2_hints >> 2) & 3u);
            WorkCursor cur = work_begin(p, unit, krank);
            WorkCoord  c;
            for (uint32_t w = unit; ok && work_next(p, cur, unit, units, wn, tile_m, c); w += units) {
                const int32_t   am = static_cast<int32_t>(c.m0 + rank * BLOCK_M);
                const int32_t   bn = static_cast<int32_t>(c.n0 + rank * sub_rows);
                // Streaming (HBM-bound) problems rotate each work unit's K order so that the CTAs
                // running at the same time read different K offsets: rows of a K-major operand
                // are a power of two apart, and same-offset reads from thousands of rows land on
                // a few memory channels.
                const uint32_t nkb = c.kb1 - c.kb0;
                if constexpr (SLOT) {
                    // One slot = kc k-blocks of A' (p.bm rows) and of B' (BN rows),
                    // one TMA instruction per operand (per 64-row half for an MN-major operand).
                    // Boxes that reach past K read zeros, so a ragged last slot needs no care.
                    // Two cluster K partitions are interleaved: rank r takes the ring-slot-sized K
                    // steps r, r + 2, r + 4, ... so that the two CTAs, which run in step, read
                    // neighbouring pieces of the same operand rows at the same time.  (Measured
                    // 1 - 5 % faster than two contiguous halves on 128x8192x8192; four interleaved
                    // partitions measured 8 % slower than four contiguous quarters.)
                    const bool     ileave = KS && p.split_k == 2u;
                    const uint32_t nst  = ileave ? ((p.k_blocks + kc - 1u) / kc + 1u - krank) / 2u : (nkb + kc - 1u) / kc;
                    const uint32_t rot  = (p.k_skew && nst) ? static_cast<uint32_t>((static_cast<uint64_t>(w) * p.k_skew) % nst) : 0u;
                    const uint32_t half = kc * (64u * BLOCK_K * 2u); // bytes of one 64-row half of an MN-major operand
                    for (uint32_t i = 0; i < nst; ++i) {
                        const uint32_t rel = i + rot >= nst ? i + rot - nst : i + rot;
                        const int32_t  kb  = ileave ? static_cast<int32_t>((krank + rel * 2u) * kc)
                                                    : static_cast<int32_t>(c.kb0 + rel * kc);
                        const int32_t  k0  = kb * BLOCK_K;
                        ok = bounded_wait(ptx::smem_u32(&s_empty[stage]), phase ^ 1u, &s_abort,
                                          p.status, ST_PRODUCER_WAIT);
                        if (!ok) break;
                        const uint32_t sa  = ring + stage * pitch;
                        const uint32_t sb  = sa + kc * a_bytes;
                        const uint32_t bar = ptx::smem_u32(&s_full[stage]);
                        ptx::mbar_expect_tx(bar, pitch);
                        if (issued == 0) B200_TLG(15);
                        dep_wait();
                        if (issued == 0) {
                            B200_TL(3);
                            B200_TL_CTA(0);
                        }
                        if (p.a_mn_major == 0u) {
                            if (p.k4d) ptx::tma_load_4d(sa, &tmA, bar, 0, am, kb, c.z_in, pol_a);
                            else ptx::tma_load_3d(sa, &tmA, bar, k0, am, c.z_in, pol_a);
                        } else {
                            ptx::tma_load_3d(sa, &tmA, bar, am, k0, c.z_in, pol_a);
                            if (p.bm > 64u) ptx::tma_load_3d(sa + half, &tmA, bar, am + 64, k0, c.z_in, pol_a);
                        }
                        if (p.b_mn_major == 0u) {
                            if (p.k4d) ptx::tma_load_4d(sb, &tmB, bar, 0, bn, kb, c.z_in, pol_b);
                            else ptx::tma_load_3d(sb, &tmB, bar, k0, bn, c.z_in, pol_b);
                        } else {
#pragma unroll
                            for (int j = 0; j < SUB_ROWS / 64; ++j)
                                ptx::tma_load_3d(sb + j * half, &tmB, bar, bn + j * 64, k0, c.z_in, pol_b);
                        }
                        if (issued == 0) B200_TL(4);
                        ++issued;
                        B200_TL(5);
                        if (++stage == stages) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                    continue;
                }
                const uint32_t rot = p.k_skew ? static_cast<uint32_t>((static_cast<uint64_t>(w) * p.k_skew) % nkb) : 0u;
                const uint32_t stg_x  = (NSUB == 2) ? min(p.stagger, nkb) : 0u;
                const uint32_t nsteps = nkb + stg_x;
                for (uint32_t i = 0; i < nsteps; ++i) {
                    const TileStep ts   = (NSUB == 2) ? tile_step(i, nkb, stg_x) : TileStep{i, 1u};
                    const uint32_t rel  = ts.kb_rel + rot >= nkb ? ts.kb_rel + rot - nkb : ts.kb_rel + rot;
                    const uint32_t kb   = c.kb0 + rel;
                    const uint32_t nsub = (NSUB == 2) ? __popc(ts.mask) : 1u;
                    ok = bounded_wait(ptx::smem_u32(&s_empty[stage]), phase ^ 1u, &s_abort,
                                      p.status, ST_PRODUCER_WAIT);
                    if (!ok) break;
                    const uint32_t sa = ring + stage * pitch;
                    const uint32_t sb = sa + a_bytes;
                    const int32_t  k0 = static_cast<int32_t>(kb * BLOCK_K);
                    const uint32_t step_bytes = a_bytes + nsub * sub_bytes; // this CTA's share
                    uint32_t       bar = ptx::smem_u32(&s_full[stage]);
                    if constexpr (CL == 2) {
                        // Rank 0 owns the pair's full barrier and expects both CTAs' bytes.
                        if (rank == 0) ptx::mbar_expect_tx(bar, 2 * step_bytes);
                        bar = ptx::mapa_u32(bar, 0);
                    } else {
                        ptx::mbar_expect_tx(bar, step_bytes);
                    }
                    if (issued == 0) B200_TLG(15);
                    dep_wait();
                    if (issued == 0) {
                        B200_TL(3);
                        B200_TL_CTA(0);
                    }
                    if (p.a_mn_major == 0u) {
                        tma_load<CL>(sa, &tmA, bar, k0, am, c.z_in, pol_a);
                    } else {
#pragma unroll
                        for (int j = 0; j < BLOCK_M / 64; ++j)
                            tma_load<CL>(sa + j * (64 * BLOCK_K * 2), &tmA, bar, am + j * 64, k0,
                                         c.z_in, pol_a);
                    }
#pragma unroll
                    for (int h = 0; h < NSUB; ++h) {
                        if (NSUB == 2 && !((ts.mask >> h) & 1u)) continue;
                        const int32_t  bh = bn + h * UMMA_N; // first B' row of sub-tile h
                        const uint32_t sh = sb + h * SUB_BYTES;
                        if (p.b_mn_major == 0u) {
                            tma_load<CL>(sh, &tmB, bar, k0, bh, c.z_in, pol_b);
                        } else {
#pragma unroll
                            for (int j = 0; j < SUB_ROWS / 64; ++j)
                                if (!FLEX || static_cast<uint32_t>(j) * 64u < sub_rows)
                                    tma_load<CL>(sh + j * (64 * BLOCK_K * 2), &tmB, bar, bh + j * 64,
                                                 k0, c.z_in, pol_b);
                        }
                    }
                    if (issued == 0) B200_TL(4);
                    ++issued;
                    B200_TL(5);
                    if (++stage == stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (s_abort != 0u && rank == 0) {
                // Gave up somewhere: let the loads already in flight land before the CTA exits.
                const uint32_t pending = min(issued, stages);
                for (uint32_t i = 0; i < pending; ++i) {
                    if (stage == 0) {
                        stage = stages;
                        phase ^= 1u;
                    }
                    --stage;
                    const uint64_t t0 = ptx::global_timer_ns();
                    while (!ptx::mbar_try_wait(ptx::smem_u32(&s_full[stage]), phase)) {
                        if (ptx::global_timer_ns() - t0 > WAIT_LIMIT_NS) {
                            atomicOr(p.status, ST_DRAIN_WAIT);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (ptx::elect_one() && rank == 0) {
            // K-major swizzled tiles ignore the leading offset (canonical value: 16 bytes).
            const uint32_t a_lbo   = p.a_mn_major ? 64u * BLOCK_K * 2u : 16u;
            const uint32_t b_lbo   = p.b_mn_major ? 64u * BLOCK_K * 2u : 16u;
            // Descriptor start-address step (16-byte units) per K = 16 slice.
            const uint32_t a_kstep = p.a_mn_major ? (2u * 1024u) >> 4 : (UMMA_K * 2u) >> 4;
            const uint32_t b_kstep = p.b_mn_major ? (2u * 1024u) >> 4 : (UMMA_K * 2u) >> 4;
            uint32_t       stage = 0, phase = 0, it = 0;
            bool           ok = true;
            WorkCursor cur = work_begin(p, unit, krank);
            WorkCoord  c;
            for (; ok && work_next(p, cur, unit, units, wn, tile_m, c); ++it) {
                if constexpr (NSUB == 2) {
                    // Two column halves with their own full / empty barriers (s_tfull[h],
                    // s_tempty[h]), staggered by stg_x k-blocks: see TileStep.  Three
                    // straight-line loops (half 0 alone, both, half 1 alone): the MMAs of one
                    // step must be issued back to back, with no branch between the two halves
                    // that share an A' tile — a conditional in this loop costs 10 % of the
                    // kernel's throughput.
                    const uint32_t nkb    = c.kb1 - c.kb0;
                    const uint32_t stg_x  = min(p.stagger, nkb);
                    const uint32_t tphase = it & 1u;
                    auto step = [&](auto mask_c, uint32_t acc0, uint32_t acc1) -> bool {
                        constexpr uint32_t MASK = decltype(mask_c)::value;
                        if (!bounded_wait(ptx::smem_u32(&s_full[stage]), phase, &s_abort, p.status,
                                          ST_MMA_WAIT_FULL))
                            return false;
                        ptx::tc_fence_after();
                        const uint32_t sa = ring + stage * pitch;
                        const uint32_t sb = sa + a_bytes;
                        const uint64_t ad = ptx::make_smem_desc(sa, a_lbo, 1024u);
                        const uint64_t bd = ptx::make_smem_desc(sb, b_lbo, 1024u);
#pragma unroll
                        for (uint32_t k = 0; k < BLOCK_K / UMMA_K; ++k) {
                            if constexpr ((MASK & 1u) != 0u)
                                ptx::umma_f16<CL>(tmem_base, ad + k * a_kstep, bd + k * b_kstep, p.idesc,
                                                  (acc0 | k) ? 1u : 0u);
                            if constexpr ((MASK & 2u) != 0u)
                                ptx::umma_f16<CL>(tmem_base + UMMA_N, ad + k * a_kstep,
                                                  bd + (SUB_BYTES >> 4) + k * b_kstep, p.idesc,
                                                  (acc1 | k) ? 1u : 0u);
                        }
                        umma_arrive<CL>(ptx::smem_u32(&s_empty[stage]));
                        if (++stage == stages) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        return true;
                    };
                    // half 0 starts: its columns must have been drained
                    ok = bounded_wait<CL == 2>(ptx::smem_u32(&s_tempty[0]), tphase ^ 1u, &s_abort, p.status,
                                               ST_MMA_WAIT_ACC);
                    for (uint32_t i = 0; ok && i < stg_x; ++i)
                        ok = step(std::integral_constant<uint32_t, 1u>{}, i > 0u ? 1u : 0u, 0u);
                    if (!ok) break;
                    // half 1 starts
                    ok = bounded_wait<CL == 2>(ptx::smem_u32(&s_tempty[1]), tphase ^ 1u, &s_abort, p.status,
                                               ST_MMA_WAIT_ACC);
                    for (uint32_t i = stg_x; ok && i < nkb; ++i)
                        ok = step(std::integral_constant<uint32_t, 3u>{}, i > 0u ? 1u : 0u, i > stg_x ? 1u : 0u);
                    if (!ok) break;
                    umma_arrive<CL>(ptx::smem_u32(&s_tfull[0])); // half 0 complete
                    for (uint32_t i = 0; ok && i < stg_x; ++i)
                        ok = step(std::integral_constant<uint32_t, 2u>{}, 0u, (nkb > stg_x || i > 0u) ? 1u : 0u);
                    if (!ok) break;
                    umma_arrive<CL>(ptx::smem_u32(&s_tfull[1])); // half 1 complete
                    B200_TL(7);
                    continue;
                }
                const uint32_t buf    = it % NUM_ACC;
                const uint32_t aphase = (it / NUM_ACC) & 1u;
                ok = bounded_wait<CL == 2>(ptx::smem_u32(&s_tempty[buf]), aphase ^ 1u, &s_abort,
                                           p.status, ST_MMA_WAIT_ACC);
                if (!ok) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * ACC_COLS;
                if constexpr (SLOT) {
                    // kc k-blocks per slot; see the producer for the slot layout.
                    const uint32_t nst    = (KS && p.split_k == 2u) ? ((p.k_blocks + kc - 1u) / kc + 1u - krank) / 2u // interleaved, see the producer
                                                                    : (c.kb1 - c.kb0 + kc - 1u) / kc;
                    const uint32_t half   = kc * (64u * BLOCK_K * 2u);
                    const uint32_t a_blk  = p.a_mn_major ? 64u * BLOCK_K * 2u : a_bytes;
                    const uint32_t b_blk  = p.b_mn_major ? 64u * BLOCK_K * 2u : B_TILE_BYTES;
                    const uint32_t a_lbo2 = p.a_mn_major ? half : 16u;
                    const uint32_t b_lbo2 = p.b_mn_major ? half : 16u;
                    for (uint32_t i = 0; i < nst; ++i) {
                        ok = bounded_wait(ptx::smem_u32(&s_full[stage]), phase, &s_abort, p.status,
                                          ST_MMA_WAIT_FULL);
                        if (!ok) break;
                        if (i == 0 && it == 0) B200_TL(6);
                        ptx::tc_fence_after();
                        const uint32_t sa = ring + stage * pitch;
                        const uint32_t sb = sa + kc * a_bytes;
                        for (uint32_t c2 = 0; c2 < kc; ++c2) {
                            const uint64_t ad = ptx::make_smem_desc(sa + c2 * a_blk, a_lbo2, 1024u);
                            const uint64_t bd = ptx::make_smem_desc(sb + c2 * b_blk, b_lbo2, 1024u);
#pragma unroll
                            for (uint32_t k = 0; k < BLOCK_K / UMMA_K; ++k) {
                                ptx::umma_f16<CL>(d_tmem, ad + k * a_kstep, bd + k * b_kstep, p.idesc,
                                                  (i | c2 | k) ? 1u : 0u);
                            }
                        }
                        umma_arrive<CL>(ptx::smem_u32(&s_empty[stage]));
                        if (++stage == stages) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                } else {
                    for (uint32_t kb = c.kb0; kb < c.kb1; ++kb) {
                        ok = bounded_wait(ptx::smem_u32(&s_full[stage]), phase, &s_abort, p.status,
                                          ST_MMA_WAIT_FULL);
                        if (!ok) break;
                        if (kb == c.kb0 && it == 0) B200_TL(6);
                        ptx::tc_fence_after();
                        const uint32_t sa = ring + stage * pitch;
                        const uint32_t sb = sa + a_bytes;
                        const uint64_t ad = ptx::make_smem_desc(sa, a_lbo, 1024u);
                        const uint64_t bd = ptx::make_smem_desc(sb, b_lbo, 1024u);
#pragma unroll
                        for (uint32_t k = 0; k < BLOCK_K / UMMA_K; ++k) {
                            ptx::umma_f16<CL>(d_tmem, ad + k * a_kstep, bd + k * b_kstep, p.idesc,
                                              (kb > c.kb0 || k > 0u) ? 1u : 0u);
                        }
                        // Slot free (in both CTAs of a pair) once these MMAs retire.
                        umma_arrive<CL>(ptx::smem_u32(&s_empty[stage]));
                        if (++stage == stages) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                }
                if (!ok) break;
                umma_arrive<CL>(ptx::smem_u32(&s_tfull[buf])); // accumulator complete
                B200_TL(7);
            }
            // All MMAs must have retired before TMEM is released and shared memory goes away.
            if constexpr (CL == 2) ptx::umma_commit_pair(ptx::smem_u32(&s_drain), 0x1);
            else ptx::umma_commit(ptx::smem_u32(&s_drain));
            const uint64_t t0 = ptx::global_timer_ns();
            while (!ptx::mbar_try_wait(ptx::smem_u32(&s_drain), 0u)) {
                if (ptx::global_timer_ns() - t0 > WAIT_LIMIT_NS) {
                    atomicOr(p.status, ST_DRAIN_WAIT);
                    break;
                }
            }
            B200_TL(8);
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const uint32_t q    = warp & 3u; // TMEM lane quarter this warp may read
        const uint32_t stg  = epi + q * 2u * EPI_BUF_BYTES;
        uint32_t       it   = 0, nstore = 0;
        bool           ok   = true;
        const uint64_t pol_d = ptx::make_l2_policy((p.l2_hints >> 4) & 3u);
        WorkCursor cur = work_begin(p, unit, krank);
        WorkCoord  c;
        if constexpr (KS) {
            // One tile per cluster: wait for this CTA's partial accumulator; the partials are
            // summed after the cluster barrier below.
            if (work_next(p, cur, unit, units, wn, tile_m, c)) {
                ok = bounded_wait(ptx::smem_u32(&s_tfull[0]), 0u, &s_abort, p.status, ST_EPI_WAIT);
                ok = __all_sync(0xffffffffu, ok);
                ptx::tc_fence_after();
                ks_c  = c;
                ks_ok = ok;
                if (warp == 2 && lane == 0) {
                    B200_TL(9);
                    B200_TL_CTA(2);
                }
            }
        } else
        for (; ok && work_next(p, cur, unit, units, wn, tile_m, c); ++it) {
            const uint32_t  buf    = it % NUM_ACC;
            const uint32_t  aphase = (it / NUM_ACC) & 1u;
            // A 512-wide tile is drained as two 256-column halves, each published (s_tfull[h])
            // and handed back (s_tempty[h]) on its own; narrower tiles have one accumulator per
            // barrier pair.
#pragma unroll 1
            for (uint32_t hh = 0; hh < static_cast<uint32_t>(NSUB); ++hh) {
            const uint32_t bar_i  = (NSUB == 2) ? hh : buf;
            const uint32_t parity = (NSUB == 2) ? (it & 1u) : aphase;
            const uint32_t colh   = hh * UMMA_N; // first column of this half within the tile
            ok = bounded_wait(ptx::smem_u32(&s_tfull[bar_i]), parity, &s_abort, p.status,
                              ST_EPI_WAIT);
            ok = __all_sync(0xffffffffu, ok); // warp-uniform: the TMEM loads below are aligned
            if (!ok) break;
            if (warp == 2 && lane == 0 && it == 0) {
                B200_TL(9);
                B200_TL_CTA(2);
            }
            ptx::tc_fence_after();
            const uint32_t row0     = c.m0 + rank * BLOCK_M + q * 32u;
            // 32-row groups at and beyond the slab height belong to the next tile (narrow staged
            // tiles may use slabs of 32, 64 or 96 rows; p.bm is 128 everywhere else).
            const bool     row_live = row0 < p.M && q * 32u < p.bm;
            const uint32_t tacc = tmem_base + ((q * 32u) << 16) + buf * ACC_COLS + colh;
            if constexpr (TR) {
                // Transposed epilogue: D(i, j) goes to out[j * M + i].  Each lane owns row i, so
                // for a fixed column j the warp writes 32 consecutive elements: coalesced stores
                // straight from registers, no staging.  Used when the caller's small dimension
                // had to become the MMA's N extent (skinny problems).
                // Rows at and beyond p.bm belong to the next slab (the MMA computed them from
                // whatever follows the slab in shared memory): never stored.
                const uint32_t i      = c.m0 + q * 32u + lane;
                const bool     i_live = (q * 32u + lane) < p.bm && i < p.M;
                dep_wait();
#pragma unroll 1
                for (int ch = 0; ch < (BN + 31) / 32; ++ch) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32(tacc + ch * 32, v);
                    ptx::tmem_ld_wait(v);
                    if (ch == (BN + 31) / 32 - 1) {
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&s_tempty[buf]));
                    }
                    if (i_live) {
                        const size_t base = (static_cast<size_t>(c.z_out) * p.N + c.n0 + ch * 32) * p.M + i;
#pragma unroll
                        for (int r = 0; r < 32; ++r) {
                            if (ch * 32 + r < BN && c.n0 + ch * 32 + r < p.N) {
                                const size_t at = base + static_cast<size_t>(r) * p.M;
                                if constexpr (OUT == OUT_F32) {
                                    static_cast<float*>(p.out)[at] = __uint_as_float(v[r]);
                                } else if constexpr (OUT == OUT_F16) {
                                    static_cast<__half*>(p.out)[at] = __float2half_rn(__uint_as_float(v[r]));
                                } else {
                                    static_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(__uint_as_float(v[r]));
                                }
                            }
                        }
                    }
                }
                continue;
            }
            // Software pipeline over 128-byte column chunks: the TMEM load of chunk ch + 1 is
            // in flight while chunk ch is converted, staged and handed to the TMA store.  `O` is
            // the element kind written: the kernel's output type, or f32 for a partial tile of
            // the balanced schedule (tile-local coordinates in the workspace map `tm`).
            auto drain = [&](auto out_tag, const CUtensorMap* tm, bool tile_local) {
            constexpr int O    = decltype(out_tag)::value;
            constexpr int O_CH = (O == OUT_F32) ? 32 : 64; // output columns per 128-byte chunk
            uint32_t       n0[32], n1[32]; // raw accumulator words of the chunk in flight
            ptx::tmem_ld_32x32(tacc, n0);
            if constexpr (O != OUT_F32) ptx::tmem_ld_32x32(tacc + 32u, n1);
            const int NCH_H = FLEX ? static_cast<int>(wn) / O_CH : (BN < O_CH ? 1 : BN / O_CH) / NSUB; // chunks per half
#pragma unroll 1
            for (int ch = 0; ch < NCH_H; ++ch) {
                uint32_t v[32];
                ptx::tmem_ld_wait(n0);
                if constexpr (O == OUT_F32) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = n0[j];
                } else {
                    ptx::tmem_ld_wait(n1);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        v[j]      = pack2<O>(n0[2 * j], n0[2 * j + 1]);
                        v[16 + j] = pack2<O>(n1[2 * j], n1[2 * j + 1]);
                    }
                }
                if (ch + 1 < NCH_H) {
                    ptx::tmem_ld_32x32(tacc + (ch + 1) * O_CH, n0);
                    if constexpr (O != OUT_F32) ptx::tmem_ld_32x32(tacc + (ch + 1) * O_CH + 32u, n1);
                }
                if (ch == NCH_H - 1) {
                    // Accumulator (half) fully read: hand it back to the MMA issuer (rank 0).
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (CL == 2) ptx::mbar_arrive_cluster(ptx::smem_u32(&s_tempty[bar_i]), 0);
                        else ptx::mbar_arrive(ptx::smem_u32(&s_tempty[bar_i]));
                    }
                }
                const uint32_t col0 = c.n0 + colh + ch * O_CH;
                if (row_live && col0 < p.N) {
                    const uint32_t sbuf = stg + (nstore & 1u) * EPI_BUF_BYTES;
                    // The store that last used this buffer (two stores ago) must have read it.
                    if (lane == 0) ptx::tma_store_wait_read<1>();
                    __syncwarp();
                    const uint32_t rowaddr = sbuf + lane * 128u;
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) {
                        st_shared_v4(rowaddr + ((j ^ (lane & 7u)) << 4), v[4 * j], v[4 * j + 1],
                                     v[4 * j + 2], v[4 * j + 3]);
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        dep_wait();
                        if constexpr (GATHER) {
                            // The tile goes to every copy of the full matrix (this GPU's and its
                            // peers', over NVLink) at the slab's offset: the all-gather of the
                            // output happens tile by tile under the main loop of the next tile.
                            for (uint32_t d = 0; d < p.ndst; ++d)
                                ptx::tma_store_3d(&tmDs[d], sbuf, col0 + p.dst_col0, row0 + p.dst_row0, c.z_out, pol_d);
                        } else if (tile_local) {
                            ptx::tma_store_3d(tm, sbuf, col0 - c.n0, row0 - c.m0, c.z_out, pol_d);
                        } else {
                            ptx::tma_store_3d(tm, sbuf, col0, row0, c.z_out, pol_d);
                        }
                        ptx::tma_store_commit();
                        if (warp == 2) {
                            if (nstore == 0) B200_TL(10);
                            B200_TL(11);
                        }
                    }
                    ++nstore;
                }
            }
            }; // drain
            if constexpr (!GATHER && NSUB == 1 && !TR) {
                // balanced schedule: partial segments go to the workspace as f32, whole tiles to C
                if (c.partial) drain(std::integral_constant<int, OUT_F32>{}, &tmW, true);
                else drain(std::integral_constant<int, OUT>{}, &tmD, false);
            } else {
                drain(std::integral_constant<int, OUT>{}, &tmD, false);
            }
            } // halves
        }
        // The staging buffers may go away once the stores have READ them; the writes themselves
        // are complete when the grid is (and a dependent grid waits for exactly that).
        if (lane == 0) ptx::tma_store_wait_read<0>();
        if (warp == 2 && lane == 0) B200_TL(12);
    }

    if constexpr (KS) {
        // ------------------------------------------------------ sum of the cluster's K partitions
        // Every CTA of the cluster holds an f32 partial of the same tile in TMEM.  The tile's
        // 128-byte output chunks are dealt round-robin to the CTAs (chunk ch belongs to rank
        // ch % split_k); each CTA sends the chunks it does not own to their owners' shared memory
        // (the operand ring, free once every CTA's MMAs have retired: first barrier), and after the
        // second barrier adds the partials of its own chunks in partition order - whichever CTA
        // owns a chunk, the sum is ((p0 + p1) + p2) + ... - converts and stores them to C.  No
        // workspace in global memory and no second kernel.  All threads of the cluster pass both
        // barriers whatever happened before (a role that gave up a bounded wait included).
        // (the transposed epilogue stores element by element: its chunks are 32 f32 columns)
        constexpr int      O_CH  = (TR || OUT == OUT_F32) ? 32 : 64; // output columns per chunk
        constexpr int      NCH   = TR ? (BN + 31) / 32 : BN / O_CH; // (a 16-column slab is one chunk, half of it unused)
        constexpr uint32_t ROW_B = O_CH * 4u;                  // bytes of one row of an f32 chunk
        constexpr uint32_t WSLOT = 32u * ROW_B;                // one warp's 32 rows of a chunk
        const uint32_t ks   = p.split_k;
        const uint32_t q    = warp & 3u;
        const uint32_t tacc = tmem_base + ((q * 32u) << 16);
        __syncwarp();
        if (warp == 2 && lane == 0) B200_TL(16);
        ptx::cluster_arrive();
        ptx::cluster_wait();
        if (warp == 2 && lane == 0) B200_TL(17);
        if (warp >= 2 && ks_ok) {
#pragma unroll 1
            for (uint32_t ch = 0; ch < static_cast<uint32_t>(NCH); ++ch) {
                const uint32_t owner = ch % ks;
                if (owner == krank) continue;
                // (within a warp's slot the 16-byte units are laid out [unit][lane]: every store and
                // load instruction of the warp covers 512 contiguous bytes)
                const uint32_t local  = ring + (((ch / ks) * ks + krank) * 4u + q) * WSLOT + lane * 16u;
                const uint32_t remote = ptx::mapa_u32(local, owner);
#pragma unroll
                for (uint32_t h = 0; h < static_cast<uint32_t>(O_CH / 32); ++h) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32(tacc + ch * O_CH + h * 32u, v);
                    ptx::tmem_ld_wait(v);
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j)
                        ptx::st_cluster_v4(remote + (h * 8u + j) * 512u, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
        }
        __syncwarp();
        if (warp == 2 && lane == 0) B200_TL(18);
        ptx::cluster_arrive();
        ptx::cluster_wait();
        if (warp == 2 && lane == 0) B200_TL(19);
        if (warp >= 2 && ks_ok) {
            const uint32_t stg      = epi + q * 2u * EPI_BUF_BYTES;
            const uint32_t row0     = ks_c.m0 + q * 32u;
            const bool     row_live = row0 < p.M;
            uint32_t       nstore   = 0;
#pragma unroll 1
            for (uint32_t ch = krank; ch < static_cast<uint32_t>(NCH); ch += ks) {
                uint32_t own[O_CH];
                float    acc[O_CH];
#pragma unroll
                for (uint32_t h = 0; h < static_cast<uint32_t>(O_CH / 32); ++h) {
                    uint32_t t[32];
                    ptx::tmem_ld_32x32(tacc + ch * O_CH + h * 32u, t);
                    ptx::tmem_ld_wait(t);
#pragma unroll
                    for (int j = 0; j < 32; ++j) own[h * 32 + j] = t[j];
                }
#pragma unroll 1
                for (uint32_t s = 0; s < ks; ++s) {
                    if (s == krank) {
#pragma unroll
                        for (int j = 0; j < O_CH; ++j)
                            acc[j] = (s == 0u) ? __uint_as_float(own[j]) : acc[j] + __uint_as_float(own[j]);
                    } else {
                        const uint32_t src = ring + (((ch / ks) * ks + s) * 4u + q) * WSLOT + lane * 16u;
#pragma unroll
                        for (uint32_t h = 0; h < static_cast<uint32_t>(O_CH / 32); ++h) {
#pragma unroll
                            for (uint32_t j = 0; j < 8; ++j) {
                                uint32_t x0, x1, x2, x3;
                                ptx::ld_shared_v4(src + (h * 8u + j) * 512u, x0, x1, x2, x3);
                                const int at = h * 32 + 4 * j;
                                acc[at]     = (s == 0u) ? __uint_as_float(x0) : acc[at] + __uint_as_float(x0);
                                acc[at + 1] = (s == 0u) ? __uint_as_float(x1) : acc[at + 1] + __uint_as_float(x1);
                                acc[at + 2] = (s == 0u) ? __uint_as_float(x2) : acc[at + 2] + __uint_as_float(x2);
                                acc[at + 3] = (s == 0u) ? __uint_as_float(x3) : acc[at + 3] + __uint_as_float(x3);
                            }
                        }
                    }
                }
                if constexpr (TR) {
                    // D(i, j) goes to out[j * M + i]: for a fixed column the warp writes 32
                    // consecutive elements (see the transposed epilogue above).
                    const uint32_t i      = ks_c.m0 + q * 32u + lane;
                    const bool     i_live = (q * 32u + lane) < p.bm && i < p.M;
                    dep_wait();
                    if (i_live) {
                        const size_t base = (static_cast<size_t>(ks_c.z_out) * p.N + ks_c.n0 + ch * 32u) * p.M + i;
#pragma unroll
                        for (int r = 0; r < 32; ++r) {
                            if (ks_c.n0 + ch * 32u + r < p.N) {
                                const size_t at = base + static_cast<size_t>(r) * p.M;
                                if constexpr (OUT == OUT_F32) static_cast<float*>(p.out)[at] = acc[r];
                                else if constexpr (OUT == OUT_F16) static_cast<__half*>(p.out)[at] = __float2half_rn(acc[r]);
                                else static_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(acc[r]);
                            }
                        }
                    }
                } else {
                uint32_t v[32];
                if constexpr (OUT == OUT_F32) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(acc[j]);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = pack2<OUT>(__float_as_uint(acc[2 * j]), __float_as_uint(acc[2 * j + 1]));
                }
                const uint32_t col0 = ks_c.n0 + ch * O_CH;
                if (row_live && col0 < p.N) {
                    const uint32_t sbuf = stg + (nstore & 1u) * EPI_BUF_BYTES;
                    if (lane == 0) ptx::tma_store_wait_read<1>();
                    __syncwarp();
                    const uint32_t rowaddr = sbuf + lane * 128u;
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j)
                        st_shared_v4(rowaddr + ((j ^ (lane & 7u)) << 4), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        dep_wait();
                        ptx::tma_store_3d(&tmD, sbuf, col0, row0, ks_c.z_out, ptx::make_l2_policy((p.l2_hints >> 4) & 3u));
                        ptx::tma_store_commit();
                    }
                    ++nstore;
                }
                } // staged store
            }
            if (warp == 2 && lane == 0) B200_TL(20);
            if (lane == 0) ptx::tma_store_wait_read<0>();
            if (warp == 2 && lane == 0) B200_TL(21);
        }
    }

    // ---------------------------------------------------------------------- tail
    ptx::tc_fence_before();
    __syncthreads();
    if constexpr (CL == 2) { // neither CTA may leave while its peer can still touch it
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
    if (threadIdx.x == 0) B200_TL(13);
    if (threadIdx.x == 64) B200_TL_CTA(1);
    if (warp == 1) {
        ptx::tc_fence_after();
        __syncwarp();
        ptx::tmem_dealloc<CL>(tmem_base, TMEM_COLS);
        if (lane == 0) B200_TL(14);
    }
}

template <int BN, int OUT, int CL, bool TR = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_umma_kernel(const __grid_constant__ CUtensorMap tmA,
                     const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmD,
                     const __grid_constant__ CUtensorMap tmW, const GemmParams p)
{
    // tmW: the balanced schedule's workspace of f32 partial tiles (any valid map otherwise)
    gemm_umma_body<BN, OUT, CL, TR, false>(tmA, tmB, &tmD, tmW, p);
}

// The same GEMM with the all-gather of its output fused into the epilogue: this GPU computes a
// slab of a larger matrix and stores every tile of it into p.ndst copies of that matrix (its own
// and, through peer mappings, the other GPUs').  Plain TMA stores to peer memory: no loads from
// a peer, no multicast, and no wait on another GPU anywhere in the kernel.
template <int BN, int OUT, int CL>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_umma_gather_kernel(const __grid_constant__ CUtensorMap tmA,
                            const __grid_constant__ CUtensorMap tmB,
                            const __grid_constant__ GatherMaps dst, const GemmParams p)
{
    gemm_umma_body<BN, OUT, CL, false, true>(tmA, tmB, dst.m, dst.m[0], p);
}

// The same GEMM with a tile's K partitions spread over the CTAs of a cluster (cluster size =
// p.split_k, one tile per cluster) and summed through distributed shared memory.
template <int BN, int OUT, bool TR = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_umma_ksplit_kernel(const __grid_constant__ CUtensorMap tmA,
                            const __grid_constant__ CUtensorMap tmB,
                            const __grid_constant__ CUtensorMap tmD, const GemmParams p)
{
    gemm_umma_body<BN, OUT, 1, TR, false, true>(tmA, tmB, &tmD, tmD, p);
}

// ---------------------------------------------------------------------------------------------
// Split-K reduction: out[z][i] = convert(sum_s ws[z][s][i]), s ascending (deterministic).
// `ws` holds batch * split_k partial matrices of `mn` f32 elements each.
// ---------------------------------------------------------------------------------------------
template <int OUT>
__global__ void __launch_bounds__(256)
    splitk_reduce_kernel(const float* __restrict__ ws, void* __restrict__ out, uint64_t mn,
                         uint32_t split_k, uint32_t batch)
{
    const uint64_t total4 = (mn * batch) >> 2; // mn is a multiple of 4
    const uint64_t mn4    = mn >> 2;
    ptx::grid_dep_wait(); // the partials are complete once the GEMM grid before this one has finished
    ptx::grid_dep_launch();
    for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < total4;
         i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint64_t z   = i / mn4;
        const uint64_t e   = i - z * mn4;
        const float4*  src = reinterpret_cast<const float4*>(ws) + z * split_k * mn4 + e;
        float4         acc = __ldg(src);
        for (uint32_t s = 1; s < split_k; ++s) {
            const float4 t = __ldg(src + s * mn4);
            acc.x += t.x;
            acc.y += t.y;
            acc.z += t.z;
            acc.w += t.w;
        }
        if constexpr (OUT == OUT_F32) {
            reinterpret_cast<float4*>(out)[i] = acc;
        } else if constexpr (OUT == OUT_F16) {
            const __half2 a = __floats2half2_rn(acc.x, acc.y);
            const __half2 b = __floats2half2_rn(acc.z, acc.w);
            uint2         u;
            u.x = *reinterpret_cast<const uint32_t*>(&a);
            u.y = *reinterpret_cast<const uint32_t*>(&b);
            reinterpret_cast<uint2*>(out)[i] = u;
        } else {
            const __nv_bfloat162 a = __floats2bfloat162_rn(acc.x, acc.y);
            const __nv_bfloat162 b = __floats2bfloat162_rn(acc.z, acc.w);
            uint2                u;
            u.x = *reinterpret_cast<const uint32_t*>(&a);
            u.y = *reinterpret_cast<const uint32_t*>(&b);
            reinterpret_cast<uint2*>(out)[i] = u;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Fix-up pass of the balanced (stream-K) schedule: for every tile that a run boundary cuts,
// out(tile) = convert(sum of the tile's partial tiles), partials added in K order (ascending
// worker), so the result does not depend on timing.  Tiles no boundary cuts were written to C
// by the GEMM kernel itself and are not touched.
//
// Job j (1 <= j < workers) belongs to the boundary between runs j - 1 and j.  The boundary cuts
// a tile unless it falls on a tile's first K step; a tile cut by several boundaries is handled
// by the job of the first of them.  The tile's contributors are the workers w0 .. w1 whose runs
// hold its first and last K step; worker w's partial sits in slot 2w if its run starts inside
// the tile, in slot 2w + 1 if its run came in through the tile's first K step (see WorkCursor).
// `ws` holds one dense tile_m x tile_n f32 tile per slot.  N is a multiple of 4, so a float4
// never straddles the matrix edge.  L2/HBM-bound: (parts x 4 + sizeof(out)) bytes per element
// of a cut tile; blockIdx.y = job, blockIdx.x strides over the tile's float4s.
// ---------------------------------------------------------------------------------------------
template <int OUT>
__global__ void __launch_bounds__(256)
    streamk_reduce_kernel(const float* __restrict__ ws, void* __restrict__ out, const GemmParams p, uint32_t tile_m,
                          uint32_t tile_n)
{
    ptx::grid_dep_wait(); // the partials are complete once the GEMM grid before this one has finished
    ptx::grid_dep_launch();
    const uint32_t j        = blockIdx.y + 1u;
    const uint32_t upt      = p.units_per_tile;
    const uint32_t boundary = run_start(p, j);
    const uint32_t tile     = boundary / upt; // over batch x tiles
    const uint32_t tile_beg = tile * upt;
    if (boundary == tile_beg) return;                             // the cut falls between two tiles
    if (j > 1u && run_start(p, j - 1u) > tile_beg) return;        // an earlier boundary owns this tile
    // workers whose runs hold the tile's first and last K step
    const uint64_t x0 = tile_beg, x1 = x0 + upt - 1u;
    const uint32_t w0 = static_cast<uint32_t>(((x0 + 1u) * p.workers + p.total_units - 1u) / p.total_units) - 1u;
    const uint32_t w1 = static_cast<uint32_t>(((x1 + 1u) * p.workers + p.total_units - 1u) / p.total_units) - 1u;
    const uint32_t tiles    = p.m_tiles * p.n_tiles;
    const uint32_t row4     = tile_n / 4u; // float4 per tile row
    const uint32_t tile_sz4 = tile_m * row4;
    uint32_t       m_idx, n_idx;
    tile_coords(p, tile % tiles, m_idx, n_idx);
    const uint32_t z    = tile / tiles;
    const float4*  ws4  = reinterpret_cast<const float4*>(ws);
    // the first contributor's run holds the tile's first K step: its partial is its run's last segment
    const uint32_t slot0 = 2u * w0 + 1u;
    for (uint32_t e = blockIdx.x * blockDim.x + threadIdx.x; e < tile_sz4; e += gridDim.x * blockDim.x) {
        const uint32_t rr = e / row4, c4 = e - rr * row4;
        const uint32_t row = m_idx * tile_m + rr, col = n_idx * tile_n + c4 * 4u;
        if (row >= p.M || col >= p.N) continue;
        float4 acc = __ldg(ws4 + static_cast<uint64_t>(slot0) * tile_sz4 + e);
        for (uint32_t w = w0 + 1u; w <= w1; ++w) { // these runs start inside the tile: slot 2w
            const float4 t = __ldg(ws4 + static_cast<uint64_t>(2u * w) * tile_sz4 + e);
            acc.x += t.x;
            acc.y += t.y;
            acc.z += t.z;
            acc.w += t.w;
        }
        const uint64_t at = (static_cast<uint64_t>(z) * p.M + row) * p.N + col; // element index; col % 4 == 0
        if constexpr (OUT == OUT_F32) {
            *reinterpret_cast<float4*>(static_cast<float*>(out) + at) = acc;
        } else if constexpr (OUT == OUT_F16) {
            const __half2 a = __floats2half2_rn(acc.x, acc.y);
            const __half2 b = __floats2half2_rn(acc.z, acc.w);
            uint2         u;
            u.x = *reinterpret_cast<const uint32_t*>(&a);
            u.y = *reinterpret_cast<const uint32_t*>(&b);
            *reinterpret_cast<uint2*>(static_cast<__half*>(out) + at) = u;
        } else {
            const __nv_bfloat162 a = __floats2bfloat162_rn(acc.x, acc.y);
            const __nv_bfloat162 b = __floats2bfloat162_rn(acc.z, acc.w);
            uint2                u;
            u.x = *reinterpret_cast<const uint32_t*>(&a);
            u.y = *reinterpret_cast<const uint32_t*>(&b);
            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + at) = u;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// CUDA-core GEMM with arbitrary element strides, f32 accumulation in ascending k.  Only used
// for shapes whose contiguous extents are not multiples of 16 bytes (TMA cannot address
// them); correctness path, not a performance path.
// ---------------------------------------------------------------------------------------------
template <class TIn, class TOut>
__global__ void __launch_bounds__(256)
    gemm_generic_kernel(TOut* __restrict__ C, const TIn* __restrict__ A,
                        const TIn* __restrict__ B, uint32_t M, uint32_t N, uint32_t K,
                        uint64_t a_sm, uint64_t a_sk, uint64_t b_sk, uint64_t b_sn, uint64_t c_sm,
                        uint64_t c_sn, uint64_t a_sb, uint64_t b_sb, uint64_t c_sb)
{
    __shared__ float sA[16][17];
    __shared__ float sB[16][17];
    const uint32_t   tx = threadIdx.x & 15u, ty = threadIdx.x >> 4;
    const uint32_t   i = blockIdx.y * 16u + ty, j = blockIdx.x * 16u + tx;
    const TIn*       Ab  = A + blockIdx.z * a_sb;
    const TIn*       Bb  = B + blockIdx.z * b_sb;
    float            acc = 0.f;
    for (uint32_t k0 = 0; k0 < K; k0 += 16u) {
        const uint32_t ka = k0 + tx, kb = k0 + ty;
        sA[ty][tx] = (i < M && ka < K) ? static_cast<float>(Ab[i * a_sm + ka * a_sk]) : 0.f;
        sB[ty][tx] = (kb < K && j < N) ? static_cast<float>(Bb[kb * b_sk + j * b_sn]) : 0.f;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) acc += sA[ty][k] * sB[k][tx];
        __syncthreads();
    }
    if (i < M && j < N) C[blockIdx.z * c_sb + i * c_sm + j * c_sn] = static_cast<TOut>(acc);
}

} // namespace b200
