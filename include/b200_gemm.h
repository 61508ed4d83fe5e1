/*
 * b200_gemm.h — C ABI of the B200 (sm_100a) half-precision GEMM library.
 *
 * The library computes C = A * B (no alpha/beta) for four (output, input) type pairs
 * and every row-/column-major combination of A (M x K), B (K x N) and C (M x N), single
 * or strided-batched, with dense-packed matrices (leading dimension == the contiguous
 * extent) and batch strides M*K, K*N and M*N elements.
 *
 * Two groups of entry points:
 *
 *  1. The four `rocm_wmma_gemm_<out>_<in>` symbols.  Name, argument order and argument
 *     meaning are those of the reference library's per-architecture shared object, so a
 *     host program that dlopen()s that object and dlsym()s these four names binds here
 *     unchanged.  They return void and never throw; a failure is recorded and can be
 *     read with b200_gemm_last_status() / b200_gemm_last_error().
 *
 *  2. `b200_gemm_*` twins that return a status code, plus helpers the reference does not
 *     have (host-buffer call, explicit config, column-slab partition, device status).
 *
 * All pointers named C/A/B in group 1 and in b200_gemm_<out>_<in> are DEVICE pointers.
 * `stream` is a POINTER TO a cudaStream_t (the reference passes `&stream`); NULL means
 * the default stream.  Layout ints: 0 = row-major, 1 = column-major.
 */
#ifndef B200_GEMM_H
#define B200_GEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------ */
enum b200_gemm_status {
    B200_GEMM_OK               = 0,
    B200_GEMM_ERR_BAD_LAYOUT   = 1, /* a layout int is not 0 or 1 (the reference ignores the call) */
    B200_GEMM_ERR_NULL_POINTER = 2,
    B200_GEMM_ERR_BAD_SIZE     = 3, /* a dimension does not fit 31 bits, or batch_count == 0 */
    B200_GEMM_ERR_MISALIGNED   = 4, /* a base pointer is not aligned to its element size */
    B200_GEMM_ERR_NO_DEVICE    = 5, /* no CUDA device, or the current device is not sm_100 */
    B200_GEMM_ERR_CUDA         = 6, /* a CUDA runtime/driver call failed; see last_error */
    B200_GEMM_ERR_BAD_CONFIG   = 7, /* explicit config outside the compiled variant set */
    B200_GEMM_ERR_DEVICE_WAIT  = 8, /* a kernel gave up on a bounded wait (device status) */
    B200_GEMM_ERR_TOO_LARGE    = 9, /* request exceeds a fixed-capacity entry point's limit */
    B200_GEMM_ERR_NO_NCCL      = 10, /* the multi-GPU driver could not load libnccl.so.2 */
    B200_GEMM_ERR_NCCL         = 11  /* an NCCL call failed; see last_error */
};

/* ---- group 1: the reference's C ABI ----------------------------------------------------
 * Replaces rocm_wmma_gemm/src/gemm.cpp:207-250 (DEFINE_C_DISPATCH) of the reference, which
 * rocm_wmma_gemm/include/rocm_wmma_gemm/kernel_loader.hpp:91-113 resolves by name.
 * Suffix is <out>_<in>.  C: M x N, A: M x K, B: K x N; batch strides M*N, M*K, K*N.
 */
void rocm_wmma_gemm_f16_f16(void* C, void* A, void* B, size_t M, size_t N, size_t K,
                            size_t batch_count, int layout_c, int layout_a, int layout_b,
                            void* stream);
void rocm_wmma_gemm_f32_f16(void* C, void* A, void* B, size_t M, size_t N, size_t K,
                            size_t batch_count, int layout_c, int layout_a, int layout_b,
                            void* stream);
void rocm_wmma_gemm_bf16_bf16(void* C, void* A, void* B, size_t M, size_t N, size_t K,
                              size_t batch_count, int layout_c, int layout_a, int layout_b,
                              void* stream);
void rocm_wmma_gemm_f32_bf16(void* C, void* A, void* B, size_t M, size_t N, size_t K,
                             size_t batch_count, int layout_c, int layout_a, int layout_b,
                             void* stream);

/* ---- group 2: status-returning twins ----------------------------------------------------
 * Same arguments as group 1 (reference: rocm_wmma_gemm/src/gemm.cpp:219-245); the return
 * value is a b200_gemm_status.  The call is asynchronous on `*stream`.
 */
int b200_gemm_f16_f16(void* C, void* A, void* B, size_t M, size_t N, size_t K,
                      size_t batch_count, int layout_c, int layout_a, int layout_b, void* stream);
int b200_gemm_f32_f16(void* C, void* A, void* B, size_t M, size_t N, size_t K,
                      size_t batch_count, int layout_c, int layout_a, int layout_b, void* stream);
int b200_gemm_bf16_bf16(void* C, void* A, void* B, size_t M, size_t N, size_t K,
                        size_t batch_count, int layout_c, int layout_a, int layout_b, void* stream);
int b200_gemm_f32_bf16(void* C, void* A, void* B, size_t M, size_t N, size_t K,
                       size_t batch_count, int layout_c, int layout_a, int layout_b, void* stream);

/* Type-pair index used by the generic entry points below; the numbering is the reference's
 * type_idx (rocm_wmma_gemm/include/rocm_wmma_gemm/kernel_launcher.hpp:78-84):
 * 0 = f16<-f16, 1 = f32<-f16, 2 = bf16<-bf16, 3 = f32<-bf16. */
enum b200_gemm_types {
    B200_GEMM_F16_F16   = 0,
    B200_GEMM_F32_F16   = 1,
    B200_GEMM_BF16_BF16 = 2,
    B200_GEMM_F32_BF16  = 3
};

/* Tunable launch configuration: the B200 counterpart of the reference's per-entry `config`
 * object {warps_m, warps_n, warp_tile_m, warp_tile_n, swizzle, bits}
 * (rocm_wmma_gemm/config/gemm_config_gfx1100_f16.json:1-22; struct gemm_params generated by
 * rocm_wmma_gemm/config/generate_config.py:94-103).
 *   tile_m   rows of C per CTA (per CTA pair when cluster == 2): 128, or 256 with cluster 2
 *   tile_n   columns of C per CTA / CTA pair: 64, 128, 256, or 512 (512: cluster 2 only); with
 *            cluster 2 also 160, 192 and 224 (the 256-column kernel at a run-time width; needs
 *            a K-major B operand in the kernel view and whole 128-byte output chunks, i.e. a
 *            multiple of 32 columns for f32 outputs, of 64 for 16-bit outputs)
 *   stages   depth of the TMA -> shared-memory ring (2 .. 12, clamped to what fits; kernels
 *            that stage several k-blocks per ring slot size the ring themselves)
 *   cluster  1 = one CTA per tile, 2 = a CTA pair shares one tile (cta_group::2 MMA)
 *   split_k  number of K partitions reduced through an f32 workspace (1 = none).  0 selects the
 *            balanced schedule (stream-K, the reference's roadmap item README.md:202): the K
 *            loops of all tiles are laid end to end and cut into one equal run per SM, so every
 *            SM does the same number of K steps whatever the tile count; tiles a run covers
 *            whole go straight to C, the tiles a run boundary cuts meet as f32 partials in a
 *            deterministic fix-up pass.  Needs tile_n <= 256 and N % 4 == 0 in the kernel view.
 *   raster   tile-rows per raster band (the reference's `swizzle` key,
 *            rocm_wmma_gemm/include/rocm_wmma_gemm/kernel/mapping.hpp:108-287); 0 = column sweep.
 *            Adding B200_GEMM_RASTER_SNAKE selects the boustrophedon order of the reference's
 *            xor_snake mappings: every other band walks its columns backwards, so a band starts
 *            on the panels of B the band before it has just read.
 */
#define B200_GEMM_RASTER_SNAKE 128
typedef struct b200_gemm_config {
    int tile_m;
    int tile_n;
    int stages;
    int cluster;
    int split_k;
    int raster;
} b200_gemm_config;

/* C = A*B with an explicit configuration (cfg == NULL: the tuned table decides, exactly as
 * the four fixed-type entry points do).  Used by the tuner and the benchmarks; counterpart
 * of the tuner's "one instantiation chosen by CLI parameters"
 * (rocm_wmma_gemm/config/tuner.cpp:458-466). */
int b200_gemm_ex(int types, void* C, const void* A, const void* B, size_t M, size_t N, size_t K,
                 size_t batch_count, int layout_c, int layout_a, int layout_b, void* stream,
                 const b200_gemm_config* cfg);

/* The configuration the tuned table selects for a problem: exact (M,N,K,type_group,layouts)
 * match, else exact match in the 16-bit-output group, else nearest K then nearest (M,N)
 * within the same layout triple, else the default.  Counterpart of
 * detail::find_best_config / get_gemm_params
 * (rocm_wmma_gemm/config/generate_config.py:174-303).  Pure host code, no GPU needed.
 * Returns the index of the chosen entry of the compiled config list (>= 0). */
int b200_gemm_select_config(size_t M, size_t N, size_t K, int types, int layout_c, int layout_a,
                            int layout_b, b200_gemm_config* out);

/* What a call with these arguments would launch (operands assumed 16-byte aligned): the
 * kernel family, the tile it cuts the kernel view into, the K partitions, the ring geometry
 * and the CTA count - after the table lookup, the check of a borrowed entry against the cost
 * model, the narrow-tile and row-slab rules.  Pure host code: `sm_count` 0 means the current
 * device's SM count, or 148 when the process has no usable device.  No reference counterpart
 * (the reference's launch is fully described by its config entry,
 * rocm_wmma_gemm/src/gemm.cpp:38-92). */
enum b200_gemm_kernel_kind {
    B200_GEMM_KERNEL_NONE       = 0, /* nothing to launch (empty C, or K == 0: C is zero-filled) */
    B200_GEMM_KERNEL_GENERIC    = 1, /* CUDA-core kernel: a leading dimension TMA cannot address */
    B200_GEMM_KERNEL_STAGED     = 2, /* tcgen05 kernel, TMA-store epilogue */
    B200_GEMM_KERNEL_TRANSPOSED = 3  /* tcgen05 kernel on swapped operands, transposing epilogue (skinny problems) */
};
typedef struct b200_gemm_plan_info {
    int       kernel;            /* b200_gemm_kernel_kind */
    int       tile_m;            /* kernel-view rows per tile: 128 x cluster, or the slab height (8..128) */
    int       tile_n;            /* kernel-view columns per tile */
    int       cluster;           /* CTAs per tile (1 or 2) */
    int       split_k;           /* K partitions (> 1: a reduction pass follows unless cluster_k is set) */
    int       slots;             /* ring depth */
    int       k_blocks_per_slot; /* 64-deep k-blocks staged per ring slot (1, 2 or 4) */
    int       raster;            /* tile-row band height (0: column sweep) */
    int       ctas;              /* CTAs launched (persistent: at most one per SM) */
    long long work_units;        /* tiles x K partitions x batch */
    int       cluster_k;         /* 1: the K partitions of a tile are the CTAs of one thread-block cluster and are
                                    summed through distributed shared memory: no workspace, no reduction pass */
} b200_gemm_plan_info;
int b200_gemm_plan(int types, size_t M, size_t N, size_t K, size_t batch_count, int layout_c,
                   int layout_a, int layout_b, int sm_count, b200_gemm_plan_info* out);

/* Host-buffer call: A, B, C are HOST pointers (pageable or pinned).  Copies A and B to the
 * device, runs the GEMM, copies C back and synchronises; device buffers are cached per
 * device and grow on demand.  This is the path a caller without device memory of its own
 * uses, and the one the end-to-end benchmark times.  Calls on the same device are serialised
 * (the staging buffers and copy streams are per device): a second thread's call waits for the
 * first to return.  No reference counterpart (the reference's tests do the copies themselves,
 * test/gemm/test_float_accum.cpp:95-119). */
int b200_gemm_host(int types, void* C, const void* A, const void* B, size_t M, size_t N, size_t K,
                   size_t batch_count, int layout_c, int layout_a, int layout_b);

/* Column-slab partition of C = A*B over `world` devices with A replicated: device `rank`
 * owns columns [*n_begin, *n_begin + *n_count) of B and C.  Slab widths are multiples of
 * `align` columns except the last.  No reference counterpart (the reference is single-GPU). */
int b200_gemm_slab(size_t N, int world, int rank, size_t align, size_t* n_begin, size_t* n_count);

/* ---- multi-GPU column-slab driver ----------------------------------------------------------
 * C = A*B over `world` GPUs of one box, one host process (or thread) per GPU: A replicated,
 * GPU `rank` owns the columns b200_gemm_slab assigns it of B and C.  The slab GEMM itself is the
 * ordinary single-GPU call on (A, B slab, C slab) and needs nothing from this section; what is
 * here is the exchange around it.  None of it has a counterpart in the reference, which is a
 * single-GPU library.  NCCL is loaded at run time (libnccl.so.2 on the loader path), so programs
 * that never create a communicator do not need it.
 *
 * Communicator: rank 0 obtains an id (b200_gemm_comm_id), the caller hands the 128 bytes to the
 * other ranks by whatever channel it has, every rank calls b200_gemm_comm_create with its
 * device current.  b200_gemm_comm_barrier enqueues a 4-byte all-reduce on `*stream`: work queued
 * after it starts only when every rank's stream has reached its barrier.
 * b200_gemm_comm_allgather_inplace all-gathers `bytes_per_rank` bytes per rank inside `buf`
 * (rank r's block at buf + r * bytes_per_rank already holds its own data): with row-major A cut
 * into `world` row blocks, each GPU uploads one block from the host and NVLink carries the rest. */
#define B200_GEMM_COMM_ID_BYTES 128
#define B200_GEMM_IPC_HANDLE_BYTES 64
typedef struct b200_gemm_comm b200_gemm_comm;
int b200_gemm_comm_id(void* id /* B200_GEMM_COMM_ID_BYTES out */);
int b200_gemm_comm_create(const void* id, int world, int rank, b200_gemm_comm** out);
int b200_gemm_comm_destroy(b200_gemm_comm* comm);
int b200_gemm_comm_barrier(b200_gemm_comm* comm, void* stream);
int b200_gemm_comm_allgather_inplace(b200_gemm_comm* comm, void* buf, size_t bytes_per_rank, void* stream);

/* Device memory other processes of the box can map: b200_gemm_peer_alloc allocates on the
 * current device and fills `handle` (B200_GEMM_IPC_HANDLE_BYTES, to be sent to the other
 * processes); b200_gemm_peer_open maps a buffer another process allocated and returns its
 * address in this process (valid on the current device; peer access is enabled on demand).
 * Close every mapping before the owner frees the buffer. */
int b200_gemm_peer_alloc(size_t bytes, void** dptr, void* handle);
int b200_gemm_peer_open(const void* handle, void** dptr);
int b200_gemm_peer_close(void* dptr);
int b200_gemm_peer_free(void* dptr);

/* The optional gather of C, three ways.  All leave the full M x N matrix (layout_c) on every
 * GPU; slabs are those of b200_gemm_slab(N, world, rank, align); `types` picks the element size
 * of C.
 *
 * b200_gemm_slab_allgather: NCCL all-gather of the C slabs (slab = dense M x n_count matrix in
 *   layout_c).  Column-major slabs land in place.  Row-major slabs interleave row by row: they
 *   are gathered into `staging` (M x N elements, caller-owned) and a re-layout kernel writes
 *   C_full.  Unequal slabs (N not a multiple of world x align) go as one grouped broadcast per
 *   slab.
 * b200_gemm_slab_push: this GPU's slab is copied into C_full[d] of every GPU d (C_full[rank] is
 *   local, the others are peer mappings) by the copy engines: strided device-to-device copies,
 *   no staging, no kernel, no SM taken from a GEMM that runs beside them.  The matrices are
 *   complete once every rank's copies have finished (b200_gemm_comm_barrier).
 * b200_gemm_slab_gather: the slab GEMM with the gather fused into its epilogue: every tile of
 *   the slab is stored straight into C_full[d] of all GPUs while the next tile is computed, so
 *   the exchange rides under the GEMM and there is no slab buffer at all.  Runs on the
 *   256 x 256 / 256 x 512 CTA-pair tiles (cfg NULL: the table's entry, moved onto one of them if
 *   needed) without K partitions; slab boundaries must be multiples of 64 columns (align 64 or
 *   a multiple).  C_full complete once every rank's kernel has finished
 *   (b200_gemm_comm_barrier). */
int b200_gemm_slab_allgather(b200_gemm_comm* comm, int types, void* C_full, const void* C_slab, void* staging,
                             size_t M, size_t N, int layout_c, size_t align, void* stream);
int b200_gemm_slab_push(int types, void* const* C_full, const void* C_slab, size_t M, size_t N, int layout_c,
                        int world, int rank, size_t align, void* stream);
int b200_gemm_slab_gather(int types, void* const* C_full, const void* A, const void* B_slab, size_t M, size_t N,
                          size_t K, int layout_c, int layout_a, int layout_b, int world, int rank, size_t align,
                          void* stream, const b200_gemm_config* cfg);

/* Host-buffer slab call, the multi-GPU counterpart of b200_gemm_host: every rank passes the
 * whole A (host memory, the same matrix on every rank), its own dense B slab (K x n_count,
 * layout_b) and room for its own dense C slab (M x n_count, layout_c); pointers may be pageable
 * or pinned.  Each GPU uploads only 1/world of A's storage over PCIe; an in-place NCCL all-gather
 * over NVLink completes the replica while the B slab comes up.  Collective: every rank of the
 * communicator must call it with the same M, N, K, layouts and align.  Synchronous. */
int b200_gemm_slab_host(b200_gemm_comm* comm, int types, void* C_slab, const void* A, const void* B_slab, size_t M,
                        size_t N, size_t K, int layout_c, int layout_a, int layout_b, size_t align);

/* Bytes of f32 split-K workspace a call would use (0 when the chosen config has split_k 1). */
size_t b200_gemm_workspace_bytes(int types, size_t M, size_t N, size_t K, size_t batch_count,
                                 int layout_c, int layout_a, int layout_b,
                                 const b200_gemm_config* cfg);

/* Bytes of the built-in split-K workspace used by b200_gemm_splitk_static. */
#define B200_GEMM_STATIC_WORKSPACE_BYTES (16u << 20)

/* C = A*B like b200_gemm_ex, for callers that must not allocate device memory while they run:
 * a server whose device memory was partitioned once at start-up, a latency-critical thread
 * that may not wait on the driver's allocator, a plugin inside a framework that owns all
 * allocations.  This entry point never calls cudaMalloc, cudaFree, their stream-ordered forms
 * or any allocating library routine.  Where the chosen configuration splits K, the f32
 * partial results go to a workspace that is part of the library image
 * (B200_GEMM_STATIC_WORKSPACE_BYTES on every GPU that loads the library, held until the
 * process exits) instead of a freshly allocated one.
 *   - A request whose partials (batch_count x split_k x M x N x 4 bytes) exceed the workspace
 *     is refused with B200_GEMM_ERR_TOO_LARGE; nothing runs.  Shapes the tensor-copy engine
 *     cannot address (pointers not 16-byte aligned, contiguous extents not multiples of 8
 *     elements) are refused with B200_GEMM_ERR_MISALIGNED, and K == 0 with BAD_SIZE.
 *   - The first call on each device looks up the workspace's device address and sets kernel
 *     attributes; make that first call once per device before any stream capture begins.
 *   - All calls on a device share the one workspace and it keeps whatever the previous call
 *     left there.  Nothing in it needs to start at zero (every partial is fully overwritten
 *     before it is read), but two calls that overlap on the GPU — different streams, or
 *     different threads — race on it: serialise them on one stream or with events.
 *   - Failures of device-side waits are recorded in a status word of this entry point's own
 *     (also part of the library image); read it with b200_gemm_static_status.
 *   - Planning and launch are those of b200_gemm_ex (same kernels, tiles, operand swap for
 *     skinny problems, raster); only the sources of the workspace and the status word differ.
 * cfg == NULL lets the tuned table choose.  This entry point has no counterpart in the
 * reference library, which never uses scratch memory. */
int b200_gemm_splitk_static(int types, void* C, const void* A, const void* B, size_t M, size_t N,
                            size_t K, size_t batch_count, int layout_c, int layout_a, int layout_b,
                            void* stream, const b200_gemm_config* cfg);

/* b200_gemm_device_status for the kernels launched by b200_gemm_splitk_static: synchronises
 * the current device, reads that entry point's own status word (a plain copy from the library
 * image: nothing is allocated), returns B200_GEMM_ERR_DEVICE_WAIT and clears the word if a
 * kernel gave up on a bounded wait.  No reference counterpart. */
int b200_gemm_static_status(unsigned int* detail);

/* Synchronises the current device and returns B200_GEMM_ERR_DEVICE_WAIT if any kernel of
 * this library has given up on a bounded wait since the last call (then clears the flag),
 * else B200_GEMM_OK.  `detail`, if not NULL, receives the raw device status word. */
int b200_gemm_device_status(unsigned int* detail);

/* Status / message of the last failing call on the calling thread (group 1 included). */
int         b200_gemm_last_status(void);
const char* b200_gemm_last_error(void);

/* Library version and the number of kernel launches issued so far by this process
 * (used by the benchmark to report how many of its own kernels ran in a timed region). */
const char*        b200_gemm_version(void);
unsigned long long b200_gemm_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_GEMM_H */
