/*
 * TEST INFRASTRUCTURE — NOT PRODUCT CODE.
 *
 * CPU restatement of the reference's host-side GEMM check path, in plain C:
 *   - input generation        test/test.hpp:33-54      (init_matrix: mt19937(1), uniform[-1,1))
 *   - the CPU reference GEMM  test/test.hpp:59-129     (hgemm_cpu, four type pairs)
 *   - matrix indexing         common/matrix.hpp:154-164 (row- / column-major get_index)
 *   - cosine similarity       test/test.hpp:134-196    (calculate_cosine_similarity)
 *   - benchmark input pattern benchmark/bench.hpp:37-52 (five-value cyclic fill)
 * of adelj88/rocm_wmma_gemm.  Only tests, the smoke check and the benchmark's CPU-baseline
 * leg may load this file's library; the GEMM library itself never does.
 *
 * Parity pin: every function here is compared bit-for-bit with the reference's own
 * test/test.hpp compiled unmodified (oracle/_ref, built by oracle/build.py) in
 * tests/test_oracle.py, and against the fixtures under tests/golden/ that the same
 * compiled reference produced.
 *
 * Arithmetic contract (what "the same result as the reference" means):
 *   acc = 0.0f; for k ascending: acc += (float)A(i,k) * (float)B(k,j)   — separate multiply
 *   and add in binary32 (build with -ffp-contract=off), then ONE rounding to the output
 *   type (round-to-nearest-even for f16 / bf16).  Inputs are widened exactly.
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- 16-bit float conversions ------------------------------------------------------------ */

static inline uint32_t f32_bits(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

static inline float bits_f32(uint32_t u)
{
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* IEEE binary16 -> binary32, exact. */
float oracle_f16_to_f32(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t       exp  = (h >> 10) & 0x1Fu;
    uint32_t       man  = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: normalise */
        int e = -1;
        do {
            man <<= 1;
            ++e;
        } while (!(man & 0x400u));
        man &= 0x3FFu;
        return bits_f32(sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13));
    }
    if (exp == 31) return bits_f32(sign | 0x7F800000u | (man << 13));
    return bits_f32(sign | ((exp + 127 - 15) << 23) | (man << 13));
}

/* binary32 -> binary16, round-to-nearest-even (what static_cast<half>(float) does). */
uint16_t oracle_f32_to_f16(float f)
{
    const uint32_t x    = f32_bits(f);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    const uint32_t ax   = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | (ax > 0x7F800000u ? 0x200u | ((ax >> 13) & 0x3FFu) : 0));
    if (ax >= 0x477FF000u) /* >= 65520: rounds to inf */
        return (uint16_t)(sign | 0x7C00u);
    if (ax < 0x33000001u) /* <= 2^-25: rounds to zero (ties-to-even at exactly 2^-25) */
        return sign;
    int32_t  exp = (int32_t)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u; /* 24-bit significand */
    uint32_t shift;
    uint32_t hexp;
    if (exp < -14) { /* subnormal result */
        shift = (uint32_t)(13 + (-14 - exp));
        hexp  = 0;
    } else {
        shift = 13;
        hexp  = (uint32_t)(exp + 15);
    }
    uint32_t       q    = man >> shift;
    const uint32_t rem  = man & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    /* q includes the implicit bit for normal results; adding it to the exponent field
     * handles the carry into the next binade. */
    uint32_t out = (hexp == 0) ? q : ((hexp - 1) << 10) + q;
    return (uint16_t)(sign | out);
}

float oracle_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* binary32 -> bfloat16, round-to-nearest-even (what __float2bfloat16 does). */
uint16_t oracle_f32_to_bf16(float f)
{
    const uint32_t x = f32_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFFu; /* NaN -> canonical */
    const uint32_t lsb = (x >> 16) & 1u;
    return (uint16_t)((x + 0x7FFFu + lsb) >> 16);
}

/* ---- mt19937 + libstdc++ uniform_real_distribution<float>(-1, 1) ------------------------- */

typedef struct {
    uint32_t mt[624];
    int      idx;
} mt19937_t;

static void mt_seed(mt19937_t* g, uint32_t seed)
{
    g->mt[0] = seed;
    for (int i = 1; i < 624; ++i)
        g->mt[i] = 1812433253u * (g->mt[i - 1] ^ (g->mt[i - 1] >> 30)) + (uint32_t)i;
    g->idx = 624;
}

static uint32_t mt_next(mt19937_t* g)
{
    if (g->idx >= 624) {
        for (int i = 0; i < 624; ++i) {
            const uint32_t y = (g->mt[i] & 0x80000000u) | (g->mt[(i + 1) % 624] & 0x7FFFFFFFu);
            g->mt[i]         = g->mt[(i + 397) % 624] ^ (y >> 1) ^ ((y & 1u) ? 0x9908B0DFu : 0u);
        }
        g->idx = 0;
    }
    uint32_t y = g->mt[g->idx++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9D2C5680u;
    y ^= (y << 15) & 0xEFC60000u;
    y ^= y >> 18;
    return y;
}

/* generate_canonical<float, 24>(mt19937): one 32-bit draw converted to float (rounding to
 * nearest), divided by 2^32, clamped below 1; then scaled to [a, b) as r * (b - a) + a. */
static float uniform_pm1(mt19937_t* g)
{
    float r = (float)mt_next(g) / 4294967296.0f;
    if (r >= 1.0f) r = nextafterf(1.0f, 0.0f);
    return r * (1.0f - -1.0f) + -1.0f;
}

/* ---- shared helpers ----------------------------------------------------------------------- */

/* Type-pair index: 0 = f16<-f16, 1 = f32<-f16, 2 = bf16<-bf16, 3 = f32<-bf16. */
static inline int in_is_bf16(int types) { return types >= 2; }
static inline int out_is_f32(int types) { return types == 1 || types == 3; }

/* Linear index of logical element (i, j) of a rows x cols matrix (common/matrix.hpp:154-164). */
static inline size_t at(size_t i, size_t j, size_t rows, size_t cols, int layout)
{
    return layout == 0 ? i * cols + j : j * rows + i;
}

/* init_matrix (test/test.hpp:33-54): a freshly seeded mt19937(1) per call, values drawn in
 * logical row-then-column order whatever the storage layout.  `bf16` selects the 16-bit
 * format of `data`. */
void oracle_init_matrix(uint16_t* data, size_t rows, size_t cols, int layout, int bf16)
{
    mt19937_t g;
    mt_seed(&g, 1u);
    for (size_t m = 0; m < rows; ++m)
        for (size_t n = 0; n < cols; ++n) {
            const float v = uniform_pm1(&g);
            data[at(m, n, rows, cols, layout)] = bf16 ? oracle_f32_to_bf16(v) : oracle_f32_to_f16(v);
        }
}

/* Benchmark fill (benchmark/bench.hpp:37-52): {0.1, 0.125, 0.15, 0.175, 0.2} cyclic in
 * logical row-then-column order. */
void oracle_init_matrix_cyclic(uint16_t* data, size_t rows, size_t cols, int layout, int bf16)
{
    static const float values[5] = {0.1f, 0.125f, 0.15f, 0.175f, 0.2f};
    size_t             idx       = 0;
    for (size_t m = 0; m < rows; ++m)
        for (size_t n = 0; n < cols; ++n) {
            const float v = values[idx % 5];
            data[at(m, n, rows, cols, layout)] = bf16 ? oracle_f32_to_bf16(v) : oracle_f32_to_f16(v);
            ++idx;
        }
}

/* ---- hgemm_cpu ---------------------------------------------------------------------------- */

typedef struct {
    int             types;
    void*           C;
    const float*    Af; /* widened A, row i contiguous in k:  Af[i * K + k]           */
    const float*    Bf; /* widened B, column j contiguous in k: Bf[j * K + k]          */
    size_t          M, N, K;
    int             lc;
    const uint32_t* rows; /* optional list of rows to compute (NULL: range)            */
    size_t          row_begin, row_end;
    const uint32_t* cols; /* optional list of columns (NULL: all)                       */
    size_t          n_cols;
} job_t;

static void store_c(const job_t* jb, size_t i, size_t j, float acc)
{
    const size_t idx = at(i, j, jb->M, jb->N, jb->lc);
    if (out_is_f32(jb->types))
        ((float*)jb->C)[idx] = acc;
    else if (in_is_bf16(jb->types))
        ((uint16_t*)jb->C)[idx] = oracle_f32_to_bf16(acc);
    else
        ((uint16_t*)jb->C)[idx] = oracle_f32_to_f16(acc);
}

/* The triple loop of test/test.hpp:59-129 for one row: j ascending, k ascending, float acc. */
static void do_row(const job_t* jb, size_t i)
{
    const float* a  = jb->Af + i * jb->K;
    const size_t nj = jb->cols ? jb->n_cols : jb->N;
    for (size_t jj = 0; jj < nj; ++jj) {
        const size_t j   = jb->cols ? jb->cols[jj] : jj;
        const float* b   = jb->Bf + j * jb->K;
        float        acc = 0.0f;
        for (size_t k = 0; k < jb->K; ++k) acc += a[k] * b[k];
        store_c(jb, i, j, acc);
    }
}

typedef struct {
    const job_t* jb;
    size_t       t, nt;
} worker_t;

static void* worker(void* arg)
{
    const worker_t* w  = (const worker_t*)arg;
    const job_t*    jb = w->jb;
    if (jb->rows) {
        for (size_t r = w->t; r < jb->row_end; r += w->nt) do_row(jb, jb->rows[r]);
    } else {
        for (size_t i = jb->row_begin + w->t; i < jb->row_end; i += w->nt) do_row(jb, i);
    }
    return NULL;
}

static float widen(const uint16_t* p, size_t idx, int bf16)
{
    return bf16 ? oracle_bf16_to_f32(p[idx]) : oracle_f16_to_f32(p[idx]);
}

/* Core: computes C(i, j) for i in `rows` (or [row_begin, row_end)) and j in `cols` (or all),
 * over `threads` host threads (rows are independent, so threading does not change any
 * result).  Inputs are widened to float once (exactly); the arithmetic per element is the
 * reference's.  Returns 0, or -1 on allocation failure / bad arguments. */
int oracle_hgemm_select(int types, void* C, const uint16_t* A, const uint16_t* B, size_t M, size_t N,
                        size_t K, int lc, int la, int lb, const uint32_t* rows, size_t n_rows,
                        size_t row_begin, size_t row_end, const uint32_t* cols, size_t n_cols,
                        int threads)
{
    if (types < 0 || types > 3 || !C || (K && (!A || !B))) return -1;
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    const int bf16 = in_is_bf16(types);
    /* Widen only what is needed: all of B (or the selected columns), the selected rows of A. */
    float* Af = (float*)malloc(sizeof(float) * (M * K ? M * K : 1));
    float* Bf = (float*)malloc(sizeof(float) * (N * K ? N * K : 1));
    if (!Af || !Bf) {
        free(Af);
        free(Bf);
        return -1;
    }
    if (rows) {
        for (size_t r = 0; r < n_rows; ++r) {
            const size_t i = rows[r];
            for (size_t k = 0; k < K; ++k) Af[i * K + k] = widen(A, at(i, k, M, K, la), bf16);
        }
    } else {
        for (size_t i = row_begin; i < row_end; ++i)
            for (size_t k = 0; k < K; ++k) Af[i * K + k] = widen(A, at(i, k, M, K, la), bf16);
    }
    if (cols) {
        for (size_t c = 0; c < n_cols; ++c) {
            const size_t j = cols[c];
            for (size_t k = 0; k < K; ++k) Bf[j * K + k] = widen(B, at(k, j, K, N, lb), bf16);
        }
    } else if (lb == 1) {
        for (size_t j = 0; j < N; ++j)
            for (size_t k = 0; k < K; ++k) Bf[j * K + k] = widen(B, j * K + k, bf16);
    } else {
        for (size_t k = 0; k < K; ++k)
            for (size_t j = 0; j < N; ++j) Bf[j * K + k] = widen(B, k * N + j, bf16);
    }

    job_t jb;
    jb.types     = types;
    jb.C         = C;
    jb.Af        = Af;
    jb.Bf        = Bf;
    jb.M         = M;
    jb.N         = N;
    jb.K         = K;
    jb.lc        = lc;
    jb.rows      = rows;
    jb.row_begin = rows ? 0 : row_begin;
    jb.row_end   = rows ? n_rows : row_end;
    jb.cols      = cols;
    jb.n_cols    = n_cols;

    pthread_t th[256];
    worker_t  ws[256];
    int       started = 0;
    for (int t = 0; t < threads; ++t) {
        ws[t].jb = &jb;
        ws[t].t  = (size_t)t;
        ws[t].nt = (size_t)threads;
        if (t == threads - 1) {
            worker(&ws[t]); /* the calling thread takes the last share */
        } else if (pthread_create(&th[t], NULL, worker, &ws[t]) == 0) {
            ++started;
        } else {
            worker(&ws[t]);
            th[t] = 0;
        }
    }
    for (int t = 0; t < threads - 1; ++t)
        if (th[t]) pthread_join(th[t], NULL);
    (void)started;
    free(Af);
    free(Bf);
    return 0;
}

/* hgemm_cpu (test/test.hpp:59-129): the whole of C. */
int oracle_hgemm(int types, void* C, const uint16_t* A, const uint16_t* B, size_t M, size_t N, size_t K,
                 int lc, int la, int lb, int threads)
{
    return oracle_hgemm_select(types, C, A, B, M, N, K, lc, la, lb, NULL, 0, 0, M, NULL, 0, threads);
}

/* Same loop restricted to rows [row_begin, row_end) of C (other elements untouched). */
int oracle_hgemm_rows(int types, void* C, const uint16_t* A, const uint16_t* B, size_t M, size_t N,
                      size_t K, int lc, int la, int lb, size_t row_begin, size_t row_end, int threads)
{
    if (row_end > M || row_begin > row_end) return -1;
    return oracle_hgemm_select(types, C, A, B, M, N, K, lc, la, lb, NULL, 0, row_begin, row_end, NULL, 0,
                               threads);
}

/* ---- calculate_cosine_similarity (test/test.hpp:134-196) --------------------------------- */

/* `kind`: 0 = f16, 1 = f32, 2 = bf16 elements.  Float accumulators, logical row-then-column
 * order, as in the reference. */
float oracle_cosine_similarity(const void* gpu, const void* cpu, size_t M, size_t N, int layout, int kind)
{
    float dot = 0.0f, ng = 0.0f, nc = 0.0f;
    for (size_t i = 0; i < M; ++i)
        for (size_t j = 0; j < N; ++j) {
            const size_t idx = at(i, j, M, N, layout);
            float        g, c;
            if (kind == 1) {
                g = ((const float*)gpu)[idx];
                c = ((const float*)cpu)[idx];
            } else {
                g = widen((const uint16_t*)gpu, idx, kind == 2);
                c = widen((const uint16_t*)cpu, idx, kind == 2);
            }
            dot += g * c;
            ng += g * g;
            nc += c * c;
        }
    if (ng < 1e-10f || nc < 1e-10f) {
        float mg = 0.0f, mc = 0.0f;
        for (size_t i = 0; i < M; ++i)
            for (size_t j = 0; j < N; ++j) {
                const size_t idx = at(i, j, M, N, layout);
                float        g, c;
                if (kind == 1) {
                    g = ((const float*)gpu)[idx];
                    c = ((const float*)cpu)[idx];
                } else {
                    g = widen((const uint16_t*)gpu, idx, kind == 2);
                    c = widen((const uint16_t*)cpu, idx, kind == 2);
                }
                mg = fmaxf(mg, fabsf(g));
                mc = fmaxf(mc, fabsf(c));
            }
        const float tol = (kind == 2) ? 1e-2f : 1e-4f;
        return (mg < tol && mc < tol) ? 1.0f : 0.0f;
    }
    return dot / (sqrtf(ng) * sqrtf(nc));
}
