/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE. CPU restatement of the arithmetic of k0zi/Vulkanizer's cuBLAS GEMM path,
 * used only as the checker in tests/, in the smoke test and as the timed CPU baseline of the benchmark. Nothing
 * under vulkanizer_b200/ links, loads or calls it.
 *
 * What is restated, and from where (paths inside the Vulkanizer tree):
 *   - f16 / bf16 <-> f32 conversions with round-to-nearest-even: src/npu/host.cpp:15-67
 *     (the same integer algorithm as the shaders' roundToBits, src/cublas/shaders/gemm.comp:52-74);
 *   - the reference's own CPU GEMM, `CpuBackend::gemm`: src/npu/backend.cpp:28-52 with `epilogue`
 *     src/npu/host.cpp:161-184: operands widened to f32, f32 accumulation with k ascending for each
 *     element, v = alpha * acc, then v += beta * C only when beta != 0, one rounding to C's type;
 *   - the fp64 reference of the reference's acceptance test: tests/cublas.cpp:121-136 (double
 *     accumulation, float(alpha * acc + beta * C), one rounding to C's type) and its cuBLASLt form with
 *     bias / ReLU / tanh-GELU applied after D was rounded once: tests/cublas.cpp:456-475;
 *   - the test's data generator, a 32-bit LCG: tests/cublas.cpp:64-78.
 *
 * Pins: the conversions are checked against the known answers of tests/npu.cpp:110-121, and oracle_gemm_f32
 * is checked bit for bit against the reference's CpuBackend::gemm compiled from its own sources
 * (oracle/_ref, built by oracle/Makefile) and against golden vectors generated from it (tests/golden).
 *
 * int8 -> int32: PARITY UNPINNED. Vulkanizer has no int8 GEMM (src/cublas/cublas.cpp:178-185 and 304-308 answer
 * CUBLAS_STATUS_NOT_SUPPORTED), so oracle_gemm_s8 is exact integer arithmetic, checked against mathematics only.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#pragma STDC FP_CONTRACT OFF

#include <pthread.h>
#include <unistd.h>

/* A plain parallel-for over [0, count) on the host's cores (pthreads; the toolchain here has no OpenMP runtime). */
typedef void (*oracle_body)(int64_t index, void* ctx);
struct oracle_span { oracle_body body; void* ctx; int64_t first, last; };
static void* oracle_run_span(void* arg) {
    struct oracle_span* s = (struct oracle_span*)arg;
    for (int64_t i = s->first; i < s->last; ++i) s->body(i, s->ctx);
    return 0;
}
static void oracle_parallel_for(int64_t count, oracle_body body, void* ctx) {
    long cores = sysconf(_SC_NPROCESSORS_ONLN);
    int64_t threads = cores < 1 ? 1 : cores > 64 ? 64 : cores;
    if (threads > count) threads = count > 0 ? count : 1;
    pthread_t ids[64];
    struct oracle_span spans[64];
    for (int64_t t = 0; t < threads; ++t) {
        spans[t].body = body, spans[t].ctx = ctx;
        spans[t].first = count * t / threads, spans[t].last = count * (t + 1) / threads;
        if (t > 0 && pthread_create(&ids[t], 0, oracle_run_span, &spans[t]) != 0) {
            oracle_run_span(&spans[t]); /* could not start a thread: do the span here */
            ids[t] = ids[0];
            spans[t].first = spans[t].last = -1;
        }
    }
    oracle_run_span(&spans[0]);
    for (int64_t t = 1; t < threads; ++t)
        if (spans[t].first != -1 || spans[t].last != -1) pthread_join(ids[t], 0);
}

enum { ORACLE_F32 = 0, ORACLE_F16 = 1, ORACLE_BF16 = 2 };

/* ---- conversions (src/npu/host.cpp:15-67) ---- */

float oracle_half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, mant = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0x1F) bits = sign | 0x7F800000u | (mant << 13);
    else if (exp != 0) bits = sign | ((exp + 112u) << 23) | (mant << 13);
    else if (mant == 0) bits = sign;
    else { /* subnormal half: normalise */
        int shift = 0;
        uint32_t m = mant;
        while (!(m & 0x400u)) m <<= 1, ++shift;
        bits = sign | ((uint32_t)(113 - shift) << 23) | ((m & 0x3FFu) << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t oracle_float_to_half(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    const uint32_t sign = (u >> 16) & 0x8000u, mag = u & 0x7FFFFFFFu;
    if (mag > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);  /* NaN */
    if (mag >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to infinity */
    if (mag < 0x38800000u) {                                   /* result is subnormal or zero */
        if (mag < 0x33000000u) return (uint16_t)sign;
        const uint32_t e = mag >> 23, mant = (mag & 0x7FFFFFu) | 0x800000u, shift = 126u - e;
        uint32_t v = mant >> shift;
        const uint32_t rest = mant & ((1u << shift) - 1u), half = 1u << (shift - 1u);
        if (rest > half || (rest == half && (v & 1u))) ++v;
        return (uint16_t)(sign | v);
    }
    uint32_t v = (mag - 0x38000000u) >> 13;
    const uint32_t rest = mag & 0x1FFFu;
    if (rest > 0x1000u || (rest == 0x1000u && (v & 1u))) ++v;
    return (uint16_t)(sign | v);
}

float oracle_bf16_to_float(uint16_t h) {
    const uint32_t bits = (uint32_t)h << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t oracle_float_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u); /* quiet NaN */
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static float load_elem(const void* base, int type, int64_t i) {
    switch (type) {
    case ORACLE_F16: return oracle_half_to_float(((const uint16_t*)base)[i]);
    case ORACLE_BF16: return oracle_bf16_to_float(((const uint16_t*)base)[i]);
    default: return ((const float*)base)[i];
    }
}

static void store_elem(void* base, int type, int64_t i, float v) {
    switch (type) {
    case ORACLE_F16: ((uint16_t*)base)[i] = oracle_float_to_half(v); break;
    case ORACLE_BF16: ((uint16_t*)base)[i] = oracle_float_to_bf16(v); break;
    default: ((float*)base)[i] = v; break;
    }
}

static size_t elem_size(int type) { return type == ORACLE_F32 ? 4 : 2; }

/* Rounds a float to `type` and back. */
float oracle_round_to(float v, int type) {
    if (type == ORACLE_F16) return oracle_half_to_float(oracle_float_to_half(v));
    if (type == ORACLE_BF16) return oracle_bf16_to_float(oracle_float_to_bf16(v));
    return v;
}

/* ---- data of the reference's acceptance test (tests/cublas.cpp:64-78) ----
 * seed <- seed * 1664525 + 1013904223; value (int(seed >> 24) - 128) / 64, rounded to the storage type.
 * Writes the storage bytes and, when `values` is not null, the float each element actually holds. */
void oracle_fill_lcg(int type, int64_t count, uint32_t seed, void* bytes, float* values) {
    for (int64_t i = 0; i < count; ++i) {
        seed = seed * 1664525u + 1013904223u;
        float v = (float)((int)(seed >> 24) - 128) / 64.0f;
        store_elem(bytes, type, i, v);
        if (values) values[i] = load_elem(bytes, type, i);
    }
}

/* ---- the reference's CPU GEMM (src/npu/backend.cpp:28-52, src/npu/host.cpp:161-184) ----
 * Column-major C = alpha op(A) op(B) + beta C over `batch` strided entries; strides in elements. */
void oracle_gemm_f32(int transA, int transB, int64_t m, int64_t n, int64_t k, int64_t batch, float alpha, const void* A,
                     int typeA, int64_t lda, int64_t strideA, const void* B, int typeB, int64_t ldb, int64_t strideB,
                     float beta, void* C, int typeC, int64_t ldc, int64_t strideC) {
    float* acol = (float*)malloc((size_t)(k > 0 ? k : 1) * sizeof(float));
    float* bcol = (float*)malloc((size_t)(k > 0 ? k : 1) * sizeof(float));
    for (int64_t e = 0; e < batch; ++e) {
        const char* a = (const char*)A + e * strideA * (int64_t)elem_size(typeA);
        const char* b = (const char*)B + e * strideB * (int64_t)elem_size(typeB);
        char* c = (char*)C + e * strideC * (int64_t)elem_size(typeC);
        for (int64_t j = 0; j < n; ++j) {
            for (int64_t l = 0; l < k; ++l) bcol[l] = load_elem(b, typeB, transB ? j + l * ldb : l + j * ldb);
            for (int64_t i = 0; i < m; ++i) {
                for (int64_t l = 0; l < k; ++l) acol[l] = load_elem(a, typeA, transA ? l + i * lda : i + l * lda);
                /* the reference adds l * r into out[q] for p = 0 .. k-1 in order, l from op(B), r from op(A); product
                 * and sum are two roundings there (its -O2 x86-64 build has no fused multiply-add), hence
                 * FP_CONTRACT OFF above and -ffp-contract=off in the Makefile */
                float acc = 0.0f;
                for (int64_t l = 0; l < k; ++l) acc += bcol[l] * acol[l];
                float v = alpha * acc;
                if (beta != 0.0f) v += beta * load_elem(c, typeC, i + j * ldc);
                store_elem(c, typeC, i + j * ldc, v);
            }
        }
    }
    free(acol);
    free(bcol);
}

/* ---- the acceptance test's fp64 reference (tests/cublas.cpp:121-136) ----
 * want = round_to_C(float(alpha * sum_l double(a) * double(b) + double(beta) * C)). `want` holds floats, one
 * per element of C's storage (elements outside the m x n window keep C's value); `wantAbs`, when not null,
 * receives |alpha| * sum |a b| for the test's fp16-math allowance. */
struct fp64_job {
    int transA, transB, typeA, typeB, typeC;
    int64_t m, n, k, lda, ldb, ldc, strideA, strideB, strideC;
    float alpha, beta;
    const void *A, *B;
    float *want, *wantAbs;
};
static void fp64_column(int64_t index, void* ctx) {
    const struct fp64_job* g = (const struct fp64_job*)ctx;
    const int64_t e = index / g->n, j = index % g->n;
    const char* a = (const char*)g->A + e * g->strideA * (int64_t)elem_size(g->typeA);
    const char* b = (const char*)g->B + e * g->strideB * (int64_t)elem_size(g->typeB);
    double* bcol = (double*)malloc((size_t)(g->k > 0 ? g->k : 1) * sizeof(double));
    for (int64_t l = 0; l < g->k; ++l) bcol[l] = (double)load_elem(b, g->typeB, g->transB ? j + l * g->ldb : l + j * g->ldb);
    for (int64_t i = 0; i < g->m; ++i) {
        double acc = 0.0, absAcc = 0.0;
        for (int64_t l = 0; l < g->k; ++l) {
            const double p = (double)load_elem(a, g->typeA, g->transA ? l + i * g->lda : i + l * g->lda) * bcol[l];
            acc += p;
            absAcc += fabs(p);
        }
        const int64_t at = e * g->strideC + i + j * g->ldc;
        g->want[at] = oracle_round_to((float)((double)g->alpha * acc + (double)g->beta * (double)g->want[at]), g->typeC);
        if (g->wantAbs) g->wantAbs[at] = (float)(fabs((double)g->alpha) * absAcc);
    }
    free(bcol);
}
void oracle_gemm_fp64(int transA, int transB, int64_t m, int64_t n, int64_t k, int64_t batch, float alpha, const void* A,
                      int typeA, int64_t lda, int64_t strideA, const void* B, int typeB, int64_t ldb, int64_t strideB,
                      float beta, const void* C, int typeC, int64_t ldc, int64_t strideC, float* want, float* wantAbs) {
    if (batch <= 0 || n <= 0) return;
    for (int64_t i = 0; i < strideC * (batch - 1) + ldc * n; ++i) want[i] = load_elem(C, typeC, i);
    struct fp64_job g = {transA, transB, typeA, typeB, typeC, m, n, k, lda, ldb, ldc, strideA, strideB, strideC,
                         alpha, beta, A, B, want, wantAbs};
    oracle_parallel_for(batch * n, fp64_column, &g);
}

/* fp64 dot products for a sample of C: rows[i] x cols[j] -> out[i + j * nrows] (double, before alpha / beta),
 * the way the reference's large test looks at every 7th row and column only (tests/cublas.cpp:550-585).
 * Type codes as above, plus 3 for int8 operands. */
struct dots_job {
    int transA, transB, typeA, typeB;
    int64_t k, lda, ldb, nrows;
    const void *A, *B;
    const int64_t *rows, *cols;
    double* out;
};
static double load_any(const void* base, int type, int64_t i) {
    return type == 3 ? (double)((const int8_t*)base)[i] : (double)load_elem(base, type, i);
}
static void dots_column(int64_t jj, void* ctx) {
    const struct dots_job* g = (const struct dots_job*)ctx;
    const int64_t j = g->cols[jj];
    for (int64_t ii = 0; ii < g->nrows; ++ii) {
        const int64_t i = g->rows[ii];
        double acc = 0.0;
        for (int64_t l = 0; l < g->k; ++l)
            acc += load_any(g->A, g->typeA, g->transA ? l + i * g->lda : i + l * g->lda) *
                   load_any(g->B, g->typeB, g->transB ? j + l * g->ldb : l + j * g->ldb);
        g->out[ii + jj * g->nrows] = acc;
    }
}
void oracle_dots_fp64(int transA, int transB, int64_t k, const void* A, int typeA, int64_t lda, const void* B, int typeB,
                      int64_t ldb, const int64_t* rows, int64_t nrows, const int64_t* cols, int64_t ncols, double* out) {
    struct dots_job g = {transA, transB, typeA, typeB, k, lda, ldb, nrows, A, B, rows, cols, out};
    oracle_parallel_for(ncols, dots_column, &g);
}

/* ---- cuBLASLt expectation (tests/cublas.cpp:456-475): D = act(round_D(alpha * acc + beta * C) + bias[row]) ----
 * epilogue bits: 1 bias, 2 ReLU, 4 GELU. All matrices of one storage type, dense (ld = rows). */
void oracle_lt_fp64(int transA, int transB, int64_t m, int64_t n, int64_t k, int64_t batch, float alpha, const void* A,
                    const void* B, float beta, const void* C, const void* bias, int type, int epilogue, float* want) {
    const int64_t rowsA = transA ? k : m, rowsB = transB ? n : k;
    const int64_t sA = rowsA * (transA ? m : k), sB = rowsB * (transB ? k : n), sC = m * n;
    for (int64_t e = 0; e < batch; ++e)
        for (int64_t j = 0; j < n; ++j)
            for (int64_t i = 0; i < m; ++i) {
                double acc = 0.0;
                for (int64_t l = 0; l < k; ++l)
                    acc += (double)load_elem(A, type, e * sA + (transA ? l + i * rowsA : i + l * rowsA)) *
                           (double)load_elem(B, type, e * sB + (transB ? j + l * rowsB : l + j * rowsB));
                double v = (double)alpha * acc + (double)beta * (double)load_elem(C, type, e * sC + i + j * m);
                if (type != ORACLE_F32) v = oracle_round_to((float)v, type);
                if (epilogue & 1) v += load_elem(bias, type, i);
                if (epilogue & 2) v = v > 0.0 ? v : 0.0;
                if (epilogue & 4) v = 0.5 * v * (1.0 + tanh(0.7978845608 * (v + 0.044715 * v * v * v)));
                want[e * sC + i + j * m] = type != ORACLE_F32 ? oracle_round_to((float)v, type) : (float)v;
            }
}

/* ---- int8 x int8 -> int32, exact (no reference counterpart: parity unpinned) ---- */
struct s8_job {
    int transA, transB;
    int64_t m, n, k, lda, ldb, ldc, strideA, strideB, strideC;
    int32_t alpha, beta;
    const int8_t *A, *B;
    int32_t* C;
};
static void s8_column(int64_t index, void* ctx) {
    const struct s8_job* g = (const struct s8_job*)ctx;
    const int64_t e = index / g->n, j = index % g->n;
    const int8_t* a = g->A + e * g->strideA;
    const int8_t* b = g->B + e * g->strideB;
    int32_t* c = g->C + e * g->strideC;
    for (int64_t i = 0; i < g->m; ++i) {
        int64_t acc = 0;
        for (int64_t l = 0; l < g->k; ++l)
            acc += (int64_t)a[g->transA ? l + i * g->lda : i + l * g->lda] * (int64_t)b[g->transB ? j + l * g->ldb : l + j * g->ldb];
        const int64_t v = (int64_t)g->alpha * acc + (g->beta != 0 ? (int64_t)g->beta * (int64_t)c[i + j * g->ldc] : 0);
        c[i + j * g->ldc] = (int32_t)(uint32_t)(uint64_t)v; /* wraps like 32-bit hardware arithmetic */
    }
}
void oracle_gemm_s8(int transA, int transB, int64_t m, int64_t n, int64_t k, int64_t batch, int32_t alpha, const int8_t* A,
                    int64_t lda, int64_t strideA, const int8_t* B, int64_t ldb, int64_t strideB, int32_t beta, int32_t* C,
                    int64_t ldc, int64_t strideC) {
    if (batch <= 0 || n <= 0) return;
    struct s8_job g = {transA, transB, m, n, k, lda, ldb, ldc, strideA, strideB, strideC, alpha, beta, A, B, C};
    oracle_parallel_for(batch * n, s8_column, &g);
}
