/* cpu_ref.c -- plain-C CPU restatement of the decode linear-layer arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY: this file is the checker (and the "port"-kind CPU
 * baseline of the benchmark).  Nothing in the product library links or calls it.
 *
 * What it restates (paths relative to the reference project root):
 *   - threaded row-parallel GEMV, one sequential fp32 sum per output row:
 *       native/tests/reference_forward.cpp:49-75
 *   - e4m3 decode by integer bit construction:
 *       native/kernels/sm120/kernels.h:131-148
 *   - fp8 GEMV with double accumulation, row scale applied to the finished sum:
 *       native/tests/kernel_ops.cpp:842-850
 *   - bf16 GEMV with double accumulation:
 *       native/tests/gemv_bench.cpp:122-138
 *   - SwiGLU on bf16-rounded gate/up:  native/kernels/sm120/swiglu.cu:57-70
 *   - residual add + RMSNorm:          native/kernels/sm120/rmsnorm.cu:130-166
 *   - greedy argmax, ties to the lowest index: native/kernels/sm120/sampling.cu:70-99
 *
 * Parity pin: checked against the numpy oracle (itself pinned bit-for-bit on
 * the reference's Python implementation) and against the reference's native
 * CPU cross-check compiled in place (oracle/_ref) by the CPU test-suite.
 *
 * Build: see oracle/Makefile (gcc -O2 -fno-fast-math -pthread -shared).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_widen(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t bf16_narrow(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* e4m3 code -> f32: sign | rebias(exp) | mantissa; subnormals are normalised
 * by shifting the mantissa up (at most three steps). */
static inline float e4m3_widen(uint8_t c) {
    uint32_t sign = (uint32_t)(c & 0x80u) << 24;
    uint32_t e = (c >> 3) & 0xFu, m = c & 7u, bits;
    if (e == 0) {
        if (m == 0) {
            bits = sign;
        } else {
            uint32_t sh = 0;
            while ((m & 8u) == 0) { m <<= 1; ++sh; }
            bits = sign | ((127u - 6u - sh) << 23) | ((m & 7u) << 20);
        }
    } else {
        bits = sign | ((e + 120u) << 23) | (m << 20);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

float oracle_e4m3_to_f32(uint8_t c) { return e4m3_widen(c); }
uint16_t oracle_f32_to_bf16(float f) { return bf16_narrow(f); }

/* ------------------------------------------------------------------ threads */
typedef void (*row_fn)(uint32_t row, void* ctx);
typedef struct { row_fn fn; void* ctx; uint32_t rows; volatile uint32_t next; } job_t;

static void* worker(void* p) {
    job_t* j = (job_t*)p;
    for (;;) {
        /* rows handed out in blocks of 16 to keep the atomic cold */
        uint32_t r0 = __atomic_fetch_add(&j->next, 16u, __ATOMIC_RELAXED);
        if (r0 >= j->rows) break;
        uint32_t r1 = r0 + 16u < j->rows ? r0 + 16u : j->rows;
        for (uint32_t r = r0; r < r1; ++r) j->fn(r, j->ctx);
    }
    return NULL;
}

static void parallel_rows(uint32_t rows, int threads, row_fn fn, void* ctx) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    job_t j = {fn, ctx, rows, 0};
    if (threads == 1) { worker(&j); return; }
    pthread_t t[256];
    for (int i = 0; i < threads; ++i) pthread_create(&t[i], NULL, worker, &j);
    for (int i = 0; i < threads; ++i) pthread_join(t[i], NULL);
}

/* --------------------------------------------------------------- bf16 GEMV */
typedef struct {
    const uint16_t* w; const uint8_t* q; const float* scale;
    const uint16_t* x; uint16_t* y; float* y32;
    uint32_t M, N, K; int use_double;
} lin_t;

static void row_bf16(uint32_t n, void* p) {
    lin_t* a = (lin_t*)p;
    const uint16_t* wr = a->w + (size_t)n * a->K;
    for (uint32_t m = 0; m < a->M; ++m) {
        const uint16_t* xr = a->x + (size_t)m * a->K;
        float r;
        if (a->use_double) {
            double acc = 0.0;
            for (uint32_t k = 0; k < a->K; ++k)
                acc += (double)bf16_widen(xr[k]) * (double)bf16_widen(wr[k]);
            r = (float)acc;
        } else {
            float acc = 0.f;
            for (uint32_t k = 0; k < a->K; ++k) acc += bf16_widen(xr[k]) * bf16_widen(wr[k]);
            r = acc;
        }
        if (a->y) a->y[(size_t)m * a->N + n] = bf16_narrow(r);
        if (a->y32) a->y32[(size_t)m * a->N + n] = r;
    }
}

/* y[M,N] = bf16( x[M,K] . W[N,K]^T ).  use_double=0: sequential fp32 sum per
 * row (the native CPU cross-check's rule); 1: double sum (the kernel tests'
 * rule).  y32 (optional) receives the unrounded fp32 result. */
void oracle_linear_bf16(const uint16_t* w, const uint16_t* x, uint16_t* y, float* y32,
                        uint32_t M, uint32_t N, uint32_t K, int use_double, int threads) {
    lin_t a = {w, NULL, NULL, x, y, y32, M, N, K, use_double};
    parallel_rows(N, threads, row_bf16, &a);
}

/* ---------------------------------------------------------------- fp8 GEMV */
static void row_fp8(uint32_t n, void* p) {
    lin_t* a = (lin_t*)p;
    const uint8_t* qr = a->q + (size_t)n * a->K;
    for (uint32_t m = 0; m < a->M; ++m) {
        const uint16_t* xr = a->x + (size_t)m * a->K;
        float r;
        if (a->use_double) {
            double acc = 0.0;
            for (uint32_t k = 0; k < a->K; ++k)
                acc += (double)e4m3_widen(qr[k]) * (double)bf16_widen(xr[k]);
            r = (float)(acc * (double)a->scale[n]);
        } else {
            float acc = 0.f;
            for (uint32_t k = 0; k < a->K; ++k) acc += e4m3_widen(qr[k]) * bf16_widen(xr[k]);
            r = acc * a->scale[n];
        }
        if (a->y) a->y[(size_t)m * a->N + n] = bf16_narrow(r);
        if (a->y32) a->y32[(size_t)m * a->N + n] = r;
    }
}

/* y[M,N] = bf16( scale[n] * sum_k e4m3(q[n,k]) * x[m,k] ). */
void oracle_linear_fp8(const uint8_t* q, const float* scale, const uint16_t* x, uint16_t* y,
                       float* y32, uint32_t M, uint32_t N, uint32_t K, int use_double,
                       int threads) {
    lin_t a = {NULL, q, scale, x, y, y32, M, N, K, use_double};
    parallel_rows(N, threads, row_fp8, &a);
}

/* ------------------------------------------------------------ elementwise */
/* out[m,d] = bf16( silu(g) * u ), g = src[m, d], u = src[m, inter + d] */
void oracle_swiglu_gated(const uint16_t* src, uint16_t* out, uint32_t M, uint32_t inter) {
    for (uint32_t m = 0; m < M; ++m)
        for (uint32_t d = 0; d < inter; ++d) {
            float g = bf16_widen(src[(size_t)m * 2 * inter + d]);
            float u = bf16_widen(src[(size_t)m * 2 * inter + inter + d]);
            float s = g / (1.0f + expf(-g));
            out[(size_t)m * inter + d] = bf16_narrow(s * u);
        }
}

/* res = bf16(res + add) in place (add may be NULL), then
 * out = bf16( res * rsqrt(mean(res^2) + eps) * w ) on the ROUNDED residual. */
void oracle_residual_rmsnorm(uint16_t* res, const uint16_t* add, const uint16_t* w,
                             uint16_t* out, uint32_t n, float eps) {
    if (add)
        for (uint32_t i = 0; i < n; ++i) res[i] = bf16_narrow(bf16_widen(res[i]) + bf16_widen(add[i]));
    float ss = 0.f;
    for (uint32_t i = 0; i < n; ++i) { float v = bf16_widen(res[i]); ss += v * v; }
    float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (uint32_t i = 0; i < n; ++i) out[i] = bf16_narrow(bf16_widen(res[i]) * inv * bf16_widen(w[i]));
}

/* argmax over bf16 logits compared as f32; ties -> lowest index; NaN never wins;
 * returns INT32_MAX only when every logit is NaN (all -inf yields index 0). */
int32_t oracle_argmax_bf16(const uint16_t* logits, int32_t n) {
    float best = -INFINITY;
    int32_t bi = INT32_MAX;
    for (int32_t i = 0; i < n; ++i) {
        float v = bf16_widen(logits[i]);
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    return bi;
}
