/*
 * CPU oracle for the block-quantized linear operators (TEST INFRASTRUCTURE).
 *
 * PARITY UNPINNED: the makepad/makepad snapshot this build was specified
 * against holds no implementation, golden vector or known-answer test of this
 * path (no quantised-linear code anywhere in the tree; the only "AI" code is
 * the HTTP chat client studio/src/ai_chat/ai_chat_manager.rs:778-967).  This
 * file therefore restates the formats exactly as the task configuration words
 * them -- Q4: 4-bit signed codes in [-8,7] packed two per byte along K, one
 * fp16 scale per 32 K-elements; NVFP4: e2m1 codes, one e4m3 scale per 16
 * K-elements, one fp32 tensor scale -- using only the public IEEE-754 binary16,
 * bfloat16, OCP e4m3 (finite-only, max 448) and e2m1 definitions.  The
 * scalar-oracle-vs-accelerated-kernel relationship follows the reference's own
 * test idiom (libs/zune-jpeg/src/idct.rs:79-127: scalar idct_int compared with
 * the AVX2/NEON kernels on the same coefficients).  The number conversions are
 * pinned against numpy's float16 and torch's float8_e4m3fn / bfloat16 over
 * their full code spaces by the CPU tests.
 *
 * Nothing in the shipped library links, loads or calls this file.  Only the
 * tests, the smoke check and the benchmark's CPU-baseline leg use it.
 *
 * Row-parallel CPU threading (rows -> std threads) mirrors the reference's
 * tile-on-a-thread-pool idiom (examples/fractal_zoom/src/mandelbrot.rs:142-172).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ */
/* number formats                                                      */
/* ------------------------------------------------------------------ */

static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* IEEE binary16 -> binary32, exact (subnormals, inf, nan included). */
float orc_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: man * 2^-24 */
        float v = (float)man * 5.9604644775390625e-8f;
        return sign ? -v : v;
    }
    if (exp == 31) return bits_f32(sign | 0x7F800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* binary32 -> binary16, round to nearest even, overflow to inf. */
uint16_t orc_f32_to_f16(float f)
{
    uint32_t u = f32_bits(f);
    uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    uint32_t a = u & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (a > 0x7F800000u ? 0x200u | ((a >> 13) & 0x3FFu) : 0));
    if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);            /* >= 65520 rounds to inf */
    if (a < 0x33000001u) return sign;                                  /* <= 2^-25 rounds to 0 */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;                          /* 24-bit significand */
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;                     /* bits dropped */
    uint32_t kept = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (kept & 1u))) kept++;
    uint32_t out;
    if (e < -14) out = kept;                                           /* subnormal (may carry into normal) */
    else out = ((uint32_t)(e + 15) << 10) + (kept - 0x400u);           /* carry propagates into exponent */
    return (uint16_t)(sign | out);
}

/* binary32 -> bfloat16 bits, round to nearest even (nan kept quiet). */
uint16_t orc_f32_to_bf16(float f)
{
    uint32_t u = f32_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return (uint16_t)(u >> 16);
}

float orc_bf16_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }

/* OCP e4m3 (finite-only: S.EEEE.MMM, bias 7, 0x7F/0xFF = nan, max 448). */
float orc_e4m3_to_f32(uint8_t b)
{
    uint32_t exp = (b >> 3) & 0xFu, man = b & 7u;
    float v;
    if (exp == 15 && man == 7) return bits_f32(0x7FC00000u);
    if (exp == 0) v = (float)man * 0.001953125f;                      /* man * 2^-9 */
    else v = ldexpf((float)(8u + man), (int)exp - 10);                /* (1+man/8) * 2^(exp-7) */
    return (b & 0x80u) ? -v : v;
}

/* binary32 -> e4m3, round to nearest even, saturate to +-448, nan -> 0x7F. */
uint8_t orc_f32_to_e4m3(float f)
{
    uint32_t u = f32_bits(f);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return (uint8_t)(sign | 0x7Fu);
    float x = bits_f32(a);
    if (x >= 448.0f) return (uint8_t)(sign | 0x7Eu);
    /* grid spacing: 2^-9 below 2^-6, else 2^(e-3) */
    int e;
    (void)frexpf(x, &e);            /* x = m * 2^e, m in [0.5,1) -> floor(log2 x) = e-1 */
    int le = e - 1;
    if (x == 0.0f || le < -6) le = -6;
    float q = ldexpf(1.0f, le - 3);
    float r = rintf(x / q);         /* exact division by a power of two; rintf = RNE */
    float y = r * q;
    if (y >= 448.0f) y = 448.0f;    /* cannot exceed, kept for clarity */
    /* encode y */
    if (y == 0.0f) return sign;
    int ye;
    (void)frexpf(y, &ye);
    int yle = ye - 1;
    if (yle < -6) return (uint8_t)(sign | (uint8_t)(y * 512.0f));       /* subnormal */
    uint32_t man = (uint32_t)(ldexpf(y, 3 - yle)) - 8u;
    return (uint8_t)(sign | ((uint32_t)(yle + 7) << 3) | man);
}

/* e2m1: S.EE.M -> {0, .5, 1, 1.5, 2, 3, 4, 6} with sign. */
float orc_e2m1_to_f32(uint8_t nib)
{
    static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float v = mag[nib & 7u];
    return (nib & 8u) ? -v : v;
}

/* binary32 -> e2m1 nibble, round to nearest even (ties to the even mantissa), saturating. */
uint8_t orc_f32_to_e2m1(float f)
{
    uint8_t sign = (f32_bits(f) >> 31) ? 8u : 0u;
    float x = fabsf(f);
    uint8_t m;
    if (!(x == x)) return (uint8_t)(sign | 7u);
    if (x <= 0.25f) m = 0;
    else if (x < 0.75f) m = 1;
    else if (x <= 1.25f) m = 2;
    else if (x < 1.75f) m = 3;
    else if (x <= 2.5f) m = 4;
    else if (x < 3.5f) m = 5;
    else if (x <= 5.0f) m = 6;
    else m = 7;
    return (uint8_t)(sign | m);
}

/* Q4 code of element k in a packed row: element 2j is the LOW nibble of byte j,
 * element 2j+1 the HIGH nibble; a nibble is a two's-complement 4-bit integer. */
static inline int q4_code(const uint8_t* row, int64_t k)
{
    uint8_t b = row[k >> 1];
    int nib = (k & 1) ? (b >> 4) : (b & 0xF);
    return (nib ^ 8) - 8;
}

static inline uint8_t fp4_nib(const uint8_t* row, int64_t k)
{
    uint8_t b = row[k >> 1];
    return (uint8_t)((k & 1) ? (b >> 4) : (b & 0xF));
}

/* ------------------------------------------------------------------ */
/* a tiny row-range thread pool                                        */
/* ------------------------------------------------------------------ */

typedef void (*row_fn)(void* arg, int64_t r0, int64_t r1);
typedef struct { row_fn fn; void* arg; int64_t r0, r1; } row_job;
static void* row_thread(void* p) { row_job* j = (row_job*)p; j->fn(j->arg, j->r0, j->r1); return NULL; }

static void run_rows(row_fn fn, void* arg, int64_t rows, int threads)
{
    if (threads < 1) threads = 1;
    if (threads > rows) threads = (int)(rows > 0 ? rows : 1);
    if (threads == 1) { fn(arg, 0, rows); return; }
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)threads);
    row_job* jobs = (row_job*)malloc(sizeof(row_job) * (size_t)threads);
    for (int t = 0; t < threads; ++t) {
        jobs[t].fn = fn; jobs[t].arg = arg;
        jobs[t].r0 = rows * t / threads; jobs[t].r1 = rows * (t + 1) / threads;
        pthread_create(&th[t], NULL, row_thread, &jobs[t]);
    }
    for (int t = 0; t < threads; ++t) pthread_join(th[t], NULL);
    free(th); free(jobs);
}

/* ------------------------------------------------------------------ */
/* Q4                                                                  */
/* ------------------------------------------------------------------ */

/* W~[n,k] = fp32(scale[n,k/32]) * fp32(code[n,k]); the product is exact in
 * binary32 (11-bit by 4-bit significands), so this export is the bit-exact
 * criterion for every device layout. */
void orc_q4_dequantize(int64_t N, int64_t K, const uint8_t* codes, const uint16_t* scales, float* out)
{
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* row = codes + n * (K / 2);
        for (int64_t k = 0; k < K; ++k)
            out[n * K + k] = orc_f16_to_f32(scales[n * (K / 32) + k / 32]) * (float)q4_code(row, k);
    }
}

typedef struct {
    int64_t M, N, K; const uint8_t* codes; const uint16_t* scales; const float* X;
    double* Y64; float* Y32;
} q4_args;

/* Y[m,n] = sum_k W~[n,k] * X[m,k], accumulated in binary64: the arbiter for tolerance tests. */
static void q4_rows_f64(void* p, int64_t n0, int64_t n1)
{
    q4_args* a = (q4_args*)p;
    int64_t K = a->K;
    for (int64_t n = n0; n < n1; ++n) {
        const uint8_t* row = a->codes + n * (K / 2);
        for (int64_t m = 0; m < a->M; ++m) {
            const float* x = a->X + m * K;
            double acc = 0.0;
            for (int64_t b = 0; b < K / 32; ++b) {
                double s = (double)orc_f16_to_f32(a->scales[n * (K / 32) + b]);
                double part = 0.0;
                for (int64_t k = b * 32; k < b * 32 + 32; ++k) part += (double)q4_code(row, k) * (double)x[k];
                acc += s * part;
            }
            a->Y64[m * a->N + n] = acc;
        }
    }
}

void orc_q4_matmul_f64(int64_t M, int64_t N, int64_t K, const uint8_t* codes, const uint16_t* scales,
                       const float* X, double* Y, int threads)
{
    q4_args a = {M, N, K, codes, scales, X, Y, NULL};
    run_rows(q4_rows_f64, &a, N, threads);
}

/* The CPU path as the task configuration describes it: dequantise a block to
 * fp32 (w = fp32(scale) * fp32(code)), multiply-accumulate in fp32.  Eight
 * interleaved partial sums (element j of a block goes to lane j mod 8) keep
 * the order fixed while letting the compiler use the host's vector units.
 * This is the timed CPU baseline. */
static void q4_rows_f32(void* p, int64_t n0, int64_t n1)
{
    q4_args* a = (q4_args*)p;
    int64_t K = a->K;
    for (int64_t n = n0; n < n1; ++n) {
        const uint8_t* row = a->codes + n * (K / 2);
        const uint16_t* srow = a->scales + n * (K / 32);
        for (int64_t m = 0; m < a->M; ++m) {
            const float* x = a->X + m * K;
            float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int64_t b = 0; b < K / 32; ++b) {
                float s = orc_f16_to_f32(srow[b]);
                const uint8_t* q = row + b * 16;
                float wbuf[32];
                for (int j = 0; j < 16; ++j) {
                    wbuf[2 * j] = s * (float)(((q[j] & 0xF) ^ 8) - 8);
                    wbuf[2 * j + 1] = s * (float)(((q[j] >> 4) ^ 8) - 8);
                }
                const float* xb = x + b * 32;
                for (int j = 0; j < 32; j += 8)
                    for (int l = 0; l < 8; ++l) lane[l] += wbuf[j + l] * xb[j + l];
            }
            a->Y32[m * a->N + n] = ((lane[0] + lane[1]) + (lane[2] + lane[3])) + ((lane[4] + lane[5]) + (lane[6] + lane[7]));
        }
    }
}

void orc_q4_matmul_f32(int64_t M, int64_t N, int64_t K, const uint8_t* codes, const uint16_t* scales,
                       const float* X, float* Y, int threads)
{
    q4_args a = {M, N, K, codes, scales, X, NULL, Y};
    run_rows(q4_rows_f32, &a, N, threads);
}

/* ------------------------------------------------------------------ */
/* NVFP4                                                               */
/* ------------------------------------------------------------------ */

/* value[r,k] = fp32(e2m1[r,k]) * fp32(e4m3[r,k/16]) * tensor_scale.  The first
 * product is exact in binary32; the tensor scale multiplies last. */
void orc_nvfp4_dequantize(int64_t R, int64_t K, const uint8_t* codes, const uint8_t* sf, float tscale, float* out)
{
    for (int64_t r = 0; r < R; ++r) {
        const uint8_t* row = codes + r * (K / 2);
        for (int64_t k = 0; k < K; ++k)
            out[r * K + k] = orc_e2m1_to_f32(fp4_nib(row, k)) * orc_e4m3_to_f32(sf[r * (K / 16) + k / 16]) * tscale;
    }
}

typedef struct {
    int64_t M, N, K; const uint8_t *a, *sfa, *b, *sfb; float ta, tb; float* C32; uint16_t* C16;
} fp4_args;

/* C[m,n] = tsA*tsB * sum_k A~[m,k] * B~[n,k]  (B stored [N][K/2], K contiguous).
 * Every block partial (16 products of small dyadic rationals) is exact in
 * binary64 and so is the block's scaled value; the running sum is binary64. */
static void fp4_rows(void* p, int64_t m0, int64_t m1)
{
    fp4_args* g = (fp4_args*)p;
    int64_t K = g->K, KB = K / 16;
    float* arow = (float*)malloc(sizeof(float) * (size_t)K);
    for (int64_t m = m0; m < m1; ++m) {
        for (int64_t k = 0; k < K; ++k) arow[k] = orc_e2m1_to_f32(fp4_nib(g->a + m * (K / 2), k));
        for (int64_t n = 0; n < g->N; ++n) {
            const uint8_t* brow = g->b + n * (K / 2);
            double acc = 0.0;
            for (int64_t kb = 0; kb < KB; ++kb) {
                float part = 0.0f;                       /* |part| <= 16*36: exact in fp32 */
                for (int64_t k = kb * 16; k < kb * 16 + 16; ++k) part += arow[k] * orc_e2m1_to_f32(fp4_nib(brow, k));
                acc += (double)part * (double)orc_e4m3_to_f32(g->sfa[m * KB + kb]) * (double)orc_e4m3_to_f32(g->sfb[n * KB + kb]);
            }
            float c = (float)(acc * (double)g->ta * (double)g->tb);
            if (g->C32) g->C32[m * g->N + n] = c;
            if (g->C16) g->C16[m * g->N + n] = orc_f32_to_bf16(c);
        }
    }
    free(arow);
}

void orc_nvfp4_gemm(int64_t M, int64_t N, int64_t K, const uint8_t* a, const uint8_t* sfa, float ta,
                    const uint8_t* b, const uint8_t* sfb, float tb, float* C32, uint16_t* C16, int threads)
{
    fp4_args g = {M, N, K, a, sfa, b, sfb, ta, tb, C32, C16};
    run_rows(fp4_rows, &g, M, threads);
}

/* ------------------------------------------------------------------ */
/* vectorised conversions for the tests                                */
/* ------------------------------------------------------------------ */

/* Activation quantisation to NVFP4 (the usual recipe, stated here because the snapshot holds none): per row and
 * 16-element block, amax = max |x|; the block scale is e4m3(amax / (6 * tscale)) (round to nearest even, saturating,
 * 6 = the largest e2m1 magnitude); every element becomes e2m1(x / (e4m3_value * tscale)), round to nearest even,
 * saturating; a block whose scale encodes to 0 gets all-zero codes.  All arithmetic in binary32. */
void orc_nvfp4_quantize(int64_t R, int64_t K, const float* x, float tscale, uint8_t* codes, uint8_t* sf)
{
    for (int64_t r = 0; r < R; ++r)
        for (int64_t b = 0; b < K / 16; ++b) {
            const float* xb = x + r * K + 16 * b;
            float amax = 0.0f;
            for (int i = 0; i < 16; ++i) { float a = fabsf(xb[i]); if (a > amax) amax = a; }
            uint8_t s8 = orc_f32_to_e4m3(amax / (6.0f * tscale));
            float d = orc_e4m3_to_f32(s8) * tscale;
            sf[r * (K / 16) + b] = s8;
            for (int i = 0; i < 16; i += 2) {
                uint8_t lo = d > 0.0f ? orc_f32_to_e2m1(xb[i] / d) : 0;
                uint8_t hi = d > 0.0f ? orc_f32_to_e2m1(xb[i + 1] / d) : 0;
                codes[r * (K / 2) + 8 * b + i / 2] = (uint8_t)(lo | (hi << 4));
            }
        }
}

void orc_f16_to_f32_n(const uint16_t* in, float* out, int64_t n) { for (int64_t i = 0; i < n; ++i) out[i] = orc_f16_to_f32(in[i]); }
void orc_f32_to_f16_n(const float* in, uint16_t* out, int64_t n) { for (int64_t i = 0; i < n; ++i) out[i] = orc_f32_to_f16(in[i]); }
void orc_f32_to_bf16_n(const float* in, uint16_t* out, int64_t n) { for (int64_t i = 0; i < n; ++i) out[i] = orc_f32_to_bf16(in[i]); }
void orc_e4m3_to_f32_n(const uint8_t* in, float* out, int64_t n) { for (int64_t i = 0; i < n; ++i) out[i] = orc_e4m3_to_f32(in[i]); }
void orc_f32_to_e4m3_n(const float* in, uint8_t* out, int64_t n) { for (int64_t i = 0; i < n; ++i) out[i] = orc_f32_to_e4m3(in[i]); }
void orc_f32_to_e2m1_n(const float* in, uint8_t* out, int64_t n) { for (int64_t i = 0; i < n; ++i) out[i] = orc_f32_to_e2m1(in[i]); }
