/*
 * CPU oracle for Y = X * W^T (X row-major MxK, W row-major NxK, FP32 accumulate).
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke
 * check and the benchmark's CPU-baseline leg may call it; the GPU library never does.
 *
 * Parity status: the reference project ships no golden vectors, known-answer files
 * or host GEMM.  Its check is a GPU kernel whose loop body is
 *     acc = 0; for k in 0..K-1: acc += float(X[row*K+k]) * float(W[col*K+k]); Y[row*N+col] = acc
 * (reference src/bench.cu:68-85, loop at :77-84).  This file restates that loop on
 * the host.  The strict mode keeps the k-ascending FP32 order exactly; the fast mode
 * lets the compiler reorder the additions inside one dot product (vector lanes),
 * which is inside the rounding noise the tolerances allow.  The restatement is
 * pinned by hand-computable known answers and by fixtures under tests/golden/
 * that were produced by an independent float64 computation.
 *
 * The quantised variants (FP8 e4m3 per-tensor, MXFP8, W4A16, W4A4/MX-FP4) have no
 * counterpart in the reference at all ("parity unpinned" by the reference); their
 * oracle is "dequantise on the host, then the same FP32 GEMM", as the task states.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t v)
{
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even float -> bf16, NaN kept quiet (matches __float2bfloat16_rn) */
static inline uint16_t f32_to_bf16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u)
        return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_bf16_to_f32(const uint16_t *src, float *dst, size_t n)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++)
        dst[i] = bf16_to_f32(src[i]);
}

void oracle_f32_to_bf16(const float *src, uint16_t *dst, size_t n)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++)
        dst[i] = f32_to_bf16(src[i]);
}

/*
 * Fast mode building block: a 4-row x 4-column block of dot products over the full K, sixteen
 * FP32 accumulators, every operand element converted to FP32 where it is used (as the
 * reference loop does, src/bench.cu:79-81).  Additions inside one dot product are reordered
 * across SIMD lanes only.
 */
#define DOT4(T, CVT)                                                                               \
    static void dot_block_##T(const T *const x[4], const T *const w[4], int K, float out[4][4])    \
    {                                                                                              \
        float a00 = 0, a01 = 0, a02 = 0, a03 = 0, a10 = 0, a11 = 0, a12 = 0, a13 = 0;              \
        float a20 = 0, a21 = 0, a22 = 0, a23 = 0, a30 = 0, a31 = 0, a32 = 0, a33 = 0;              \
        const T *x0 = x[0], *x1 = x[1], *x2 = x[2], *x3 = x[3];                                    \
        const T *w0 = w[0], *w1 = w[1], *w2 = w[2], *w3 = w[3];                                    \
        _Pragma("omp simd reduction(+ : a00, a01, a02, a03, a10, a11, a12, a13, a20, a21, a22, a23, a30, a31, a32, a33)") \
        for (int k = 0; k < K; k++) {                                                              \
            float p0 = CVT(x0[k]), p1 = CVT(x1[k]), p2 = CVT(x2[k]), p3 = CVT(x3[k]);              \
            float q0 = CVT(w0[k]), q1 = CVT(w1[k]), q2 = CVT(w2[k]), q3 = CVT(w3[k]);              \
            a00 += p0 * q0; a01 += p0 * q1; a02 += p0 * q2; a03 += p0 * q3;                        \
            a10 += p1 * q0; a11 += p1 * q1; a12 += p1 * q2; a13 += p1 * q3;                        \
            a20 += p2 * q0; a21 += p2 * q1; a22 += p2 * q2; a23 += p2 * q3;                        \
            a30 += p3 * q0; a31 += p3 * q1; a32 += p3 * q2; a33 += p3 * q3;                        \
        }                                                                                          \
        out[0][0] = a00; out[0][1] = a01; out[0][2] = a02; out[0][3] = a03;                        \
        out[1][0] = a10; out[1][1] = a11; out[1][2] = a12; out[1][3] = a13;                        \
        out[2][0] = a20; out[2][1] = a21; out[2][2] = a22; out[2][3] = a23;                        \
        out[3][0] = a30; out[3][1] = a31; out[3][2] = a32; out[3][3] = a33;                        \
    }
#define CVT_F32(v) (v)
#define CVT_BF16(v) bf16_to_f32(v)
typedef uint16_t bf16_t;
DOT4(float, CVT_F32)
DOT4(bf16_t, CVT_BF16)

/*
 * Shared driver: Y[i, :] = X[rows[i], :] . W^T for i < n_rows (rows == NULL: rows 0..n_rows-1).
 * Work is cut into (16-row block) x (256-column chunk) tasks so a block of X stays in cache
 * while W streams past it once per row block.
 */
#define GEMM_ROWS(NAME, T, DOTFN, CVT)                                                              \
    static void NAME(int N, int K, const T *X, const T *W, float *Y, const int *rows, int n_rows, int strict) \
    {                                                                                               \
        const int RB = 16, CB = 256;                                                                \
        const int nrb = (n_rows + RB - 1) / RB, ncb = (N + CB - 1) / CB;                            \
        _Pragma("omp parallel for collapse(2) schedule(dynamic, 1)")                                \
        for (int rb = 0; rb < nrb; rb++)                                                            \
            for (int cb = 0; cb < ncb; cb++) {                                                      \
                const int i1 = (rb + 1) * RB < n_rows ? (rb + 1) * RB : n_rows;                     \
                const int c1 = (cb + 1) * CB < N ? (cb + 1) * CB : N;                               \
                for (int c = cb * CB; c < c1; c += 4)                                               \
                    for (int i = rb * RB; i < i1; i += 4) {                                         \
                        const T *xp[4], *wp[4];                                                     \
                        for (int u = 0; u < 4; u++) {                                               \
                            int ii = i + u < i1 ? i + u : i1 - 1;                                   \
                            int cc = c + u < c1 ? c + u : c1 - 1;                                   \
                            xp[u] = X + (size_t)(rows ? rows[ii] : ii) * K;                         \
                            wp[u] = W + (size_t)cc * K;                                             \
                        }                                                                           \
                        float out[4][4];                                                            \
                        if (strict) {                                                               \
                            for (int u = 0; u < 4; u++)                                             \
                                for (int v = 0; v < 4; v++) {                                       \
                                    volatile float acc = 0.0f; /* k ascending, no reassociation */  \
                                    for (int k = 0; k < K; k++) {                                   \
                                        float pr = CVT(xp[u][k]) * CVT(wp[v][k]);                   \
                                        acc = acc + pr;                                             \
                                    }                                                               \
                                    out[u][v] = acc;                                                \
                                }                                                                   \
                        } else {                                                                    \
                            DOTFN(xp, wp, K, out);                                                  \
                        }                                                                           \
                        for (int u = 0; u < 4 && i + u < i1; u++)                                   \
                            for (int v = 0; v < 4 && c + v < c1; v++)                               \
                                Y[(size_t)(i + u) * N + c + v] = out[u][v];                         \
                    }                                                                               \
            }                                                                                       \
    }
GEMM_ROWS(gemm_rows_f32, float, dot_block_float, CVT_F32)
GEMM_ROWS(gemm_rows_bf16, bf16_t, dot_block_bf16_t, CVT_BF16)

/* FP32 operands (the dequantise-then-GEMM oracle of the quantised variants) */
void oracle_gemm_f32_rows(int N, int K, const float *X, const float *W, float *Y,
                          const int *rows, int n_rows, int strict)
{
    gemm_rows_f32(N, K, X, W, Y, rows, n_rows, strict);
}

/*
 * bf16 in, FP32 out.  The reference's oracle signature (src/bench.cu:87-95:
 * naive_gemm_f32(M,N,K,X,W,Y)) with two additions: a row list and the strict flag.
 */
int oracle_gemm_bf16_rows(int M, int N, int K, const uint16_t *X, const uint16_t *W,
                          float *Y, const int *rows, int n_rows, int strict)
{
    (void)M;
    gemm_rows_bf16(N, K, X, W, Y, rows, n_rows, strict);
    return 0;
}

int oracle_gemm_bf16(int M, int N, int K, const uint16_t *X, const uint16_t *W, float *Y, int strict)
{
    return oracle_gemm_bf16_rows(M, N, K, X, W, Y, NULL, M, strict);
}

/*
 * Diagnostic mode: the same products (bf16 x bf16 is exact in FP32, hence in double) summed in
 * DOUBLE, k ascending, result kept in double.  Not the reference's arithmetic (its loop adds in
 * FP32, src/bench.cu:77-84); it exists to tell apart the two error sources when an FP32-summed
 * reference is itself uncertain by more than the tolerance under test (K = 16384 with unit-variance
 * inputs: the FP32 sum carries ~1e-3 of absolute noise, more than the bf16 spacing of the outputs
 * nearest zero).  With 53 significand bits the sum of K <= 2^20 such products is exact to ~1e-13.
 */
void oracle_gemm_bf16_rows_f64(int N, int K, const uint16_t *X, const uint16_t *W, double *Y,
                               const int *rows, int n_rows)
{
#pragma omp parallel for collapse(2) schedule(dynamic, 16)
    for (int i = 0; i < n_rows; i++)
        for (int c = 0; c < N; c++) {
            const uint16_t *x = X + (size_t)(rows ? rows[i] : i) * K, *w = W + (size_t)c * K;
            double a0 = 0, a1 = 0, a2 = 0, a3 = 0;
            int k = 0;
            for (; k + 4 <= K; k += 4) {
                a0 += (double)bf16_to_f32(x[k]) * (double)bf16_to_f32(w[k]);
                a1 += (double)bf16_to_f32(x[k + 1]) * (double)bf16_to_f32(w[k + 1]);
                a2 += (double)bf16_to_f32(x[k + 2]) * (double)bf16_to_f32(w[k + 2]);
                a3 += (double)bf16_to_f32(x[k + 3]) * (double)bf16_to_f32(w[k + 3]);
            }
            for (; k < K; k++) a0 += (double)bf16_to_f32(x[k]) * (double)bf16_to_f32(w[k]);
            Y[(size_t)i * N + c] = (a0 + a1) + (a2 + a3);
        }
}

/* ------------------------------------------------------------------------------------------
 * Number formats of the quantised variants (no reference counterpart; OCP MX v1.0 and the
 * OFP8 e4m3 "fn" format: no infinities, 0x7f/0xff = NaN, max finite 448).
 * ---------------------------------------------------------------------------------------- */

float oracle_e4m3_to_f32(uint8_t v)
{
    int s = v >> 7, e = (v >> 3) & 0xf, m = v & 7;
    float r;
    if (e == 0xf && m == 7) return NAN;
    if (e == 0) r = ldexpf((float)m, -9);           /* subnormal: m/8 * 2^-6 */
    else r = ldexpf((float)(8 + m), e - 7 - 3);
    return s ? -r : r;
}

/* round-to-nearest-even, saturating to +-448 (satfinite), NaN -> 0x7f */
uint8_t oracle_f32_to_e4m3(float f)
{
    if (isnan(f)) return 0x7f;
    uint8_t s = signbit(f) ? 0x80 : 0;
    float a = fabsf(f);
    if (a >= 464.0f) return s | 0x7e;                /* beyond the midpoint above 448: saturate */
    if (a < ldexpf(1.0f, -10)) return s;             /* below half the smallest subnormal */
    int e;
    (void)frexpf(a, &e);                             /* a = f * 2^e, f in [0.5,1) */
    int E = e - 1;                                   /* a in [2^E, 2^(E+1)) */
    if (E < -6) E = -6;                              /* subnormal range shares exponent -6 */
    float q = ldexpf(a, 3 - E);                      /* units of the 3-bit mantissa step */
    float rq = nearbyintf(q);                        /* RNE in the default rounding mode */
    int qi = (int)rq;
    if (qi >= 16) { qi = 8; E += 1; }                /* mantissa overflow */
    uint8_t bits;
    if (E == -6 && qi < 8) bits = (uint8_t)qi;       /* subnormal */
    else bits = (uint8_t)(((E + 7) << 3) | (qi - 8));
    if (bits > 0x7e) bits = 0x7e;
    return s | bits;
}

/* e2m1 (FP4): values +-{0, .5, 1, 1.5, 2, 3, 4, 6} */
static const float E2M1_LUT[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};

float oracle_e2m1_to_f32(uint8_t v)
{
    float r = E2M1_LUT[v & 7];
    return (v & 8) ? -r : r;
}

/* round-to-nearest, ties to the even code, saturating at 6 */
uint8_t oracle_f32_to_e2m1(float f)
{
    uint8_t s = signbit(f) ? 8 : 0;
    float a = fabsf(f);
    if (isnan(a)) return s | 7;
    uint8_t best = 0;
    float bd = INFINITY;
    for (uint8_t c = 0; c < 8; c++) {
        float d = fabsf(a - E2M1_LUT[c]);
        if (d < bd || (d == bd && (c & 1) == 0)) { bd = d; best = c; }
    }
    return s | best;
}

/* ue8m0: value 2^(v-127); 0xff = NaN */
float oracle_ue8m0_to_f32(uint8_t v)
{
    if (v == 0xff) return NAN;
    return ldexpf(1.0f, (int)v - 127);
}

/* smallest power of two >= amax/elem_max (so the scaled block fits), clamped to the format */
uint8_t oracle_ue8m0_for_block(float amax, float elem_max)
{
    if (!(amax > 0.f)) return 127;                   /* all-zero block: scale 1 */
    float t = amax / elem_max;
    int e;
    float m = frexpf(t, &e);                         /* t = m * 2^e, m in [0.5,1) */
    int p = (m == 0.5f) ? e - 1 : e;                 /* ceil(log2 t) */
    p += 127;
    if (p < 0) p = 0;
    if (p > 254) p = 254;
    return (uint8_t)p;
}

/*
 * MX quantisation of a row-major R x K matrix along K in blocks of 32:
 *   kind 8: elements e4m3 (1 byte each),   out_elems has R*K bytes
 *   kind 4: elements e2m1, two per byte (low nibble = even k), out_elems has R*K/2 bytes
 * scales: R x K/32 ue8m0 bytes, row-major.
 */
void oracle_mx_quantise(const float *src, int R, int K, int kind, uint8_t *out_elems, uint8_t *scales)
{
    const float emax = (kind == 8) ? 448.0f : 6.0f;
    int KB = K / 32;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < R; r++) {
        for (int b = 0; b < KB; b++) {
            const float *p = src + (size_t)r * K + b * 32;
            float amax = 0.f;
            for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(p[i]));
            uint8_t sc = oracle_ue8m0_for_block(amax, emax);
            scales[(size_t)r * KB + b] = sc;
            float inv = ldexpf(1.0f, 127 - (int)sc);
            if (kind == 8) {
                for (int i = 0; i < 32; i++)
                    out_elems[(size_t)r * K + b * 32 + i] = oracle_f32_to_e4m3(p[i] * inv);
            } else {
                for (int i = 0; i < 32; i += 2) {
                    uint8_t lo = oracle_f32_to_e2m1(p[i] * inv);
                    uint8_t hi = oracle_f32_to_e2m1(p[i + 1] * inv);
                    out_elems[((size_t)r * K + b * 32 + i) / 2] = (uint8_t)(lo | (hi << 4));
                }
            }
        }
    }
}

void oracle_mx_dequantise(const uint8_t *elems, const uint8_t *scales, int R, int K, int kind, float *dst)
{
    int KB = K / 32;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < R; r++) {
        for (int k = 0; k < K; k++) {
            float s = oracle_ue8m0_to_f32(scales[(size_t)r * KB + k / 32]);
            float v;
            if (kind == 8) v = oracle_e4m3_to_f32(elems[(size_t)r * K + k]);
            else {
                uint8_t byte = elems[((size_t)r * K + k) / 2];
                v = oracle_e2m1_to_f32((k & 1) ? (byte >> 4) : (byte & 0xf));
            }
            dst[(size_t)r * K + k] = v * s;
        }
    }
}

/* per-tensor e4m3: q = e4m3(src / scale) */
void oracle_e4m3_quantise(const float *src, size_t n, float scale, uint8_t *dst)
{
    float inv = 1.0f / scale;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++)
        dst[i] = oracle_f32_to_e4m3(src[i] * inv);
}

void oracle_e4m3_dequantise(const uint8_t *src, size_t n, float scale, float *dst)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++)
        dst[i] = oracle_e4m3_to_f32(src[i]) * scale;
}

/*
 * W4A16 weights: signed int4 in [-8,7], two per byte along K (low nibble = even k),
 * one bf16 scale per `group` K-elements: w[n,k] = q[n,k] * float(scale[n, k/group]).
 */
void oracle_int4_dequantise(const uint8_t *packed, const uint16_t *scales, int N, int K, int group, float *dst)
{
    int G = K / group;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        for (int k = 0; k < K; k++) {
            uint8_t byte = packed[((size_t)n * K + k) / 2];
            int q = (k & 1) ? (byte >> 4) : (byte & 0xf);
            if (q >= 8) q -= 16;
            dst[(size_t)n * K + k] = (float)q * bf16_to_f32(scales[(size_t)n * G + k / group]);
        }
    }
}

/*
 * Symmetric int4 quantisation of W4A16 weights, group-wise along K: s = bf16(max|w| / 7) (1 for an
 * all-zero group), q = clamp(rint(w * (1 / s)), -8, 7), packed two per byte (low nibble = even k).
 */
void oracle_int4_quantise(const float *w, int N, int K, int group, uint8_t *packed, uint16_t *scales)
{
    int G = K / group;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        for (int g = 0; g < G; g++) {
            const float *p = w + (size_t)n * K + (size_t)g * group;
            float amax = 0.f;
            for (int i = 0; i < group; i++) amax = fmaxf(amax, fabsf(p[i]));
            uint16_t sb = f32_to_bf16(amax > 0.f ? amax / 7.0f : 1.0f);
            scales[(size_t)n * G + g] = sb;
            float inv = 1.0f / bf16_to_f32(sb);
            for (int i = 0; i < group; i += 2) {
                float a = nearbyintf(p[i] * inv), b = nearbyintf(p[i + 1] * inv);
                a = fminf(fmaxf(a, -8.f), 7.f);
                b = fminf(fmaxf(b, -8.f), 7.f);
                packed[((size_t)n * K + (size_t)g * group + i) / 2] = (uint8_t)(((int)a & 0xf) | (((int)b & 0xf) << 4));
            }
        }
    }
}

/* number of OpenMP threads the library may use from now on (a launcher may have exported OMP_NUM_THREADS=1) */
void oracle_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
