/*
 * tb200_oracle.c -- TEST INFRASTRUCTURE, not product code.
 *
 * CPU restatement, in plain C, of the TornadoVM Java kernels on the dense /
 * quantised matrix-vector and matrix-matrix path.  It is the checker that the
 * CUDA library is compared with and the CPU baseline that is timed beside it.
 * Nothing in the shipped library or its host bindings may call into this file.
 *
 * Compile with -ffp-contract=off: the JVM never fuses a multiply with an add,
 * and every "ref" function below keeps the reference's fp32 evaluation order.
 * The "*_f64" twins evaluate the same formula with double accumulation and are
 * the yard-stick for relative-L2 error.
 *
 * Reference files followed (paths inside the TornadoVM project):
 *   tornado-examples/.../compute/MatrixVectorRowMajor.java      (mat-vec, Q8_0, DP4A)
 *   tornado-examples/.../compute/MatrixMultiplication2D.java    (SGEMM)
 *   tornado-examples/.../compute/MatrixMultiplicationMMA.java   (FP16 GEMM reference loop)
 *   tornado-api/.../utils/QuantizationUtils.java                (dp4a)
 *   tornado-api/.../types/HalfFloat.java                        (fp16 conversions)
 * Third-party arithmetic that is not part of the TornadoVM tree and is restated
 * from its public specification: java.util.Random (JDK 21 Javadoc: 48-bit LCG)
 * and Float.floatToFloat16 / float16ToFloat (IEEE 754 binary16, round to
 * nearest even).
 *
 * Parity status: pinned for fp16 conversion, dp4a, the Q8_0 quantiser and the
 * GEMM/GEMV loops by the closed-form vectors of the reference's own unit tests
 * (see tests/test_oracle_golden.py).  Q4_0, batched GEMV and per-block
 * activation quantisation do not exist in the reference: parity unpinned.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* java.util.Random (JDK Javadoc: class Random, methods next, nextInt,        */
/* nextFloat, nextDouble, nextGaussian).                                      */
/* ------------------------------------------------------------------------- */
typedef struct {
    uint64_t seed;
    int have_next_gaussian;
    double next_gaussian;
} orc_jrand;

#define JR_MULT 0x5DEECE66DULL
#define JR_MASK ((1ULL << 48) - 1)

ORC_API void orc_jrand_init(orc_jrand *r, int64_t seed) {
    r->seed = ((uint64_t)seed ^ JR_MULT) & JR_MASK;
    r->have_next_gaussian = 0;
    r->next_gaussian = 0.0;
}

static inline int32_t jr_next(orc_jrand *r, int bits) {
    r->seed = (r->seed * JR_MULT + 0xBULL) & JR_MASK;
    return (int32_t)((int64_t)r->seed >> (48 - bits));
}

ORC_API int32_t orc_jrand_next_int(orc_jrand *r) { return jr_next(r, 32); }

ORC_API int32_t orc_jrand_next_int_bound(orc_jrand *r, int32_t bound) {
    int32_t bits = jr_next(r, 31);
    int32_t m = bound - 1;
    if ((bound & m) == 0) {
        return (int32_t)(((int64_t)bound * (int64_t)bits) >> 31);
    }
    int32_t val = bits % bound;
    /* Java: while (bits - val + m < 0) with 32-bit wrap-around */
    while ((int32_t)((uint32_t)bits - (uint32_t)val + (uint32_t)m) < 0) {
        bits = jr_next(r, 31);
        val = bits % bound;
    }
    return val;
}

ORC_API float orc_jrand_next_float(orc_jrand *r) {
    return (float)jr_next(r, 24) / (float)(1 << 24);
}

ORC_API double orc_jrand_next_double(orc_jrand *r) {
    int64_t hi = (int64_t)jr_next(r, 26) << 27;
    int64_t lo = jr_next(r, 27);
    return (double)(hi + lo) * 0x1.0p-53;
}

/* The JDK evaluates the polar method with StrictMath.log / sqrt; libm's log can
 * differ from it in the last bit, so Gaussian draws match Java to 1 ulp, not
 * bit for bit.  They only shape synthetic operands. */
ORC_API double orc_jrand_next_gaussian(orc_jrand *r) {
    if (r->have_next_gaussian) {
        r->have_next_gaussian = 0;
        return r->next_gaussian;
    }
    double v1, v2, s;
    do {
        v1 = 2 * orc_jrand_next_double(r) - 1;
        v2 = 2 * orc_jrand_next_double(r) - 1;
        s = v1 * v1 + v2 * v2;
    } while (s >= 1 || s == 0);
    double multiplier = sqrt(-2 * log(s) / s);
    r->next_gaussian = v2 * multiplier;
    r->have_next_gaussian = 1;
    return v1 * multiplier;
}

/* fillRandomData: array[i] = min + nextFloat() * (max - min)
 * (MatrixVectorRowMajor.java:66-71). */
ORC_API void orc_fill_uniform_f32(orc_jrand *r, float *out, int64_t n, float lo, float hi) {
    float range = hi - lo;
    for (int64_t i = 0; i < n; i++) out[i] = lo + orc_jrand_next_float(r) * range;
}

/* Two arrays filled element by element in lock-step, a[i] then b[i]
 * (MatrixMultiplication2D.java:91-97 fills A and B inside one loop). */
ORC_API void orc_fill_uniform_f32_interleaved(orc_jrand *r, float *a, float *b, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        a[i] = orc_jrand_next_float(r);
        b[i] = orc_jrand_next_float(r);
    }
}

/* out[i] = nextInt(bound) */
ORC_API void orc_fill_int_bound(orc_jrand *r, int32_t *out, int64_t n, int32_t bound) {
    for (int64_t i = 0; i < n; i++) out[i] = orc_jrand_next_int_bound(r, bound);
}

ORC_API void orc_fill_gaussian_f32(orc_jrand *r, float *out, int64_t n, float mul) {
    for (int64_t i = 0; i < n; i++) out[i] = (float)(orc_jrand_next_gaussian(r) * (double)mul);
}

/* ------------------------------------------------------------------------- */
/* IEEE binary16 <-> binary32, round to nearest even                          */
/* (HalfFloat.java:41-43 -> Float.floatToFloat16; :189-191 -> float16ToFloat) */
/* ------------------------------------------------------------------------- */
ORC_API uint16_t orc_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) { /* inf / nan */
        if (absx == 0x7F800000u) return (uint16_t)(sign | 0x7C00u);
        return (uint16_t)(sign | 0x7E00u | ((absx >> 13) & 0x03FFu)); /* quiet NaN */
    }
    if (absx >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to inf: >= 65520 */
    if (absx < 0x33000001u) return (uint16_t)sign;              /* <= 2^-25 rounds to zero */
    int32_t exp = (int32_t)(absx >> 23) - 127;
    uint32_t man = absx & 0x007FFFFFu;
    uint32_t half;
    if (exp < -14) { /* subnormal half */
        man |= 0x00800000u;
        int shift = -exp - 14 + 13; /* 14 .. 24 */
        uint32_t q = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (q & 1))) q++;
        half = q;
    } else {
        uint32_t q = ((uint32_t)(exp + 15) << 10) | (man >> 13);
        uint32_t rem = man & 0x1FFFu;
        if (rem > 0x1000u || (rem == 0x1000u && (q & 1))) q++;
        half = q;
    }
    return (uint16_t)(sign | half);
}

ORC_API float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1F;
    uint32_t man = h & 0x3FF;
    uint32_t x;
    if (exp == 0) {
        if (man == 0) {
            x = sign;
        } else {
            int e = -1;
            do {
                e++;
                man <<= 1;
            } while ((man & 0x400) == 0);
            man &= 0x3FF;
            x = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        x = sign | 0x7F800000u | (man << 13);
    } else {
        x = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

ORC_API void orc_f32_to_f16_n(const float *in, uint16_t *out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = orc_f32_to_f16(in[i]);
}
ORC_API void orc_f16_to_f32_n(const uint16_t *in, float *out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = orc_f16_to_f32(in[i]);
}

/* N(0,1) * mul rounded to fp16, the FP16 GEMM operand distribution. */
ORC_API void orc_fill_gaussian_f16(orc_jrand *r, uint16_t *out, int64_t n, float mul) {
    for (int64_t i = 0; i < n; i++) out[i] = orc_f32_to_f16((float)(orc_jrand_next_gaussian(r) * (double)mul));
}

/* ------------------------------------------------------------------------- */
/* FP32 matrix-vector                                                         */
/* ------------------------------------------------------------------------- */

/* matrixVectorSequential (MatrixVectorRowMajor.java:83-92) == README mxv
 * (README.md:35-47): one fp32 accumulator per row, ascending j. */
ORC_API void orc_sgemv_seq(const float *w, const float *x, float *out, int n, int d) {
    for (int i = 0; i < d; i++) {
        float sum = 0.0f;
        const float *row = w + (int64_t)i * n;
        for (int j = 0; j < n; j++) sum += row[j] * x[j];
        out[i] = sum;
    }
}

/* The same loop split over host threads by rows: the decomposition of
 * TornadoVM's multi-core CPU device (one chunk of the outer @Parallel loop per
 * compute unit, tornado-drivers/opencl/.../scheduler/OCLCPUScheduler.java:41). */
ORC_API void orc_sgemv_seq_mt(const float *w, const float *x, float *out, int n, int d) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < d; i++) {
        float sum = 0.0f;
        const float *row = w + (int64_t)i * n;
        for (int j = 0; j < n; j++) sum += row[j] * x[j];
        out[i] = sum;
    }
}

/* matrixVectorRowMajorOptimized (MatrixVectorRowMajor.java:129-158): work-group
 * per row, lane l sums j = l, l+L, ...; tree reduction stride L/2 .. 1. */
ORC_API void orc_sgemv_workgroup(const float *w, const float *x, float *out, int n, int d, int L) {
    float *part = (float *)malloc(sizeof(float) * (size_t)L);
    for (int i = 0; i < d; i++) {
        const float *row = w + (int64_t)i * n;
        for (int l = 0; l < L; l++) {
            float p = 0.0f;
            for (int j = l; j < n; j += L) p += row[j] * x[j];
            part[l] = p;
        }
        for (int s = L / 2; s > 0; s >>= 1)
            for (int l = 0; l < s; l++) part[l] += part[l + s];
        out[i] = part[0];
    }
    free(part);
}

ORC_API void orc_sgemv_f64(const float *w, const float *x, double *out, int n, int d) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < d; i++) {
        double sum = 0.0;
        const float *row = w + (int64_t)i * n;
        for (int j = 0; j < n; j++) sum += (double)row[j] * (double)x[j];
        out[i] = sum;
    }
}

/* ------------------------------------------------------------------------- */
/* Q8_0                                                                       */
/* ------------------------------------------------------------------------- */

static inline int32_t java_round_f32(float a) {
    /* Math.round(float): nearest int, ties toward +inf; exact in double */
    double r = floor((double)a + 0.5);
    if (r > 2147483647.0) return 2147483647;
    if (r < -2147483648.0) return (int32_t)(-2147483647 - 1);
    return (int32_t)r;
}

/* quantizeWeightsToQ8 (MatrixVectorRowMajor.java:363-407).  Fills the split
 * layout (q: rows*cols int8, scales: rows*cols/32 fp16) and the unified layout
 * (34-byte blocks: fp16 scale little-endian, then 32 int8).  Any output may be
 * NULL. */
ORC_API void orc_q8_quantize(const float *w, int8_t *q, uint16_t *scales, uint8_t *blocks, int rows, int cols) {
    int bpr = cols / 32;
    for (int r = 0; r < rows; r++) {
        for (int b = 0; b < bpr; b++) {
            const float *src = w + (int64_t)r * cols + b * 32;
            float max_abs = 0.0f;
            for (int i = 0; i < 32; i++) {
                float a = fabsf(src[i]);
                if (a > max_abs) max_abs = a;
            }
            float scale = (max_abs == 0.0f) ? 0.0f : (max_abs / 127.0f);
            uint16_t hs = orc_f32_to_f16(scale);
            int64_t gb = (int64_t)r * bpr + b;
            if (scales) scales[gb] = hs;
            if (blocks) {
                blocks[gb * 34] = (uint8_t)(hs & 0xFF);
                blocks[gb * 34 + 1] = (uint8_t)(hs >> 8);
            }
            float inv = (scale == 0.0f) ? 0.0f : 1.0f / scale;
            for (int i = 0; i < 32; i++) {
                int32_t v = java_round_f32(src[i] * inv);
                if (v > 127) v = 127;
                else if (v < -127) v = -127;
                if (q) q[(int64_t)r * cols + b * 32 + i] = (int8_t)v;
                if (blocks) blocks[gb * 34 + 2 + i] = (uint8_t)(int8_t)v;
            }
        }
    }
}

/* Re-pack split Q8_0 into 34-byte blocks (pure byte movement). */
ORC_API void orc_q8_pack_blocks(const int8_t *q, const uint16_t *scales, uint8_t *blocks, int64_t nblocks) {
    for (int64_t b = 0; b < nblocks; b++) {
        blocks[b * 34] = (uint8_t)(scales[b] & 0xFF);
        blocks[b * 34 + 1] = (uint8_t)(scales[b] >> 8);
        memcpy(blocks + b * 34 + 2, q + b * 32, 32);
    }
}

/* matrixVectorRowMajorOptimizedQ8_0Final (MatrixVectorRowMajor.java:530-578):
 * lanes l = 0..L-1, four interleaved accumulators over j = 4l, 4l+4L, ...,
 * per-element dequantise ((float)q * scale) * x, sum (p1+p2+p3+p4), tail loop,
 * tree reduction.  The unified ByteArray kernel (:447-524) does the same
 * arithmetic on the same values, so one restatement serves both layouts. */
ORC_API void orc_q8_gemv_ref(const int8_t *q, const uint16_t *scales, const float *x, float *out, int n, int d, int L) {
    float *part = (float *)malloc(sizeof(float) * (size_t)L);
    int bpr = n / 32;
    for (int r = 0; r < d; r++) {
        const int8_t *qr = q + (int64_t)r * n;
        const uint16_t *sr = scales + (int64_t)r * bpr;
        for (int l = 0; l < L; l++) {
            float p1 = 0.0f, p2 = 0.0f, p3 = 0.0f, p4 = 0.0f;
            for (int j = l * 4; j < n - 3; j += L * 4) {
                float s = orc_f16_to_f32(sr[j / 32]);
                p1 += ((float)qr[j] * s) * x[j];
                p2 += ((float)qr[j + 1] * s) * x[j + 1];
                p3 += ((float)qr[j + 2] * s) * x[j + 2];
                p4 += ((float)qr[j + 3] * s) * x[j + 3];
            }
            float p = p1 + p2 + p3 + p4;
            for (int j = (n / 4) * 4 + l; j < n; j += L) {
                float s = orc_f16_to_f32(sr[j / 32]);
                p += ((float)qr[j] * s) * x[j];
            }
            part[l] = p;
        }
        for (int s = L / 2; s > 0; s >>= 1)
            for (int l = 0; l < s; l++) part[l] += part[l + s];
        out[r] = part[0];
    }
    free(part);
}

/* Plain sequential form of the same product, one accumulator, ascending j:
 * what "sequential Java" computes for Q8_0, and the CPU baseline that is timed. */
ORC_API void orc_q8_gemv_seq(const int8_t *q, const uint16_t *scales, const float *x, float *out, int n, int d) {
    int bpr = n / 32;
    for (int r = 0; r < d; r++) {
        const int8_t *qr = q + (int64_t)r * n;
        const uint16_t *sr = scales + (int64_t)r * bpr;
        float sum = 0.0f;
        for (int b = 0; b < bpr; b++) {
            float s = orc_f16_to_f32(sr[b]);
            for (int i = 0; i < 32; i++) sum += ((float)qr[b * 32 + i] * s) * x[b * 32 + i];
        }
        out[r] = sum;
    }
}

ORC_API void orc_q8_gemv_seq_mt(const int8_t *q, const uint16_t *scales, const float *x, float *out, int n, int d) {
    int bpr = n / 32;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < d; r++) {
        const int8_t *qr = q + (int64_t)r * n;
        const uint16_t *sr = scales + (int64_t)r * bpr;
        float sum = 0.0f;
        for (int b = 0; b < bpr; b++) {
            float s = orc_f16_to_f32(sr[b]);
            for (int i = 0; i < 32; i++) sum += ((float)qr[b * 32 + i] * s) * x[b * 32 + i];
        }
        out[r] = sum;
    }
}

ORC_API void orc_q8_gemv_f64(const int8_t *q, const uint16_t *scales, const float *x, double *out, int n, int d) {
    int bpr = n / 32;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < d; r++) {
        const int8_t *qr = q + (int64_t)r * n;
        const uint16_t *sr = scales + (int64_t)r * bpr;
        double sum = 0.0;
        for (int b = 0; b < bpr; b++) {
            double s = (double)orc_f16_to_f32(sr[b]);
            for (int i = 0; i < 32; i++) sum += ((double)qr[b * 32 + i] * s) * (double)x[b * 32 + i];
        }
        out[r] = sum;
    }
}

/* ------------------------------------------------------------------------- */
/* DP4A and integer block dots                                                */
/* ------------------------------------------------------------------------- */

/* QuantizationUtils.dp4a (QuantizationUtils.java:29-39). */
ORC_API int32_t orc_dp4a(const int8_t *a, const int8_t *b, int32_t c) {
    int32_t dot = 0;
    for (int i = 0; i < 4; i++) dot += (int32_t)a[i] * (int32_t)b[i];
    return c + dot;
}

/* QuantizationUtils.dp4a_packed (QuantizationUtils.java:57-66). */
ORC_API int32_t orc_dp4a_packed(int32_t a, int32_t b, int32_t c) {
    int32_t sum = c;
    for (int i = 0; i < 4; i++) {
        int8_t ab = (int8_t)((a >> (i * 8)) & 0xFF);
        int8_t bb = (int8_t)((b >> (i * 8)) & 0xFF);
        sum += (int32_t)ab * (int32_t)bb;
    }
    return sum;
}

/* performDP4A of the unit test: result[i] = dp4a(a, 4i, b, 4i, 0)
 * (QuantizationTests.java testDP4A, :517-549). */
ORC_API void orc_dp4a_n(const int8_t *a, const int8_t *b, int32_t *out, int64_t n4) {
    for (int64_t i = 0; i < n4; i++) out[i] = orc_dp4a(a + 4 * i, b + 4 * i, 0);
}

/* Per-tensor activation quantiser: reductionCalculateMax + quantizeKernelContext
 * (MatrixVectorRowMajor.java:308-354): scale = max|x|/127 (1 if 0),
 * q = (byte) floor(x * (1/scale) + 0.5). */
ORC_API void orc_quantize_x_tensor(const float *x, int8_t *xq, float *scale_out, int n) {
    float m = 0.0f;
    for (int i = 0; i < n; i++) m = fmaxf(m, fabsf(x[i]));
    float scale = (m == 0.0f) ? 1.0f : m / 127.0f;
    float inv = 1.0f / scale;
    for (int i = 0; i < n; i++) xq[i] = (int8_t)(int32_t)floorf(x[i] * inv + 0.5f);
    *scale_out = scale;
}

/* The same rule applied per 32-element block (parity unpinned: the reference
 * only has the per-tensor form). xs[b] is the fp32 scale of block b. */
ORC_API void orc_quantize_x_block(const float *x, int8_t *xq, float *xs, int n) {
    for (int b = 0; b < n / 32; b++) {
        float m = 0.0f;
        for (int i = 0; i < 32; i++) m = fmaxf(m, fabsf(x[b * 32 + i]));
        float scale = (m == 0.0f) ? 1.0f : m / 127.0f;
        float inv = 1.0f / scale;
        for (int i = 0; i < 32; i++) xq[b * 32 + i] = (int8_t)(int32_t)floorf(x[b * 32 + i] * inv + 0.5f);
        xs[b] = scale;
    }
}

/* int32 dot of every 32-element weight block with the matching activation
 * block: eight chained dp4a calls. dots is rows * cols/32. */
ORC_API void orc_q8_blockdots_i32(const int8_t *q, const int8_t *xq, int32_t *dots, int n, int d) {
    int bpr = n / 32;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < d; r++)
        for (int b = 0; b < bpr; b++) {
            int32_t acc = 0;
            for (int i = 0; i < 32; i += 4) acc = orc_dp4a(q + (int64_t)r * n + b * 32 + i, xq + b * 32 + i, acc);
            dots[(int64_t)r * bpr + b] = acc;
        }
}

/* y[r] = sum_b (float)dot[r,b] * wscale[r,b] * xscale[b], each term evaluated
 * as dequantizeFusedResult does (QuantizationUtils.java:53-55:
 * (float) dot * wScale * xScale), summed in double. */
ORC_API void orc_blockdots_combine_f64(const int32_t *dots, const uint16_t *wscales, const float *xs, double *out, int bpr, int d) {
    for (int r = 0; r < d; r++) {
        double sum = 0.0;
        for (int b = 0; b < bpr; b++) {
            double ws = (double)orc_f16_to_f32(wscales[(int64_t)r * bpr + b]);
            sum += (double)dots[(int64_t)r * bpr + b] * ws * (double)xs[b];
        }
        out[r] = sum;
    }
}

/* ------------------------------------------------------------------------- */
/* Q4_0 (not in the reference; block format fixed by this project: 18-byte    */
/* blocks, fp16 scale little-endian then 16 bytes, byte i holding element i   */
/* in its low nibble and element i+16 in its high nibble; value = nibble - 8) */
/* ------------------------------------------------------------------------- */
static inline int q4_val(const uint8_t *blk, int i) {
    uint8_t byte = blk[2 + (i & 15)];
    return (int)((i < 16) ? (byte & 0x0F) : (byte >> 4)) - 8;
}

ORC_API void orc_q4_pack_blocks(const uint8_t *nibbles, const uint16_t *scales, uint8_t *blocks, int64_t nblocks) {
    /* nibbles: one value 0..15 per element, nblocks*32 of them */
    for (int64_t b = 0; b < nblocks; b++) {
        uint8_t *blk = blocks + b * 18;
        blk[0] = (uint8_t)(scales[b] & 0xFF);
        blk[1] = (uint8_t)(scales[b] >> 8);
        for (int i = 0; i < 16; i++) blk[2 + i] = (uint8_t)((nibbles[b * 32 + i] & 0x0F) | (nibbles[b * 32 + i + 16] << 4));
    }
}

ORC_API void orc_q4_gemv_seq(const uint8_t *blocks, const float *x, float *out, int n, int d) {
    int bpr = n / 32;
    for (int r = 0; r < d; r++) {
        float sum = 0.0f;
        for (int b = 0; b < bpr; b++) {
            const uint8_t *blk = blocks + ((int64_t)r * bpr + b) * 18;
            float s = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
            for (int i = 0; i < 32; i++) sum += ((float)q4_val(blk, i) * s) * x[b * 32 + i];
        }
        out[r] = sum;
    }
}

ORC_API void orc_q4_gemv_seq_mt(const uint8_t *blocks, const float *x, float *out, int n, int d) {
    int bpr = n / 32;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < d; r++) {
        float sum = 0.0f;
        for (int b = 0; b < bpr; b++) {
            const uint8_t *blk = blocks + ((int64_t)r * bpr + b) * 18;
            float s = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
            for (int i = 0; i < 32; i++) sum += ((float)q4_val(blk, i) * s) * x[b * 32 + i];
        }
        out[r] = sum;
    }
}

ORC_API void orc_q4_gemv_f64(const uint8_t *blocks, const float *x, double *out, int n, int d) {
    int bpr = n / 32;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < d; r++) {
        double sum = 0.0;
        for (int b = 0; b < bpr; b++) {
            const uint8_t *blk = blocks + ((int64_t)r * bpr + b) * 18;
            double s = (double)orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
            for (int i = 0; i < 32; i++) sum += ((double)q4_val(blk, i) * s) * (double)x[b * 32 + i];
        }
        out[r] = sum;
    }
}

ORC_API void orc_q4_blockdots_i32(const uint8_t *blocks, const int8_t *xq, int32_t *dots, int n, int d) {
    int bpr = n / 32;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < d; r++)
        for (int b = 0; b < bpr; b++) {
            const uint8_t *blk = blocks + ((int64_t)r * bpr + b) * 18;
            int32_t acc = 0;
            for (int i = 0; i < 32; i++) acc += q4_val(blk, i) * (int32_t)xq[b * 32 + i];
            dots[(int64_t)r * bpr + b] = acc;
        }
}

/* fp16 scales of a unified-block matrix gathered into a dense array. */
ORC_API void orc_block_scales(const uint8_t *blocks, uint16_t *scales, int64_t nblocks, int block_bytes) {
    for (int64_t b = 0; b < nblocks; b++) scales[b] = (uint16_t)(blocks[b * block_bytes] | (blocks[b * block_bytes + 1] << 8));
}

/* ------------------------------------------------------------------------- */
/* FP32 SGEMM: matrixMultiplication (MatrixMultiplication2D.java:48-58)       */
/* ------------------------------------------------------------------------- */
ORC_API void orc_sgemm_seq(const float *a, const float *b, float *c, int m, int n, int k, int row0, int row1) {
    for (int i = row0; i < row1; i++)
        for (int j = 0; j < n; j++) {
            float sum = 0.0f;
            for (int kk = 0; kk < k; kk++) sum += a[(int64_t)i * k + kk] * b[(int64_t)kk * n + j];
            c[(int64_t)i * n + j] = sum;
        }
}

/* parallelStreamsMxM (MatrixMultiplication2D.java:60-70): rows over threads. */
ORC_API void orc_sgemm_seq_mt(const float *a, const float *b, float *c, int m, int n, int k, int row0, int row1) {
#pragma omp parallel for schedule(static)
    for (int i = row0; i < row1; i++)
        for (int j = 0; j < n; j++) {
            float sum = 0.0f;
            for (int kk = 0; kk < k; kk++) sum += a[(int64_t)i * k + kk] * b[(int64_t)kk * n + j];
            c[(int64_t)i * n + j] = sum;
        }
}

/* Double-accumulated twin; loops reordered (i,k,j) for speed, which does not
 * change a double sum beyond ~1e-16 relative. c is (row1-row0) x n. */
ORC_API void orc_sgemm_f64(const float *a, const float *b, double *c, int m, int n, int k, int row0, int row1) {
#pragma omp parallel for schedule(static)
    for (int i = row0; i < row1; i++) {
        double *crow = c + (int64_t)(i - row0) * n;
        for (int j = 0; j < n; j++) crow[j] = 0.0;
        for (int kk = 0; kk < k; kk++) {
            double av = (double)a[(int64_t)i * k + kk];
            const float *brow = b + (int64_t)kk * n;
            for (int j = 0; j < n; j++) crow[j] += av * (double)brow[j];
        }
    }
}

/* ------------------------------------------------------------------------- */
/* FP16 GEMM: gemmReference (MatrixMultiplicationMMA.java:616-627,            */
/* TestMatrixMultiplicationMMA.java:266-279): fp16 -> fp32, fp32 accumulate,  */
/* ascending k.  c is (row1-row0) x n.                                        */
/* ------------------------------------------------------------------------- */
ORC_API void orc_hgemm_ref(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int row0, int row1) {
    float *bf = (float *)malloc(sizeof(float) * (size_t)k * (size_t)n);
    orc_f16_to_f32_n(b, bf, (int64_t)k * n);
#pragma omp parallel for schedule(static)
    for (int i = row0; i < row1; i++) {
        float *crow = c + (int64_t)(i - row0) * n;
        for (int j = 0; j < n; j++) crow[j] = 0.0f;
        /* (i,k,j) order performs, for each (i,j), the same fp32 additions in the
         * same ascending-k order as the reference's (i,j,k) loop. */
        for (int kk = 0; kk < k; kk++) {
            float av = orc_f16_to_f32(a[(int64_t)i * k + kk]);
            const float *brow = bf + (int64_t)kk * n;
            for (int j = 0; j < n; j++) crow[j] += av * brow[j];
        }
    }
    free(bf);
}

ORC_API void orc_hgemm_f64(const uint16_t *a, const uint16_t *b, double *c, int m, int n, int k, int row0, int row1) {
    float *bf = (float *)malloc(sizeof(float) * (size_t)k * (size_t)n);
    orc_f16_to_f32_n(b, bf, (int64_t)k * n);
#pragma omp parallel for schedule(static)
    for (int i = row0; i < row1; i++) {
        double *crow = c + (int64_t)(i - row0) * n;
        for (int j = 0; j < n; j++) crow[j] = 0.0;
        for (int kk = 0; kk < k; kk++) {
            double av = (double)orc_f16_to_f32(a[(int64_t)i * k + kk]);
            const float *brow = bf + (int64_t)kk * n;
            for (int j = 0; j < n; j++) crow[j] += av * (double)brow[j];
        }
    }
    free(bf);
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
