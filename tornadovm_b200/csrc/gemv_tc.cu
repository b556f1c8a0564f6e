// Batched Q8_0 / Q4_0 mat-vec on the tensor cores with the activations in registers.
//
// Serves the integer mode from two activation vectors on (exact int32 block dots by
// mma.sync.m16n8k32.s8) and the float mode (fp32 activations as fp16 hi + lo pairs,
// mma.sync.m16n8k16.f16 with fp32 accumulation).  The kernels are HBM-bound: the tensor
// cores only take the multiply-adds off the issue slots, so the legacy mma.sync path is
// the right tool; tcgen05 needs its operands in canonical 16-byte aligned shared-memory
// tiles, which 34- and 18-byte blocks are not.
//
// Work layout.  A CTA owns a contiguous range of rows, walked in units of 16 rows.  K is cut
// into chunks of 8 blocks (256 columns); consumer warp w owns chunk w of every unit
// (chunk w + KS * p in phase p when there are more chunks than warps) and keeps the
// activations of its chunk -- MMA B fragments and, in integer mode, the per-block scales --
// in REGISTERS for the whole launch.  Nothing but weights ever passes through shared memory, so
// up to 16 vectors cost no shared memory and no shared-memory bandwidth.  The weights of a unit
// (16 rows: one contiguous piece of global memory) arrive in a CTA-wide ring by bulk async copies
// issued by one thread of a copy warp, so global memory is read in long sequential runs.  The KS
// partial tiles of a unit are summed in a fixed order by a seventeenth warp (mbarrier hand-off,
// bounded waits), which also writes y; results therefore do not depend on warp timing.
//
// Algorithmic bytes per launch: block bytes * rows * cols / 32 + 4 * batch * (cols + rows).
#include <cstdlib>
#include <type_traits>

#include "gemv_common.cuh"

#ifndef TB200_OP_CLASS
#define TB200_OP_CLASS TB200_PREPARE_GEMV_QUANT
#endif

TB200_TU_STATUS(gemv_tc)

namespace tb200 {

constexpr int TC_KS_MAX = 16;                       // consumer warps = K chunks in flight per unit
constexpr int TC_THREADS = (TC_KS_MAX + 2) * 32;    // + the reducing warp + the copy-issuing warp
constexpr int TC_MAX_STAGES = 8;
constexpr int TC_KB = 8;                            // blocks per K chunk
constexpr int TC_NB = 2;                            // partial-tile buffers between consumers and reducer

constexpr int X_INT_WS = 0;     // int8 activations and their scales read from global memory (already quantised)
constexpr int X_INT_FUSED = 1;  // fp32 activations quantised per 32-block while they are loaded
constexpr int X_FLOAT = 2;      // fp32 activations split into fp16 hi + lo

template <int FMT>
struct TcTraits {
    static constexpr int BB = FMT == FMT_Q4B ? 18 : (FMT == FMT_Q8B ? 34 : 32);
    static constexpr int WROW = TC_KB * BB;                           // weight bytes per row and chunk (272 / 144 / 256)
};

template <int FMT, int NT>
struct TcConfig {
    static constexpr size_t PARTIAL = (size_t)TC_NB * TC_KS_MAX * NT * 512;
};

struct TcArgs {
    QGemvArgs g;
    int ks;        // consumer warps in use (K chunks per phase)
    int phases;    // ceil(chunks / ks)
    int max_units; // most 16-row units any CTA walks (sizes the running sums when phases > 1)
    int stages;    // stages of the CTA-wide ring
    int wshift;    // 0, or 8 when the weights sit 8 bytes past a 16-byte boundary (an array behind a 24-byte header)
    int sshift;    // the same for the scale array of the split layout
    TcGroup grp;   // count > 0: the rows of several matrices laid end to end (block formats)
};

// matrix of row r of a grouped launch (r < row_start[count])
__device__ __forceinline__ int tc_matrix_of(const TcGroup &grp, int r) {
    int m = 0;
    while (r >= grp.row_start[m + 1]) ++m;
    return m;
}

__device__ __forceinline__ float4 ldg_f4(const float *p, bool vec) {
    if (vec) return __ldg(reinterpret_cast<const float4 *>(p));
    return make_float4(__ldg(p), __ldg(p + 1), __ldg(p + 2), __ldg(p + 3));
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// Activation fragments of one K chunk (blocks blk0 .. blk0 + 7) for this lane.
//   integer modes: bf[kb][j][0..1] = the B fragment of mma.m16n8k32 (column g of tile j = vector 8j + g, bytes
//                  4t..4t+3 and 16+4t..19+4t of the block); xsr[kb][j][0..1] = scales of vectors 8j + 2t, 8j + 2t + 1
//   float mode:    bf[kb][j][0..3] = B fragments of the block's two mma.m16n8k16 (column g of tile j = the hi part
//                  (g even) or lo part (g odd) of vector 4j + g / 2); every x is first multiplied by vscale[vector]
// The fp32 activations of half a chunk (four blocks of one tile) are requested together -- eight 128-bit loads
// in flight per lane -- and only then converted: the prologue of the kernel costs two round trips to L2 per tile,
// not one per block.  Float mode: every half chunk of a vector gets its own power-of-two prescale 2^-e (e from
// the largest magnitude of those 128 values), so that the fp16 hi + lo pairs stay inside the normal range for
// any fp32 input; the warp multiplies the half chunk's sums by 2^e before they join its accumulators.
constexpr int TC_HB = TC_KB / 2;  // blocks per half chunk

// vector whose fp32 activations this lane loads for tile j
template <int XSRC>
__device__ __forceinline__ int x_vector_of_lane(int j, int g) { return XSRC == X_FLOAT ? j * 4 + (g >> 1) : j * 8 + g; }

template <int XSRC>
__device__ __forceinline__ void load_x_raw(const QGemvArgs &a, int blk0, int lane, int j, float4 (&v)[TC_HB][2]) {
    const int g = lane >> 2, t = lane & 3;
    const int n = x_vector_of_lane<XSRC>(j, g);
    const bool vec = (((uintptr_t)a.x | ((uintptr_t)a.cols << 2)) & 15) == 0;
    const float *p = a.x + (size_t)n * a.cols + (size_t)blk0 * 32 + 4 * t;
#pragma unroll
    for (int kb = 0; kb < TC_HB; ++kb) {
        v[kb][0] = v[kb][1] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n < a.batch) v[kb][0] = ldg_f4(p + kb * 32, vec), v[kb][1] = ldg_f4(p + kb * 32 + 16, vec);
    }
}

__device__ __forceinline__ float absmax8(const float4 &a, const float4 &b) {
    return fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                 fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
}

// half = 0 / 1: blocks 0..3 / 4..7 of the chunk.  Float mode returns 2^e of vector 4j + t for this half.
template <int FMT, int NT, int XSRC>
__device__ __forceinline__ float convert_x(const QGemvArgs &a, int lane, int j, int half, const float4 (&v)[TC_HB][2],
                                           uint32_t (&bf)[TC_KB][NT][XSRC == X_FLOAT ? 4 : 2], float (&xsr)[TC_KB][NT][2]) {
    const int g = lane >> 2, t = lane & 3;
    const int n = x_vector_of_lane<XSRC>(j, g);
    const float wfix = FMT == FMT_Q4B ? 0.0625f : 1.0f;  // Q4_0 nibbles enter the MMA as 16 * (nibble - 8)
    float prescale = 1.f, unscale = 1.f;
    if constexpr (XSRC == X_FLOAT) {
        float m = 0.f;
#pragma unroll
        for (int kb = 0; kb < TC_HB; ++kb) m = fmaxf(m, absmax8(v[kb][0], v[kb][1]));
        // the eight lanes of a vector (its hi and lo columns, four lanes each) hold all of the half chunk
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
        int e = ((__float_as_int(m) >> 23) & 0xFF) - 127;  // max |x| = 1.f * 2^e
        if (m == 0.f || e > 127) e = 0;                    // all zero, or inf / NaN: leave the values alone
        e = e < -126 ? -126 : (e > 126 ? 126 : e);
        prescale = __int_as_float((127 - e) << 23);        // every |x| * 2^-e < 4
        unscale = __shfl_sync(0xffffffffu, __int_as_float((127 + e) << 23), 8 * t);  // from a lane of vector 4j + t
    }
#pragma unroll
    for (int kh = 0; kh < TC_HB; ++kh) {
        const int kb = half * TC_HB + kh;
        if constexpr (XSRC == X_INT_FUSED) {
            float m = absmax8(v[kh][0], v[kh][1]);
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
            // the rule of the separate quantiser kernel, operation for operation
            const float scale = (m == 0.0f) ? 1.0f : __fdiv_rn(m, 127.0f);
            const float inv = __fdiv_rn(1.0f, scale);
            const float4 v0 = v[kh][0], v1 = v[kh][1];
            bf[kb][j][0] = quantize_byte(v0.x, inv) | (quantize_byte(v0.y, inv) << 8) | (quantize_byte(v0.z, inv) << 16) | (quantize_byte(v0.w, inv) << 24);
            bf[kb][j][1] = quantize_byte(v1.x, inv) | (quantize_byte(v1.y, inv) << 8) | (quantize_byte(v1.z, inv) << 16) | (quantize_byte(v1.w, inv) << 24);
            const float sc = n < a.batch ? wfix * scale : 0.f;
            xsr[kb][j][0] = __shfl_sync(0xffffffffu, sc, 8 * t);      // lane of column 2t
            xsr[kb][j][1] = __shfl_sync(0xffffffffu, sc, 8 * t + 4);  // lane of column 2t + 1
        } else {
            const float4 r0 = v[kh][0], r1 = v[kh][1];
            const float w[8] = {r0.x * prescale, r0.y * prescale, r0.z * prescale, r0.w * prescale,
                                r1.x * prescale, r1.y * prescale, r1.z * prescale, r1.w * prescale};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // packed conversions only (the single-value ones run on the slow conversion unit)
                const __half2 hi = __floats2half2_rn(w[2 * i], w[2 * i + 1]);
                if (g & 1) {
                    const float2 back = __half22float2(hi);
                    bf[kb][j][i] = pack_h2(w[2 * i] - back.x, w[2 * i + 1] - back.y);  // the lo part
                } else {
                    bf[kb][j][i] = *reinterpret_cast<const uint32_t *>(&hi);
                }
            }
            xsr[kb][j][0] = xsr[kb][j][1] = 0.f;
        }
    }
    return unscale;
}

// already quantised activations: the fragments are loaded straight into their registers (all loads in flight at once)
template <int FMT, int NT>
__device__ __forceinline__ void load_x_quantised(const QGemvArgs &a, int blk0, int lane, uint32_t (&bf)[TC_KB][NT][2], float (&xsr)[TC_KB][NT][2]) {
    const int g = lane >> 2, t = lane & 3;
    const int bpr = a.cols / 32;
    const float wfix = FMT == FMT_Q4B ? 0.0625f : 1.0f;
    const bool word_ok = (((uintptr_t)a.xq | (uintptr_t)a.cols) & 3) == 0;
    // a.xlayout = 1: xq[block][vector][32], xs[block][vector] (the library's own quantiser in front of this kernel):
    // the eight vectors of a tile are 256 contiguous bytes, two cache lines per load instead of eight
    const bool inter = a.xlayout != 0;
#pragma unroll
    for (int kb = 0; kb < TC_KB; ++kb) {
        const int blk = blk0 + kb;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int col = j * 8 + g;
            bf[kb][j][0] = bf[kb][j][1] = 0;
            if (col < a.batch) {
                const int8_t *p = inter ? a.xq + ((size_t)blk * a.batch + col) * 32 + 4 * t : a.xq + (size_t)col * a.cols + (size_t)blk * 32 + 4 * t;
                if (word_ok) {
                    bf[kb][j][0] = __ldg(reinterpret_cast<const uint32_t *>(p));
                    bf[kb][j][1] = __ldg(reinterpret_cast<const uint32_t *>(p + 16));
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        bf[kb][j][0] |= (uint32_t)(uint8_t)p[i] << (8 * i);
                        bf[kb][j][1] |= (uint32_t)(uint8_t)p[16 + i] << (8 * i);
                    }
                }
            }
            const int c0 = j * 8 + 2 * t;
            xsr[kb][j][0] = (c0 < a.batch && a.xs) ? __ldg(inter ? a.xs + (size_t)blk * a.batch + c0 : a.xs + (size_t)c0 * bpr + blk) : 0.f;
            xsr[kb][j][1] = (c0 + 1 < a.batch && a.xs) ? __ldg(inter ? a.xs + (size_t)blk * a.batch + c0 + 1 : a.xs + (size_t)(c0 + 1) * bpr + blk) : 0.f;
        }
    }
#pragma unroll
    for (int kb = 0; kb < TC_KB; ++kb)
#pragma unroll
        for (int j = 0; j < NT; ++j) xsr[kb][j][0] *= wfix, xsr[kb][j][1] *= wfix;
}

// A fragments (rows g and g + 8 of the unit, block kb of the warp's chunk) and the two rows' block scales.
// rp0 / rp1 point at the chunk's weight bytes of the two rows, sp0 / sp1 (split layout) at its eight fp16 scales.
template <int FMT>
__device__ __forceinline__ void load_a_fragments(const unsigned char *rp0, const unsigned char *rp1, const unsigned char *sp0,
                                                 const unsigned char *sp1, int kb, int t, uint32_t &a0, uint32_t &a1, uint32_t &a2,
                                                 uint32_t &a3, float &sw0, float &sw1) {
    if (FMT == FMT_Q8B) {
        const int off = kb * 34 + 2 + 4 * t;
        if (kb % 2 == 0) {  // 34 * kb + 2 is 2 modulo 4
            a0 = lds_u32_at<1>(rp0, off), a1 = lds_u32_at<1>(rp1, off);
            a2 = lds_u32_at<1>(rp0, off + 16), a3 = lds_u32_at<1>(rp1, off + 16);
        } else {
            a0 = lds_u32_at<0>(rp0, off), a1 = lds_u32_at<0>(rp1, off);
            a2 = lds_u32_at<0>(rp0, off + 16), a3 = lds_u32_at<0>(rp1, off + 16);
        }
        sw0 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(rp0 + kb * 34));
        sw1 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(rp1 + kb * 34));
    } else if (FMT == FMT_Q4B) {
        const int off = kb * 18 + 2 + 4 * t;
        uint32_t w0, w1;
        if (kb % 2 == 0) w0 = lds_u32_at<1>(rp0, off), w1 = lds_u32_at<1>(rp1, off);
        else w0 = lds_u32_at<0>(rp0, off), w1 = lds_u32_at<0>(rp1, off);
        // byte i holds element i (low nibble) and element i + 16 (high nibble): raw nibbles here, the
        // caller turns them into signed bytes or halves
        a0 = w0 & 0x0F0F0F0Fu, a2 = (w0 >> 4) & 0x0F0F0F0Fu;
        a1 = w1 & 0x0F0F0F0Fu, a3 = (w1 >> 4) & 0x0F0F0F0Fu;
        sw0 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(rp0 + kb * 18));
        sw1 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(rp1 + kb * 18));
    } else {
        const int off = kb * 32 + 4 * t;
        a0 = lds_u32_at<0>(rp0, off), a1 = lds_u32_at<0>(rp1, off);
        a2 = lds_u32_at<0>(rp0, off + 16), a3 = lds_u32_at<0>(rp1, off + 16);
        sw0 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(sp0 + kb * 2));
        sw1 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(sp1 + kb * 2));
    }
}

// int32 -> fp32 for |d| < 2^22 without the conversion unit: 1.5 * 2^23 + d is exact, and so is the subtraction
__device__ __forceinline__ float small_int_to_float(int d) { return __int_as_float(0x4B400000 + d) - 12582912.0f; }

// One (unit, chunk) item: eight block dots of a 16-row x 8*NT-column tile, scaled and accumulated.
template <int FMT, int NT, bool FLT, bool DOTS>
__device__ __forceinline__ void consume_chunk(const QGemvArgs &a, const unsigned char *rp0, const unsigned char *rp1,
                                              const unsigned char *sp0, const unsigned char *sp1, int t, int r0, int r1, int row_end,
                                              int blk0, const uint32_t (&bf)[TC_KB][NT][FLT ? 4 : 2], const float (&xsr)[TC_KB][NT][2],
                                              const float (&unscale)[2][NT], float (&acc)[NT][4]) {
    const int bpr = a.cols / 32;
    float half_acc[NT][2];  // float mode: sums of the running half chunk, in its prescaled units
#pragma unroll
    for (int kb = 0; kb < TC_KB; ++kb) {
        if (FLT && kb % TC_HB == 0) {
#pragma unroll
            for (int j = 0; j < NT; ++j) half_acc[j][0] = half_acc[j][1] = 0.f;
        }
        uint32_t a0, a1, a2, a3;
        float sw0, sw1;
        load_a_fragments<FMT>(rp0, rp1, sp0, sp1, kb, t, a0, a1, a2, a3, sw0, sw1);
        if constexpr (FLT) {
            uint32_t p0, p1, p2, p3, q0, q1, q2, q3;
            if (FMT == FMT_Q4B) {
                u8x4_to_h2x2(a0, 0x64086408u, p0, p2), u8x4_to_h2x2(a1, 0x64086408u, p1, p3);
                u8x4_to_h2x2(a2, 0x64086408u, q0, q2), u8x4_to_h2x2(a3, 0x64086408u, q1, q3);
            } else {
                u8x4_to_h2x2(a0 ^ 0x80808080u, 0x64806480u, p0, p2), u8x4_to_h2x2(a1 ^ 0x80808080u, 0x64806480u, p1, p3);
                u8x4_to_h2x2(a2 ^ 0x80808080u, 0x64806480u, q0, q2), u8x4_to_h2x2(a3 ^ 0x80808080u, 0x64806480u, q1, q3);
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                float d[4] = {0.f, 0.f, 0.f, 0.f};
                mma_f16_16816(d, p0, p1, p2, p3, bf[kb][j][0], bf[kb][j][1]);
                mma_f16_16816(d, q0, q1, q2, q3, bf[kb][j][2], bf[kb][j][3]);
                // columns 2t (hi part) and 2t + 1 (lo part) belong to vector 4j + t
                half_acc[j][0] = fmaf(d[0] + d[1], sw0, half_acc[j][0]);
                half_acc[j][1] = fmaf(d[2] + d[3], sw1, half_acc[j][1]);
                if (kb % TC_HB == TC_HB - 1) {
                    acc[j][0] = fmaf(half_acc[j][0], unscale[kb / TC_HB][j], acc[j][0]);
                    acc[j][2] = fmaf(half_acc[j][1], unscale[kb / TC_HB][j], acc[j][2]);
                }
            }
        } else {
            if (FMT == FMT_Q4B) {
                // nibble n -> the signed byte 16 * (n - 8): (n << 4) ^ 0x80; the 1/16 sits in xsr
                a0 = (a0 << 4) ^ 0x80808080u, a1 = (a1 << 4) ^ 0x80808080u;
                a2 = (a2 << 4) ^ 0x80808080u, a3 = (a3 << 4) ^ 0x80808080u;
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                int d[4];
                mma_s8_16832(d, a0, a1, a2, a3, bf[kb][j][0], bf[kb][j][1]);
                if constexpr (DOTS) {
                    // dots[vector][row][block]; Q4_0 fragments carry 16 * (nibble - 8)
                    const int sh = FMT == FMT_Q4B ? 4 : 0;
                    const int n0 = j * 8 + 2 * t;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int n = n0 + (i & 1), r = i < 2 ? r0 : r1;
                        if (n < a.batch && r < row_end) a.dots[((size_t)n * a.rows + r) * bpr + blk0 + kb] = d[i] >> sh;
                    }
                } else {
                    // One column tile: the conversion unit has room for four conversions per block (one issue slot
                    // each).  Two tiles would saturate it: there the conversion is an integer add and an exact
                    // float subtract on the ordinary pipes.
                    auto cvt = [](int v) { return NT == 1 ? __int2float_rn(v) : small_int_to_float(v); };
                    acc[j][0] = fmaf(cvt(d[0]), sw0 * xsr[kb][j][0], acc[j][0]);
                    acc[j][1] = fmaf(cvt(d[1]), sw0 * xsr[kb][j][1], acc[j][1]);
                    acc[j][2] = fmaf(cvt(d[2]), sw1 * xsr[kb][j][0], acc[j][2]);
                    acc[j][3] = fmaf(cvt(d[3]), sw1 * xsr[kb][j][1], acc[j][3]);
                }
            }
        }
    }
}

// Shared-memory pitch of a row that holds `ks` chunks of `wrow` bytes: padded so that the eight rows a warp
// reads together start 4 banks apart (wrow is 16 modulo 128 for the block formats, 0 for the split quants)
__host__ __device__ __forceinline__ int tc_row_pitch(int ks, int wrow) {
    const int raw = ks * wrow;
    return raw + (((raw / 4 + 4) % 32) % 8 == 4 ? 16 : 32);
}

// The weights of a unit -- 16 consecutive rows, one contiguous piece of global memory per phase -- arrive in a
// CTA-wide ring as one bulk async copy per row (TMA engine, evict-first), issued by one thread of an eighteenth
// warp; every consumer warp reads its own chunk of the 16 rows and releases the stage through an mbarrier.  Global
// memory is therefore read in long sequential runs, and no consumer spends issue slots on copies.
// Weights that sit 8 bytes past a 16-byte boundary (a TornadoVM array behind a 24-byte header) keep that phase in
// shared memory: the bulk copy moves the 16-byte aligned middle of a row, and two lanes of the copy warp add the
// row's first and last 8 bytes with 8-byte cp.async copies that arrive on the same mbarrier.
template <int FMT, int NT, int XSRC, bool DOTS>
__global__ void __launch_bounds__(TC_THREADS, 1) qtc_gemv_kernel(const __grid_constant__ TcArgs args) {
    using T = TcTraits<FMT>;
    constexpr bool FLT = XSRC == X_FLOAT;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[TC_MAX_STAGES];   // a stage has landed
    __shared__ __align__(8) uint64_t empty_bar[TC_MAX_STAGES];  // every consumer is done with a stage
    __shared__ __align__(8) uint64_t pfull_bar[TC_NB];          // partial tiles of an item are complete
    __shared__ __align__(8) uint64_t pempty_bar[TC_NB];

    const QGemvArgs &a = args.g;
    const int cols = a.cols, rows = a.rows;
    const int bpr = cols / 32, nch = bpr / TC_KB;
    const int KS = args.ks, phases = args.phases, S = args.stages;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    const int row_begin = (int)((long long)rows * blockIdx.x / gridDim.x);
    const int row_end = (int)((long long)rows * (blockIdx.x + 1) / gridDim.x);
    const int nunits = (row_end - row_begin + 15) / 16;
    const int total = nunits * phases;  // items every warp walks: (phase, unit), phase-major
    const size_t row_bytes = (size_t)bpr * T::BB;

    // stage = [16 rows x wpitch weights][split layout: 16 rows x spitch scales]; both pitches leave at least 16 bytes
    // beyond a row's data, so a row shifted by 8 bytes still fits
    const int wpitch = tc_row_pitch(KS, T::WROW), spitch = FMT == FMT_Q8S ? KS * 16 + 16 : 0;
    const int stage_bytes = 16 * (wpitch + spitch);
    const size_t ring_bytes = (size_t)S * stage_bytes;
    const bool shifted = (args.wshift | args.sshift) != 0;
    float4 *partial = reinterpret_cast<float4 *>(smem_raw + ((ring_bytes + 127) & ~(size_t)127));  // [buffer][warp][tile][lane]
    float4 *ysum = partial + (size_t)TC_NB * TC_KS_MAX * NT * 32;                                  // [unit][tile][lane], phases > 1

    if (tid == 0) {
        for (int i = 0; i < TC_MAX_STAGES; ++i) {
            mbar_init(&full_bar[i], shifted ? 33 : 1);  // the copy thread, + every lane of its warp for the row ends
            mbar_init(&empty_bar[i], KS);
        }
        for (int i = 0; i < TC_NB; ++i) {
            mbar_init(&pfull_bar[i], KS);
            mbar_init(&pempty_bar[i], 1);
        }
        mbar_fence_init();
    }
    __syncthreads();  // barriers exist before the producer's first copy can signal one

    const bool consumer = warp < KS;

    if (warp == TC_KS_MAX + 1) {
        // ================= producer =================
        // Lane r issues the copy of row r: sixteen requests leave together instead of one after the other.
        const bool has_scales = FMT == FMT_Q8S && !DOTS;
        const uint32_t wcut = args.wshift ? 16u : 0u, scut = args.sshift ? 16u : 0u;  // bytes of a row the bulk copy leaves out
        const uint64_t policy = l2_evict_first_policy();
        // (phase, unit) and (stage, use count of the stage) advance as counters: no divisions in the loop
        int p = 0, u = 0, st = 0, use = 0;
        for (int it = 0; it < total; ++it, (++u == nunits ? (u = 0, ++p) : 0), (++st == S ? (st = 0, ++use) : 0)) {
            bool ok = true;
            if (lane == 0) {
                if (use > 0) ok = mbar_wait(&empty_bar[st], (use - 1) & 1);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0) != 0;  // also orders the other lanes' copies after the wait
            if (!ok) break;
            const int row_first = row_begin + u * 16;
            const int nrows = min(16, row_end - row_first);
            const int nvalid = min(KS, nch - p * KS);
            const uint32_t wbytes = (uint32_t)nvalid * T::WROW, sbytes = has_scales ? (uint32_t)nvalid * 16 : 0;
            unsigned char *dst = smem_raw + (size_t)st * stage_bytes;
            const unsigned char *src = a.w + (size_t)row_first * row_bytes + (size_t)p * KS * T::WROW;
            const unsigned char *ssrc = has_scales ? reinterpret_cast<const unsigned char *>(a.scales + (size_t)row_first * bpr + (size_t)p * KS * TC_KB) : nullptr;
            if (lane == 0) mbar_expect_tx(&full_bar[st], (uint32_t)nrows * (wbytes - wcut + (sbytes ? sbytes - scut : 0)));
            __syncwarp();
            // lanes 0..15: the 16-byte aligned part of row `lane`, at the same phase in shared memory as in global
            // memory; lanes 16..31: the scales of row lane - 16 (split layout)
            // first byte of row `r` of the unit in this phase; grouped: the row's matrix is looked up (a unit may span two)
            auto row_src = [&](int r) -> const unsigned char * {
                if (args.grp.count == 0) return src + (size_t)r * row_bytes;
                const int vr = row_first + r, m = tc_matrix_of(args.grp, vr);
                return args.grp.w[m] + (size_t)(vr - args.grp.row_start[m]) * row_bytes + (size_t)p * KS * T::WROW;
            };
            if (lane < nrows)
                bulk_g2s_stream(dst + (size_t)lane * wpitch + wcut, row_src(lane) + (wcut >> 1), wbytes - wcut, &full_bar[st], policy);
            if (sbytes && lane >= 16 && lane - 16 < nrows)
                bulk_g2s_stream(dst + 16 * (size_t)wpitch + (size_t)(lane - 16) * spitch + scut, ssrc + (size_t)(lane - 16) * bpr * 2 + (scut >> 1), sbytes - scut,
                                &full_bar[st], policy);
            if (shifted) {
                // lane 2r copies the first 8 bytes of row r, lane 2r + 1 its last 8 bytes
                const int r = lane >> 1, last = lane & 1;
                if (r < nrows) {
                    if (args.wshift) {
                        const uint32_t off = last ? wbytes - 8 : 0u;  // relative to the row's first byte
                        cp_async_8(smem_u32(dst + (size_t)r * wpitch + 8 + off), row_src(r) + off);
                    }
                    if (args.sshift && sbytes) {
                        const uint32_t off = last ? sbytes - 8 : 0u;
                        cp_async_8(smem_u32(dst + 16 * (size_t)wpitch + (size_t)r * spitch + 8 + off), ssrc + (size_t)r * bpr * 2 + off);
                    }
                }
                // counts as this lane's arrival once its copies above have landed (at once if it made none)
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full_bar[st])) : "memory");
            }
        }
        if (shifted) asm volatile("cp.async.wait_all;" ::: "memory");
        return;
    }

    pdl_launch_dependents();
    pdl_wait();  // activations and outputs may belong to the kernel before this one

    if (warp < TC_KS_MAX) {
        if (!consumer) return;  // fewer K chunks than warps: no barrier below counts this warp
        // ================= consumer =================
        uint32_t bf[TC_KB][NT][FLT ? 4 : 2];
        float xsr[TC_KB][NT][2];
        float acc[NT][4];
        float unscale[2][NT];  // float mode: 2^e of vector 4j + t for each half chunk
        int phase_loaded = -1;
        int p = 0, u = 0, st = 0, use = 0;  // (phase, unit) of the item, its stage and the stage's use count
        for (int it = 0; it < total; ++it, (++u == nunits ? (u = 0, ++p) : 0), (++st == S ? (st = 0, ++use) : 0)) {
            const int kc = p * KS + warp;
            const bool valid = kc < nch;  // the last phase may have fewer chunks than warps
            if (p != phase_loaded) {
                // before the wait below: the activation loads overlap the weights' flight
                if (valid) {
                    if constexpr (XSRC == X_INT_WS) {
                        load_x_quantised<FMT, NT>(a, kc * TC_KB, lane, bf, xsr);
                    } else {
                        // half a chunk at a time: requesting both halves before the first conversion measured slower
                        // (the fragments under construction and 64 raw values do not fit the register budget)
                        float4 xraw[TC_HB][2];  // fp32 activations of half a chunk on their way into fragments
#pragma unroll
                        for (int j = 0; j < NT; ++j)
#pragma unroll
                            for (int half = 0; half < 2; ++half) {
                                load_x_raw<XSRC>(a, kc * TC_KB + half * TC_HB, lane, j, xraw);
                                unscale[half][j] = convert_x<FMT, NT, XSRC>(a, lane, j, half, xraw, bf, xsr);
                            }
                    }
                }
                phase_loaded = p;
            }
            if (!mbar_wait(&full_bar[st], use & 1)) break;
            const unsigned char *base = smem_raw + (size_t)st * stage_bytes;
            const unsigned char *rp0 = base + g * wpitch + warp * T::WROW + args.wshift;
            const unsigned char *sp0 = base + 16 * wpitch + g * spitch + warp * 16 + args.sshift;
            const int wp = wpitch, sp = spitch;
#pragma unroll
            for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
            const int r0 = row_begin + u * 16 + g;
            if (valid)
                consume_chunk<FMT, NT, FLT, DOTS>(a, rp0, rp0 + 8 * wp, sp0, sp0 + 8 * sp, t, r0, r0 + 8, row_end, kc * TC_KB, bf, xsr, unscale, acc);
            __syncwarp();  // every lane has read its fragments
            if (lane == 0) mbar_arrive(&empty_bar[st]);
            if (!DOTS) {
                // hand the partial tiles to the reducer
                const int buf = it % TC_NB;
                if (it >= TC_NB && !mbar_wait(&pempty_bar[buf], ((it / TC_NB) - 1) & 1)) break;
                if (valid) {
#pragma unroll
                    for (int j = 0; j < NT; ++j)
                        partial[((size_t)(buf * TC_KS_MAX + warp) * NT + j) * 32 + lane] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&pfull_bar[buf]);
            }
        }
    } else if (!DOTS) {
        // ================= reducer =================
        int p = 0, u = 0;
        for (int it = 0; it < total; ++it, (++u == nunits ? (u = 0, ++p) : 0)) {
            const int buf = it % TC_NB;
            if (!mbar_wait(&pfull_bar[buf], (it / TC_NB) & 1)) break;
            const int nvalid = min(KS, nch - p * KS);
            float4 sum[NT];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                sum[j] = (phases > 1 && p > 0) ? ysum[((size_t)u * NT + j) * 32 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
                for (int w = 0; w < nvalid; ++w) {  // fixed order: the result does not depend on warp timing
                    const float4 v = partial[((size_t)(buf * TC_KS_MAX + w) * NT + j) * 32 + lane];
                    sum[j].x += v.x, sum[j].y += v.y, sum[j].z += v.z, sum[j].w += v.w;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&pempty_bar[buf]);
            if (p + 1 < phases) {
#pragma unroll
                for (int j = 0; j < NT; ++j) ysum[((size_t)u * NT + j) * 32 + lane] = sum[j];
                continue;
            }
            const int r0 = row_begin + u * 16 + g, r1 = r0 + 8;
            // y[vector][row]; for matrices laid back to back (group_rows > 0) y[matrix][vector][row of the matrix]: a
            // base per row and the distance between two vectors
            long long y0 = r0, y1 = r1;
            size_t ystep0 = (size_t)rows, ystep1 = (size_t)rows;
            if (a.group_rows > 0) {
                const int m0 = r0 / a.group_rows, m1 = r1 / a.group_rows;
                ystep0 = ystep1 = (size_t)a.group_rows;
                y0 = (long long)m0 * a.batch * a.group_rows + (r0 - m0 * a.group_rows);
                y1 = (long long)m1 * a.batch * a.group_rows + (r1 - m1 * a.group_rows);
            } else if (args.grp.count > 0) {
                // the table of a grouped launch: matrix m writes its [batch][rows of m] block at y + y_off[m]
                if (r0 < row_end) {
                    const int m0 = tc_matrix_of(args.grp, r0);
                    ystep0 = (size_t)(args.grp.row_start[m0 + 1] - args.grp.row_start[m0]);
                    y0 = args.grp.y_off[m0] + (r0 - args.grp.row_start[m0]);
                }
                if (r1 < row_end) {
                    const int m1 = tc_matrix_of(args.grp, r1);
                    ystep1 = (size_t)(args.grp.row_start[m1 + 1] - args.grp.row_start[m1]);
                    y1 = args.grp.y_off[m1] + (r1 - args.grp.row_start[m1]);
                }
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                if (FLT) {
                    const int n = j * 4 + t;
                    if (n < a.batch) {
                        if (r0 < row_end) a.y[(long long)(n * ystep0) + y0] = sum[j].x;
                        if (r1 < row_end) a.y[(long long)(n * ystep1) + y1] = sum[j].z;
                    }
                } else {
                    const int n0 = j * 8 + 2 * t, n1 = n0 + 1;
                    if (n0 < a.batch) {
                        if (r0 < row_end) a.y[(long long)(n0 * ystep0) + y0] = sum[j].x;
                        if (r1 < row_end) a.y[(long long)(n0 * ystep1) + y1] = sum[j].z;
                    }
                    if (n1 < a.batch) {
                        if (r0 < row_end) a.y[(long long)(n1 * ystep0) + y0] = sum[j].y;
                        if (r1 < row_end) a.y[(long long)(n1 * ystep1) + y1] = sum[j].w;
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------------
struct TcPlan {
    int ks, phases, grid, max_units, stages;
    size_t smem;
};

template <int FMT, int NT>
static bool tc_plan(const QGemvArgs &a, const DeviceInfo *di, TcPlan &p) {
    using T = TcTraits<FMT>;
    using Cfg = TcConfig<FMT, NT>;
    const int nch = a.cols / 256;
    p.phases = (nch + TC_KS_MAX - 1) / TC_KS_MAX;
    p.ks = (nch + p.phases - 1) / p.phases;
    const int units = (a.rows + 15) / 16;
    p.grid = units < di->sm_count ? units : di->sm_count;
    // Every CTA walks ceil(units / grid) units, whole or not: with 896 units on 148 CTAs that is a seventh unit of a
    // single row each, a full item's latency for 1 % of its bytes.  Among the grids that keep at least four fifths
    // of the SMs busy, take the one that leaves the fewest unit slots empty (896 units: 128 CTAs of 7 whole units).
    // Q8_0 blocks only, where the launch is bound by memory (measured at 14336 x 4096: 8 vectors 15.0 -> 14.4 us); the
    // split layout and Q4_0 are bound by their consumer warps and lose 2-4 % on fewer SMs.
    if (FMT == FMT_Q8B && units > di->sm_count) {
        long long best_waste = -1;
        for (int g = di->sm_count; g >= di->sm_count * 4 / 5; --g) {
            const long long waste = (long long)((units + g - 1) / g) * g - units;
            if (best_waste < 0 || waste < best_waste) best_waste = waste, p.grid = g;
        }
    }
    const int rows_per_cta = (a.rows + p.grid - 1) / p.grid;
    p.max_units = (rows_per_cta + 15) / 16 + 1;
    const size_t tail = Cfg::PARTIAL + (p.phases > 1 ? (size_t)p.max_units * NT * 512 : 0) + 128;
    const size_t limit = (size_t)di->max_smem_optin - 1024;  // the kernel's static shared memory and slack
    const size_t stage = 16 * ((size_t)tc_row_pitch(p.ks, T::WROW) + (FMT == FMT_Q8S ? p.ks * 16 + 16 : 0));
    if (tail + 2 * stage > limit) return false;
    const size_t n = (limit - tail) / stage;
    p.stages = (int)(n > TC_MAX_STAGES ? TC_MAX_STAGES : n);
    p.smem = (size_t)p.stages * stage + tail;
    return p.smem <= limit;
}

template <int FMT, int NT, int XSRC, bool DOTS>
static int tc_launch(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s, bool overlap, const TcGroup *grp = nullptr) {
    TcPlan p;
    if (!tc_plan<FMT, NT>(a, di, p)) return TB200_ERR_INVALID_ARG;
    // pointers are 0 or 8 modulo 16 here (tc_eligible)
    const int wshift = (int)((uintptr_t)a.w & 15), sshift = (FMT == FMT_Q8S && a.scales) ? (int)((uintptr_t)a.scales & 15) : 0;
    TcArgs args{a, p.ks, p.phases, p.max_units, p.stages, wshift, sshift};
    if (grp) args.grp = *grp;
    constexpr auto kernel = qtc_gemv_kernel<FMT, NT, XSRC, DOTS>;
    const int st = ensure_smem_optin<kernel>(di);
    if (st) return st;
    return launch_kernel(kernel, dim3(p.grid), dim3(TC_THREADS), p.smem, s, overlap, args);
}

template <int FMT>
static bool tc_eligible(int mode, const QGemvArgs &a, const DeviceInfo *di) {
    if (a.cols < 256 || a.cols % 256 != 0 || a.rows < 1 || !a.w || !aligned_to(a.w, 8)) return false;
    if (FMT == FMT_Q8S && !a.dots && (!a.scales || !aligned_to(a.scales, 8))) return false;
    const int cap = mode == MODE_FLOAT ? 8 : kMaxBatch;
    if (a.batch < 1 || a.batch > cap) return false;
    if (mode == MODE_INT ? !a.xq : (!a.x || !aligned_to(a.x, 4))) return false;
    if (a.dots ? mode != MODE_INT : !a.y) return false;
    const bool two = mode == MODE_FLOAT ? a.batch > 4 : a.batch > 8;
    TcPlan p;
    return two ? tc_plan<FMT, 2>(a, di, p) : tc_plan<FMT, 1>(a, di, p);
}

template <int FMT>
static int tc_dispatch(int mode, const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s, bool overlap) {
    if (a.dots)
        return a.batch <= 8 ? tc_launch<FMT, 1, X_INT_WS, true>(a, di, s, overlap)
                            : tc_launch<FMT, 2, X_INT_WS, true>(a, di, s, overlap);
    if (mode == MODE_FLOAT)
        return a.batch <= 4 ? tc_launch<FMT, 1, X_FLOAT, false>(a, di, s, overlap)
                            : tc_launch<FMT, 2, X_FLOAT, false>(a, di, s, overlap);
    if (mode == MODE_INT)
        return a.batch <= 8 ? tc_launch<FMT, 1, X_INT_WS, false>(a, di, s, overlap)
                            : tc_launch<FMT, 2, X_INT_WS, false>(a, di, s, overlap);
    return a.batch <= 8 ? tc_launch<FMT, 1, X_INT_FUSED, false>(a, di, s, overlap)
                        : tc_launch<FMT, 2, X_INT_FUSED, false>(a, di, s, overlap);
}

bool qtc_eligible(int fmt, int mode, const QGemvArgs &a, const DeviceInfo *di) {
    return fmt == FMT_Q8S ? tc_eligible<FMT_Q8S>(mode, a, di) : fmt == FMT_Q8B ? tc_eligible<FMT_Q8B>(mode, a, di) : tc_eligible<FMT_Q4B>(mode, a, di);
}

int qtc_dispatch(int fmt, int mode, const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s, bool overlap) {
    return fmt == FMT_Q8S ? tc_dispatch<FMT_Q8S>(mode, a, di, s, overlap)
                          : fmt == FMT_Q8B ? tc_dispatch<FMT_Q8B>(mode, a, di, s, overlap) : tc_dispatch<FMT_Q4B>(mode, a, di, s, overlap);
}

int qtc_dispatch_group(int fmt, const QGemvArgs &a, const TcGroup &grp, const DeviceInfo *di, cudaStream_t s, bool overlap) {
    if (fmt == FMT_Q8S || a.batch > kMaxBatch || grp.count < 1 || grp.count > kTcMaxGroup) return TB200_ERR_INVALID_ARG;
    if (a.batch > 8) return fmt == FMT_Q8B ? tc_launch<FMT_Q8B, 2, X_INT_WS, false>(a, di, s, overlap, &grp) : tc_launch<FMT_Q4B, 2, X_INT_WS, false>(a, di, s, overlap, &grp);
    return fmt == FMT_Q8B ? tc_launch<FMT_Q8B, 1, X_INT_WS, false>(a, di, s, overlap, &grp) : tc_launch<FMT_Q4B, 1, X_INT_WS, false>(a, di, s, overlap, &grp);
}

}  // namespace tb200


extern "C" int tb200_blockdots_i32_batched(int format, int rows, int cols, int batch, const void *weights, const int8_t *xq,
                                           int32_t *dots, tb200_stream_t stream) {
    using namespace tb200;
    if (format < FMT_Q8S || format > FMT_Q4B || rows < 0 || cols < 0 || batch < 1 || batch > kMaxBatch) return TB200_ERR_INVALID_ARG;
    if (rows == 0 || cols == 0) return TB200_OK;
    if (!weights || !xq || !dots) return TB200_ERR_INVALID_ARG;
    if (!aligned_to(dots, 4)) return TB200_ERR_ALIGNMENT;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    QGemvArgs a{reinterpret_cast<const uint8_t *>(weights), nullptr, nullptr, xq, nullptr, nullptr, dots, rows, cols, batch};
    if (!qtc_eligible(format, MODE_INT, a, di)) return TB200_ERR_INVALID_ARG;  // cols % 256 == 0, 8-byte aligned weights
    return qtc_dispatch(format, MODE_INT, a, di, (cudaStream_t)stream, false);
}
