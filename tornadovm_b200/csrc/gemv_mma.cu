// Batched Q8_0 / Q4_0 mat-vec on the integer tensor-core path (batch 5..16).
//
// With several activation vectors the dp4a kernels run out of integer issue
// slots long before HBM is busy, so each 32-element block dot of a 16-row x
// 8-vector tile is one mma.sync.m16n8k32 (s8 x s8 -> s32): the int32 block dots
// stay exact, and one fp32 FMA per output applies wscale * xscale, exactly as in
// the dp4a kernels.  (mma.sync is the legacy tensor path; the arithmetic here is
// tiny -- the kernel is HBM-bound -- so tcgen05 would add nothing.)
//
// One CTA per SM.  A CTA owns a contiguous range of 16-row units; in each round
// its eight warps take one unit each and walk K together in chunks of 8 blocks
// (256 columns): all threads cp.async the chunk's weights (8 units x 16 rows)
// and the chunk of the quantised activations into a 4-stage shared-memory ring,
// one __syncthreads per chunk.  Two warps share a unit and take half of the
// chunk's blocks each (more warps per scheduler hide the shared-memory and mma
// latencies); their partial sums are added in a fixed order when the unit is
// complete.  Rows are padded to a 272- / 144-byte pitch in shared memory so
// that the fragment loads are bank-conflict free.
#define TB200_OP_CLASS TB200_PREPARE_GEMV_QUANT
#include "gemv_common.cuh"

TB200_TU_STATUS(gemv_mma)

namespace tb200 {

constexpr int MM_WARPS = 8 /* 16-row units per round */, MM_KSPLIT = 2 /* warps per unit */;
constexpr int MM_THREADS = MM_WARPS * MM_KSPLIT * 32, MM_KB = 8 /* blocks per chunk */;
constexpr int MM_STAGES = 4;

template <int FMT>
struct MmaTraits {
    static constexpr int BB = FMT == FMT_Q4B ? 18 : (FMT == FMT_Q8B ? 34 : 32);  // weight bytes per block in the row chunk
    static constexpr int ROWB = MM_KB * BB;                                       // bytes per row chunk (272 / 144 / 256)
    static constexpr int WS = FMT == FMT_Q4B ? 144 : 272;                         // shared-memory row pitch
    static constexpr int PP = ROWB / 16 + (FMT == FMT_Q8S ? 1 : 0);              // 16-byte pieces per row (+ scales piece)
    static constexpr int W_BYTES = MM_WARPS * 16 * WS;
    static constexpr int SC_BYTES = FMT == FMT_Q8S ? MM_WARPS * 16 * 16 : 0;     // split layout: 8 fp16 scales per row
};

template <int FMT, int NT>
struct MmaStage {
    using T = MmaTraits<FMT>;
    static constexpr int BP = NT * 8;
    static constexpr int X_OFF = T::W_BYTES + T::SC_BYTES;
    static constexpr int XS_OFF = X_OFF + BP * 272;
    static constexpr int BYTES = (XS_OFF + BP * 32 + 127) & ~127;
    static constexpr int W_ONLY_BYTES = (X_OFF + 127) & ~127;  // a stage without the activation chunk
};

// XFULL: all quantised activations (and their scales) are staged in shared memory once, in the prologue.
// Otherwise every K chunk re-reads its slice of them from L2 -- which all CTAs then do at the same moment
// for the same addresses; that hot spot costs about a microsecond per chunk, so XFULL is used whenever
// the vectors fit beside the weight ring.
//
// XM selects how the activations reach the tensor cores:
//   0  int8, one slice per K chunk (the vectors do not fit in shared memory)
//   1  int8, resident
//   2  fp32 activations ("float mode"), resident as fp16 pairs: x = hi + lo with hi = fp16(x) and
//      lo = fp16(x - hi), relative error 2^-22.  Weights are exact in fp16, every product is exact in
//      fp32, so one m16n8k16 fp16 MMA with fp32 accumulation per 16 columns computes the reference's
//      fp32 dot products to fp32 accuracy; column 2b of the MMA's B operand carries hi of vector b and
//      column 2b+1 its lo part, and the two result columns are added.
template <int FMT, int NT, int XM>
__global__ void __launch_bounds__(MM_THREADS, 1) qmma_gemv_kernel(QGemvArgs a) {
    constexpr bool XFULL = XM != 0, FLT = XM == 2;
    using T = MmaTraits<FMT>;
    using S = MmaStage<FMT, NT>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int cols = a.cols, rows = a.rows, batch = a.batch;
    const int bpr = cols / 32;
    const int nkc = bpr / MM_KB;  // cols % 256 == 0
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = (tid >> 5) % MM_WARPS;   // unit slot of this warp
    const int khalf = (tid >> 5) / MM_WARPS;  // which blocks of a chunk it takes
    const int g = lane >> 2, t = lane & 3;

    const int nunits = (rows + 15) / 16;
    const int ubeg = (int)((long long)nunits * blockIdx.x / gridDim.x);
    const int uend = (int)((long long)nunits * (blockIdx.x + 1) / gridDim.x);
    const int nrounds = (uend - ubeg + MM_WARPS - 1) / MM_WARPS;
    const int total = nrounds * nkc;
    constexpr int STAGE_BYTES = XFULL ? S::W_ONLY_BYTES : S::BYTES;
    float *red = reinterpret_cast<float *>(smem_raw + (size_t)MM_STAGES * STAGE_BYTES);  // [unit slot][lane][NT*4]
    // resident activations: int8 rows with a pitch of cols + 16 bytes (bank spread), then fp32 scales [vector][block]
    const int xpitch = FLT ? cols * 2 + 32 : cols + 16;  // float mode: 8-byte reads, rows 8 banks apart
    unsigned char *xfull = reinterpret_cast<unsigned char *>(red + MM_WARPS * 32 * NT * 4);
    float *xsfull = reinterpret_cast<float *>(xfull + (size_t)S::BP * xpitch);

    // Copy plan of this thread: it always moves the same (row, piece) slots of a chunk, so the source
    // pointers are set up once per round and only advance along K afterwards.
    constexpr int NW = (MM_WARPS * 16 * T::PP + MM_THREADS - 1) / MM_THREADS;  // weight pieces per thread and chunk
    constexpr int NX = (S::BP * 18 + MM_THREADS - 1) / MM_THREADS;            // activation pieces per thread and chunk
    const unsigned char *wsrc[NW];
    uint32_t wdst[NW];
    int wstep[NW];
    const unsigned char *xsrc[NX];
    uint32_t xdst[NX];
    int xstep[NX];
#pragma unroll
    for (int m = 0; m < NX; ++m) {
        const int i = tid + m * MM_THREADS;
        const int b = i / 18, p = i - b * 18;
        xsrc[m] = nullptr, xdst[m] = 0, xstep[m] = 0;
        if (i < S::BP * 18 && b < batch) {
            if (p < 16) {
                xsrc[m] = reinterpret_cast<const unsigned char *>(a.xq) + (size_t)b * cols + p * 16;
                xdst[m] = S::X_OFF + b * 272 + p * 16, xstep[m] = 256;
            } else {
                xsrc[m] = reinterpret_cast<const unsigned char *>(a.xs + (size_t)b * bpr + (p - 16) * 4);
                xdst[m] = S::XS_OFF + b * 32 + (p - 16) * 16, xstep[m] = MM_KB * 4;
            }
        }
    }
    auto plan_round = [&](int round) {
        const int ufirst = ubeg + round * MM_WARPS;
#pragma unroll
        for (int m = 0; m < NW; ++m) {
            const int i = tid + m * MM_THREADS;
            const int rl = i / T::PP, p = i - rl * T::PP;
            wsrc[m] = nullptr;
            // unit slots past the end of this CTA's range copy nothing (their warps idle through the round)
            if (i < MM_WARPS * 16 * T::PP && ufirst + (rl >> 4) < uend) {
                const size_t grow = (size_t)min((ufirst + (rl >> 4)) * 16 + (rl & 15), rows - 1);
                if (FMT == FMT_Q8S) {
                    if (p < 16) {
                        wsrc[m] = a.w + grow * cols + p * 16, wdst[m] = rl * T::WS + p * 16, wstep[m] = 256;
                    } else {
                        wsrc[m] = reinterpret_cast<const unsigned char *>(a.scales + grow * bpr);
                        wdst[m] = T::W_BYTES + rl * 16, wstep[m] = MM_KB * 2;
                    }
                } else {
                    wsrc[m] = a.w + grow * bpr * T::BB + p * 16, wdst[m] = rl * T::WS + p * 16, wstep[m] = T::ROWB;
                }
            }
        }
    };

    // one chunk (8 units x 16 rows x 8 blocks of weights, 8 blocks of every activation vector) into a stage
    int issue_kc = 0, issue_round = 0;
    plan_round(0);
    auto issue = [&](int it) {
        if (it < total) {
            const uint32_t base_s = smem_u32(smem_raw + (size_t)(it % MM_STAGES) * STAGE_BYTES);
#pragma unroll
            for (int m = 0; m < NW; ++m)
                if (wsrc[m]) cp_async_16(base_s + wdst[m], wsrc[m] + (size_t)issue_kc * wstep[m]);
#pragma unroll
            for (int m = 0; m < NX; ++m)
                if (!XFULL && xsrc[m]) cp_async_16(base_s + xdst[m], xsrc[m] + (size_t)issue_kc * xstep[m]);
            if (++issue_kc == nkc) {
                issue_kc = 0;
                if (++issue_round < nrounds) plan_round(issue_round);
            }
        }
        cp_async_commit();
    };

#pragma unroll
    for (int s = 0; s < MM_STAGES - 1; ++s) issue(s);
    if (FLT) {
        // weights are on their way; the activations may come from the kernel before this one
        pdl_launch_dependents();
        pdl_wait();
        const int n4 = cols / 4;
        for (int i = tid; i < batch * n4; i += MM_THREADS) {
            const int b = i / n4, c4 = i - b * n4;
            const float4 v = __ldg(reinterpret_cast<const float4 *>(a.x + (size_t)b * cols) + c4);
            const __half h0 = __float2half_rn(v.x), h1 = __float2half_rn(v.y), h2 = __float2half_rn(v.z), h3 = __float2half_rn(v.w);
            const __half l0 = __float2half_rn(v.x - __half2float(h0)), l1 = __float2half_rn(v.y - __half2float(h1));
            const __half l2 = __float2half_rn(v.z - __half2float(h2)), l3 = __float2half_rn(v.w - __half2float(h3));
            __half2 *hp = reinterpret_cast<__half2 *>(xfull + (size_t)(2 * b) * xpitch + c4 * 8);
            __half2 *lp = reinterpret_cast<__half2 *>(xfull + (size_t)(2 * b + 1) * xpitch + c4 * 8);
            hp[0] = __halves2half2(h0, h1), hp[1] = __halves2half2(h2, h3);
            lp[0] = __halves2half2(l0, l1), lp[1] = __halves2half2(l2, l3);
        }
    } else if (XFULL) {
        // visible to all warps after the first chunk's __syncthreads
        const int n16 = cols / 16;
        for (int i = tid; i < batch * n16; i += MM_THREADS) {
            const int b = i / n16, p = i - b * n16;
            *reinterpret_cast<uint4 *>(xfull + (size_t)b * xpitch + p * 16) =
                __ldg(reinterpret_cast<const uint4 *>(a.xq + (size_t)b * cols) + p);
        }
        for (int i = tid; i < batch * bpr; i += MM_THREADS) xsfull[i] = __ldg(a.xs + i);
    }

    float acc[NT][4];
    for (int it = 0; it < total; ++it) {
        cp_async_wait<MM_STAGES - 2>();
        __syncthreads();             // chunk `it` has landed for everyone; chunk it-1 is no longer read
        issue(it + MM_STAGES - 1);   // refills the stage of chunk it-1
        const int round = it / nkc, kc = it - round * nkc;
        const unsigned char *base = smem_raw + (size_t)(it % MM_STAGES) * STAGE_BYTES;
        const int unit = ubeg + round * MM_WARPS + warp;
        const bool active = unit < uend;  // warp-uniform; an idle warp still takes part in copies and barriers
        if (kc == 0) {
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
        }
        const unsigned char *rp0 = base + (warp * 16 + g) * T::WS;
        const unsigned char *rp1 = rp0 + 8 * T::WS;
#pragma unroll
        for (int kbi = 0; kbi < (active ? MM_KB / MM_KSPLIT : 0); ++kbi) {
            const int kb = khalf * (MM_KB / MM_KSPLIT) + kbi;  // kb % 2 == kbi % 2
            uint32_t a0, a1, a2, a3;
            float sw0, sw1;
            if (FMT == FMT_Q8B) {
                constexpr int dummy = 0;
                (void)dummy;
                const int off = kb * 34 + 2 + 4 * t;
                if (kbi % 2 == 0) {  // 34*kb + 2 is 2 modulo 4
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
                if (kbi % 2 == 0) w0 = lds_u32_at<1>(rp0, off), w1 = lds_u32_at<1>(rp1, off);
                else w0 = lds_u32_at<0>(rp0, off), w1 = lds_u32_at<0>(rp1, off);
                // byte i holds element i (low nibble) and element i + 16 (high nibble)
                a0 = w0 & 0x0F0F0F0Fu, a2 = (w0 >> 4) & 0x0F0F0F0Fu;
                a1 = w1 & 0x0F0F0F0Fu, a3 = (w1 >> 4) & 0x0F0F0F0Fu;
                sw0 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(rp0 + kb * 18));
                sw1 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(rp1 + kb * 18));
            } else {
                const int off = kb * 32 + 4 * t;
                a0 = lds_u32_at<0>(rp0, off), a1 = lds_u32_at<0>(rp1, off);
                a2 = lds_u32_at<0>(rp0, off + 16), a3 = lds_u32_at<0>(rp1, off + 16);
                const unsigned char *sp = base + T::W_BYTES + (warp * 16 + g) * 16 + kb * 2;
                sw0 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(sp));
                sw1 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(sp + 8 * 16));
            }
            if (FLT) {
                // group 0 = elements 0..15 of the block, group 1 = elements 16..31; within a group this thread
                // owns elements 4t..4t+3, which it feeds to the MMA as k = {2t, 2t+1} and {2t+8, 2t+9}
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
                    const unsigned char *xrow = xfull + (size_t)(j * 8 + g) * xpitch + ((kc * MM_KB + kb) * 32 + 4 * t) * 2;
                    const uint2 bA = *reinterpret_cast<const uint2 *>(xrow);
                    const uint2 bB = *reinterpret_cast<const uint2 *>(xrow + 32);
                    float d[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_f16_16816(d, p0, p1, p2, p3, bA.x, bA.y);
                    mma_f16_16816(d, q0, q1, q2, q3, bB.x, bB.y);
                    // columns 2t (hi part) and 2t+1 (lo part) belong to vector j*4 + t
                    acc[j][0] = fmaf(d[0] + d[1], sw0, acc[j][0]);
                    acc[j][2] = fmaf(d[2] + d[3], sw1, acc[j][2]);
                }
                continue;
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const unsigned char *xrow = XFULL ? xfull + (size_t)(j * 8 + g) * xpitch + (kc * MM_KB + kb) * 32 + 4 * t
                                                  : base + S::X_OFF + (j * 8 + g) * 272 + kb * 32 + 4 * t;
                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(xrow);
                const uint32_t b1 = *reinterpret_cast<const uint32_t *>(xrow + 16);
                int d[4];
                mma_s8_16832(d, a0, a1, a2, a3, b0, b1);
                if (FMT == FMT_Q4B) {
                    // nibbles are 0..15: subtract 8 * sum(xq) of the block, itself one mma against all-ones rows
                    int sx[4];
                    mma_s8_16832(sx, 0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u, b0, b1);
                    d[0] -= 8 * sx[0], d[1] -= 8 * sx[1], d[2] -= 8 * sx[0], d[3] -= 8 * sx[1];
                }
                float x0, x1;
                if (XFULL) {
                    // vectors beyond the batch read shared memory that was never written: their outputs are dropped
                    const float *xsp = xsfull + (size_t)(j * 8 + 2 * t) * bpr + kc * MM_KB + kb;
                    x0 = xsp[0], x1 = xsp[bpr];
                } else {
                    const float *xsp = reinterpret_cast<const float *>(base + S::XS_OFF) + (j * 8 + 2 * t) * 8 + kb;
                    x0 = xsp[0], x1 = xsp[8];
                }
                acc[j][0] = fmaf((float)d[0], sw0 * x0, acc[j][0]);
                acc[j][1] = fmaf((float)d[1], sw0 * x1, acc[j][1]);
                acc[j][2] = fmaf((float)d[2], sw1 * x0, acc[j][2]);
                acc[j][3] = fmaf((float)d[3], sw1 * x1, acc[j][3]);
            }
        }
        if (kc == nkc - 1) {
            // the round is complete: the second warp of each unit hands its partial tile to the first
            float *tile = red + (size_t)warp * 32 * NT * 4 + lane * NT * 4;
            if (khalf == 1) {
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) tile[j * 4 + i] = acc[j][i];
            }
            __syncthreads();
            if (khalf == 0 && active) {
                const int r0 = unit * 16 + g, r1 = r0 + 8;
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const float c0 = acc[j][0] + tile[j * 4 + 0], c1 = acc[j][1] + tile[j * 4 + 1];
                    const float c2 = acc[j][2] + tile[j * 4 + 2], c3 = acc[j][3] + tile[j * 4 + 3];
                    if (FLT) {
                        const int n = j * 4 + t;
                        if (n < batch) {
                            if (r0 < rows) a.y[(size_t)n * rows + r0] = c0;
                            if (r1 < rows) a.y[(size_t)n * rows + r1] = c2;
                        }
                        continue;
                    }
                    const int n0 = j * 8 + 2 * t, n1 = n0 + 1;
                    if (n0 < batch) {
                        if (r0 < rows) a.y[(size_t)n0 * rows + r0] = c0;
                        if (r1 < rows) a.y[(size_t)n0 * rows + r1] = c2;
                    }
                    if (n1 < batch) {
                        if (r0 < rows) a.y[(size_t)n1 * rows + r0] = c1;
                        if (r1 < rows) a.y[(size_t)n1 * rows + r1] = c3;
                    }
                }
            }
            // `red` is written again only at the end of the next round, behind that round's barriers
        }
    }
    cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------------------
// Warp-autonomous form of the same computation, used whenever the activations fit in shared memory next to
// the rings.  Every warp owns whole 16-row units (a contiguous run of them) and streams their K chunks
// through its OWN 4-stage cp.async ring: no CTA-wide barrier after the prologue, warps drift apart and hide
// one another's shared-memory and MMA latencies, and a slow unit delays nobody else.  With 14336 rows there
// are 896 units for 148 x 8 warps: most warps stream exactly one unit from start to end.
// FLT = false: int8 activations (xq, xs) -> mma.sync s8;  FLT = true: fp32 activations as fp16 hi/lo pairs.
// Measured against two variants that were dropped: rings of 5 to 8 stages (slower by about 1 us) and the
// CTA working on one unit at a time with its warps on interleaved K chunks (slower by 2 to 3 us).
// ---------------------------------------------------------------------------------------------------------
constexpr int WM_WARPS = 8, WM_THREADS = WM_WARPS * 32, WM_STAGES = 4;

template <int FMT>
struct WmTraits {
    using T = MmaTraits<FMT>;
    static constexpr int STAGE = 16 * T::WS;                    // 4352 / 2304 bytes: 16 rows of one 8-block chunk
    static constexpr int PIECES = 16 * T::PP;                   // 16-byte pieces per stage (272 / 144)
    static constexpr int NP = (PIECES + 31) / 32;               // pieces per lane
    static constexpr int RING = WM_WARPS * WM_STAGES * STAGE;   // bytes of all rings of a CTA
};

template <int FMT, int NT, bool FLT>
static size_t wm_smem_bytes(int cols) {
    const size_t x = FLT ? (size_t)NT * 8 * (cols * 2 + 32) : (size_t)NT * 8 * (cols + 16) + (size_t)NT * 8 * (cols / 32) * 4;
    return (size_t)WmTraits<FMT>::RING + x;
}

template <int FMT, int NT, bool FLT>
__global__ void __launch_bounds__(WM_THREADS, 1) qmmaw_gemv_kernel(QGemvArgs a) {
    using T = MmaTraits<FMT>;
    using W = WmTraits<FMT>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int cols = a.cols, rows = a.rows, batch = a.batch;
    const int bpr = cols / 32;
    const int nkc = bpr / MM_KB;  // cols % 256 == 0
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    unsigned char *ring = smem_raw + (size_t)warp * WM_STAGES * W::STAGE;
    const uint32_t ring_s = smem_u32(ring);
    const int xpitch = FLT ? cols * 2 + 32 : cols + 16;
    unsigned char *xfull = smem_raw + W::RING;
    float *xsfull = reinterpret_cast<float *>(xfull + (size_t)NT * 8 * xpitch);  // int mode: fp32 scales [vector][block]

    // this warp's run of units
    const int nunits = (rows + 15) / 16;
    const long long gw = (long long)blockIdx.x * WM_WARPS + warp, nw = (long long)gridDim.x * WM_WARPS;
    const int ubeg = (int)(nunits * gw / nw), uend = (int)(nunits * (gw + 1) / nw);
    const int total = (uend - ubeg) * nkc;

    // copy plan: lane l moves pieces l, l + 32, ... of a stage; per unit only the row base changes
    const unsigned char *src[W::NP];
    uint32_t dst[W::NP];
    int step[W::NP];
    auto plan_unit = [&](int unit) {
#pragma unroll
        for (int j = 0; j < W::NP; ++j) {
            const int i = lane + 32 * j;
            const int rl = i / T::PP, p = i - rl * T::PP;
            src[j] = nullptr;
            if (i < W::PIECES) {
                const size_t grow = (size_t)min(unit * 16 + rl, rows - 1);
                dst[j] = rl * T::WS + p * 16;
                if (FMT == FMT_Q8S) {
                    if (p < 16) src[j] = a.w + grow * cols + p * 16, step[j] = 256;
                    else src[j] = reinterpret_cast<const unsigned char *>(a.scales + grow * bpr), step[j] = MM_KB * 2;
                } else {
                    src[j] = a.w + grow * bpr * T::BB + p * 16, step[j] = T::ROWB;
                }
            }
        }
    };
    int iu = ubeg, ikc = 0;
    if (total > 0) plan_unit(iu);
    auto issue = [&](int it) {
        if (it < total) {
            const uint32_t base_s = ring_s + (it % WM_STAGES) * W::STAGE;
#pragma unroll
            for (int j = 0; j < W::NP; ++j)
                if (src[j]) cp_async_16(base_s + dst[j], src[j] + (size_t)ikc * step[j]);
            if (++ikc == nkc) {
                ikc = 0;
                if (++iu < uend) plan_unit(iu);
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < WM_STAGES - 1; ++s) issue(s);

    // ---- activations into shared memory, once per CTA ----
    if (FLT) {
        pdl_launch_dependents();
        pdl_wait();  // weights are on their way; the activations may come from the kernel before this one
        const int n4 = cols / 4;
        for (int i = tid; i < batch * n4; i += WM_THREADS) {
            const int b = i / n4, c4 = i - b * n4;
            const float4 v = __ldg(reinterpret_cast<const float4 *>(a.x + (size_t)b * cols) + c4);
            const __half h0 = __float2half_rn(v.x), h1 = __float2half_rn(v.y), h2 = __float2half_rn(v.z), h3 = __float2half_rn(v.w);
            const __half l0 = __float2half_rn(v.x - __half2float(h0)), l1 = __float2half_rn(v.y - __half2float(h1));
            const __half l2 = __float2half_rn(v.z - __half2float(h2)), l3 = __float2half_rn(v.w - __half2float(h3));
            __half2 *hp = reinterpret_cast<__half2 *>(xfull + (size_t)(2 * b) * xpitch + c4 * 8);
            __half2 *lp = reinterpret_cast<__half2 *>(xfull + (size_t)(2 * b + 1) * xpitch + c4 * 8);
            hp[0] = __halves2half2(h0, h1), hp[1] = __halves2half2(h2, h3);
            lp[0] = __halves2half2(l0, l1), lp[1] = __halves2half2(l2, l3);
        }
    } else {
        const int n16 = cols / 16;
        for (int i = tid; i < batch * n16; i += WM_THREADS) {
            const int b = i / n16, p = i - b * n16;
            *reinterpret_cast<uint4 *>(xfull + (size_t)b * xpitch + p * 16) = __ldg(reinterpret_cast<const uint4 *>(a.xq + (size_t)b * cols) + p);
        }
        for (int i = tid; i < batch * bpr; i += WM_THREADS) xsfull[i] = __ldg(a.xs + i);
    }
    __syncthreads();  // the only CTA-wide barrier

    float acc[NT][4];
    for (int it = 0; it < total; ++it) {
        cp_async_wait<WM_STAGES - 2>();
        __syncwarp();               // chunk `it` is visible to every lane; every lane is done with chunk it-1
        issue(it + WM_STAGES - 1);  // refills the stage of chunk it-1
        const int u = it / nkc, kc = it - u * nkc;
        const int unit = ubeg + u;
        const unsigned char *base = ring + (size_t)(it % WM_STAGES) * W::STAGE;
        if (kc == 0) {
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
        }
        const unsigned char *rp0 = base + g * T::WS;
        const unsigned char *rp1 = rp0 + 8 * T::WS;
#pragma unroll 4
        for (int kb = 0; kb < MM_KB; ++kb) {
            uint32_t a0, a1, a2, a3;
            float sw0, sw1;
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
                // byte i holds element i (low nibble) and element i + 16 (high nibble)
                a0 = w0 & 0x0F0F0F0Fu, a2 = (w0 >> 4) & 0x0F0F0F0Fu;
                a1 = w1 & 0x0F0F0F0Fu, a3 = (w1 >> 4) & 0x0F0F0F0Fu;
                sw0 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(rp0 + kb * 18));
                sw1 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(rp1 + kb * 18));
            } else {
                const int off = kb * 32 + 4 * t;
                a0 = lds_u32_at<0>(rp0, off), a1 = lds_u32_at<0>(rp1, off);
                a2 = lds_u32_at<0>(rp0, off + 16), a3 = lds_u32_at<0>(rp1, off + 16);
                sw0 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(rp0 + 256 + kb * 2));
                sw1 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(rp1 + 256 + kb * 2));
            }
            const int blk = kc * MM_KB + kb;
            if (FLT) {
                // group 0 = elements 0..15 of the block, group 1 = elements 16..31; within a group this thread
                // owns elements 4t..4t+3, which it feeds to the MMA as k = {2t, 2t+1} and {2t+8, 2t+9}
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
                    const unsigned char *xrow = xfull + (size_t)(j * 8 + g) * xpitch + (blk * 32 + 4 * t) * 2;
                    const uint2 bA = *reinterpret_cast<const uint2 *>(xrow);
                    const uint2 bB = *reinterpret_cast<const uint2 *>(xrow + 32);
                    float d[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_f16_16816(d, p0, p1, p2, p3, bA.x, bA.y);
                    mma_f16_16816(d, q0, q1, q2, q3, bB.x, bB.y);
                    // columns 2t (hi part) and 2t+1 (lo part) belong to vector j*4 + t
                    acc[j][0] = fmaf(d[0] + d[1], sw0, acc[j][0]);
                    acc[j][2] = fmaf(d[2] + d[3], sw1, acc[j][2]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const unsigned char *xrow = xfull + (size_t)(j * 8 + g) * xpitch + blk * 32 + 4 * t;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t *>(xrow);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t *>(xrow + 16);
                    int d[4];
                    mma_s8_16832(d, a0, a1, a2, a3, b0, b1);
                    if (FMT == FMT_Q4B) {
                        // nibbles are 0..15: subtract 8 * sum(xq) of the block, itself one mma against all-ones rows
                        int sx[4];
                        mma_s8_16832(sx, 0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u, b0, b1);
                        d[0] -= 8 * sx[0], d[1] -= 8 * sx[1], d[2] -= 8 * sx[0], d[3] -= 8 * sx[1];
                    }
                    // vectors beyond the batch read shared memory that was never written: their outputs are dropped
                    const float *xsp = xsfull + (size_t)(j * 8 + 2 * t) * bpr + blk;
                    const float x0 = xsp[0], x1 = xsp[bpr];
                    acc[j][0] = fmaf((float)d[0], sw0 * x0, acc[j][0]);
                    acc[j][1] = fmaf((float)d[1], sw0 * x1, acc[j][1]);
                    acc[j][2] = fmaf((float)d[2], sw1 * x0, acc[j][2]);
                    acc[j][3] = fmaf((float)d[3], sw1 * x1, acc[j][3]);
                }
            }
        }
        if (kc == nkc - 1) {
            const int r0 = unit * 16 + g, r1 = r0 + 8;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                if (FLT) {
                    const int n = j * 4 + t;
                    if (n < batch) {
                        if (r0 < rows) a.y[(size_t)n * rows + r0] = acc[j][0];
                        if (r1 < rows) a.y[(size_t)n * rows + r1] = acc[j][2];
                    }
                } else {
                    const int n0 = j * 8 + 2 * t, n1 = n0 + 1;
                    if (n0 < batch) {
                        if (r0 < rows) a.y[(size_t)n0 * rows + r0] = acc[j][0];
                        if (r1 < rows) a.y[(size_t)n0 * rows + r1] = acc[j][2];
                    }
                    if (n1 < batch) {
                        if (r0 < rows) a.y[(size_t)n1 * rows + r0] = acc[j][1];
                        if (r1 < rows) a.y[(size_t)n1 * rows + r1] = acc[j][3];
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
}

template <int FMT, int NT, bool FLT>
static int launch_qmmaw(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s, bool overlap) {
    constexpr auto kernel = qmmaw_gemv_kernel<FMT, NT, FLT>;
    int st = ensure_smem_optin<kernel>(di);
    if (st) return st;
    const int nunits = (a.rows + 15) / 16;
    const int grid = nunits < di->sm_count ? nunits : di->sm_count;  // units spread over all SMs, a few per CTA
    return launch_kernel(kernel, dim3(grid), dim3(WM_THREADS), wm_smem_bytes<FMT, NT, FLT>(a.cols), s, overlap, a);
}

template <int FMT, int NT, bool FLT>
static bool qmmaw_fits(const QGemvArgs &a, const DeviceInfo *di) {
    return option_value(TB200_OPT_MMA_WARP_RINGS) && wm_smem_bytes<FMT, NT, FLT>(a.cols) + 1024 <= (size_t)di->max_smem_optin;
}

template <int FMT, int NT, int XM>
static int launch_qmma_x(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s, size_t smem, bool overlap = false) {
    constexpr auto kernel = qmma_gemv_kernel<FMT, NT, XM>;
    int st = ensure_smem_optin<kernel>(di);
    if (st) return st;
    const int nunits = (a.rows + 15) / 16;
    const int grid = nunits < di->sm_count ? nunits : di->sm_count;
    return launch_kernel(kernel, dim3(grid), dim3(MM_THREADS), smem, s, overlap, a);  // int modes follow the quantiser kernel: plain stream order
}

template <int FMT, int NT>
static int launch_qmma(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    using S = MmaStage<FMT, NT>;
    const size_t red = (size_t)MM_WARPS * 32 * NT * 4 * sizeof(float);
    const size_t xfull = (size_t)S::BP * (a.cols + 16) + (size_t)S::BP * (a.cols / 32) * 4;
    const size_t resident = (size_t)MM_STAGES * S::W_ONLY_BYTES + red + xfull;
    if (qmmaw_fits<FMT, NT, false>(a, di)) return launch_qmmaw<FMT, NT, false>(a, di, s, false);  // follows the quantiser kernel
    if (resident + 1024 <= (size_t)di->max_smem_optin) return launch_qmma_x<FMT, NT, 1>(a, di, s, resident);
    return launch_qmma_x<FMT, NT, 0>(a, di, s, (size_t)MM_STAGES * S::BYTES + red);
}

// Entry used by the dispatcher of gemv_quant.cu: already quantised activations (xq, xs), 5 <= batch <= 16.
template <int FMT>
static int qmma_dispatch_t(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    return a.batch <= 8 ? launch_qmma<FMT, 1>(a, di, s) : launch_qmma<FMT, 2>(a, di, s);
}

// Shapes and alignments the tensor-core kernel takes.
template <int FMT>
static bool qmma_eligible_t(const QGemvArgs &a) {
    if (a.batch < option_value(TB200_OPT_INT_TENSOR_CORE_MIN_BATCH) || a.cols % 256 != 0 || !aligned_to(a.w, 16) || !aligned_to(a.xq, 16) || !a.xs || !aligned_to(a.xs, 16)) return false;
    if (FMT == FMT_Q8S && (!a.scales || !aligned_to(a.scales, 16))) return false;
    return a.y != nullptr;
}

// Float mode (fp32 activations): batch <= 8 and vectors that stay resident in shared memory.
template <int FMT>
static bool qmma_float_eligible_t(const QGemvArgs &a, const DeviceInfo *di) {
    if (a.batch < 1 || a.batch > 8 || a.cols % 256 != 0 || !aligned_to(a.w, 16) || !a.x || !aligned_to(a.x, 16) || !a.y) return false;
    if (FMT == FMT_Q8S && (!a.scales || !aligned_to(a.scales, 16))) return false;
    const int nt = a.batch <= 4 ? 1 : 2;
    const size_t need = (size_t)MM_STAGES * (nt == 1 ? MmaStage<FMT, 1>::W_ONLY_BYTES : MmaStage<FMT, 2>::W_ONLY_BYTES) +
                        (size_t)MM_WARPS * 32 * nt * 4 * sizeof(float) + (size_t)nt * 8 * (a.cols * 2 + 32);
    return need + 1024 <= (size_t)di->max_smem_optin;
}

template <int FMT, int NT>
static int launch_qmma_float(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s, bool overlap) {
    using S = MmaStage<FMT, NT>;
    if (qmmaw_fits<FMT, NT, true>(a, di)) return launch_qmmaw<FMT, NT, true>(a, di, s, overlap);
    const size_t smem = (size_t)MM_STAGES * S::W_ONLY_BYTES + (size_t)MM_WARPS * 32 * NT * 4 * sizeof(float) +
                        (size_t)S::BP * (a.cols * 2 + 32);
    return launch_qmma_x<FMT, NT, 2>(a, di, s, smem, overlap);
}

template <int FMT>
static int qmma_float_dispatch_t(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s, bool overlap) {
    return a.batch <= 4 ? launch_qmma_float<FMT, 1>(a, di, s, overlap) : launch_qmma_float<FMT, 2>(a, di, s, overlap);
}

bool qmma_eligible(int fmt, const QGemvArgs &a) {
    return fmt == FMT_Q8S ? qmma_eligible_t<FMT_Q8S>(a) : fmt == FMT_Q8B ? qmma_eligible_t<FMT_Q8B>(a) : qmma_eligible_t<FMT_Q4B>(a);
}
int qmma_dispatch(int fmt, const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    return fmt == FMT_Q8S ? qmma_dispatch_t<FMT_Q8S>(a, di, s) : fmt == FMT_Q8B ? qmma_dispatch_t<FMT_Q8B>(a, di, s) : qmma_dispatch_t<FMT_Q4B>(a, di, s);
}
bool qmma_float_eligible(int fmt, const QGemvArgs &a, const DeviceInfo *di) {
    return fmt == FMT_Q8S ? qmma_float_eligible_t<FMT_Q8S>(a, di)
                          : fmt == FMT_Q8B ? qmma_float_eligible_t<FMT_Q8B>(a, di) : qmma_float_eligible_t<FMT_Q4B>(a, di);
}
int qmma_float_dispatch(int fmt, const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s, bool overlap) {
    return fmt == FMT_Q8S ? qmma_float_dispatch_t<FMT_Q8S>(a, di, s, overlap)
                          : fmt == FMT_Q8B ? qmma_float_dispatch_t<FMT_Q8B>(a, di, s, overlap) : qmma_float_dispatch_t<FMT_Q4B>(a, di, s, overlap);
}

}  // namespace tb200
