// Q8_0 / Q4_0 matrix-vector products, HBM-bound.
//
// Replaces the work-group-per-row Q8_0 kernels of the reference
// (MatrixVectorRowMajor.java:409-578) and its DP4A kernels (:580-838).
//
// Three weight formats:
//   Q8S  split   int8 q[rows][cols] + fp16 scale[rows][cols/32]
//   Q8B  blocks  34-byte blocks  (fp16 scale, 32 x int8)
//   Q4B  blocks  18-byte blocks  (fp16 scale, 16 nibble bytes)
// Two arithmetic modes:
//   float  fp32 activations, weights dequantised in registers, fp32 FMA
//   int    activations quantised to int8 per 32-block, exact int32 block dots
//          (dp4a), one fp32 multiply-add per block for the two scales
//
// Kernel families:
//   q8s_gemv_kernel   split layout; each lane streams 16 quants per row with one
//                     128-bit load that bypasses L1; R rows share every
//                     activation read from shared memory.
//   qblk_gemv_kernel  block layouts; rows are 2-byte aligned records, so each
//                     warp runs its own bulk-async-copy (TMA) pipeline that
//                     lands row chunks of 64 blocks in shared memory; a lane
//                     decodes one pair of blocks (a 4-byte aligned 68 / 36 byte
//                     record) per row.
//   q*_generic_kernel any alignment and any cols % 32 == 0; byte loads.
//
// Activations are staged once per CTA in shared memory in a lane-interleaved
// order, so that the 128-bit shared loads of a warp touch consecutive 16-byte
// slots (no bank conflicts).
//
// Algorithmic bytes per launch:
//   Q8: 34 * rows*cols/32 + 4*batch*(cols + rows)
//   Q4: 18 * rows*cols/32 + 4*batch*(cols + rows)
#include "common.cuh"

namespace tb200 {

constexpr int FMT_Q8S = 0, FMT_Q8B = 1, FMT_Q4B = 2;
constexpr int kMaxBatch = 16;

struct QGemvArgs {
    const uint8_t *w;        // quants (split) or blocks
    const uint16_t *scales;  // split layout only
    const float *x;          // float mode: [batch][cols]
    const int8_t *xq;        // int mode:   [batch][cols]
    const float *xs;         // int mode:   [batch][cols/32]
    float *y;                // [batch][rows]; may be null when dots is set
    int32_t *dots;           // optional [rows][cols/32] (batch 1, int mode)
    int rows, cols, batch;
};

__device__ __forceinline__ int dp4a_s8(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }

// ---------------------------------------------------------------------------
// Generic kernels: one warp per row, one lane per block, byte loads.
// ---------------------------------------------------------------------------
template <int FMT>
__device__ __forceinline__ void load_block_generic(const QGemvArgs &a, size_t row, int blk, int bpr, float &scale,
                                                   int (&v)[32]) {
    if (FMT == FMT_Q8S) {
        scale = a.scales ? half_bits_to_float(a.scales[row * bpr + blk]) : 1.0f;
        const int8_t *p = reinterpret_cast<const int8_t *>(a.w) + row * (size_t)a.cols + (size_t)blk * 32;
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = p[i];
    } else if (FMT == FMT_Q8B) {
        const uint8_t *p = a.w + (row * bpr + blk) * 34;
        scale = half_bits_to_float((uint16_t)(p[0] | (p[1] << 8)));
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = (int8_t)p[2 + i];
    } else {
        const uint8_t *p = a.w + (row * bpr + blk) * 18;
        scale = half_bits_to_float((uint16_t)(p[0] | (p[1] << 8)));
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            uint8_t byte = p[2 + i];
            v[i] = (int)(byte & 0x0F) - 8;
            v[i + 16] = (int)(byte >> 4) - 8;
        }
    }
}

template <int FMT, bool INT>
__global__ void __launch_bounds__(256) qgemv_generic_kernel(QGemvArgs a) {
    const int lane = threadIdx.x & 31;
    const int bpr = a.cols / 32;
    const int wpc = blockDim.x / 32;
    for (int row = blockIdx.x * wpc + (threadIdx.x >> 5); row < a.rows; row += gridDim.x * wpc) {
        float acc[kMaxBatch];
#pragma unroll
        for (int b = 0; b < kMaxBatch; ++b) acc[b] = 0.f;
        for (int blk = lane; blk < bpr; blk += 32) {
            float scale;
            int v[32];
            load_block_generic<FMT>(a, (size_t)row, blk, bpr, scale, v);
#pragma unroll
            for (int b = 0; b < kMaxBatch; ++b) {
                if (b < a.batch) {
                    if (INT) {
                        const int8_t *xq = a.xq + (size_t)b * a.cols + blk * 32;
                        int isum = 0;
#pragma unroll
                        for (int i = 0; i < 32; ++i) isum += v[i] * (int)xq[i];
                        if (a.dots) a.dots[(size_t)row * bpr + blk] = isum;
                        acc[b] = fmaf((float)isum, scale * (a.xs ? a.xs[(size_t)b * bpr + blk] : 1.0f), acc[b]);
                    } else {
                        const float *x = a.x + (size_t)b * a.cols + blk * 32;
                        float s = 0.f;
#pragma unroll
                        for (int i = 0; i < 32; ++i) s = fmaf((float)v[i], __ldg(x + i), s);
                        acc[b] = fmaf(scale, s, acc[b]);
                    }
                }
            }
        }
        if (a.y) {
#pragma unroll
            for (int b = 0; b < kMaxBatch; ++b) {
                if (b < a.batch) {
                    float s = warp_sum(acc[b]);
                    if (lane == 0) a.y[(size_t)b * a.rows + row] = s;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Activation staging in shared memory.
//
// CPL = contiguous columns owned by one lane inside a warp-wide segment of
// 32*CPL columns.  16-byte piece k of lane l of segment s is stored at slot
// s*(32*CPL/PIECE) + k*32 + l, PIECE = columns per 16 bytes (4 floats or 16
// int8).  A warp reading "its piece k" therefore touches 32 consecutive slots.
// ---------------------------------------------------------------------------
template <int CPL, int PIECE>
__device__ __forceinline__ int permuted_slot(int col) {
    constexpr int SEG = 32 * CPL;
    int seg = col / SEG;
    int in = col - seg * SEG;
    int l = in / CPL;
    int k = (in - l * CPL) / PIECE;
    return seg * (SEG / PIECE) + k * 32 + l;
}

__host__ __device__ __forceinline__ int round_up(int v, int m) { return (v + m - 1) / m * m; }

// float mode: xs4[b * slots_per_vec + slot]
template <int CPL>
__device__ __forceinline__ void stage_x_float(float4 *xs4, const float *x, int cols, int batch, int slots_per_vec) {
    const int n4 = cols / 4;
    const bool vec_ok = (((uintptr_t)x & 15) == 0);
    for (int b = 0; b < batch; ++b) {
        const float *xb = x + (size_t)b * cols;
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            float4 v;
            if (vec_ok) {
                v = __ldg(reinterpret_cast<const float4 *>(xb) + i);
            } else {
                v.x = __ldg(xb + 4 * i);
                v.y = __ldg(xb + 4 * i + 1);
                v.z = __ldg(xb + 4 * i + 2);
                v.w = __ldg(xb + 4 * i + 3);
            }
            xs4[(size_t)b * slots_per_vec + permuted_slot<CPL, 4>(4 * i)] = v;
        }
    }
}

// int mode: xq16[b * slots_per_vec + slot] (16 int8 per slot); xq is 16-byte
// aligned by construction of the workspace.
template <int CPL>
__device__ __forceinline__ void stage_x_int(uint4 *xq16, const int8_t *xq, int cols, int batch, int slots_per_vec) {
    const int n16 = cols / 16;
    for (int b = 0; b < batch; ++b) {
        const uint4 *src = reinterpret_cast<const uint4 *>(xq + (size_t)b * cols);
        for (int i = threadIdx.x; i < n16; i += blockDim.x)
            xq16[(size_t)b * slots_per_vec + permuted_slot<CPL, 16>(16 * i)] = __ldg(src + i);
    }
}

// ---------------------------------------------------------------------------
// Family 1: split Q8_0.
// Tile = R rows x one 512-column segment per lane load (16 quants per lane).
// ---------------------------------------------------------------------------
constexpr int kQ8SThreads = 256;

template <int B, int R, bool INT, bool DOTS>
__global__ void __launch_bounds__(kQ8SThreads) q8s_gemv_kernel(QGemvArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int cols = a.cols, rows = a.rows;
    const int bpr = cols / 32;
    const int nseg = (cols + 511) / 512;
    const int lane = threadIdx.x & 31;

    // ---- stage activations -------------------------------------------------
    const int slots = nseg * (INT ? 32 : 128);  // 16-byte slots per activation vector
    float *xs_scales = nullptr;
    if (INT) {
        uint4 *xq16 = reinterpret_cast<uint4 *>(smem_raw);
        xs_scales = reinterpret_cast<float *>(smem_raw + (size_t)B * slots * 16);
        stage_x_int<16>(xq16, a.xq, cols, B, slots);
        if (!DOTS)
            for (int i = threadIdx.x; i < B * bpr; i += blockDim.x) xs_scales[i] = a.xs[i];
    } else {
        stage_x_float<16>(reinterpret_cast<float4 *>(smem_raw), a.x, cols, B, slots);
    }
    __syncthreads();

    const int wpc = kQ8SThreads / 32;
    const int ngroups = (rows + R - 1) / R;
    const int8_t *q = reinterpret_cast<const int8_t *>(a.w);

    for (int g = blockIdx.x * wpc + (threadIdx.x >> 5); g < ngroups; g += gridDim.x * wpc) {
        size_t rowi[R];
#pragma unroll
        for (int r = 0; r < R; ++r) rowi[r] = (size_t)min(g * R + r, rows - 1);
        float acc[R][B];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int b = 0; b < B; ++b) acc[r][b] = 0.f;

        // two segments per trip: 2*R independent 128-bit loads in flight per lane
        for (int seg = 0; seg < nseg; seg += 2) {
            uint4 w[2][R];
            float sc[2][R];
            bool valid[2];
            unsigned vmask[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int col0 = (seg + u) * 512 + lane * 16;
                valid[u] = (seg + u) < nseg && col0 < cols;
                vmask[u] = __ballot_sync(0xffffffffu, valid[u]);  // lanes come in whole pairs per block
                if (valid[u]) {
#pragma unroll
                    for (int r = 0; r < R; ++r) w[u][r] = ldg_stream_v4(q + rowi[r] * cols + col0);
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int col0 = (seg + u) * 512 + lane * 16;
                if (valid[u]) {
#pragma unroll
                    for (int r = 0; r < R; ++r)
                        sc[u][r] = DOTS ? 1.0f : half_bits_to_float(__ldg(a.scales + rowi[r] * bpr + (col0 >> 5)));
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (!valid[u]) continue;
                const int s = seg + u;
                const int blk = (s * 512 + lane * 16) >> 5;
                if (INT) {
                    const uint4 *xq16 = reinterpret_cast<const uint4 *>(smem_raw);
#pragma unroll
                    for (int b = 0; b < B; ++b) {
                        const uint4 xv = xq16[(size_t)b * slots + s * 32 + lane];
                        const float xscale = DOTS ? 1.0f : xs_scales[b * bpr + blk];
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            int isum = dp4a_s8(w[u][r].x, xv.x, 0);
                            isum = dp4a_s8(w[u][r].y, xv.y, isum);
                            isum = dp4a_s8(w[u][r].z, xv.z, isum);
                            isum = dp4a_s8(w[u][r].w, xv.w, isum);
                            if (DOTS) {
                                // a block is shared by two neighbouring lanes
                                int full = isum + __shfl_xor_sync(vmask[u], isum, 1);
                                if ((lane & 1) == 0 && b == 0 && g * R + r < rows) a.dots[rowi[r] * bpr + blk] = full;
                            }
                            acc[r][b] = fmaf((float)isum, sc[u][r] * xscale, acc[r][b]);
                        }
                    }
                } else {
                    const float4 *xs4 = reinterpret_cast<const float4 *>(smem_raw);
                    float part[R][B];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float wf[R][4];
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            const uint32_t word = k == 0 ? w[u][r].x : k == 1 ? w[u][r].y : k == 2 ? w[u][r].z : w[u][r].w;
                            s8x4_to_f32(word, wf[r][0], wf[r][1], wf[r][2], wf[r][3]);
                        }
#pragma unroll
                        for (int b = 0; b < B; ++b) {
                            const float4 xv = xs4[(size_t)b * slots + s * 128 + k * 32 + lane];
#pragma unroll
                            for (int r = 0; r < R; ++r) {
                                float p = k == 0 ? wf[r][0] * xv.x : fmaf(wf[r][0], xv.x, part[r][b]);
                                p = fmaf(wf[r][1], xv.y, p);
                                p = fmaf(wf[r][2], xv.z, p);
                                part[r][b] = fmaf(wf[r][3], xv.w, p);
                            }
                        }
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int b = 0; b < B; ++b) acc[r][b] = fmaf(sc[u][r], part[r][b], acc[r][b]);
                }
            }
        }
        if (a.y) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int b = 0; b < B; ++b) {
                    float s = warp_sum(acc[r][b]);
                    if (lane == 0 && g * R + r < rows) a.y[(size_t)b * rows + g * R + r] = s;
                }
        }
    }
}

// ---------------------------------------------------------------------------
// Family 2: block layouts (Q8B, Q4B) through a per-warp bulk-copy pipeline.
// ---------------------------------------------------------------------------
constexpr int kBlkWarps = 8;
constexpr int kBlkThreads = kBlkWarps * 32;
constexpr int kBlkStages = 2;
constexpr int kChunkBlocks = 64;  // blocks per row chunk = 2048 columns

template <int FMT>
struct BlkTraits {
    static constexpr int BB = FMT == FMT_Q8B ? 34 : 18;  // bytes per block
    static constexpr int PW = BB / 2;                    // 32-bit words per block pair
    static constexpr int CB = kChunkBlocks * BB;         // bytes per full row chunk
    static constexpr int QW = FMT == FMT_Q8B ? 8 : 4;    // quant words per block
};

// Pull one block pair (PW words, 4-byte aligned) out of shared memory and
// split it into the two scales and the realigned quant words of each block.
template <int FMT>
__device__ __forceinline__ void load_pair(const uint32_t *p, float (&scale)[2], uint32_t (&qa)[BlkTraits<FMT>::QW],
                                          uint32_t (&qb)[BlkTraits<FMT>::QW]) {
    constexpr int PW = BlkTraits<FMT>::PW, QW = BlkTraits<FMT>::QW;
    uint32_t wds[PW];
#pragma unroll
    for (int i = 0; i < PW; ++i) wds[i] = p[i];
    // block A: scale in the low half of word 0, quants from byte 2
    scale[0] = half_bits_to_float((uint16_t)(wds[0] & 0xFFFFu));
#pragma unroll
    for (int i = 0; i < QW; ++i) qa[i] = __byte_perm(wds[i], wds[i + 1], 0x5432);
    // block B: scale in the high half of word QW, quants in the following words
    scale[1] = half_bits_to_float((uint16_t)(wds[QW] >> 16));
#pragma unroll
    for (int i = 0; i < QW; ++i) qb[i] = wds[QW + 1 + i];
}

template <int FMT, int B, int R, bool INT, bool DOTS>
__global__ void __launch_bounds__(kBlkThreads) qblk_gemv_kernel(QGemvArgs a) {
    using T = BlkTraits<FMT>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[kBlkWarps][kBlkStages];

    const int cols = a.cols, rows = a.rows;
    const int bpr = cols / 32;
    const int nch = (bpr + kChunkBlocks - 1) / kChunkBlocks;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const size_t row_bytes = (size_t)bpr * T::BB;

    // ---- shared memory carve-up ---------------------------------------------
    // [ weight pipeline: warps x stages x R x CB ][ activations ][ activation scales ]
    unsigned char *wbuf = smem_raw + (size_t)warp * kBlkStages * R * T::CB;
    unsigned char *xbase = smem_raw + (size_t)kBlkWarps * kBlkStages * R * T::CB;
    const int slots = nch * (INT ? 128 : 512);  // 16-byte slots per activation vector
    float *xs_scales = nullptr;
    if (INT) {
        xs_scales = reinterpret_cast<float *>(xbase + (size_t)B * slots * 16);
        stage_x_int<64>(reinterpret_cast<uint4 *>(xbase), a.xq, cols, B, slots);
        if (!DOTS)
            for (int i = threadIdx.x; i < B * bpr; i += blockDim.x) xs_scales[i] = a.xs[i];
    } else {
        stage_x_float<64>(reinterpret_cast<float4 *>(xbase), a.x, cols, B, slots);
    }
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kBlkStages; ++s) mbar_init(&bars[warp][s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const int ngroups = (rows + R - 1) / R;
    const int gw = blockIdx.x * kBlkWarps + warp;
    const int gstride = gridDim.x * kBlkWarps;
    const int mine = gw < ngroups ? (ngroups - gw + gstride - 1) / gstride : 0;
    const int total = mine * nch;  // pipeline steps of this warp

    // issue step t: R bulk copies (one per row) of chunk c of group g
    auto issue = [&](int t) {
        const int gi = t / nch, c = t - gi * nch;
        const int g = gw + gi * gstride;
        const int nblk = min(kChunkBlocks, bpr - c * kChunkBlocks);
        const uint32_t bytes = (uint32_t)nblk * T::BB;
        const int st = t % kBlkStages;
        if (lane == 0) {
            mbar_expect_tx(&bars[warp][st], bytes * R);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const size_t row = (size_t)min(g * R + r, rows - 1);
                bulk_g2s_stream(wbuf + ((size_t)st * R + r) * T::CB, a.w + row * row_bytes + (size_t)c * T::CB, bytes,
                                &bars[warp][st]);
            }
        }
    };

    for (int t = 0; t < kBlkStages && t < total; ++t) issue(t);

    float acc[R][B];
    bool alive = true;
    for (int t = 0; t < total && alive; ++t) {
        const int gi = t / nch, c = t - gi * nch;
        const int g = gw + gi * gstride;
        const int st = t % kBlkStages;
        const int nblk = min(kChunkBlocks, bpr - c * kChunkBlocks);
        if (c == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int b = 0; b < B; ++b) acc[r][b] = 0.f;
        }
        alive = __all_sync(0xffffffffu, mbar_wait(&bars[warp][st], (uint32_t)((t / kBlkStages) & 1)));

        const bool active = 2 * lane < nblk;
        float scale[R][2];
        uint32_t qa[R][T::QW], qb[R][T::QW];
        if (active) {
#pragma unroll
            for (int r = 0; r < R; ++r)
                load_pair<FMT>(reinterpret_cast<const uint32_t *>(wbuf + ((size_t)st * R + r) * T::CB) + lane * T::PW,
                               scale[r], qa[r], qb[r]);
        }
        __syncwarp();
        if (t + kBlkStages < total) issue(t + kBlkStages);  // the stage is free again

        if (active) {
            const int blk0 = c * kChunkBlocks + 2 * lane;
            if (INT) {
                const uint4 *xq16 = reinterpret_cast<const uint4 *>(xbase);
#pragma unroll
                for (int b = 0; b < B; ++b) {
                    // 64 activation bytes of this lane: pieces k = 0..3
                    uint32_t xw[16];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint4 v = xq16[(size_t)b * slots + c * 128 + k * 32 + lane];
                        xw[4 * k] = v.x, xw[4 * k + 1] = v.y, xw[4 * k + 2] = v.z, xw[4 * k + 3] = v.w;
                    }
                    const float2 xsc = DOTS ? make_float2(1.f, 1.f) : *reinterpret_cast<const float2 *>(xs_scales + b * bpr + blk0);
                    int xsum[2] = {0, 0};
                    if (FMT == FMT_Q4B) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            xsum[0] = dp4a_s8(0x01010101u, xw[i], xsum[0]);
                            xsum[1] = dp4a_s8(0x01010101u, xw[8 + i], xsum[1]);
                        }
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        int d0 = 0, d1 = 0;
                        if (FMT == FMT_Q8B) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                d0 = dp4a_s8(qa[r][i], xw[i], d0);
                                d1 = dp4a_s8(qb[r][i], xw[8 + i], d1);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                d0 = dp4a_s8(qa[r][i] & 0x0F0F0F0Fu, xw[i], d0);
                                d0 = dp4a_s8((qa[r][i] >> 4) & 0x0F0F0F0Fu, xw[4 + i], d0);
                                d1 = dp4a_s8(qb[r][i] & 0x0F0F0F0Fu, xw[8 + i], d1);
                                d1 = dp4a_s8((qb[r][i] >> 4) & 0x0F0F0F0Fu, xw[12 + i], d1);
                            }
                            d0 -= 8 * xsum[0];
                            d1 -= 8 * xsum[1];
                        }
                        if (DOTS && b == 0 && g * R + r < rows) {
                            int32_t *dp = a.dots + (size_t)(g * R + r) * bpr + blk0;
                            dp[0] = d0;
                            dp[1] = d1;
                        }
                        acc[r][b] = fmaf((float)d0, scale[r][0] * xsc.x, acc[r][b]);
                        acc[r][b] = fmaf((float)d1, scale[r][1] * xsc.y, acc[r][b]);
                    }
                }
            } else {
                const float4 *xs4 = reinterpret_cast<const float4 *>(xbase);
                float part[R][B];
                // k indexes the lane's sixteen float4 activation pieces: 0..7 block A, 8..15 block B
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    float wf[R][4];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        if (FMT == FMT_Q8B) {
                            const uint32_t word = k < 8 ? qa[r][k] : qb[r][k - 8];
                            s8x4_to_f32(word, wf[r][0], wf[r][1], wf[r][2], wf[r][3]);
                        } else {
                            // elements 4j..4j+3 are the low nibbles of word j, 16+4j.. the high nibbles
                            const int kk = k & 7;
                            const uint32_t word = k < 8 ? qa[r][kk & 3] : qb[r][kk & 3];
                            const uint32_t nib = (kk < 4 ? word : (word >> 4)) & 0x0F0F0F0Fu;
                            u8x4_to_f32(nib, 8388616.0f, wf[r][0], wf[r][1], wf[r][2], wf[r][3]);
                        }
                    }
#pragma unroll
                    for (int b = 0; b < B; ++b) {
                        const float4 xv = xs4[(size_t)b * slots + c * 512 + k * 32 + lane];
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            float p = (k & 7) == 0 ? wf[r][0] * xv.x : fmaf(wf[r][0], xv.x, part[r][b]);
                            p = fmaf(wf[r][1], xv.y, p);
                            p = fmaf(wf[r][2], xv.z, p);
                            part[r][b] = fmaf(wf[r][3], xv.w, p);
                        }
                    }
                    if ((k & 7) == 7) {
#pragma unroll
                        for (int r = 0; r < R; ++r)
#pragma unroll
                            for (int b = 0; b < B; ++b) acc[r][b] = fmaf(scale[r][k >> 3], part[r][b], acc[r][b]);
                    }
                }
            }
        }
        if (c == nch - 1 && a.y) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int b = 0; b < B; ++b) {
                    float s = warp_sum(acc[r][b]);
                    if (lane == 0 && g * R + r < rows) a.y[(size_t)b * rows + g * R + r] = s;
                }
        }
    }
}

// ---------------------------------------------------------------------------
// Activation quantiser: one warp per 32-element block.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_x_kernel(const float *__restrict__ x, int8_t *__restrict__ xq,
                                                         float *__restrict__ xs, int nblocks) {
    const int lane = threadIdx.x & 31;
    const int wpc = blockDim.x / 32;
    for (int blk = blockIdx.x * wpc + (threadIdx.x >> 5); blk < nblocks; blk += gridDim.x * wpc) {
        const float v = x[(size_t)blk * 32 + lane];
        float m = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float scale = (m == 0.0f) ? 1.0f : __fdiv_rn(m, 127.0f);
        const float inv = __fdiv_rn(1.0f, scale);
        const float r = floorf(__fadd_rn(__fmul_rn(v, inv), 0.5f));
        xq[(size_t)blk * 32 + lane] = (int8_t)(int)r;
        if (lane == 0) xs[blk] = scale;
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------

// Pick a CTA count <= max_ctas that wastes the fewest warp slots in the last
// round of a grid-stride loop over `units` (row groups).
static int balanced_grid(int units, int warps_per_cta, int max_ctas) {
    int need = (units + warps_per_cta - 1) / warps_per_cta;
    if (need <= max_ctas) return need > 0 ? need : 1;
    int best = max_ctas;
    double best_eff = 0.0;
    for (int g = max_ctas; g >= (max_ctas * 3) / 4; --g) {
        long long w = (long long)g * warps_per_cta;
        long long rounds = (units + w - 1) / w;
        double eff = (double)units / (double)(rounds * w);
        if (eff > best_eff + 1e-9) {
            best_eff = eff;
            best = g;
        }
    }
    return best;
}

static int occupancy_ctas(const DeviceInfo *di, size_t smem, int cap) {
    // shared memory per SM is 228 KB, 1 KB of it reserved per resident CTA
    int by_smem = (int)((size_t)(di->max_smem_optin + 1024) / (smem + 1024));
    if (by_smem < 1) by_smem = 1;
    return by_smem < cap ? by_smem : cap;
}

template <int B, int R, bool INT, bool DOTS>
static int launch_q8s(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    const int nseg = (a.cols + 511) / 512;
    size_t smem = INT ? (size_t)B * nseg * 32 * 16 + (size_t)B * (a.cols / 32) * 4 : (size_t)B * nseg * 128 * 16;
    if (smem + 256 > (size_t)di->max_smem_optin) return TB200_ERR_INVALID_ARG;
    auto kernel = q8s_gemv_kernel<B, R, INT, DOTS>;
    int st = ensure_smem_optin(kernel, di);
    if (st) return st;
    int ctas = occupancy_ctas(di, smem, 4);
    int grid = balanced_grid((a.rows + R - 1) / R, kQ8SThreads / 32, di->sm_count * ctas);
    kernel<<<grid, kQ8SThreads, smem, s>>>(a);
    return check_launch();
}

template <int FMT, int B, int R, bool INT, bool DOTS>
static int launch_qblk(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    using T = BlkTraits<FMT>;
    const int bpr = a.cols / 32;
    const int nch = (bpr + kChunkBlocks - 1) / kChunkBlocks;
    size_t smem = (size_t)kBlkWarps * kBlkStages * R * T::CB;
    smem += INT ? (size_t)B * nch * 128 * 16 + (size_t)B * bpr * 4 : (size_t)B * nch * 512 * 16;
    if (smem + 256 > (size_t)di->max_smem_optin) return TB200_ERR_INVALID_ARG;
    auto kernel = qblk_gemv_kernel<FMT, B, R, INT, DOTS>;
    int st = ensure_smem_optin(kernel, di);
    if (st) return st;
    int ctas = occupancy_ctas(di, smem, 2);
    int grid = balanced_grid((a.rows + R - 1) / R, kBlkWarps, di->sm_count * ctas);
    kernel<<<grid, kBlkThreads, smem, s>>>(a);
    return check_launch();
}

template <int FMT, bool INT>
static int launch_generic(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    int need = (a.rows + 7) / 8;
    int grid = di->sm_count * 8 < need ? di->sm_count * 8 : need;
    qgemv_generic_kernel<FMT, INT><<<grid, 256, 0, s>>>(a);
    return check_launch();
}

// Largest batch the fast kernels can hold in shared memory next to the weight
// pipeline, for one launch.
template <int FMT, bool INT>
static int max_fast_batch(int cols, const DeviceInfo *di) {
    size_t per_vec, fixed = 0;
    if (FMT == FMT_Q8S) {
        const int nseg = (cols + 511) / 512;
        per_vec = INT ? (size_t)nseg * 512 + (size_t)(cols / 32) * 4 : (size_t)nseg * 2048;
    } else {
        const int nch = (cols / 32 + kChunkBlocks - 1) / kChunkBlocks;
        per_vec = INT ? (size_t)nch * 2048 + (size_t)(cols / 32) * 4 : (size_t)nch * 8192;
        fixed = (size_t)kBlkWarps * kBlkStages * 4 * BlkTraits<FMT == FMT_Q8S ? FMT_Q8B : FMT>::CB;
    }
    size_t room = (size_t)di->max_smem_optin > fixed + 256 ? (size_t)di->max_smem_optin - fixed - 256 : 0;
    int b = (int)(room / per_vec);
    return b > 8 ? 8 : b;
}

template <int FMT, bool INT, bool DOTS, int B>
static int launch_fast_b(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    if constexpr (FMT == FMT_Q8S) {
        return launch_q8s<B, (B <= 2 ? 4 : 2), INT, DOTS>(a, di, s);
    } else if constexpr (FMT == FMT_Q8B) {
        return launch_qblk<FMT_Q8B, B, 2, INT, DOTS>(a, di, s);
    } else {
        return launch_qblk<FMT_Q4B, B, (B <= 4 ? 4 : 2), INT, DOTS>(a, di, s);
    }
}

template <int FMT, bool INT, bool DOTS>
static int launch_fast(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    switch (a.batch) {
        case 1: return launch_fast_b<FMT, INT, DOTS, 1>(a, di, s);
        case 2: return launch_fast_b<FMT, INT, false, 2>(a, di, s);
        case 3: return launch_fast_b<FMT, INT, false, 3>(a, di, s);
        case 4: return launch_fast_b<FMT, INT, false, 4>(a, di, s);
        case 5: return launch_fast_b<FMT, INT, false, 5>(a, di, s);
        case 6: return launch_fast_b<FMT, INT, false, 6>(a, di, s);
        case 7: return launch_fast_b<FMT, INT, false, 7>(a, di, s);
        case 8: return launch_fast_b<FMT, INT, false, 8>(a, di, s);
        default: return TB200_ERR_INVALID_ARG;
    }
}

// Shared front end: validation, path choice, batch splitting.
template <int FMT, bool INT, bool DOTS>
static int qgemv_dispatch(QGemvArgs a, tb200_stream_t stream) {
    if (a.rows < 0 || a.cols < 0 || a.batch < 1 || a.batch > kMaxBatch) return TB200_ERR_INVALID_ARG;
    if (a.cols % 32 != 0) return TB200_ERR_INVALID_ARG;
    if (a.rows == 0) return TB200_OK;
    if (!a.w || (FMT == FMT_Q8S && !DOTS && !a.scales) || (!DOTS && !a.y)) return TB200_ERR_INVALID_ARG;
    if (INT ? (!a.xq || (!DOTS && !a.xs)) : !a.x) return TB200_ERR_INVALID_ARG;
    if (DOTS && !a.dots) return TB200_ERR_INVALID_ARG;
    if (FMT == FMT_Q8S && a.scales && !aligned_to(a.scales, 2)) return TB200_ERR_ALIGNMENT;
    if ((a.y && !aligned_to(a.y, 4)) || (!INT && !aligned_to(a.x, 4))) return TB200_ERR_ALIGNMENT;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    cudaStream_t s = (cudaStream_t)stream;
    if (a.cols == 0) {
        if (a.y) {
            cudaError_t e = cudaMemsetAsync(a.y, 0, sizeof(float) * (size_t)a.rows * a.batch, s);
            return (int)e;
        }
        return TB200_OK;
    }
    // fast path: rows of a whole number of 16-byte units starting on a 16-byte boundary
    const bool fast = aligned_to(a.w, 16) && (FMT == FMT_Q8S ? true : (a.cols % 256 == 0)) &&
                      (!INT || aligned_to(a.xq, 16));
    if (!fast) return launch_generic<FMT, INT>(a, di, s);
    const int maxb = max_fast_batch<FMT, INT>(a.cols, di);
    if (maxb < 1) return launch_generic<FMT, INT>(a, di, s);
    // more activation vectors than fit next to the pipeline: several passes over the weights
    int passes = (a.batch + maxb - 1) / maxb;
    int per = (a.batch + passes - 1) / passes;
    for (int b0 = 0; b0 < a.batch; b0 += per) {
        QGemvArgs p = a;
        p.batch = a.batch - b0 < per ? a.batch - b0 : per;
        if (INT) {
            p.xq = a.xq + (size_t)b0 * a.cols;
            p.xs = a.xs + (size_t)b0 * (a.cols / 32);
        } else {
            p.x = a.x + (size_t)b0 * a.cols;
        }
        if (a.y) p.y = a.y + (size_t)b0 * a.rows;
        st = launch_fast<FMT, INT, DOTS>(p, di, s);
        if (st) return st;
    }
    return TB200_OK;
}

static int split_workspace(int cols, int batch, void *workspace, size_t workspace_bytes, int8_t **xq, float **xs) {
    if (cols < 0 || cols % 32 != 0 || batch < 1 || batch > kMaxBatch) return TB200_ERR_INVALID_ARG;
    if (!workspace || workspace_bytes < tb200_qx_workspace_bytes(cols, batch)) return TB200_ERR_WORKSPACE;
    if (!aligned_to(workspace, 16)) return TB200_ERR_ALIGNMENT;
    *xq = reinterpret_cast<int8_t *>(workspace);
    *xs = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(workspace) + round_up(cols * batch, 16));
    return TB200_OK;
}

static int quantize_x(int cols, int batch, const float *x, int8_t *xq, float *xs, cudaStream_t s) {
    if (!x) return TB200_ERR_INVALID_ARG;
    if (!aligned_to(x, 4)) return TB200_ERR_ALIGNMENT;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    int nblocks = cols / 32 * batch;
    if (nblocks == 0) return TB200_OK;
    int grid = (nblocks + 7) / 8;
    if (grid > di->sm_count * 8) grid = di->sm_count * 8;
    quantize_x_kernel<<<grid, 256, 0, s>>>(x, xq, xs, nblocks);
    return check_launch();
}

template <int FMT>
static int qgemv_i8(int rows, int cols, int batch, const void *w, const uint16_t *scales, const float *x, float *y,
                    void *workspace, size_t workspace_bytes, tb200_stream_t stream) {
    int8_t *xq;
    float *xs;
    int st = split_workspace(cols, batch, workspace, workspace_bytes, &xq, &xs);
    if (st) return st;
    if (rows < 0) return TB200_ERR_INVALID_ARG;
    if (rows == 0) return TB200_OK;
    st = quantize_x(cols, batch, x, xq, xs, (cudaStream_t)stream);
    if (st) return st;
    QGemvArgs a{reinterpret_cast<const uint8_t *>(w), scales, nullptr, xq, xs, y, nullptr, rows, cols, batch};
    return qgemv_dispatch<FMT, true, false>(a, stream);
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_q8_gemv(int rows, int cols, int batch, const int8_t *q, const uint16_t *scales, const float *x,
                             float *y, tb200_stream_t stream) {
    QGemvArgs a{reinterpret_cast<const uint8_t *>(q), scales, x, nullptr, nullptr, y, nullptr, rows, cols, batch};
    return qgemv_dispatch<FMT_Q8S, false, false>(a, stream);
}

extern "C" int tb200_q8b_gemv(int rows, int cols, int batch, const uint8_t *blocks, const float *x, float *y,
                              tb200_stream_t stream) {
    if (blocks && !aligned_to(blocks, 2)) return TB200_ERR_ALIGNMENT;
    QGemvArgs a{blocks, nullptr, x, nullptr, nullptr, y, nullptr, rows, cols, batch};
    return qgemv_dispatch<FMT_Q8B, false, false>(a, stream);
}

extern "C" int tb200_q4b_gemv(int rows, int cols, int batch, const uint8_t *blocks, const float *x, float *y,
                              tb200_stream_t stream) {
    if (blocks && !aligned_to(blocks, 2)) return TB200_ERR_ALIGNMENT;
    QGemvArgs a{blocks, nullptr, x, nullptr, nullptr, y, nullptr, rows, cols, batch};
    return qgemv_dispatch<FMT_Q4B, false, false>(a, stream);
}

extern "C" size_t tb200_qx_workspace_bytes(int cols, int batch) {
    if (cols < 0 || batch < 0) return 0;
    return (size_t)round_up(cols * batch, 16) + (size_t)(cols / 32) * batch * sizeof(float);
}

extern "C" int tb200_quantize_x(int cols, int batch, const float *x, void *workspace, size_t workspace_bytes,
                                tb200_stream_t stream) {
    int8_t *xq;
    float *xs;
    int st = split_workspace(cols, batch, workspace, workspace_bytes, &xq, &xs);
    if (st) return st;
    return quantize_x(cols, batch, x, xq, xs, (cudaStream_t)stream);
}

extern "C" int tb200_q8_gemv_i8(int rows, int cols, int batch, const int8_t *q, const uint16_t *scales,
                                const float *x, float *y, void *workspace, size_t workspace_bytes,
                                tb200_stream_t stream) {
    return qgemv_i8<FMT_Q8S>(rows, cols, batch, q, scales, x, y, workspace, workspace_bytes, stream);
}

extern "C" int tb200_q8b_gemv_i8(int rows, int cols, int batch, const uint8_t *blocks, const float *x, float *y,
                                 void *workspace, size_t workspace_bytes, tb200_stream_t stream) {
    if (blocks && !aligned_to(blocks, 2)) return TB200_ERR_ALIGNMENT;
    return qgemv_i8<FMT_Q8B>(rows, cols, batch, blocks, nullptr, x, y, workspace, workspace_bytes, stream);
}

extern "C" int tb200_q4b_gemv_i8(int rows, int cols, int batch, const uint8_t *blocks, const float *x, float *y,
                                 void *workspace, size_t workspace_bytes, tb200_stream_t stream) {
    if (blocks && !aligned_to(blocks, 2)) return TB200_ERR_ALIGNMENT;
    return qgemv_i8<FMT_Q4B>(rows, cols, batch, blocks, nullptr, x, y, workspace, workspace_bytes, stream);
}

// The block-dot entries take an already quantised activation vector and write
// only `dots`: scales do not enter an integer dot, so none are passed.
template <int FMT>
static int blockdots(int rows, int cols, const void *w, const int8_t *xq, int32_t *dots, tb200_stream_t stream) {
    QGemvArgs a{reinterpret_cast<const uint8_t *>(w), nullptr, nullptr, xq, nullptr, nullptr, dots, rows, cols, 1};
    return qgemv_dispatch<FMT, true, true>(a, stream);
}

extern "C" int tb200_q8_blockdots_i32(int rows, int cols, const int8_t *q, const int8_t *xq, int32_t *dots,
                                      tb200_stream_t stream) {
    return blockdots<FMT_Q8S>(rows, cols, q, xq, dots, stream);
}

extern "C" int tb200_q8b_blockdots_i32(int rows, int cols, const uint8_t *blocks, const int8_t *xq, int32_t *dots,
                                       tb200_stream_t stream) {
    return blockdots<FMT_Q8B>(rows, cols, blocks, xq, dots, stream);
}

extern "C" int tb200_q4b_blockdots_i32(int rows, int cols, const uint8_t *blocks, const int8_t *xq, int32_t *dots,
                                       tb200_stream_t stream) {
    return blockdots<FMT_Q4B>(rows, cols, blocks, xq, dots, stream);
}
