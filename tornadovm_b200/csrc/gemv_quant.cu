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
//   q8s_gemv_kernel   split layout, 16-byte aligned weights: per-lane cp.async rings.
//   qblk_gemv_kernel  block layouts when cols % 256 == 0 and the weights are
//                     16-byte aligned: per-warp cp.async rings, block pairs
//                     decoded from shared memory.
//                     Both keep the bytes in flight in shared memory, not in
//                     registers, and the integer mode can quantise the
//                     activations in the kernel's own prologue.
//   q*_generic_kernel any alignment and any cols % 32 == 0; byte loads.
//
// Activations are staged once per CTA in shared memory in a lane-interleaved
// order, so that the 128-bit shared loads of a warp touch consecutive 16-byte
// slots (no bank conflicts).
//
// Algorithmic bytes per launch:
//   Q8: 34 * rows*cols/32 + 4*batch*(cols + rows)
//   Q4: 18 * rows*cols/32 + 4*batch*(cols + rows)
#include <type_traits>

#define TB200_OP_CLASS TB200_PREPARE_GEMV_QUANT
#include "gemv_common.cuh"

TB200_TU_STATUS(gemv_quant)

namespace tb200 {

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

// Integer activations into shared memory.  Eight consecutive threads share a
// 32-element block, four elements each: quantise on the fly (QUANTIZE) or copy
// the workspace's int8 values; write the four bytes to their lane-interleaved
// slot, the block's fp32 scale, and the block's int32 sum (Q4_0 needs sum(xq)
// for the "- 8" of its nibbles).
template <int CPL, bool QUANTIZE, bool WANT_SUM>
__device__ __forceinline__ void stage_x_blocks(unsigned char *xq_smem, float *xs_smem, int *xsum_smem,
                                               const QGemvArgs &a, int batch, int slots_per_vec, bool want_scales) {
    const int total4 = batch * a.cols / 4;  // groups of four elements, all vectors back to back
    const bool x_vec = QUANTIZE && (((uintptr_t)a.x & 15) == 0);
    const bool q_vec = !QUANTIZE && (((uintptr_t)a.xq & 3) == 0);
    const int lane = threadIdx.x & 31;
    constexpr int T = 4;  // trips whose global loads are issued together
    // blockDim.x is a multiple of 32 and a.cols of 32: the eight threads of a block sit in one warp and
    // take the same trips; trip counts are warp-uniform
    for (int base = threadIdx.x & ~31; base < total4; base += T * blockDim.x) {
        float4 v[T];
        uint32_t qw[T];
        float sc[T];
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const int i4 = base + t * blockDim.x + lane;
            v[t] = make_float4(0.f, 0.f, 0.f, 0.f), qw[t] = 0, sc[t] = 1.0f;
            if (i4 < total4) {
                const int flat = i4 * 4;
                if (QUANTIZE) {
                    if (x_vec) {
                        v[t] = __ldg(reinterpret_cast<const float4 *>(a.x + flat));
                    } else {
                        v[t].x = __ldg(a.x + flat), v[t].y = __ldg(a.x + flat + 1);
                        v[t].z = __ldg(a.x + flat + 2), v[t].w = __ldg(a.x + flat + 3);
                    }
                } else {
                    if (q_vec) {
                        qw[t] = __ldg(reinterpret_cast<const uint32_t *>(a.xq + flat));
                    } else {
                        qw[t] = (uint32_t)(uint8_t)a.xq[flat] | ((uint32_t)(uint8_t)a.xq[flat + 1] << 8) |
                                ((uint32_t)(uint8_t)a.xq[flat + 2] << 16) | ((uint32_t)(uint8_t)a.xq[flat + 3] << 24);
                    }
                    if (want_scales) sc[t] = a.xs[flat >> 5];
                }
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const int i4 = base + t * blockDim.x + lane;
            const unsigned mask = __ballot_sync(0xffffffffu, i4 < total4);  // whole groups of eight lanes
            if (i4 >= total4) continue;
            const int flat = i4 * 4;
            const int b = flat / a.cols, col = flat - b * a.cols;
            const int blk_flat = flat >> 5;  // == b * (cols / 32) + col / 32
            uint32_t packed = qw[t];
            float scale = sc[t];
            if (QUANTIZE) {
                float m = fmaxf(fmaxf(fabsf(v[t].x), fabsf(v[t].y)), fmaxf(fabsf(v[t].z), fabsf(v[t].w)));
                m = fmaxf(m, __shfl_xor_sync(mask, m, 1));
                m = fmaxf(m, __shfl_xor_sync(mask, m, 2));
                m = fmaxf(m, __shfl_xor_sync(mask, m, 4));
                scale = (m == 0.0f) ? 1.0f : __fdiv_rn(m, 127.0f);
                const float inv = __fdiv_rn(1.0f, scale);
                packed = quantize_byte(v[t].x, inv) | (quantize_byte(v[t].y, inv) << 8) | (quantize_byte(v[t].z, inv) << 16) |
                         (quantize_byte(v[t].w, inv) << 24);
            }
            *reinterpret_cast<uint32_t *>(xq_smem + ((size_t)b * slots_per_vec + permuted_slot<CPL, 16>(col)) * 16 + (col & 15)) = packed;
            if (WANT_SUM) {
                int sum = dp4a_s8(packed, 0x01010101u, 0);
                sum += __shfl_xor_sync(mask, sum, 1);
                sum += __shfl_xor_sync(mask, sum, 2);
                sum += __shfl_xor_sync(mask, sum, 4);
                if ((lane & 7) == 0) xsum_smem[blk_flat] = sum;
            }
            if (want_scales && (lane & 7) == 0) xs_smem[blk_flat] = scale;
        }
    }
}

// ---------------------------------------------------------------------------
// Family 1: split Q8_0 through per-lane cp.async rings.
//
// A CTA owns a contiguous range of rows and each of its warps a contiguous run
// of row groups (R rows).  A ring stage holds one trip of one group: U segments
// of 512 columns, i.e. R*U 16-byte pieces (16 quants each) per lane.  A lane
// copies its pieces into its own slots of the warp's shared-memory ring with
// cp.async and keeps STAGES stages in flight: no registers are held while the
// bytes travel and no cross-lane synchronisation is needed, because a lane
// reads back only what it copied.  The fp16 scales ride in registers.  Rows
// longer than one trip are accumulated in registers by the same warp, so a
// row's sum never depends on warp timing.
// ---------------------------------------------------------------------------
constexpr int kQ8SThreads = 256;
constexpr int kQ8SWarps = kQ8SThreads / 32;

// SA: the scales of a trip are 16-byte aligned runs and travel through the ring as well (cols % 256 == 0,
// 16-byte aligned scale array); otherwise they are loaded into registers when the trip is requested.
template <int B, int R, int U, int MODE, bool DOTS, int STAGES, bool SA>
__global__ void __launch_bounds__(kQ8SThreads) q8s_gemv_kernel(QGemvArgs a) {
    constexpr bool INT = MODE != MODE_FLOAT;
    static_assert(STAGES >= 2 && STAGES <= 4, "ring depth");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int cols = a.cols;
    const int bpr = cols / 32;
    const int nseg = (cols + 511) / 512;
    const int ntrips = (nseg + U - 1) / U;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int8_t *q = reinterpret_cast<const int8_t *>(a.w);

    // rows of the CTA, row groups of the warp
    const int row_begin = (int)((long long)a.rows * blockIdx.x / gridDim.x);
    const int row_end = (int)((long long)a.rows * (blockIdx.x + 1) / gridDim.x);
    const int ngroups = (row_end - row_begin + R - 1) / R;
    const int g_begin = ngroups * warp / kQ8SWarps, g_end = ngroups * (warp + 1) / kQ8SWarps;

    // ---- shared memory: [ activations ][ activation scales ][ rings: warps x stages x R x U x 512 ] ----
    const int slots = nseg * (INT ? 32 : 128);  // 16-byte slots per activation vector
    float *xs_scales = reinterpret_cast<float *>(smem_raw + (size_t)B * slots * 16);
    const uint32_t ring_off = (uint32_t)(((size_t)B * slots * 16 + (size_t)(INT ? B * bpr : 0) * 4 + 127) & ~(size_t)127);
    constexpr int REC = U * 512 + (SA ? U * 32 : 0);  // bytes per row and stage: quants, then the trip's scales
    unsigned char *ring = smem_raw + ring_off + (size_t)warp * STAGES * R * REC + lane * 16;
    const uint32_t ring_s = smem_u32(ring);

    // ---- issue side ----------------------------------------------------------------
    uint16_t sc[SA ? 1 : STAGES][R][U];
    int ig = g_begin, itrip = 0;  // next (group, trip) to request
    auto issue = [&](auto stage_c) {
        constexpr int st = decltype(stage_c)::value;
        if (ig < g_end) {
            const int colbase = itrip * (U * 512) + lane * 16;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const size_t row = (size_t)min(row_begin + ig * R + r, row_end - 1);
                const int8_t *qrow = q + row * cols + colbase;
                const uint16_t *srow = a.scales + row * bpr + (colbase >> 5);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (colbase + u * 512 < cols) {
                        cp_async_16(ring_s + (st * R + r) * REC + u * 512, qrow + u * 512);
                        if (!DOTS && !SA) sc[SA ? 0 : st][r][u] = __ldg(srow + u * 16);
                    }
                }
                if (SA && !DOTS) {
                    // the trip's U*16 scales: 16-byte pieces of eight, copied by the first lanes
                    const int blk = itrip * (U * 16) + lane * 8;
                    if (lane < U * 2 && blk < bpr)
                        cp_async_16(ring_s + (st * R + r) * REC + U * 512, a.scales + row * bpr + blk);
                }
            }
            if (++itrip == ntrips) itrip = 0, ++ig;
        }
        cp_async_commit();
    };

    // ring primed before anything else: weights do not depend on the predecessor kernel
    issue(std::integral_constant<int, 0>{});
    issue(std::integral_constant<int, 1>{});
    if (STAGES > 2) issue(std::integral_constant<int, 2 % STAGES>{});
    if (STAGES > 3) issue(std::integral_constant<int, 3 % STAGES>{});

    // dependents may start (they only prefetch weights); activations and outputs wait for the predecessor
    pdl_launch_dependents();
    pdl_wait();

    if (MODE == MODE_FLOAT) {
        stage_x_float<16>(reinterpret_cast<float4 *>(smem_raw), a.x, cols, B, slots);
    } else if (MODE == MODE_INT_FUSED) {
        stage_x_blocks<16, true, false>(smem_raw, xs_scales, nullptr, a, B, slots, true);
    } else {
        stage_x_blocks<16, false, false>(smem_raw, xs_scales, nullptr, a, B, slots, !DOTS);
    }
    __syncthreads();

    // ---- consume side ----------------------------------------------------------------
    float acc[R][B];
    int cg = g_begin, ctrip = 0;
    auto consume = [&](auto stage_c) {
        constexpr int st = decltype(stage_c)::value;
        const int row0 = row_begin + cg * R;
        if (ctrip == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int b = 0; b < B; ++b) acc[r][b] = 0.f;
        }
        const int colbase = ctrip * (U * 512) + lane * 16;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int col0 = colbase + u * 512;
            const bool valid = col0 < cols;
            const unsigned vmask = __ballot_sync(0xffffffffu, valid);  // lanes come in whole pairs per block
            if (!valid) continue;
            const int piece = col0 >> 4;  // 16-column piece index within the row
            uint4 w[R];
#pragma unroll
            for (int r = 0; r < R; ++r) w[r] = *reinterpret_cast<const uint4 *>(ring + (st * R + r) * REC + u * 512);
            float wsc[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (DOTS) wsc[r] = 1.0f;
                else if (SA) wsc[r] = half_bits_to_float(*reinterpret_cast<const uint16_t *>(
                    ring - lane * 16 + (st * R + r) * REC + U * 512 + (u * 16 + (lane >> 1)) * 2));
                else wsc[r] = half_bits_to_float(sc[SA ? 0 : st][r][u]);
            }
            if (INT) {
                const uint4 *xq16 = reinterpret_cast<const uint4 *>(smem_raw);
#pragma unroll
                for (int b = 0; b < B; ++b) {
                    const uint4 xv = xq16[b * slots + piece];
                    const float xscale = DOTS ? 1.0f : xs_scales[b * bpr + (piece >> 1)];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        int isum = dp4a_s8(w[r].x, xv.x, 0);
                        isum = dp4a_s8(w[r].y, xv.y, isum);
                        isum = dp4a_s8(w[r].z, xv.z, isum);
                        isum = dp4a_s8(w[r].w, xv.w, isum);
                        if (DOTS) {
                            const int full = isum + __shfl_xor_sync(vmask, isum, 1);  // a block spans two lanes
                            if ((lane & 1) == 0 && b == 0 && row0 + r < row_end)
                                a.dots[(size_t)(row0 + r) * bpr + (piece >> 1)] = full;
                        }
                        acc[r][b] = fmaf((float)isum, wsc[r] * xscale, acc[r][b]);
                    }
                }
            } else {
                const float4 *xs4 = reinterpret_cast<const float4 *>(smem_raw);
                const int seg = piece >> 5;  // 512-column segment
                float p[R][B];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float wf[R][4];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const uint32_t word = k == 0 ? w[r].x : k == 1 ? w[r].y : k == 2 ? w[r].z : w[r].w;
                        s8x4_to_f32(word, wf[r][0], wf[r][1], wf[r][2], wf[r][3]);
                    }
#pragma unroll
                    for (int b = 0; b < B; ++b) {
                        const float4 xv = xs4[b * slots + seg * 128 + k * 32 + lane];
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            float t = k == 0 ? wf[r][0] * xv.x : fmaf(wf[r][0], xv.x, p[r][b]);
                            t = fmaf(wf[r][1], xv.y, t);
                            t = fmaf(wf[r][2], xv.z, t);
                            p[r][b] = fmaf(wf[r][3], xv.w, t);
                        }
                    }
                }
#pragma unroll
                for (int r = 0; r < R; ++r) {
#pragma unroll
                    for (int b = 0; b < B; ++b) acc[r][b] = fmaf(wsc[r], p[r][b], acc[r][b]);
                }
            }
        }
        if (++ctrip == ntrips) {
            ctrip = 0;
            if (!DOTS) {
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int b = 0; b < B; ++b) {
                        const float s = warp_sum(acc[r][b]);
                        if (lane == 0 && row0 + r < row_end) a.y[(size_t)b * a.rows + row0 + r] = s;
                    }
            }
            ++cg;
        }
    };

    // With SA a lane reads scales that other lanes copied: the warp synchronises after the wait and
    // again before the stage is requested anew.
    auto step = [&](auto stage_c) {
        cp_async_wait<STAGES - 1>();
        if (SA) __syncwarp();
        consume(stage_c);
        if (SA) __syncwarp();
        issue(stage_c);
    };
    while (cg < g_end) {
        step(std::integral_constant<int, 0>{});
        if (cg >= g_end) break;
        step(std::integral_constant<int, 1>{});
        if (STAGES > 2) {
            if (cg >= g_end) break;
            step(std::integral_constant<int, 2 % STAGES>{});
        }
        if (STAGES > 3) {
            if (cg >= g_end) break;
            step(std::integral_constant<int, 3 % STAGES>{});
        }
    }
    cp_async_wait<0>();
}

// ---------------------------------------------------------------------------
// Family 2: block layouts (Q8B 34-byte, Q4B 18-byte blocks) through per-warp
// cp.async rings.
//
// A CTA owns a contiguous range of rows and each of its warps a contiguous run
// of row groups (R rows).  A ring stage holds one chunk of 128 blocks (4096
// columns) of the R rows: the lanes copy it as consecutive 16-byte pieces
// (coalesced cp.async, no registers held while the bytes travel), STAGES chunks
// are in flight per warp.  Blocks are 2-byte aligned records, so after the
// copies of a stage have landed (cp.async.wait_group + __syncwarp) a lane
// decodes whole block *pairs* -- 4-byte aligned records of 68 / 36 bytes read
// with conflict-free 32-bit shared loads -- pairs `lane` and `lane + 32`.
// ---------------------------------------------------------------------------
constexpr int kChunkBlocks = 128;  // blocks per row chunk = 4096 columns

template <int FMT>
struct RingTraits {
    static constexpr int BB = FMT == FMT_Q4B ? 18 : 34;   // bytes per block
    static constexpr int PW = BB / 2;                     // 32-bit words per block pair
    static constexpr int CB = kChunkBlocks * BB;          // bytes per full row chunk (4352 / 2304)
    static constexpr int QW = FMT == FMT_Q4B ? 4 : 8;     // quant words per block
    static constexpr int CPL = 64;                        // contiguous columns per lane and pair
    static constexpr int PIECES = (CB / 16 + 31) / 32;    // 16-byte pieces per lane and row chunk (9 / 5)
};

// Pull one block pair (PW words, 4-byte aligned) out of shared memory and
// split it into the two scales and the realigned quant words of each block.
template <int FMT>
__device__ __forceinline__ void load_pair(const uint32_t *p, float (&scale)[2], uint32_t (&qa)[RingTraits<FMT>::QW],
                                          uint32_t (&qb)[RingTraits<FMT>::QW]) {
    constexpr int PW = RingTraits<FMT>::PW, QW = RingTraits<FMT>::QW;
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

template <int FMT, int B, int R, int MODE, bool DOTS, int STAGES, bool GROUPED, int SHR>
__device__ __forceinline__ void qblk_gemv_body(const QGemvArgs a, const QGroupArgs *grp) {
    // GROUPED: a.rows counts the rows of all matrices laid end to end; a.w and a.y are unused
    using T = RingTraits<FMT>;
    constexpr bool INT = MODE != MODE_FLOAT;
    static_assert(STAGES >= 2 && STAGES <= 4, "ring depth");
    static_assert(T::PIECES * 32 * 16 >= T::CB + 128 && T::CB % 128 == 0, "a shifted chunk starts up to 120 bytes into its slot");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int cols = a.cols;
    const int bpr = cols / 32;
    const int nch = (bpr + kChunkBlocks - 1) / kChunkBlocks;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t row_bytes = (size_t)bpr * T::BB;

    const int row_begin = (int)((long long)a.rows * blockIdx.x / gridDim.x);
    const int row_end = (int)((long long)a.rows * (blockIdx.x + 1) / gridDim.x);
    const int ngroups = (row_end - row_begin + R - 1) / R;
    const int g_begin = ngroups * warp / kQ8SWarps, g_end = ngroups * (warp + 1) / kQ8SWarps;

    // ---- shared memory: [ activations ][ scales ][ block sums ][ rings: warps x stages x R x CB ] ----
    const int slots = (cols + 2047) / 2048 * 2048 / (INT ? 16 : 4);  // 16-byte slots per activation vector
    float *xs_scales = reinterpret_cast<float *>(smem_raw + (size_t)B * slots * 16);
    int *xsum = reinterpret_cast<int *>(xs_scales + B * bpr);
    const uint32_t ring_off = (uint32_t)(((size_t)B * slots * 16 + (size_t)(INT ? B * bpr : 0) * 8 + 127) & ~(size_t)127);
    // SHR: ring slots are 128 bytes longer and a chunk starts a.wshift bytes into its slot (see below)
    constexpr int CBS = SHR ? T::CB + 128 : T::CB;
    unsigned char *ring = smem_raw + ring_off + (size_t)warp * STAGES * R * CBS;
    const uint32_t ring_s = smem_u32(ring);
    // SHR: every row chunk starts a.wshift bytes (a multiple of 8 below 128) past a 128-byte boundary -- weights behind
    // an array header of 16 or 24 bytes in a 256-byte aligned buffer.  A warp's 32 pieces of 16 bytes then would span
    // five 128-byte lines instead of four (measured: 12-17 % more time per launch).  The chunk therefore keeps its
    // phase inside the ring slot: the pieces are the aligned 16-byte units of the lines that hold the chunk, the ones
    // wholly outside it are skipped and, at an 8-byte phase (SHR == 2), the first and last travel as 8-byte copies.
    // Template parameters: the aligned form keeps its slots and its instruction count, and the 16-byte phases do not
    // carry the 8-byte copies (the Q4_0 kernels are bound by their instruction count).
    const uint32_t wsh = SHR ? (uint32_t)a.wshift : 0u;

    // ---- issue side ------------------------------------------------------------------
    int ig = g_begin, ich = 0;
    int im = 0;  // GROUPED: matrix of the first row of the group being requested; groups only move forward
    auto issue = [&](int st) {
        if (ig < g_end) {
            const int nblk = min(kChunkBlocks, bpr - ich * kChunkBlocks);
            const int npieces = nblk * T::BB / 16;  // nblk is a multiple of 8: whole 16-byte pieces
            // SHR: the chunk's bytes are [wsh, hi) of its slot
            const uint32_t hi = wsh + 16u * npieces, lo_up = (wsh + 15u) & ~15u;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int vrow = min(row_begin + ig * R + r, row_end - 1);
                const unsigned char *src;  // this lane's first piece; SHR: counted from the boundary below the chunk
                if constexpr (GROUPED) {
                    int m = im;
                    while (vrow >= grp->row_start[m + 1]) ++m;  // vrow < row_start[count]
                    if (r == 0) im = m;  // the later chunks of this group start from its first row again
                    src = grp->w[m] + (size_t)(vrow - grp->row_start[m]) * row_bytes + (size_t)ich * T::CB + lane * 16 - wsh;
                } else {
                    src = a.w + (size_t)vrow * row_bytes + (size_t)ich * T::CB + lane * 16 - wsh;
                }
                const uint32_t dst = ring_s + (st * R + r) * CBS + lane * 16;
                if constexpr (!SHR) {
#pragma unroll
                    for (int i = 0; i < T::PIECES; ++i)
                        if (lane + 32 * i < npieces) cp_async_16(dst + i * 512, src + i * 512);
                } else if constexpr (SHR == 1) {
#pragma unroll
                    for (int i = 0; i < T::PIECES; ++i) {
                        // the chunk starts inside the first 128 bytes of its slot: only the first round of pieces can
                        // lie in front of it (the later rounds keep the aligned form's single comparison)
                        const uint32_t p = (uint32_t)(lane + 32 * i) * 16u;
                        if ((i > 0 || p >= wsh) && p < hi) cp_async_16(dst + i * 512, src + i * 512);
                    }
                } else {
                    // 8-byte phase: the chunk begins and ends in the middle of a piece.  Its first and last 8 bytes
                    // travel as 8-byte copies, both in ONE instruction of lanes 0 and 1 (a comparison in every round
                    // of pieces instead cost the Q4_0 kernel, which is bound by its instruction count, 20 %)
                    const uint32_t hi_dn = hi - 8u;
#pragma unroll
                    for (int i = 0; i < T::PIECES; ++i) {
                        const uint32_t p = (uint32_t)(lane + 32 * i) * 16u;
                        if ((i > 0 || p >= lo_up) && p < hi_dn) cp_async_16(dst + i * 512, src + i * 512);
                    }
                    if (lane < 2) {
                        const uint32_t at = lane ? hi_dn : wsh;  // offset of the 8 bytes from the line below the chunk
                        cp_async_8(dst - lane * 16 + at, src - lane * 16 + at);
                    }
                }
            }
            if (++ich == nch) ich = 0, ++ig;
        }
        cp_async_commit();
    };
#pragma unroll
    for (int st = 0; st < STAGES; ++st) issue(st);

    pdl_launch_dependents();
    pdl_wait();  // weights were requested above; activations and outputs wait for the predecessor

    unsigned step = 0;
    if constexpr (GROUPED) {
        if (grp->flags[0]) {
            // sync[0] = s steps of this GPU are complete (all their stores performed: the launches before this one
            // have finished).  The first CTA tells every GPU so; then, before step s stores into the slot that
            // held step s - nslots, every GPU must be done reading that slot, i.e. must have started its step
            // s - nslots + 1, which is when it announced that count (bounded wait).  With two slots this holds
            // GPUs within a step of one another; a third slot gives a further step of slack.
            step = *reinterpret_cast<const volatile unsigned *>(grp->sync);
            if ((grp->handshake & 1) && warp == 0 && lane < grp->npeers) {
                if (blockIdx.x == 0) {
                    __threadfence_system();
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(grp->flags[lane] + grp->rank), "r"(step) : "memory");
                }
                if (lane != grp->rank)
                    wait_flag_at_least(grp->flags[grp->rank] + lane, step - (unsigned)(grp->nslots - 1), grp->timeout_ns);
            }
            // the other warps go on staging the activations; the barrier below joins them
        }
    }

    if (MODE == MODE_FLOAT) {
        stage_x_float<T::CPL>(reinterpret_cast<float4 *>(smem_raw), a.x, cols, B, slots);
    } else if (MODE == MODE_INT_FUSED) {
        stage_x_blocks<T::CPL, true, FMT == FMT_Q4B>(smem_raw, xs_scales, xsum, a, B, slots, true);
    } else {
        stage_x_blocks<T::CPL, false, FMT == FMT_Q4B>(smem_raw, xs_scales, xsum, a, B, slots, !DOTS);
    }
    __syncthreads();

    // ---- consume side ------------------------------------------------------------------
    float acc[R][B];
    // GROUPED: results wait in registers (lane k holds the k-th pending row) until kGroupFlushRows consecutive rows
    // of one matrix are complete, so that every destination -- peers over NVLink included -- gets whole sectors
    float pend[B];
    int pcnt = 0, pbase = 0, cm = 0;
    size_t half = 0;
    if constexpr (GROUPED) {
        // the step counter was advanced by a kernel that completed before pdl_wait() returned
        if (grp->flags[0]) half = (size_t)(step % (unsigned)grp->nslots) * grp->half_stride;
        else if (grp->epoch) half = (size_t)(*reinterpret_cast<const volatile unsigned *>(grp->epoch) & 1u) * grp->half_stride;
    }
    const int warp_row_end = min(row_begin + g_end * R, row_end);
    int cg = g_begin, cch = 0, st = 0;
    while (cg < g_end) {
        cp_async_wait<STAGES - 1>();
        __syncwarp();  // every lane's pieces of this stage have landed
        const int c = cch;
        const int nblk = min(kChunkBlocks, bpr - c * kChunkBlocks);
        const int row0 = row_begin + cg * R;
        if (c == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int b = 0; b < B; ++b) acc[r][b] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int pair = lane + 32 * j;
            if (2 * pair >= nblk) continue;
            const int blk0 = c * kChunkBlocks + 2 * pair;
            const int seg = c * 2 + j;  // 2048-column activation segment of this pair
            float scale[R][2];
            uint32_t qa[R][T::QW], qb[R][T::QW];
#pragma unroll
            for (int r = 0; r < R; ++r)
                load_pair<FMT>(reinterpret_cast<const uint32_t *>(ring + (st * R + r) * CBS + wsh) + pair * T::PW, scale[r], qa[r], qb[r]);
            if (INT) {
                const uint4 *xq16 = reinterpret_cast<const uint4 *>(smem_raw);
#pragma unroll
                for (int b = 0; b < B; ++b) {
                    uint32_t xw[16];  // the pair's 64 activation bytes: pieces k = 0..3
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint4 v = xq16[b * slots + seg * 128 + k * 32 + lane];
                        xw[4 * k] = v.x, xw[4 * k + 1] = v.y, xw[4 * k + 2] = v.z, xw[4 * k + 3] = v.w;
                    }
                    const float2 xsc = DOTS ? make_float2(1.f, 1.f) : *reinterpret_cast<const float2 *>(xs_scales + b * bpr + blk0);
                    int2 xsm = make_int2(0, 0);
                    if (FMT == FMT_Q4B) xsm = *reinterpret_cast<const int2 *>(xsum + b * bpr + blk0);
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
                            // high nibbles stay where they are: as unsigned bytes they are 16 x the nibble, so their
                            // dot is a multiple of 16 and the shift below is exact (saves a shift per word)
                            int h0 = 0, h1 = 0;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                d0 = dp4a_s8(qa[r][i] & 0x0F0F0F0Fu, xw[i], d0);
                                h0 = dp4a_u8s8(qa[r][i] & 0xF0F0F0F0u, xw[4 + i], h0);
                                d1 = dp4a_s8(qb[r][i] & 0x0F0F0F0Fu, xw[8 + i], d1);
                                h1 = dp4a_u8s8(qb[r][i] & 0xF0F0F0F0u, xw[12 + i], h1);
                            }
                            d0 += (h0 >> 4) - 8 * xsm.x;
                            d1 += (h1 >> 4) - 8 * xsm.y;
                        }
                        if (DOTS && b == 0 && row0 + r < row_end) {
                            int32_t *dp = a.dots + (size_t)(row0 + r) * bpr + blk0;
                            dp[0] = d0;
                            dp[1] = d1;
                        }
                        acc[r][b] = fmaf((float)d0, scale[r][0] * xsc.x, acc[r][b]);
                        acc[r][b] = fmaf((float)d1, scale[r][1] * xsc.y, acc[r][b]);
                    }
                }
            } else {
                const float4 *xs4 = reinterpret_cast<const float4 *>(smem_raw);
                float part[R][B];
                // k indexes the pair's sixteen float4 activation pieces: 0..7 block A, 8..15 block B
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    float wf[R][4];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        if (FMT == FMT_Q8B) {
                            const uint32_t word = k < 8 ? qa[r][k & 7] : qb[r][k & 7];
                            s8x4_to_f32(word, wf[r][0], wf[r][1], wf[r][2], wf[r][3]);
                        } else {
                            // elements 4i..4i+3 are the low nibbles of word i, 16+4i.. the high nibbles
                            const int kk = k & 7;
                            const uint32_t word = k < 8 ? qa[r][kk & 3] : qb[r][kk & 3];
                            const uint32_t nib = (kk < 4 ? word : (word >> 4)) & 0x0F0F0F0Fu;
                            u8x4_to_f32(nib, 8388616.0f, wf[r][0], wf[r][1], wf[r][2], wf[r][3]);
                        }
                    }
#pragma unroll
                    for (int b = 0; b < B; ++b) {
                        const float4 xv = xs4[b * slots + seg * 512 + k * 32 + lane];
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
        __syncwarp();  // every lane is done with this stage before it is refilled
        issue(st);
        st = st + 1 == STAGES ? 0 : st + 1;
        if (++cch == nch) {
            cch = 0;
            if constexpr (GROUPED) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int vrow = row0 + r;
                    if (vrow < row_end) {  // warp-uniform
                        if (pcnt == 0) pbase = vrow;
#pragma unroll
                        for (int b = 0; b < B; ++b) {
                            const float s = warp_sum(acc[r][b]);
                            if (lane == pcnt) pend[b] = s;
                        }
                        ++pcnt;
                        while (pbase >= grp->row_start[cm + 1]) ++cm;  // matrix of the pending run
                        if (pcnt == kGroupFlushRows || vrow + 1 == warp_row_end || vrow + 1 == grp->row_start[cm + 1]) {
                            const long long at = (long long)half + grp->out_off[cm] + grp->row_off[cm] + (pbase - grp->row_start[cm]) + lane;
                            const size_t ld = (size_t)grp->ld[cm];
                            if (lane < pcnt) {
                                for (int i = 0; i < grp->npeers; ++i) {
                                    // start with this GPU's own buffer and go round: at any moment the GPUs of a
                                    // group then store to different destinations instead of all to the same one
                                    int p = grp->rank + i;
                                    p = p >= grp->npeers ? p - grp->npeers : p;
                                    float *d = grp->dst[p] + at;  // this GPU's buffer or a peer-mapped one: plain stores
#pragma unroll
                                    for (int b = 0; b < B; ++b) d[b * ld] = pend[b];
                                }
                            }
                            pcnt = 0;
                        }
                    }
                }
            } else if (a.y) {
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int b = 0; b < B; ++b) {
                        const float s = warp_sum(acc[r][b]);
                        if (lane == 0 && row0 + r < row_end) a.y[(size_t)b * a.rows + row0 + r] = s;
                    }
            }
            ++cg;
        }
    }
    cp_async_wait<0>();
    if constexpr (GROUPED) {
        if (grp->flags[0] && (grp->handshake & 2)) {
            // The CTA that finishes last advances the step counter (local memory only: the launch that follows,
            // or tb200_peer_wait, announces it to the other GPUs once this launch has completed).
            __syncthreads();
            if (threadIdx.x == 0) {
                const unsigned done = atomicAdd(grp->sync + 1, 1u);
                if (done == gridDim.x - 1) {
                    grp->sync[1] = 0;  // ready for the next launch
                    grp->sync[0] = step + 1;
                }
            }
        }
    }
}

template <int FMT, int B, int R, int MODE, bool DOTS, int STAGES, int SHR = 0>
__global__ void __launch_bounds__(kQ8SThreads) qblk_gemv_kernel(QGemvArgs a) {
    qblk_gemv_body<FMT, B, R, MODE, DOTS, STAGES, false, SHR>(a, nullptr);
}

template <int FMT, int B, int R, int MODE, int STAGES, int SHR = 0>
__global__ void __launch_bounds__(kQ8SThreads) qblk_gemv_grouped_kernel(const QGemvArgs a, const __grid_constant__ QGroupArgs grp) {
    qblk_gemv_body<FMT, B, R, MODE, false, STAGES, true, SHR>(a, &grp);
}

// ---------------------------------------------------------------------------
// Activation quantiser: one warp per 32-element block.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_x_kernel(const float *__restrict__ x, int8_t *__restrict__ xq,
                                                         float *__restrict__ xs, int nblocks, int bpr, int batch) {
    // batch = 0: xq[vector][cols], xs[vector][cols / 32] (the layout of the public entries).
    // batch > 0: xq[block][vector][32], xs[block][vector] -- what the tensor-core mat-vec chained to this kernel reads:
    // the vectors of a column tile lie next to one another.
    const int lane = threadIdx.x & 31;
    const int wpc = blockDim.x / 32;
    pdl_launch_dependents();  // a mat-vec chained to this kernel may start and request its weights now
    for (int blk = blockIdx.x * wpc + (threadIdx.x >> 5); blk < nblocks; blk += gridDim.x * wpc) {
        const float v = x[(size_t)blk * 32 + lane];
        float m = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float scale = (m == 0.0f) ? 1.0f : __fdiv_rn(m, 127.0f);
        const float inv = __fdiv_rn(1.0f, scale);
        size_t at = (size_t)blk;
        if (batch > 0) {
            const int n = blk / bpr, b = blk - n * bpr;
            at = (size_t)b * batch + n;
        }
        xq[at * 32 + lane] = (int8_t)quantize_byte(v, inv);
        if (lane == 0) xs[at] = scale;
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------

// CTA count <= max_ctas (one resident wave) for kernels whose CTAs own contiguous row ranges and whose
// warps own contiguous runs of row groups (R rows each).  The launch is HBM-bound and every warp streams at
// the same rate, so it ends when the warp with the most groups ends: with 14336 rows on 296 x 8 warps, 128
// warps would stream a seventh row while the rest of the machine idles (a seventh of the run time at 5 % of
// the bandwidth).  Picks the count in the upper half of the wave that maximises
// rows / (warps x rows of the busiest warp); ties go to the larger count.
static int balanced_ctas(int rows, int R, int max_ctas) {
    const int groups = (rows + R - 1) / R;
    const int want = (groups + kQ8SWarps - 1) / kQ8SWarps;  // at least one group per warp
    if (want <= max_ctas) return want > 0 ? want : 1;
    int best = max_ctas;
    double best_eff = 0.0;
    for (int g = max_ctas; g >= max_ctas / 2; --g) {
        const int cta_rows = (rows + g - 1) / g;                       // the largest CTA share
        const int cta_groups = (cta_rows + R - 1) / R;
        const int warp_groups = (cta_groups + kQ8SWarps - 1) / kQ8SWarps;  // the busiest warp
        const double eff = (double)rows / ((double)g * kQ8SWarps * warp_groups * R);
        if (eff > best_eff + 1e-9) best_eff = eff, best = g;
    }
    return best;
}

template <int B, int MODE>
struct Q8SConfig {
    // rows per group x segments per trip: R*U 16-byte pieces (4 KB per warp) per ring stage
    static constexpr int R = B <= 2 ? 1 : 2;
    static constexpr int U = B <= 2 ? 8 : 4;
    static constexpr int STAGES = 3;
};

// dynamic shared memory of the split-layout kernel
template <int B, int MODE>
static size_t q8s_smem_bytes(int cols) {
    using Cfg = Q8SConfig<B, MODE>;
    const bool is_int = MODE != MODE_FLOAT;
    const int nseg = (cols + 511) / 512;
    size_t off = (size_t)B * nseg * (is_int ? 512 : 2048) + (is_int ? (size_t)B * (cols / 32) * 4 : 0);
    off = (off + 127) & ~(size_t)127;
    return off + (size_t)kQ8SWarps * Cfg::STAGES * Cfg::R * Cfg::U * (512 + 32);  // scales may ride in the ring
}

template <int B, int MODE, bool DOTS, bool SA>
static int launch_q8s_sa(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    using Cfg = Q8SConfig<B, MODE>;
    constexpr auto kernel = q8s_gemv_kernel<B, Cfg::R, Cfg::U, MODE, DOTS, Cfg::STAGES, SA>;
    int st = ensure_smem_optin<kernel>(di);
    if (st) return st;
    const size_t smem = q8s_smem_bytes<B, MODE>(a.cols);
    if (smem + 1024 > (size_t)di->max_smem_optin) return TB200_ERR_INVALID_ARG;
    // at most one resident wave, sized so that all warps own (nearly) the same number of rows
    const int grid = balanced_ctas(a.rows, Cfg::R, di->sm_count * resident_ctas<kernel>(di, kQ8SThreads, smem));
    return launch_kernel(kernel, dim3(grid), dim3(kQ8SThreads), smem, s, option_value(TB200_OPT_OVERLAP_LAUNCHES) != 0, a);
}

template <int B, int MODE, bool DOTS>
static int launch_q8s(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    if constexpr (DOTS) {
        return launch_q8s_sa<B, MODE, DOTS, false>(a, di, s);  // the block-dot entry passes no scales
    } else {
        // worth it only where the kernel is bandwidth-bound: the float mode is FFMA-bound and keeps its scales in registers
        const bool sa = MODE != MODE_FLOAT && a.cols % 256 == 0 && aligned_to(a.scales, 16);
        return sa ? launch_q8s_sa<B, MODE, DOTS, true>(a, di, s) : launch_q8s_sa<B, MODE, DOTS, false>(a, di, s);
    }
}

template <int FMT, int B, int MODE>
struct RingConfig {
    static constexpr bool INT = MODE != MODE_FLOAT;
    // rows per group: more rows share each activation read from shared memory
    static constexpr int R = INT ? (B <= 2 ? 1 : 2) : (B <= 2 ? 2 : 1);
    // about 13 KB (Q8_0) / 14 KB (Q4_0) of ring per warp
    static constexpr int STAGES = FMT == FMT_Q4B ? (R == 1 ? 4 : 3) : (R == 1 ? 3 : 2);
};

template <int FMT, int B, int MODE>
static size_t ring_smem_bytes(int cols, bool shifted = false) {
    using T = RingTraits<FMT>;
    using Cfg = RingConfig<FMT, B, MODE>;
    const size_t slots = (size_t)((cols + 2047) / 2048) * 2048 / (Cfg::INT ? 16 : 4);
    size_t off = (size_t)B * slots * 16 + (Cfg::INT ? (size_t)B * (cols / 32) * 8 : 0);  // + scales + block sums
    off = (off + 127) & ~(size_t)127;
    return off + (size_t)kQ8SWarps * Cfg::STAGES * Cfg::R * (T::CB + (shifted ? 128 : 0));
}

template <int FMT, int B, int MODE, bool DOTS, int SHR>
static int launch_ring_sh(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    using Cfg = RingConfig<FMT, B, MODE>;
    const size_t smem = ring_smem_bytes<FMT, B, MODE>(a.cols, SHR != 0);
    constexpr auto kernel = qblk_gemv_kernel<FMT, B, Cfg::R, MODE, DOTS, Cfg::STAGES, SHR>;
    int st = ensure_smem_optin<kernel>(di);
    if (st) return st;
    // at most one resident wave, sized so that all warps own (nearly) the same number of rows
    const int grid = balanced_ctas(a.rows, Cfg::R, di->sm_count * resident_ctas<kernel>(di, kQ8SThreads, smem));
    return launch_kernel(kernel, dim3(grid), dim3(kQ8SThreads), smem, s, option_value(TB200_OPT_OVERLAP_LAUNCHES) != 0, a);
}

// Byte phase of the row chunks of a block matrix for the ring kernels: the offset from the 128-byte boundary below
// when every row keeps it (rows that are whole 128-byte lines), else the offset from the 16-byte boundary (0 or 8).
template <int FMT>
static int ring_phase(const void *w, int cols) {
    const size_t row_bytes = (size_t)(cols / 32) * RingTraits<FMT>::BB;
    return (int)((uintptr_t)w & (row_bytes % 128 == 0 ? 127 : 15));
}

// weights off a 128-byte boundary: a kernel of their own for one vector (more vectors go to the tensor-core
// kernel, whose bulk copies do not depend on the phase)
template <int FMT, int B, int MODE, bool DOTS>
static int launch_ring(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    if constexpr (B == 1) {
        if (a.wshift & 8) return launch_ring_sh<FMT, B, MODE, DOTS, 2>(a, di, s);
        if (a.wshift) return launch_ring_sh<FMT, B, MODE, DOTS, 1>(a, di, s);
    }
    if (a.wshift & 15) return TB200_ERR_ALIGNMENT;  // not reached: the dispatcher keeps such launches off this path
    return launch_ring_sh<FMT, B, MODE, DOTS, 0>(a, di, s);
}

template <int FMT, int B, int MODE, int SHR>
static int launch_ring_grouped_sh(const QGemvArgs &a, const QGroupArgs &grp, const DeviceInfo *di, cudaStream_t s) {
    using Cfg = RingConfig<FMT, B, MODE>;
    const size_t smem = ring_smem_bytes<FMT, B, MODE>(a.cols, SHR != 0);
    constexpr auto kernel = qblk_gemv_grouped_kernel<FMT, B, Cfg::R, MODE, Cfg::STAGES, SHR>;
    int st = ensure_smem_optin<kernel>(di);
    if (st) return st;
    const int grid = balanced_ctas(a.rows, Cfg::R, di->sm_count * resident_ctas<kernel>(di, kQ8SThreads, smem));
    return launch_kernel(kernel, dim3(grid), dim3(kQ8SThreads), smem, s, option_value(TB200_OPT_OVERLAP_LAUNCHES) != 0, a, grp);
}

template <int FMT, int B, int MODE>
static int launch_ring_grouped(const QGemvArgs &a, const QGroupArgs &grp, const DeviceInfo *di, cudaStream_t s) {
    if (a.wshift & 8) return launch_ring_grouped_sh<FMT, B, MODE, 2>(a, grp, di, s);
    if (a.wshift) return launch_ring_grouped_sh<FMT, B, MODE, 1>(a, grp, di, s);
    return launch_ring_grouped_sh<FMT, B, MODE, 0>(a, grp, di, s);
}

template <int FMT, int MODE>
static int launch_ring_grouped_b(const QGemvArgs &a, const QGroupArgs &grp, const DeviceInfo *di, cudaStream_t s) {
    switch (a.batch) {
        case 1: return launch_ring_grouped<FMT, 1, MODE>(a, grp, di, s);
        case 2: return launch_ring_grouped<FMT, 2, MODE>(a, grp, di, s);
        case 3: return launch_ring_grouped<FMT, 3, MODE>(a, grp, di, s);
        case 4: return launch_ring_grouped<FMT, 4, MODE>(a, grp, di, s);
        default: return TB200_ERR_INVALID_ARG;
    }
}

template <int FMT, bool INT>
static int launch_generic(const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s) {
    int need = (a.rows + 7) / 8;
    int grid = di->sm_count * 8 < need ? di->sm_count * 8 : need;
    const int st = ensure_kernel<qgemv_generic_kernel<FMT, INT>, 0>(di);
    if (st) return st;
    qgemv_generic_kernel<FMT, INT><<<grid, 256, 0, s>>>(a);
    return check_launch();
}

enum Path { PATH_GENERIC, PATH_Q8S_DIRECT, PATH_RING };

// Does one fast launch with `batch` activation vectors fit in shared memory?
template <int FMT, int MODE>
static bool fast_batch_fits(int cols, int batch, Path path, const DeviceInfo *di) {
    const size_t limit = (size_t)di->max_smem_optin - 1024;
    if (path == PATH_RING) {
        // sized for the form with shifted ring slots (128 bytes more per slot), which weights off a 128-byte line take
        switch (batch) {
            case 1: return ring_smem_bytes<FMT, 1, MODE>(cols, true) <= limit;
            case 2: return ring_smem_bytes<FMT, 2, MODE>(cols, true) <= limit;
            case 3: return ring_smem_bytes<FMT, 3, MODE>(cols, true) <= limit;
            case 4: return ring_smem_bytes<FMT, 4, MODE>(cols, true) <= limit;
            case 5: return ring_smem_bytes<FMT, 5, MODE>(cols, true) <= limit;
            case 6: return ring_smem_bytes<FMT, 6, MODE>(cols, true) <= limit;
            case 7: return ring_smem_bytes<FMT, 7, MODE>(cols, true) <= limit;
            case 8: return ring_smem_bytes<FMT, 8, MODE>(cols, true) <= limit;
            default: return false;
        }
    }
    switch (batch) {
        case 1: return q8s_smem_bytes<1, MODE>(cols) <= limit;
        case 2: return q8s_smem_bytes<2, MODE>(cols) <= limit;
        case 3: return q8s_smem_bytes<3, MODE>(cols) <= limit;
        case 4: return q8s_smem_bytes<4, MODE>(cols) <= limit;
        case 5: return q8s_smem_bytes<5, MODE>(cols) <= limit;
        case 6: return q8s_smem_bytes<6, MODE>(cols) <= limit;
        case 7: return q8s_smem_bytes<7, MODE>(cols) <= limit;
        case 8: return q8s_smem_bytes<8, MODE>(cols) <= limit;
        default: return false;
    }
}

// Fewest passes over the weights such that each pass's share of the batch fits;
// returns the per-pass batch, 0 if not even one vector fits.
template <int FMT, int MODE>
static int batch_per_pass(int cols, int batch, Path path, const DeviceInfo *di) {
    for (int passes = 1; passes <= batch; ++passes) {
        const int per = (batch + passes - 1) / passes;
        if (fast_batch_fits<FMT, MODE>(cols, per, path, di)) return per;
    }
    return 0;
}

template <int FMT, int MODE, bool DOTS, int B>
static int launch_fast_b(const QGemvArgs &a, Path path, const DeviceInfo *di, cudaStream_t s) {
    if constexpr (FMT == FMT_Q8S) {
        return launch_q8s<B, MODE, DOTS>(a, di, s);
    } else {
        return launch_ring<FMT, B, MODE, DOTS>(a, di, s);
    }
}

template <int FMT, int MODE, bool DOTS>
static int launch_fast(const QGemvArgs &a, Path path, const DeviceInfo *di, cudaStream_t s) {
    switch (a.batch) {
        case 1: return launch_fast_b<FMT, MODE, DOTS, 1>(a, path, di, s);
        case 2: return launch_fast_b<FMT, MODE, false, 2>(a, path, di, s);
        case 3: return launch_fast_b<FMT, MODE, false, 3>(a, path, di, s);
        case 4: return launch_fast_b<FMT, MODE, false, 4>(a, path, di, s);
        case 5: return launch_fast_b<FMT, MODE, false, 5>(a, path, di, s);
        case 6: return launch_fast_b<FMT, MODE, false, 6>(a, path, di, s);
        case 7: return launch_fast_b<FMT, MODE, false, 7>(a, path, di, s);
        case 8: return launch_fast_b<FMT, MODE, false, 8>(a, path, di, s);
        default: return TB200_ERR_INVALID_ARG;
    }
}

// Fusing the activation quantiser into the GEMV prologue repeats it in every
// CTA; beyond this many activation elements the separate quantiser kernel and
// the workspace are cheaper.
constexpr int kFusedQuantMaxElems = 16384;

// Shared front end: validation, path choice, batch splitting.
//   MODE_FLOAT      a.x set
//   MODE_INT        a.xq / a.xs set (already quantised)
//   MODE_INT_FUSED  a.x set, quantised inside the kernel; falls back to
//                   quantiser kernel + workspace (xq_ws / xs_ws) when the fast
//                   path is not taken or the batch is large
template <int FMT, int MODE, bool DOTS>
static int qgemv_dispatch(QGemvArgs a, int8_t *xq_ws, float *xs_ws, tb200_stream_t stream);

template <int FMT, int MODE, bool DOTS>
static int qgemv_dispatch(QGemvArgs a, int8_t *xq_ws, float *xs_ws, tb200_stream_t stream) {
    constexpr bool INT = MODE != MODE_FLOAT;
    if (a.rows < 0 || a.cols < 0 || a.batch < 1 || a.batch > kMaxBatch) return TB200_ERR_INVALID_ARG;
    if (a.cols % 32 != 0) return TB200_ERR_INVALID_ARG;
    if (a.rows == 0) return TB200_OK;
    if (!a.w || (FMT == FMT_Q8S && !DOTS && !a.scales) || (!DOTS && !a.y)) return TB200_ERR_INVALID_ARG;
    if (MODE == MODE_INT ? (!a.xq || (!DOTS && !a.xs)) : !a.x) return TB200_ERR_INVALID_ARG;
    if (DOTS && !a.dots) return TB200_ERR_INVALID_ARG;
    if (FMT == FMT_Q8S && a.scales && !aligned_to(a.scales, 2)) return TB200_ERR_ALIGNMENT;
    if ((a.y && !aligned_to(a.y, 4)) || (MODE != MODE_INT && !aligned_to(a.x, 4))) return TB200_ERR_ALIGNMENT;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    cudaStream_t s = (cudaStream_t)stream;
    if (a.cols == 0) {
        if (a.y) return (int)cudaMemsetAsync(a.y, 0, sizeof(float) * (size_t)a.rows * a.batch, s);
        return TB200_OK;
    }
    // ring: every row chunk starts on a 16-byte boundary and is a whole number of 16-byte units
    // split layout: 128-bit loads need 16-byte aligned rows (cols % 32 == 0 keeps the phase)
    // block layouts: weights 8 bytes past a 16-byte boundary keep that phase inside the ring
    Path path = PATH_GENERIC;
    a.wshift = 0;
    if (FMT == FMT_Q8S) {
        if (aligned_to(a.w, 16)) path = PATH_Q8S_DIRECT;
    } else if (a.cols % 256 == 0 && (aligned_to(a.w, 16) || (aligned_to(a.w, 8) && a.batch == 1))) {
        path = PATH_RING, a.wshift = ring_phase<FMT>(a.w, a.cols);
    }
    // Tensor-core kernel with the activations in registers (gemv_tc.cu): integer mode from
    // TB200_OPT_INT_TENSOR_CORE_MIN_BATCH vectors on, float mode from one vector on, and every batch
    // when split-layout operands are only 8-byte aligned (arrays behind a 24-byte header), where the alternative
    // is the byte-load kernel.
    const bool overlap = option_value(TB200_OPT_OVERLAP_LAUNCHES) != 0;
    if (option_value(TB200_OPT_TC_REGISTER_KERNEL)) {
        const bool only8 = FMT == FMT_Q8S && (!aligned_to(a.w, 16) || (a.scales && !aligned_to(a.scales, 16)));
        if (MODE == MODE_FLOAT) {
            const int float_tc = option_value(TB200_OPT_FLOAT_TENSOR_CORES);  // 0 off, 1 / 2 on
            // measured at 14336 x 4096, one vector: Q8_0 blocks 14.5 us on the tensor cores against 16.6 us on the FFMA ring
            // kernel, Q4_0 12.6 against 13.9 us; from one vector on in every layout
            const int min_batch = 1;
            QGemvArgs p = a;
            p.batch = a.batch < 8 ? a.batch : 8;
            if ((float_tc || only8) && a.batch >= min_batch && qtc_eligible(FMT, MODE_FLOAT, p, di)) {
                // at most eight vectors (sixteen fp16 columns) per pass over the weights
                const int passes = (a.batch + 7) / 8, each = (a.batch + passes - 1) / passes;
                for (int b0 = 0; b0 < a.batch; b0 += each) {
                    p.batch = a.batch - b0 < each ? a.batch - b0 : each;
                    p.x = a.x + (size_t)b0 * a.cols, p.y = a.y + (size_t)b0 * a.rows;
                    st = qtc_dispatch(FMT, MODE_FLOAT, p, di, s, overlap && b0 == 0);
                    if (st) return st;
                }
                return TB200_OK;
            }
        } else if (a.batch >= (only8 ? 1 : option_value(TB200_OPT_INT_TENSOR_CORE_MIN_BATCH)) && (!DOTS || a.batch == 1) &&
                   qtc_eligible(FMT, MODE, a, di)) {
            if (MODE == MODE_INT_FUSED && xq_ws && xs_ws && a.batch <= 8) {
                // Quantising inside the mat-vec means every one of its CTAs converts all the vectors (measured: 5 us
                // of a 14 us launch at 8 vectors, during which the weight ring fills up and the copies stall).  Up to
                // 8 vectors the activations are therefore quantised once by a small kernel of their own, and the
                // mat-vec is chained to it with a programmatic dependent launch: it starts while the quantiser runs,
                // requests its first weights, and waits for the quantiser only where it reads the int8 activations.
                // (With two column tiles the fused form measured faster: 24.6 against 31 us at 16 vectors.)
                st = quantize_x_layout(a.cols, a.batch, a.x, xq_ws, xs_ws, s, true);
                if (st) return st;
                QGemvArgs b = a;
                b.x = nullptr, b.xq = xq_ws, b.xs = xs_ws, b.xlayout = 1;
                return qtc_dispatch(FMT, MODE_INT, b, di, s, true);
            }
            // MODE_INT follows the quantiser kernel in plain stream order; the fused form may overlap its predecessor
            return qtc_dispatch(FMT, MODE, a, di, s, MODE == MODE_INT_FUSED && overlap);
        }
    }
    const int per = path == PATH_GENERIC
                        ? 0
                        : batch_per_pass<FMT, MODE == MODE_INT_FUSED ? MODE_INT : MODE>(a.cols, a.batch, path, di);
    if (per < 1) path = PATH_GENERIC;

    if (MODE == MODE_INT_FUSED) {
        // batches of five and more go to the tensor-core kernel, which reads quantised activations from the workspace
        const bool fuse = path != PATH_GENERIC && (long long)a.batch * a.cols <= kFusedQuantMaxElems && a.batch == per && a.batch <= 4 && a.batch < option_value(TB200_OPT_INT_TENSOR_CORE_MIN_BATCH);
        if (fuse) return launch_fast<FMT, MODE_INT_FUSED, false>(a, path, di, s);
        // separate quantiser into the workspace, then the MODE_INT kernels
        st = quantize_x(a.cols, a.batch, a.x, xq_ws, xs_ws, s);
        if (st) return st;
        QGemvArgs b = a;
        b.x = nullptr, b.xq = xq_ws, b.xs = xs_ws;
        return qgemv_dispatch<FMT, MODE_INT, false>(b, nullptr, nullptr, stream);
    } else {
        if (path == PATH_GENERIC) return launch_generic<FMT, INT>(a, di, s);
        if constexpr (MODE == MODE_INT && !DOTS) {
            if (qmma_eligible(FMT, a)) return qmma_dispatch(FMT, a, di, s);
        }
        if constexpr (MODE == MODE_FLOAT && !DOTS) {
            const int float_tc = option_value(TB200_OPT_FLOAT_TENSOR_CORES);  // 0 off, 1 / 2 on
            const int min_batch = 1;
            // diagnostics only (TB200_OPT_TC_REGISTER_KERNEL = 0): this older kernel splits x into fp16 pairs without a
            // prescale, so it is accurate only for activations inside the normal fp16 range
            if (float_tc && a.batch >= min_batch && !option_value(TB200_OPT_TC_REGISTER_KERNEL)) {
                // most vectors per pass whose fp16 pairs fit in shared memory next to the weight ring
                QGemvArgs p = a;
                int cap = 0;
                for (int c = 8; c >= 4 && !cap; c -= 4) {
                    p.batch = a.batch < c ? a.batch : c;
                    if (qmma_float_eligible(FMT, p, di)) cap = c;
                }
                if (cap) {
                    const int passes = (a.batch + cap - 1) / cap, each = (a.batch + passes - 1) / passes;
                    for (int b0 = 0; b0 < a.batch; b0 += each) {
                        p.batch = a.batch - b0 < each ? a.batch - b0 : each;
                        p.x = a.x + (size_t)b0 * a.cols, p.y = a.y + (size_t)b0 * a.rows;
                        st = qmma_float_dispatch(FMT, p, di, s, option_value(TB200_OPT_OVERLAP_LAUNCHES) != 0 && b0 == 0);
                        if (st) return st;
                    }
                    return TB200_OK;
                }
            }
        }
        // more activation vectors than fit next to the ring: several passes over the weights
        for (int b0 = 0; b0 < a.batch; b0 += per) {
            QGemvArgs p = a;
            p.batch = a.batch - b0 < per ? a.batch - b0 : per;
            if (INT) {
                p.xq = a.xq + (size_t)b0 * a.cols;
                if (a.xs) p.xs = a.xs + (size_t)b0 * (a.cols / 32);
            } else {
                p.x = a.x + (size_t)b0 * a.cols;
            }
            if (a.y) p.y = a.y + (size_t)b0 * a.rows;
            st = launch_fast<FMT, MODE, DOTS>(p, path, di, s);
            if (st) return st;
        }
        return TB200_OK;
    }
}

int split_workspace(int cols, int batch, void *workspace, size_t workspace_bytes, int8_t **xq, float **xs) {
    if (cols < 0 || cols % 32 != 0 || batch < 1 || batch > kMaxBatch) return TB200_ERR_INVALID_ARG;
    if (!workspace || workspace_bytes < tb200_qx_workspace_bytes(cols, batch)) return TB200_ERR_WORKSPACE;
    if (!aligned_to(workspace, 16)) return TB200_ERR_ALIGNMENT;
    *xq = reinterpret_cast<int8_t *>(workspace);
    *xs = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(workspace) + (((size_t)cols * batch + 15) & ~(size_t)15));
    return TB200_OK;
}

int quantize_x(int cols, int batch, const float *x, int8_t *xq, float *xs, cudaStream_t s) { return quantize_x_layout(cols, batch, x, xq, xs, s, false); }

// interleaved: xq[block][vector][32], xs[block][vector] (see quantize_x_kernel)
int quantize_x_layout(int cols, int batch, const float *x, int8_t *xq, float *xs, cudaStream_t s, bool interleaved) {
    if (!x) return TB200_ERR_INVALID_ARG;
    if (!aligned_to(x, 4)) return TB200_ERR_ALIGNMENT;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    const long long nblocks_ll = (long long)(cols / 32) * batch;
    if (nblocks_ll > 0x7fffffffLL) return TB200_ERR_INVALID_ARG;
    int nblocks = (int)nblocks_ll;
    if (nblocks == 0) return TB200_OK;
    int grid = (nblocks + 7) / 8;
    if (grid > di->sm_count * 8) grid = di->sm_count * 8;
    // The mat-vec kernels that follow run with the SM's largest shared-memory carve-out.  Without this hint the
    // driver would switch the carve-out for this small kernel and back, draining the SMs twice (about 15 us).
    st = ensure_kernel<quantize_x_kernel, KERNEL_MAX_CARVEOUT>(di);
    if (st) return st;
    quantize_x_kernel<<<grid, 256, 0, s>>>(x, xq, xs, nblocks, cols / 32, interleaved ? batch : 0);
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
    QGemvArgs a{reinterpret_cast<const uint8_t *>(w), scales, x, nullptr, nullptr, y, nullptr, rows, cols, batch};
    return qgemv_dispatch<FMT, MODE_INT_FUSED, false>(a, xq, xs, stream);
}

// Integer-mode mat-vec of `count` equally shaped block matrices on the same activations, one launch,
// every output value stored to `npeers` destination buffers.
struct GroupSync {  // in-kernel hand-shake of a multi-GPU step; flags == nullptr: none
    unsigned *const *flags;
    unsigned *sync;
    int rank, handshake;
    unsigned timeout_ms;
    int nslots;
};

struct GroupShape {  // per matrix: rows in this launch, output block offset inside a slot, whole-matrix rows, first row
    int rows[kMaxGroup];
    long long out_off[kMaxGroup];
    int ld[kMaxGroup];
    int row_off[kMaxGroup];
};

template <int FMT>
static int qgemv_i8_grouped_shape(int count, const GroupShape &shape, int cols, int batch, const void *const *blocks, const float *x,
                                  float *const *dst, int npeers, long long half_stride, const unsigned *epoch, void *workspace,
                                  size_t workspace_bytes, tb200_stream_t stream, const GroupSync &gs) {
    if (count < 1 || count > kMaxGroup || npeers < 1 || npeers > kMaxPeers || !blocks || !dst || !x) return TB200_ERR_INVALID_ARG;
    if (cols < 0 || cols % 32 != 0 || batch < 1 || batch > kMaxBatch || half_stride < 0) return TB200_ERR_INVALID_ARG;
    if (!aligned_to(x, 4) || (epoch && !aligned_to(epoch, 4))) return TB200_ERR_ALIGNMENT;
    QGroupArgs grp{};
    bool fast = cols % 256 == 0 && cols > 0;
    bool same_line_phase = true;  // every matrix starts at the same offset from a 128-byte boundary
    long long total = 0;
    for (int m = 0; m < count; ++m) {
        if (!blocks[m] || shape.rows[m] < 0) return TB200_ERR_INVALID_ARG;
        if (shape.row_off[m] < 0 || shape.ld[m] < shape.rows[m] || shape.row_off[m] > shape.ld[m] - shape.rows[m]) return TB200_ERR_INVALID_ARG;
        if (!aligned_to(blocks[m], 2)) return TB200_ERR_ALIGNMENT;
        fast = fast && aligned_to(blocks[m], 8) && (((uintptr_t)blocks[m] ^ (uintptr_t)blocks[0]) & 15) == 0;  // one phase, 0 or 8
        same_line_phase = same_line_phase && (((uintptr_t)blocks[m] ^ (uintptr_t)blocks[0]) & 127) == 0;
        grp.w[m] = reinterpret_cast<const uint8_t *>(blocks[m]);
        grp.row_start[m] = (int)total;
        grp.out_off[m] = shape.out_off[m], grp.ld[m] = shape.ld[m], grp.row_off[m] = shape.row_off[m];
        total += shape.rows[m];
        if (total > 0x7fffffffLL) return TB200_ERR_INVALID_ARG;
    }
    grp.row_start[count] = (int)total;
    for (int p = 0; p < npeers; ++p) {
        if (!dst[p]) return TB200_ERR_INVALID_ARG;
        if (!aligned_to(dst[p], 4)) return TB200_ERR_ALIGNMENT;
        grp.dst[p] = dst[p];
    }
    if (gs.flags) {
        // every GPU of the group must take part in every step, and only the one-launch kernel holds the hand-shake
        if (!gs.sync || gs.rank < 0 || gs.rank >= npeers || total < 1 || !aligned_to(gs.sync, 4)) return TB200_ERR_INVALID_ARG;
        if (gs.nslots < 2 || gs.nslots > 4) return TB200_ERR_INVALID_ARG;
        grp.nslots = gs.nslots;
        for (int p = 0; p < npeers; ++p) {
            if (!gs.flags[p] || !aligned_to(gs.flags[p], 4)) return TB200_ERR_INVALID_ARG;
            grp.flags[p] = gs.flags[p];
        }
        grp.sync = gs.sync, grp.rank = gs.rank, grp.handshake = gs.handshake;
        grp.timeout_ns = (unsigned long long)(gs.timeout_ms ? gs.timeout_ms : 2000u) * 1000000ull;
        epoch = gs.sync;
    }
    if (total == 0) return TB200_OK;
    grp.epoch = epoch, grp.half_stride = half_stride, grp.count = count, grp.npeers = npeers;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    cudaStream_t s = (cudaStream_t)stream;
    // Two to eight vectors into one local buffer: the tensor-core mat-vec per matrix (it outruns the dp4a ring kernel
    // from two vectors on), all behind ONE quantiser launch and chained to one another, so that each starts
    // requesting its weights while its predecessor drains.
    // Up to 8 vectors (one column tile).  With 9 to 16 the kernel that reads quantised activations from the workspace is
    // the slower one (Q4_0 layer sweep at 16 vectors: 311 us as one launch per column count against 259 us as one launch
    // per matrix with the quantiser inside the kernel), so those groups take the per-matrix path below.
    if (batch >= option_value(TB200_OPT_INT_TENSOR_CORE_MIN_BATCH) && batch <= 8 && npeers == 1 && !epoch && !gs.flags &&
        option_value(TB200_OPT_TC_REGISTER_KERNEL) && workspace) {
        bool tc = true;
        for (int m = 0; m < count && tc; ++m) {
            QGemvArgs one{grp.w[m], nullptr, nullptr, reinterpret_cast<const int8_t *>(workspace), nullptr, dst[0], nullptr, shape.rows[m] > 0 ? shape.rows[m] : 1,
                          cols, batch};
            tc = shape.ld[m] == shape.rows[m] && qtc_eligible(FMT, MODE_INT, one, di);
        }
        // one launch over all rows: possible when the matrices share the 16-byte phase and the kernel takes that many rows
        bool table = tc && count > 1 && total <= 0x7fffffffLL;
        for (int m = 0; m < count && table; ++m) table = aligned_to(grp.w[m], 8) && (((uintptr_t)grp.w[m] ^ (uintptr_t)grp.w[0]) & 15) == 0;
        if (table) {
            QGemvArgs probe{grp.w[0], nullptr, nullptr, reinterpret_cast<const int8_t *>(workspace), nullptr, dst[0], nullptr, (int)total, cols, batch};
            table = qtc_eligible(FMT, MODE_INT, probe, di);
        }
        if (tc && (batch <= 8 || table)) {
            int8_t *xq;
            float *xs;
            st = split_workspace(cols, batch, workspace, workspace_bytes, &xq, &xs);
            if (st) return st;
            st = quantize_x_layout(cols, batch, x, xq, xs, s, true);
            if (st) return st;
            // Equally shaped matrices that lie back to back (the packed task's ByteArray) with the standard output
            // layout are ONE matrix of count * rows rows to the kernel: one launch, the activations loaded once per
            // CTA, no tail per matrix (measured, 8 matrices of 14336 x 4096, 8 vectors: 12.6 us per matrix as a chain
            // of launches); the kernel writes y[matrix][vector][row].
            bool one_launch = table;
            const size_t per = (size_t)shape.rows[0] * (size_t)(cols / 32) * RingTraits<FMT>::BB;
            for (int m = 0; m < count && one_launch; ++m)
                one_launch = shape.rows[m] == shape.rows[0] && shape.row_off[m] == 0 && grp.w[m] == grp.w[0] + (size_t)m * per &&
                             shape.out_off[m] == (long long)m * batch * shape.rows[0];
            if (one_launch) {
                QGemvArgs all{grp.w[0], nullptr, nullptr, xq, xs, dst[0], nullptr, (int)total, cols, batch};
                all.xlayout = 1, all.group_rows = shape.rows[0];
                if (qtc_eligible(FMT, MODE_INT, all, di)) return qtc_dispatch(FMT, MODE_INT, all, di, s, true);
            }
            // Any other group whose matrices share the 16-byte phase: still one launch, with a table of the matrices'
            // first rows, addresses and output blocks in the kernel's parameters (a row's matrix is looked up where
            // the row is requested and where its sums are stored).
            if (table) {
                TcGroup tg{};
                tg.count = count;
                for (int m = 0; m < count; ++m) tg.row_start[m] = grp.row_start[m], tg.w[m] = grp.w[m], tg.y_off[m] = shape.out_off[m] + shape.row_off[m];
                tg.row_start[count] = (int)total;
                QGemvArgs all{grp.w[0], nullptr, nullptr, xq, xs, dst[0], nullptr, (int)total, cols, batch};
                all.xlayout = 1;
                return qtc_dispatch_group(FMT, all, tg, di, s, true);
            }
            for (int m = 0; m < count; ++m) {
                if (shape.rows[m] == 0) continue;
                QGemvArgs one{grp.w[m], nullptr, nullptr, xq, xs, dst[0] + shape.out_off[m] + shape.row_off[m], nullptr, shape.rows[m], cols, batch};
                one.xlayout = 1;
                st = qtc_dispatch(FMT, MODE_INT, one, di, s, true);
                if (st) return st;
            }
            return TB200_OK;
        }
    }
    QGemvArgs a{nullptr, nullptr, x, nullptr, nullptr, nullptr, nullptr, (int)total, cols, batch,
                same_line_phase ? ring_phase<FMT>(blocks[0], cols) : (int)((uintptr_t)blocks[0] & 15)};
    if (fast && batch <= 4 && fast_batch_fits<FMT, MODE_INT>(cols, batch, PATH_RING, di)) {
        if ((long long)batch * cols <= kFusedQuantMaxElems) return launch_ring_grouped_b<FMT, MODE_INT_FUSED>(a, grp, di, s);
        int8_t *xq;
        float *xs;
        st = split_workspace(cols, batch, workspace, workspace_bytes, &xq, &xs);
        if (st) return st;
        st = quantize_x(cols, batch, x, xq, xs, s);
        if (st) return st;
        a.x = nullptr, a.xq = xq, a.xs = xs;
        return launch_ring_grouped_b<FMT, MODE_INT>(a, grp, di, s);
    }
    // other shapes and alignments: one launch per matrix, into the single local destination only
    if (npeers != 1 || epoch || gs.flags) return TB200_ERR_INVALID_ARG;
    int8_t *xq;
    float *xs;
    st = split_workspace(cols, batch, workspace, workspace_bytes, &xq, &xs);
    if (st) return st;
    for (int m = 0; m < count; ++m) {
        if (batch > 1 && shape.ld[m] != shape.rows[m]) return TB200_ERR_INVALID_ARG;  // the single-matrix kernels write [batch][rows]
        QGemvArgs one{grp.w[m], nullptr, x, nullptr, nullptr, dst[0] + shape.out_off[m] + shape.row_off[m], nullptr, shape.rows[m], cols, batch};
        st = qgemv_dispatch<FMT, MODE_INT_FUSED, false>(one, xq, xs, stream);
        if (st) return st;
    }
    return TB200_OK;
}

// equally shaped matrices, outputs [matrix][batch][rows_total] in every slot
template <int FMT>
static int qgemv_i8_grouped(int count, int rows, int cols, int batch, const void *const *blocks, const float *x, float *const *dst,
                            int npeers, long long half_stride, const unsigned *epoch, int rows_total, int row_offset, void *workspace,
                            size_t workspace_bytes, tb200_stream_t stream, const GroupSync &gs = GroupSync{}) {
    if (count < 1 || count > kMaxGroup || rows < 0 || batch < 1) return TB200_ERR_INVALID_ARG;
    if (row_offset < 0 || rows_total < rows || row_offset > rows_total - rows) return TB200_ERR_INVALID_ARG;
    if (gs.flags && rows < 1) return TB200_ERR_INVALID_ARG;
    GroupShape shape;
    for (int m = 0; m < count; ++m) {
        shape.rows[m] = rows, shape.out_off[m] = (long long)m * batch * rows_total, shape.ld[m] = rows_total, shape.row_off[m] = row_offset;
    }
    return qgemv_i8_grouped_shape<FMT>(count, shape, cols, batch, blocks, x, dst, npeers, half_stride, epoch, workspace, workspace_bytes,
                                       stream, gs);
}

// matrices of different row counts, each with its own [batch][rows[m]] output array on this GPU
template <int FMT>
static int qgemv_i8_grouped_rows(int count, const int *rows, int cols, int batch, const void *const *blocks, const float *x,
                                 float *const *y, void *workspace, size_t workspace_bytes, tb200_stream_t stream) {
    if (count < 1 || count > kMaxGroup || !rows || !y) return TB200_ERR_INVALID_ARG;
    GroupShape shape;
    for (int m = 0; m < count; ++m) {
        if (!y[m]) return TB200_ERR_INVALID_ARG;
        if (!aligned_to(y[m], 4)) return TB200_ERR_ALIGNMENT;
        shape.rows[m] = rows[m], shape.ld[m] = rows[m], shape.row_off[m] = 0;
        shape.out_off[m] = y[m] - y[0];  // floats; may be negative
    }
    float *base[1] = {y[0]};
    return qgemv_i8_grouped_shape<FMT>(count, shape, cols, batch, blocks, x, base, 1, 0, nullptr, workspace, workspace_bytes, stream,
                                       GroupSync{});
}

// split-layout integer mat-vec on activations that are already quantised (a.xq, a.xs)
int q8s_gemv_quantised(const QGemvArgs &a, tb200_stream_t stream) {
    return qgemv_dispatch<FMT_Q8S, MODE_INT, false>(a, nullptr, nullptr, stream);
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_q8_gemv(int rows, int cols, int batch, const int8_t *q, const uint16_t *scales, const float *x,
                             float *y, tb200_stream_t stream) {
    QGemvArgs a{reinterpret_cast<const uint8_t *>(q), scales, x, nullptr, nullptr, y, nullptr, rows, cols, batch};
    return qgemv_dispatch<FMT_Q8S, MODE_FLOAT, false>(a, nullptr, nullptr, stream);
}

extern "C" int tb200_q8b_gemv(int rows, int cols, int batch, const uint8_t *blocks, const float *x, float *y,
                              tb200_stream_t stream) {
    if (blocks && !aligned_to(blocks, 2)) return TB200_ERR_ALIGNMENT;
    QGemvArgs a{blocks, nullptr, x, nullptr, nullptr, y, nullptr, rows, cols, batch};
    return qgemv_dispatch<FMT_Q8B, MODE_FLOAT, false>(a, nullptr, nullptr, stream);
}

extern "C" int tb200_q4b_gemv(int rows, int cols, int batch, const uint8_t *blocks, const float *x, float *y,
                              tb200_stream_t stream) {
    if (blocks && !aligned_to(blocks, 2)) return TB200_ERR_ALIGNMENT;
    QGemvArgs a{blocks, nullptr, x, nullptr, nullptr, y, nullptr, rows, cols, batch};
    return qgemv_dispatch<FMT_Q4B, MODE_FLOAT, false>(a, nullptr, nullptr, stream);
}

extern "C" size_t tb200_qx_workspace_bytes(int cols, int batch) {
    if (cols < 0 || batch < 0) return 0;
    return (((size_t)cols * batch + 15) & ~(size_t)15) + (size_t)(cols / 32) * batch * sizeof(float);
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

extern "C" int tb200_q8b_gemv_i8_grouped(int count, int rows, int cols, int batch, const void *const *blocks, const float *x,
                                         float *const *dst, int npeers, long long half_stride, const unsigned *epoch, int rows_total,
                                         int row_offset, void *workspace, size_t workspace_bytes, tb200_stream_t stream) {
    return qgemv_i8_grouped<FMT_Q8B>(count, rows, cols, batch, blocks, x, dst, npeers, half_stride, epoch, rows_total, row_offset,
                                     workspace, workspace_bytes, stream);
}

extern "C" int tb200_q4b_gemv_i8_grouped(int count, int rows, int cols, int batch, const void *const *blocks, const float *x,
                                         float *const *dst, int npeers, long long half_stride, const unsigned *epoch, int rows_total,
                                         int row_offset, void *workspace, size_t workspace_bytes, tb200_stream_t stream) {
    return qgemv_i8_grouped<FMT_Q4B>(count, rows, cols, batch, blocks, x, dst, npeers, half_stride, epoch, rows_total, row_offset,
                                     workspace, workspace_bytes, stream);
}

extern "C" int tb200_q8b_gemv_i8_grouped_sync(int count, int rows, int cols, int batch, const void *const *blocks, const float *x,
                                              float *const *dst, int npeers, int rank, int nslots, long long slot_stride, unsigned *sync,
                                              unsigned *const *flags, int handshake, unsigned timeout_ms, int rows_total, int row_offset,
                                              void *workspace, size_t workspace_bytes, tb200_stream_t stream) {
    if (!flags || !sync) return TB200_ERR_INVALID_ARG;
    return qgemv_i8_grouped<FMT_Q8B>(count, rows, cols, batch, blocks, x, dst, npeers, slot_stride, nullptr, rows_total, row_offset,
                                     workspace, workspace_bytes, stream, GroupSync{flags, sync, rank, handshake, timeout_ms, nslots});
}

extern "C" int tb200_q4b_gemv_i8_grouped_sync(int count, int rows, int cols, int batch, const void *const *blocks, const float *x,
                                              float *const *dst, int npeers, int rank, int nslots, long long slot_stride, unsigned *sync,
                                              unsigned *const *flags, int handshake, unsigned timeout_ms, int rows_total, int row_offset,
                                              void *workspace, size_t workspace_bytes, tb200_stream_t stream) {
    if (!flags || !sync) return TB200_ERR_INVALID_ARG;
    return qgemv_i8_grouped<FMT_Q4B>(count, rows, cols, batch, blocks, x, dst, npeers, slot_stride, nullptr, rows_total, row_offset,
                                     workspace, workspace_bytes, stream, GroupSync{flags, sync, rank, handshake, timeout_ms, nslots});
}

extern "C" int tb200_q8b_gemv_i8_grouped_rows(int count, const int *rows, int cols, int batch, const void *const *blocks, const float *x,
                                              float *const *y, void *workspace, size_t workspace_bytes, tb200_stream_t stream) {
    return qgemv_i8_grouped_rows<FMT_Q8B>(count, rows, cols, batch, blocks, x, y, workspace, workspace_bytes, stream);
}

extern "C" int tb200_q4b_gemv_i8_grouped_rows(int count, const int *rows, int cols, int batch, const void *const *blocks, const float *x,
                                              float *const *y, void *workspace, size_t workspace_bytes, tb200_stream_t stream) {
    return qgemv_i8_grouped_rows<FMT_Q4B>(count, rows, cols, batch, blocks, x, y, workspace, workspace_bytes, stream);
}

// The block-dot entries take an already quantised activation vector and write
// only `dots`: scales do not enter an integer dot, so none are passed.
template <int FMT>
static int blockdots(int rows, int cols, const void *w, const int8_t *xq, int32_t *dots, tb200_stream_t stream) {
    QGemvArgs a{reinterpret_cast<const uint8_t *>(w), nullptr, nullptr, xq, nullptr, nullptr, dots, rows, cols, 1};
    return qgemv_dispatch<FMT, MODE_INT, true>(a, nullptr, nullptr, stream);
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
