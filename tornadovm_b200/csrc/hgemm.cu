// FP16 GEMM with fp32 accumulation and output: C[m][n] = A[m][k] * B[k][n].
//
// Replaces the reference's tile-API kernels, which issue Ampere mma.sync
// m16n8k16 from 128x128x16 CTA tiles without software pipelining
// (MatrixMultiplicationMMA.java:100-613).  Here the contraction runs on the
// 5th-generation tensor cores:
//
//   * one persistent CTA per SM, output tile 128 x 256, K step 64;
//   * warp 0 (one lane) feeds a 4-stage shared-memory ring with TMA tensor
//     copies: A[m][k] as K-major 128-byte-swizzled rows, B[k][n] as it lies in
//     memory (N contiguous = "MN-major" operand), four 64-column boxes per stage;
//   * warp 1 (one lane) issues tcgen05.mma (M128 N256 K16, fp16 x fp16 -> fp32)
//     with the accumulator in tensor memory, releases ring stages with
//     tcgen05.commit, and alternates between two 256-column accumulators so the
//     epilogue of one tile overlaps the main loop of the next;
//   * warps 2..5 read the accumulator with tcgen05.ld and store fp32 rows.
//
// Ragged M, N, K are handled by the tensor maps (out-of-range elements load as
// zero) and by bounds checks on the stores.  Every mbarrier wait is bounded: on
// expiry the CTA records TB200_ERR_TIMEOUT, all roles leave their loops, and
// tensor memory is released.
//
// flops per launch: 2*m*n*k; roofline: dense fp16 tensor throughput.
#include <cuda.h>
#include <cuda_bf16.h>

#define TB200_OP_CLASS TB200_PREPARE_GEMM_F16
#include "common.cuh"
#include "gemm_generic.cuh"

TB200_TU_STATUS(hgemm)

namespace tb200 {

constexpr int HG_BM = 128, HG_BK = 64;
constexpr int HG_THREADS = 192;
constexpr int HG_A_BYTES = HG_BM * HG_BK * 2;      // 16 KB
// Each epilogue warp owns a 32 x 32 fp32 transposition buffer (row pitch 36 floats: conflict-free float4 access both ways),
// used when tiles go to several destinations: stores to peer memory should be whole 128-byte lines, not 16-byte pieces
// of 32 different rows.
constexpr int HG_XPOSE_PITCH = 36, HG_XPOSE_BYTES = 4 * 32 * HG_XPOSE_PITCH * 4;
// Staging area of the epilogue: the transposition buffers above, or -- single destination -- two 32 x 32 fp32 tiles
// (128-byte rows, 128-byte swizzle) per epilogue warp from which finished pieces leave as TMA tensor stores.
constexpr int HG_TMA_TILE_BYTES = 32 * 128, HG_STAGING_BYTES = 4 * 2 * HG_TMA_TILE_BYTES;
static_assert(HG_STAGING_BYTES >= HG_XPOSE_BYTES, "staging area holds either form");
constexpr uint32_t HG_TMEM_COLS = 512;

// ---- PTX wrappers ------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void *dst_smem, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

// fetch a tensor map (a kernel parameter) into the descriptor cache before the first copy needs it
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_3d(void *dst_smem, const CUtensorMap *map, int x, int y, int z, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
                 : "memory");
}
// shared -> global tensor store (x must be a multiple of 16 bytes; out-of-range parts of the box are clipped)
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, const void *src_smem, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(smem_u32(src_smem)),
                 "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }


__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], M128 x N256 x K16, fp16 inputs, fp32 accumulate
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], M128 x N x K32, int8 inputs, int32 accumulate
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], M128 x N x K32, fp8 inputs (E4M3 or E5M2 by the descriptor), fp32 accumulate
__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tc_ld_32cols(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Bounded mbarrier wait that also gives up as soon as another role has given up.
__device__ __forceinline__ bool mbar_wait_abortable(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    g_device_status = TB200_ERR_TIMEOUT;
    return false;
}

// Shared-memory matrix descriptor (tcgen05), 128-byte swizzle, descriptor version 1.
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) version = 1   bits [61,64) layout = 2 (SWIZZLE_128B)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Tile order: bands of `gm` tile rows, inside a band the tile row changes fastest.  The CTAs that run
// at the same time then share a few A row-panels (which stay in L2 for the whole band) and walk along
// B together, instead of streaming all of A for every couple of B column-panels.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int gm, int &tm, int &tn) {
    const int per_band = gm * tiles_n;
    const int band = tile / per_band;
    const int in_band = tile - band * per_band;
    const int rows_here = min(gm, tiles_m - band * gm);  // the last band may be shorter
    tn = in_band / rows_here;
    tm = band * gm + (in_band - tn * rows_here);
}

// The same walk for a product whose last tile column is narrow (at most half a tile wide: a ragged N, or the four
// columns a shifted B adds): those tiles come after all the others, so that they fall to the CTAs that have a tile
// less than the rest instead of costing every CTA's schedule a whole tile.
__device__ __forceinline__ void tile_coords_edge(int tile, int tiles_m, int tiles_n, int gm, bool edge_last, int &tm, int &tn) {
    if (!edge_last) return tile_coords(tile, tiles_m, tiles_n, gm, tm, tn);
    const int main_tiles = tiles_m * (tiles_n - 1);
    if (tile >= main_tiles) {
        tn = tiles_n - 1, tm = tile - main_tiles;
        return;
    }
    tile_coords(tile, tiles_m, tiles_n - 1, gm, tm, tn);
}

// Instruction descriptor, kind::f16: D fp32, A/B fp16 or bf16, A K-major, B MN-major (N contiguous).
//   [4,6) D format 1 = F32   [7,10) A format 0 = F16, 1 = BF16   [10,13) B format likewise
//   bit 15 A major (0 = K)   bit 16 B major (1 = MN)   [17,23) N >> 3   [24,29) M >> 4
static uint32_t hg_idesc(int m, int n, bool bf16) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// What the epilogue does with a finished accumulator tile:
//     D[row][col] = act(alpha * acc + beta * C[row][col] + bias[col])        (fp32 arithmetic)
// converted to the output type and stored to every destination at dst[p][batch * batch_stride + row * ld + col_off + col].
// One local destination with ld = N is the plain GEMM; several destinations (this GPU's buffer and peer-mapped
// buffers of other GPUs) with ld = the unsharded N and col_off = the first column of this GPU's column block make
// the all-gather of a column-sharded GEMM part of the epilogue.  The fused forms follow the reference's CUTLASS
// epilogues (tornado-cutlass.cu:101-140: act(alpha * A * B + bias) with the bias row broadcast) and its alpha / beta
// GEMMs with fp16 / bf16 outputs (Cutlass.cutlassHgemm, cutlassBgemm).
constexpr int HG_MAX_DST = 8;
struct HgOut {
    void *dst[HG_MAX_DST];
    long long ld, col_off, batch_stride;  // in elements of the output type
    const void *c;                        // source of beta * C: output type, laid out like dst[0] (may be dst[0]); null: none
    const void *bias;                     // [N] of the output type; null: none
    float alpha, beta;
    int ndst;
    int xpose;      // store through the transposition buffer (whole 128-byte lines per row)
    int out_type;   // tb200_gemm_out
    int act;        // tb200_activation
    int tma_store;  // fp32, one dense destination: pieces leave shared memory as TMA tensor stores
    int line_shift; // >= 0: fp32, one destination off a 128-byte line: stores follow the destination's lines (see
                    // hg_epilogue_lines); the number of floats between a line boundary and the first column of a tile
    int line_tma;   // ... and whole lines leave as TMA stores through a map that starts line_cs floats below the
    int line_cs;    // destination (on the line boundary below it)
    int plain;      // alpha == 1, beta == 0, no bias, no activation, fp32: the accumulator is stored as it is
};

// 1 / x by the hardware approximation (1 ulp): the arguments here are 1 + something non-negative.  The IEEE-rounded
// __frcp_rn carries a slow path for denormals behind a branch, which kept the 32 values of a lane from overlapping
// (measured on an epilogue-bound product: 320 us with it for gelu, against 74 us without an activation).
__device__ __forceinline__ float hg_rcp(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// erf to about 2e-7 absolute (Abramowitz & Stegun 7.1.26) in a dozen instructions: the library erff costs
// three times as much, and the epilogue of a tile must finish within the main loop of the next one
__device__ __forceinline__ float hg_erf(float x) {
    const float ax = fabsf(x);
    const float t = hg_rcp(fmaf(0.3275911f, ax, 1.0f));
    const float poly = t * fmaf(t, fmaf(t, fmaf(t, fmaf(t, 1.061405429f, -1.453152027f), 1.421413741f), -0.284496736f), 0.254829592f);
    const float r = 1.0f - poly * __expf(-ax * ax);
    return copysignf(r, x);
}

template <int ACT>
__device__ __forceinline__ float hg_activate(float x) {
    if (ACT == TB200_ACT_RELU) return fmaxf(x, 0.f);
    if (ACT == TB200_ACT_GELU) return 0.5f * x * (1.0f + hg_erf(x * 0.70710678118654752f));
    if (ACT == TB200_ACT_SILU) return x * hg_rcp(1.0f + __expf(-x));
    if (ACT == TB200_ACT_SIGMOID) return hg_rcp(1.0f + __expf(-x));
    if (ACT == TB200_ACT_TANH) {
        const float e = __expf(-2.0f * fabsf(x));  // tanh |x| = (1 - e) / (1 + e), no overflow
        return copysignf((1.0f - e) * hg_rcp(1.0f + e), x);
    }
    if (ACT == TB200_ACT_HARDSWISH) return x * fminf(fmaxf(x + 3.0f, 0.f), 6.0f) * (1.0f / 6.0f);
    return x;
}

// Elements lo .. hi - 1 of the 32 consecutive elements of the output type that start at element index i of p, as
// floats (all lanes may read the same elements: one broadcast transaction per load).  `rows_vec`: row pitches keep
// the 16-byte phase of the base pointer; the base itself is checked here, because an array behind a 24-byte
// header starts 8 bytes off.
template <int OUT>
__device__ __forceinline__ void hg_load32(const void *p, long long i, int lo, int hi, bool rows_vec, float (&f)[32]) {
    if (OUT == TB200_OUT_F32) {
        const float *q = reinterpret_cast<const float *>(p) + i;
        if (rows_vec && lo == 0 && hi == 32 && ((uintptr_t)q & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 v = __ldg(reinterpret_cast<const float4 *>(q) + j);
                f[4 * j] = v.x, f[4 * j + 1] = v.y, f[4 * j + 2] = v.z, f[4 * j + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = (j >= lo && j < hi) ? __ldg(q + j) : 0.f;
        }
    } else {
        const uint16_t *q = reinterpret_cast<const uint16_t *>(p) + i;
        auto cvt = [](uint16_t h) { return OUT == TB200_OUT_F16 ? half_bits_to_float(h) : __uint_as_float((uint32_t)h << 16); };
        if (rows_vec && lo == 0 && hi == 32 && ((uintptr_t)q & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(q) + j);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) f[8 * j + 2 * k] = cvt((uint16_t)(w[k] & 0xFFFF)), f[8 * j + 2 * k + 1] = cvt((uint16_t)(w[k] >> 16));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = (j >= lo && j < hi) ? cvt(__ldg(q + j)) : 0.f;
        }
    }
}

// v = act(alpha * v + beta * C + bias) on the lane's 32 accumulator values (bit patterns of floats)
template <int OUT, int ACT>
__device__ __forceinline__ void hg_fuse32(uint32_t (&v)[32], const HgOut &out, long long at, int col0, int lo, int hi, bool row_ok, bool vec) {
    float x[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = out.alpha * __uint_as_float(v[j]);
    if (out.beta != 0.f && out.c && row_ok) {
        float c[32];
        hg_load32<OUT>(out.c, at, lo, hi, vec, c);
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] = fmaf(out.beta, c[j], x[j]);
    }
    if (out.bias) {
        float b[32];
        hg_load32<OUT>(out.bias, (long long)col0, lo, hi, vec, b);
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] += b[j];
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(hg_activate<ACT>(x[j]));
}

template <int OUT>
__device__ __forceinline__ void hg_fuse32_act(uint32_t (&v)[32], const HgOut &out, long long at, int col0, int lo, int hi, bool row_ok, bool vec) {
    switch (out.act) {
        case TB200_ACT_RELU: return hg_fuse32<OUT, TB200_ACT_RELU>(v, out, at, col0, lo, hi, row_ok, vec);
        case TB200_ACT_GELU: return hg_fuse32<OUT, TB200_ACT_GELU>(v, out, at, col0, lo, hi, row_ok, vec);
        case TB200_ACT_SILU: return hg_fuse32<OUT, TB200_ACT_SILU>(v, out, at, col0, lo, hi, row_ok, vec);
        case TB200_ACT_SIGMOID: return hg_fuse32<OUT, TB200_ACT_SIGMOID>(v, out, at, col0, lo, hi, row_ok, vec);
        case TB200_ACT_TANH: return hg_fuse32<OUT, TB200_ACT_TANH>(v, out, at, col0, lo, hi, row_ok, vec);
        case TB200_ACT_HARDSWISH: return hg_fuse32<OUT, TB200_ACT_HARDSWISH>(v, out, at, col0, lo, hi, row_ok, vec);
        default: return hg_fuse32<OUT, TB200_ACT_NONE>(v, out, at, col0, lo, hi, row_ok, vec);
    }
}

__device__ __forceinline__ uint16_t hg_to_out16(float x, int out_type) {
    if (out_type == TB200_OUT_F16) return __half_as_ushort(__float2half_rn(x));
    return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}

// fp32 results into ONE destination whose tile columns do not start on a 128-byte line (an array behind a 16- or
// 24-byte header, or columns shifted with B).  Storing each 32 x 32 piece where it falls writes every row as 128
// bytes that straddle two lines, with part-written 32-byte sectors at both ends; measured on products whose
// epilogue dominates (K = 256, 8192 x 8192 results): 304 us through 8-byte stores at an 8-byte phase and 115 us
// through TMA stores 16 bytes off a line, against 75 us on a line.  Here the stores follow the destination's lines
// instead: the warp's two staging tiles form a sliding window over the row -- piece c of the accumulator writes its
// first 32 - sh columns behind the sh columns that piece c - 1 left in tile c % 2, and its last sh columns into the
// other tile -- and tile c % 2 then leaves as whole 128-byte lines: one TMA tensor store through a map laid over the
// line boundary below the destination (a dense destination), else eight lanes per row, 16 bytes each.  Only the
// first and the last segment of a tile (and segments cut by the matrix edge) are partial and leave as 8-byte pieces.
//   sh        floats between the line boundary below and the tile's first column (even, 0 .. 30), the same for all tiles
template <int NCHUNK>
__device__ __forceinline__ void hg_epilogue_lines(const HgOut &out, const CUtensorMap *map_d, uint32_t taddr, int row0, int n0, int batch, int M,
                                                  int N, int rows_vec, unsigned char *staging, int lane) {
    const int row = row0 + lane;
    const int sh = out.line_shift;
    const long long boff = (long long)batch * out.batch_stride;
    float *dst = reinterpret_cast<float *>(out.dst[0]);
#pragma unroll 1
    for (int c = 0; c <= NCHUNK; ++c) {
        const int col0 = n0 + c * 32;
        if (c < NCHUNK && col0 < N && col0 + 32 > 0) {  // warp-uniform; columns beyond the matrix were not even multiplied
            uint32_t v[32];
            tc_ld_32cols(taddr + c * 32, v);
            tc_wait_ld();
            if (!out.plain) {
                const int lo = col0 < 0 ? -col0 : 0, hi = col0 + 32 <= N ? 32 : N - col0;
                const long long at = boff + (long long)row * out.ld + out.col_off + col0;
                hg_fuse32_act<TB200_OUT_F32>(v, out, at, col0, lo, hi, row < M, rows_vec != 0);
            }
            // the TMA stores that read the two tiles (segments c - 1 and c - 2) were issued before the accumulator was read
            if (out.line_tma) {
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
            }
            // lane r writes row r: column i of the piece goes to position (sh + i) % 32 of tile (c + (sh + i) / 32) % 2
            // (rows of 128 bytes, 16-byte units XOR-swizzled by the row: the layout of a 128-byte-swizzled tensor map)
            if ((sh & 3) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const int q = sh + i, pos = q & 31;
                    unsigned char *tile = staging + ((c + (q >> 5)) & 1) * HG_TMA_TILE_BYTES;
                    *reinterpret_cast<uint4 *>(tile + lane * 128 + (((pos >> 2) ^ (lane & 7)) << 4)) = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const int q = sh + i, pos = q & 31;
                    unsigned char *tile = staging + ((c + (q >> 5)) & 1) * HG_TMA_TILE_BYTES;
                    *reinterpret_cast<uint2 *>(tile + lane * 128 + (((pos >> 2) ^ (lane & 7)) << 4) + (pos & 3) * 4) = make_uint2(v[i], v[i + 1]);
                }
            }
            if (out.line_tma) fence_async_shared();  // generic-proxy writes before the TMA engine's reads
        }
        __syncwarp();
        // segment c: tile columns 32 c - sh .. 32 c - sh + 31, of which this tile owns [own_lo, own_hi)
        const int colbase = n0 + c * 32 - sh;
        const int own_lo = c == 0 ? sh : 0, own_hi = c == NCHUNK ? sh : 32;
        const int jlo = max(own_lo, -colbase), jhi = min(own_hi, N - colbase);  // both even
        const unsigned char *tile = staging + (c & 1) * HG_TMA_TILE_BYTES;
        if (jlo == 0 && jhi == 32 && out.line_tma) {
            // x = column + line_cs is a multiple of 32: whole lines; rows beyond M are clipped by the map
            if (lane == 0 && row0 < M) {
                tma_store_3d(map_d, tile, colbase + out.line_cs, row0, batch);
                tma_store_commit();
            }
        } else if (jlo == 0 && jhi == 32) {
            // eight lanes store one row's line
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int rl = i * 4 + (lane >> 3), u = lane & 7;
                const uint4 val = *reinterpret_cast<const uint4 *>(tile + rl * 128 + ((u ^ (rl & 7)) << 4));
                const int grow = row0 + rl;
                if (grow < M) *reinterpret_cast<uint4 *>(dst + boff + (long long)grow * out.ld + out.col_off + colbase + 4 * u) = val;
            }
        } else if (jlo < jhi) {
            // sixteen lanes per row, 8 bytes each, inside [jlo, jhi)
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int rl = i * 2 + (lane >> 4), j = (lane & 15) * 2;
                const uint2 val = *reinterpret_cast<const uint2 *>(tile + rl * 128 + (((j >> 2) ^ (rl & 7)) << 4) + (j & 3) * 4);
                const int grow = row0 + rl;
                if (grow < M && j >= jlo && j < jhi) *reinterpret_cast<uint2 *>(dst + boff + (long long)grow * out.ld + out.col_off + colbase + j) = val;
            }
        }
        __syncwarp();  // the tile is rewritten two pieces later
    }
}

// Epilogue of one warp for one accumulator tile: NCHUNK pieces of 32 rows (one per lane) x 32 columns.
//   taddr     tensor-memory address of the warp's lane quarter, first column of the tile's accumulator
//   row0      first row of the warp's 32 rows, n0 first column of the tile (-4 for the first tile of a product whose
//             B sits 8 bytes past a 16-byte boundary), batch index of the matrix
//   rows_vec  row pitches, column offset and batch stride keep the 16-byte phase of a destination's base pointer;
//             the pointers themselves are checked here (an array behind a 24-byte header starts 8 bytes off)
//   staging   this warp's part of the staging area (HG_STAGING_BYTES / 4 bytes, 1024-byte aligned)
//   nstores   running count of this warp's TMA stores (selects the staging tile)
template <int NCHUNK>
__device__ __forceinline__ void hg_epilogue_tile(const HgOut &out, const CUtensorMap *map_d, uint32_t taddr, int row0, int n0, int batch,
                                                 int M, int N, int rows_vec, unsigned char *staging, int lane, uint32_t &nstores) {
    if (out.line_shift >= 0) {
        hg_epilogue_lines<NCHUNK>(out, map_d, taddr, row0, n0, batch, M, N, rows_vec, staging, lane);
        return;
    }
    const int row = row0 + lane;
    const long long boff = (long long)batch * out.batch_stride;
#pragma unroll 1
    for (int c = 0; c < NCHUNK; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= N || col0 + 32 <= 0) continue;  // warp-uniform; columns beyond the matrix were not even multiplied
        uint32_t v[32];
        tc_ld_32cols(taddr + c * 32, v);
        tc_wait_ld();
        const int lo = col0 < 0 ? -col0 : 0, hi = col0 + 32 <= N ? 32 : N - col0;  // columns col0 + lo .. col0 + hi - 1 exist
        const bool full = lo == 0 && hi == 32;
        const long long at = boff + (long long)row * out.ld + out.col_off + col0;  // element index of (row, col0)
        if (!out.plain) {
            if (out.out_type == TB200_OUT_F32) hg_fuse32_act<TB200_OUT_F32>(v, out, at, col0, lo, hi, row < M, rows_vec != 0);
            else if (out.out_type == TB200_OUT_F16) hg_fuse32_act<TB200_OUT_F16>(v, out, at, col0, lo, hi, row < M, rows_vec != 0);
            else hg_fuse32_act<TB200_OUT_BF16>(v, out, at, col0, lo, hi, row < M, rows_vec != 0);
        }
        if (out.out_type != TB200_OUT_F32) {
            // 16-bit outputs: the lane's 32 values are 64 contiguous bytes of its row
            if (row < M) {
                for (int p = 0; p < out.ndst; ++p) {
                    uint16_t *dst = reinterpret_cast<uint16_t *>(out.dst[p]) + at;
                    const uintptr_t phase = (uintptr_t)dst & 15;
                    if (rows_vec && full && (phase & 7) == 0) {
                        uint32_t w[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            w[i] = (uint32_t)hg_to_out16(__uint_as_float(v[2 * i]), out.out_type) |
                                   ((uint32_t)hg_to_out16(__uint_as_float(v[2 * i + 1]), out.out_type) << 16);
                        if (phase == 0) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4 *>(dst + 8 * j) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j) *reinterpret_cast<uint2 *>(dst + 4 * j) = make_uint2(w[2 * j], w[2 * j + 1]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j >= lo && j < hi) dst[j] = hg_to_out16(__uint_as_float(v[j]), out.out_type);
                    }
                }
            }
            continue;
        }
        if (out.tma_store) {
            // (the host enables this only for columns that start at 0 and 16-byte aligned destinations)
            // lane r writes row r of a 32 x 32 tile (128-byte rows, 16-byte pieces XOR-swizzled by the row: the
            // layout of a 128-byte-swizzled tensor map), then one lane hands the tile to the TMA engine
            unsigned char *tile = staging + (nstores & 1) * HG_TMA_TILE_BYTES;
            if (lane == 0) tma_store_wait_read<1>();  // the store that last read this tile has finished reading
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4 *>(tile + lane * 128 + ((j ^ (lane & 7)) << 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            fence_async_shared();
            __syncwarp();
            if (lane == 0 && row0 < M) {
                tma_store_3d(map_d, tile, col0, row0, batch);
                tma_store_commit();
            }
            ++nstores;
            continue;
        }
        float *const *dsts = reinterpret_cast<float *const *>(out.dst);
        // whole 128-byte lines per row through the transposition buffer: for several destinations, and for a
        // destination 8 bytes past a 16-byte boundary (an array behind a 24-byte header), where the alternative is
        // one 8-byte store per lane and row.  All rows share the phase of the base pointer (rows_vec).
        uintptr_t phase = (uintptr_t)(dsts[0] + at) & 15;
        for (int p = 1; p < out.ndst; ++p)
            if ((((uintptr_t)(dsts[p] + at)) & 15) != phase) phase = 1;  // mixed
        if (rows_vec && full && ((phase == 0 && out.xpose) || phase == 8)) {
            float *stg = reinterpret_cast<float *>(staging);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *reinterpret_cast<float4 *>(stg + lane * HG_XPOSE_PITCH + 4 * j) =
                    make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
            __syncwarp();
            if (phase == 0) {
                // eight lanes store one row's 128 bytes
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rl = i * 4 + (lane >> 3), c4 = (lane & 7) * 4;
                    const float4 val = *reinterpret_cast<const float4 *>(stg + rl * HG_XPOSE_PITCH + c4);
                    const int grow = row0 + rl;
                    if (grow < M) {
                        for (int p = 0; p < out.ndst; ++p)  // plain stores, to local or peer-mapped memory
                            *reinterpret_cast<float4 *>(dsts[p] + boff + (long long)grow * out.ld + out.col_off + col0 + c4) = val;
                    }
                }
            } else {
                // sixteen lanes store one row's 128 bytes as 8-byte pieces
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int rl = i * 2 + (lane >> 4), c2 = (lane & 15) * 2;
                    const float2 val = *reinterpret_cast<const float2 *>(stg + rl * HG_XPOSE_PITCH + c2);
                    const int grow = row0 + rl;
                    if (grow < M) {
                        for (int p = 0; p < out.ndst; ++p)
                            *reinterpret_cast<float2 *>(dsts[p] + boff + (long long)grow * out.ld + out.col_off + col0 + c2) = val;
                    }
                }
            }
            __syncwarp();
        } else if (row < M) {
            for (int p = 0; p < out.ndst; ++p) {  // plain stores, to local or peer-mapped memory
                float *dst = dsts[p] + at;
                const uintptr_t phase = (uintptr_t)dst & 15;
                if (rows_vec && full && phase == 0) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float4 *>(dst + 4 * j) =
                            make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                } else if (rows_vec && full && phase == 8) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) *reinterpret_cast<float2 *>(dst + 2 * j) = make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (j >= lo && j < hi) dst[j] = __uint_as_float(v[j]);
                }
            }
        }
    }
}

// BN = 256: the standard tile.  BN = 128: for products with too few 128 x 256 tiles to fill the SMs (six ring
// stages instead of four).  `idesc` carries the operand formats (fp16 or bf16) and the tile shape.
template <int BN>
struct HgTile {
    static constexpr int STAGES = BN == 256 ? 4 : 6;
    static constexpr int B_BYTES = HG_BK * BN * 2;
    static constexpr int STAGE_BYTES = HG_A_BYTES + B_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + HG_STAGING_BYTES;
    static constexpr uint32_t TMEM_COLS = 2 * BN;
};

// Operands 8 bytes past a 16-byte boundary (TornadoVM arrays behind a 24-byte header, the reference launcher's
// default mode) cannot be the base of a tensor map, and a TMA copy cannot start 8 bytes into a 16-byte unit either.
// And operands that are 16-byte aligned but off a 128-byte line (the same arrays behind a 16-byte header) make every
// 128-byte row of a TMA box straddle two lines (measured at 8192^3: 842 instead of 1350 TFLOP/s).  The maps are
// therefore laid over an aligned address BELOW the array -- the 128-byte line boundary when every row keeps the phase,
// else the 16-byte boundary -- which shifts the matrix by kshift / nshift elements (a multiple of 4 below 64) along
// its contiguous dimension, and the kernel works in the shifted coordinates:
//   A (K contiguous): element k of a row appears at k' = k + kshift; K blocks cover k' = 0 .. K + kshift - 1, the rows
//     of B are fetched from k' - kshift (a negative row coordinate is filled with zeros), and the kshift halves in
//     front of every row of the first K block -- bytes that belong to the previous row or lie before the array --
//     are overwritten with zeros in shared memory before the first MMA reads them;
//   B (N contiguous): column n appears at n' = n + nshift; tiles cover n' = 0 .. N + nshift - 1 and the epilogue
//     stores tile column n' to column n' - nshift, skipping the nshift columns in front of the first tile.
// K8 = 1 / 2: the same pipeline for 8-bit operands -- int8 with int32 accumulation (tcgen05.mma.kind::i8) or fp8
// with fp32 accumulation (kind::f8f6f4, E4M3 / E5M2 chosen by the instruction descriptor); K = 32 per instruction,
// 128 elements per 128-byte swizzled row.  Both operands are K-major there: A[m][k] as it is, B as its transpose
// Bt[n][k] (the caller's [k][n] matrix is transposed once into workspace memory), so a stage is 128 rows of A and
// BN rows of Bt, 128 bytes each -- the byte sizes of the 16-bit stage.
template <int BN, int K8 = 0>
__global__ void __launch_bounds__(HG_THREADS, 1)
hgemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_d,
                const __grid_constant__ HgOut out, int M, int N, int K, int batches, int rows_vec, int gm, uint32_t idesc, int kshift, int nshift) {
    using TL = HgTile<BN>;
    constexpr int STAGES = TL::STAGES;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t acc_full_bar[2];
    __shared__ __align__(8) uint64_t acc_empty_bar[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    // the swizzled tiles need 1024-byte aligned bases
    unsigned char *tiles = reinterpret_cast<unsigned char *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + HG_BM - 1) / HG_BM, tiles_n = (N + nshift + BN - 1) / BN;
    const int tiles_per_matrix = tiles_m * tiles_n;
    const int num_tiles = tiles_per_matrix * batches;
    constexpr bool I8 = K8 != 0;                  // 8-bit operands
    constexpr int BKE = I8 ? 2 * HG_BK : HG_BK;  // elements of K per stage (128 bytes)
    const int k_blocks = (K + kshift + BKE - 1) / BKE;
    const int edge_cols = (N + nshift) - (tiles_n - 1) * BN;  // columns of the last tile column
    const bool edge_last = !I8 && batches == 1 && tiles_n > 1 && edge_cols <= BN / 2;

    if (threadIdx.x == 32) {  // descriptor fetches overlap the set-up below
        tma_prefetch_map(&map_a);
        tma_prefetch_map(&map_b);
        if (out.tma_store || out.line_tma) tma_prefetch_map(&map_d);
    }
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full_bar[i], 1);
            mbar_init(&acc_empty_bar[i], 4);  // one arrival per epilogue warp
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        // whole warp: allocate the tensor-memory columns of two 128 x BN fp32 accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(TL::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abortp = &abort_flag;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int batch = tile / tiles_per_matrix;
                int tm, tn;
                tile_coords_edge(tile - batch * tiles_per_matrix, tiles_m, tiles_n, gm, edge_last, tm, tn);
                const int m0 = tm * HG_BM, n0 = tn * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t use = it / STAGES;
                    if (use > 0) {
                        ok = mbar_wait_abortable(&empty_bar[s], (use - 1) & 1, abortp);
                        if (!ok) break;
                    }
                    unsigned char *a_dst = tiles + (size_t)s * TL::STAGE_BYTES;
                    unsigned char *b_dst = a_dst + HG_A_BYTES;
                    if (I8) {
                        mbar_expect_tx(&full_bar[s], TL::STAGE_BYTES);
                        tma_load_3d(a_dst, &map_a, kb * BKE, m0, batch, &full_bar[s]);
                        tma_load_3d(b_dst, &map_b, kb * BKE, n0, batch, &full_bar[s]);  // BN rows of Bt, one box
                    } else {
                        // a tile at the right edge fetches only the 64-column boxes that hold columns of the matrix
                        const int boxes = min(BN / 64, (N + nshift - n0 + 63) / 64);
                        mbar_expect_tx(&full_bar[s], HG_A_BYTES + boxes * (HG_BK * 128));
                        tma_load_3d(a_dst, &map_a, kb * BKE, m0, batch, &full_bar[s]);
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            if (j < boxes) tma_load_3d(b_dst + j * (HG_BK * 128), &map_b, n0 + j * 64, kb * HG_BK - kshift, batch, &full_bar[s]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // one lane issues; with a shifted A the whole warp walks the loop, because all lanes clear the bytes in
        // front of the rows of every tile's first K block
        if (lane == 0 || kshift) {
            uint32_t it = 0, local_tile = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
                const uint32_t acc = local_tile & 1, acc_use = local_tile >> 1;
                if (acc_use > 0) {
                    ok = mbar_wait_abortable(&acc_empty_bar[acc], (acc_use - 1) & 1, abortp);
                    if (kshift) ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t d_tmem = tmem_base + acc * BN;
                // a tile at the right edge multiplies only as many columns (a multiple of 16) as the matrix has left
                uint32_t idesc_tile = idesc;
                if (!I8) {
                    const int tile_in_matrix = tile - (tile / tiles_per_matrix) * tiles_per_matrix;
                    int tm, tn;
                    tile_coords_edge(tile_in_matrix, tiles_m, tiles_n, gm, edge_last, tm, tn);
                    const int left = N + nshift - tn * BN;
                    if (left < BN) idesc_tile = (idesc & ~(0x3Fu << 17)) | ((uint32_t)(((left + 15) & ~15) >> 3) << 17);
                }
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait_abortable(&full_bar[s], (it / STAGES) & 1, abortp);
                    if (kshift) ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    unsigned char *a_tile = tiles + (size_t)s * TL::STAGE_BYTES;
                    if (kshift && kb == 0) {
                        // row r keeps its 16-byte piece j at position j ^ (r % 8) of its 128 bytes (128-byte swizzle);
                        // the first 2 * kshift bytes of the row (whole pieces, then possibly the first 8 bytes of the
                        // next one) are the halves in front of the row
                        const int zbytes = I8 ? kshift : 2 * kshift;  // kshift counts elements
                        const int zfull = zbytes >> 4, zhalf = zbytes & 8;
#pragma unroll
                        for (int r = lane; r < HG_BM; r += 32) {
                            unsigned char *rowp = a_tile + r * 128;
                            for (int j = 0; j < zfull; ++j) *reinterpret_cast<uint4 *>(rowp + ((j ^ (r & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                            if (zhalf) *reinterpret_cast<uint2 *>(rowp + ((zfull ^ (r & 7)) << 4)) = make_uint2(0u, 0u);
                        }
                        fence_async_shared();  // generic-proxy writes before the tensor core's reads
                        __syncwarp();
                    }
                    tc_fence_after();
                    if (lane == 0) {
                        const uint32_t a_addr = smem_u32(a_tile);
                        const uint32_t b_addr = a_addr + HG_A_BYTES;
                        // A: K-major, rows of 128 bytes, 8-row groups 1024 bytes apart
                        const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024);
                        // B: N contiguous; 64-column boxes HG_BK*128 bytes apart, 8-k-row groups 1024 bytes apart
                        // (int8: Bt is K-major like A)
                        const uint64_t b_desc = I8 ? make_smem_desc(b_addr, 16, 1024) : make_smem_desc(b_addr, HG_BK * 128, 1024);
#pragma unroll
                        for (int k16 = 0; k16 < HG_BK / 16; ++k16) {
                            // A advances 32 bytes along K per instruction; B advances 16 k-rows = 2048 bytes (int8: 32 bytes along K)
                            if (K8 == 1) tc_mma_i8(d_tmem, a_desc + (uint64_t)(k16 * 2), b_desc + (uint64_t)(k16 * 2), idesc_tile, (kb > 0 || k16 > 0) ? 1u : 0u);
                            else if (K8 == 2) tc_mma_f8(d_tmem, a_desc + (uint64_t)(k16 * 2), b_desc + (uint64_t)(k16 * 2), idesc_tile, (kb > 0 || k16 > 0) ? 1u : 0u);
                            else tc_mma_f16(d_tmem, a_desc + (uint64_t)(k16 * 2), b_desc + (uint64_t)(k16 * 128), idesc_tile, (kb > 0 || k16 > 0) ? 1u : 0u);
                        }
                        tc_commit(&empty_bar[s]);  // arrives once the MMAs above have read this stage
                    }
                }
                if (ok && lane == 0) tc_commit(&acc_full_bar[acc]);  // accumulator complete
            }
        }
    } else if (warp >= 2 && warp < 6) {
        // ---------------- epilogue: warps 2..5, TMEM lane quarter = warp % 4 ----------------
        const int quarter = warp & 3;
        unsigned char *staging = tiles + (size_t)STAGES * TL::STAGE_BYTES + (warp - 2) * (HG_STAGING_BYTES / 4);
        uint32_t local_tile = 0, nstores = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
            const uint32_t acc = local_tile & 1, acc_use = local_tile >> 1;
            const int batch = tile / tiles_per_matrix;
            int tm, tn;
            tile_coords_edge(tile - batch * tiles_per_matrix, tiles_m, tiles_n, gm, edge_last, tm, tn);
            ok = __all_sync(0xffffffffu, mbar_wait_abortable(&acc_full_bar[acc], acc_use & 1, abortp));
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
            hg_epilogue_tile<BN / 32>(out, &map_d, taddr, tm * HG_BM + quarter * 32, tn * BN - nshift, batch, M, N, rows_vec, staging, lane, nstores);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
        }
        if (lane == 0) tma_store_wait_read<0>();  // shared memory stays valid until the last store has read it
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TL::TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------
// Two-CTA variant: a cluster of two CTAs (an SM pair) computes one 256 x 256 tile.
// Each CTA stages its own 128 rows of A and its own 128 columns of B (plain TMA
// loads, no multicast; both CTAs' loads signal the leader's mbarrier), the leader
// issues tcgen05.mma.cta_group::2 (M256 N256 K16), which reads B halves from both
// CTAs, and every CTA keeps the accumulator of its 128 rows in its own tensor
// memory.  Per SM this halves the shared-memory traffic for B and leaves room for
// a 6-stage ring.
// ---------------------------------------------------------------------------------
constexpr int H2_STAGES = 6;
constexpr int H2_B_BYTES = HG_BK * 128 * 2;                 // 16 KB: two 64-column boxes
constexpr int H2_STAGE_BYTES = HG_A_BYTES + H2_B_BYTES;     // 32 KB per CTA and stage
constexpr int H2_SMEM_BYTES = H2_STAGES * H2_STAGE_BYTES + 1024 + HG_STAGING_BYTES;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void *local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of one CTA of a pair; completion bytes go to the mbarrier at `bar_cluster_addr` (the leader's)
__device__ __forceinline__ void tma_load_3d_pair(void *dst_smem, const CUtensorMap *map, int x, int y, int z, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            smem_u32(dst_smem)),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar_cluster_addr)
        : "memory");
}
__device__ __forceinline__ void tc2_commit_both(uint64_t *bar) {  // arrives on `bar` in both CTAs of the pair
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     smem_u32(bar)),
                 "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void tc2_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(HG_THREADS, 1)
hgemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_d, const __grid_constant__ HgOut out, int M, int N, int K, int batches, int rows_vec,
                 int gm, uint32_t idesc, int kshift, int nshift) {
    // Shifted operands (see hgemm_tc_kernel): map_a and map_b lie over the 128-byte line below A and B.  Only
    // 16-byte aligned A (kshift a multiple of 8): the first K block of A then comes through map_a0, which lies over
    // A itself, from column -kshift -- the TMA engine fills the columns in front of the row with zeros, so no CTA has
    // to clear anything in shared memory (with A 8 bytes off, four halves per row would still have to be cleared, in
    // both CTAs, before the leader's MMA: those products take the single-CTA kernel).
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[H2_STAGES];   // used in the leader only
    __shared__ __align__(8) uint64_t empty_bar[H2_STAGES];  // one per CTA, signalled by the leader's commits
    __shared__ __align__(8) uint64_t acc_full_bar[2];       // one per CTA
    __shared__ __align__(8) uint64_t acc_empty_bar[2];      // leader only: 8 epilogue warps of the pair arrive
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    unsigned char *tiles = reinterpret_cast<unsigned char *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int tiles_m = (M + 255) / 256, tiles_n = (N + nshift + 255) / 256;
    const int tiles_per_matrix = tiles_m * tiles_n;
    const int num_tiles = tiles_per_matrix * batches;
    const int k_blocks = (K + kshift + HG_BK - 1) / HG_BK;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

    if (threadIdx.x == 32) {  // descriptor fetches overlap the set-up below
        tma_prefetch_map(&map_a);
        if (kshift) tma_prefetch_map(&map_a0);
        tma_prefetch_map(&map_b);
        if (out.tma_store || out.line_tma) tma_prefetch_map(&map_d);
    }
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < H2_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full_bar[i], 1);
            mbar_init(&acc_empty_bar[i], 8);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(HG_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abortp = &abort_flag;

    if (warp == 0) {
        // ---------------- TMA producer (one lane in each CTA) ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
                const int batch = tile / tiles_per_matrix;
                int tm, tn;
                tile_coords(tile - batch * tiles_per_matrix, tiles_m, tiles_n, gm, tm, tn);
                const int m0 = tm * 256 + (int)rank * 128;
                const int n0 = tn * 256 + (int)rank * 128;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % H2_STAGES;
                    const uint32_t use = it / H2_STAGES;
                    if (use > 0) {
                        ok = mbar_wait_abortable(&empty_bar[s], (use - 1) & 1, abortp);
                        if (!ok) break;
                    }
                    unsigned char *a_dst = tiles + (size_t)s * H2_STAGE_BYTES;
                    unsigned char *b_dst = a_dst + HG_A_BYTES;
                    if (leader) mbar_expect_tx(&full_bar[s], 2 * H2_STAGE_BYTES);  // bytes of both CTAs
                    const uint32_t bar = map_to_cta(&full_bar[s], 0);
                    if (kb == 0 && kshift) tma_load_3d_pair(a_dst, &map_a0, -kshift, m0, batch, bar);
                    else tma_load_3d_pair(a_dst, &map_a, kb * HG_BK, m0, batch, bar);
                    tma_load_3d_pair(b_dst, &map_b, n0, kb * HG_BK - kshift, batch, bar);
                    tma_load_3d_pair(b_dst + HG_BK * 128, &map_b, n0 + 64, kb * HG_BK - kshift, batch, bar);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (leader && lane == 0) {
            uint32_t it = 0, local_tile = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += npairs, ++local_tile) {
                const uint32_t acc = local_tile & 1, acc_use = local_tile >> 1;
                if (acc_use > 0) {
                    ok = mbar_wait_abortable(&acc_empty_bar[acc], (acc_use - 1) & 1, abortp);
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t d_tmem = tmem_base + acc * 256;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % H2_STAGES;
                    ok = mbar_wait_abortable(&full_bar[s], (it / H2_STAGES) & 1, abortp);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + (size_t)s * H2_STAGE_BYTES);
                    const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024);
                    const uint64_t b_desc = make_smem_desc(a_addr + HG_A_BYTES, HG_BK * 128, 1024);
#pragma unroll
                    for (int k16 = 0; k16 < HG_BK / 16; ++k16)
                        tc2_mma_f16(d_tmem, a_desc + (uint64_t)(k16 * 2), b_desc + (uint64_t)(k16 * 128), idesc,
                                    (kb > 0 || k16 > 0) ? 1u : 0u);
                    tc2_commit_both(&empty_bar[s]);  // frees this stage in both CTAs
                }
                if (ok) tc2_commit_both(&acc_full_bar[acc]);
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 of each CTA, its own 128 rows ----------------
        const int quarter = warp & 3;
        unsigned char *staging = tiles + (size_t)H2_STAGES * H2_STAGE_BYTES + (warp - 2) * (HG_STAGING_BYTES / 4);
        uint32_t local_tile = 0, nstores = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += npairs, ++local_tile) {
            const uint32_t acc = local_tile & 1, acc_use = local_tile >> 1;
            const int batch = tile / tiles_per_matrix;
            int tm, tn;
            tile_coords(tile - batch * tiles_per_matrix, tiles_m, tiles_n, gm, tm, tn);
            ok = __all_sync(0xffffffffu, mbar_wait_abortable(&acc_full_bar[acc], acc_use & 1, abortp));
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * 256;
            hg_epilogue_tile<8>(out, &map_d, taddr, tm * 256 + (int)rank * 128 + quarter * 32, tn * 256 - nshift, batch, M, N, rows_vec, staging, lane, nstores);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(&acc_empty_bar[acc], 0));
        }
        if (lane == 0) tma_store_wait_read<0>();  // shared memory stays valid until the last store has read it
    }

    // ---------------- teardown: nobody leaves while the peer may still signal or read ----------------
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(HG_TMEM_COLS) : "memory");
    }
}

// ---- host side -----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    // resolved once per process (thread-safe initialisation of a local static); tb200_prepare calls this
    // before any stream capture
    static const EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            return reinterpret_cast<EncodeTiledFn>(p);
        cudaGetLastError();
        return (EncodeTiledFn) nullptr;
    }();
    return fn;
}

int hgemm_prepare_driver() { return encode_tiled_fn() ? TB200_OK : TB200_ERR_DRIVER; }

// 3-D tensor map over `batches` row-major matrices of `outer` rows x `inner` elements, rows `pitch` elements apart
// (0: inner; a shifted matrix is 4 elements wider than its pitch, so its rows overlap) and matrices `batch_stride`
// elements apart; box of box_inner x box_rows x 1, 128-byte swizzle (box_inner elements = 128 bytes).
// Encoding goes through the driver; a task dispatches the same operands again and again, so the last maps of
// the calling thread are kept and looked up by their full key (pointer, shape, type, box).
struct MapKey {
    const void *base;
    uint64_t inner, outer, batches, batch_stride, pitch;
    uint32_t box_inner, box_rows, type;
    bool operator==(const MapKey &o) const {
        return base == o.base && inner == o.inner && outer == o.outer && batches == o.batches && batch_stride == o.batch_stride && pitch == o.pitch &&
               box_inner == o.box_inner && box_rows == o.box_rows && type == o.type;
    }
};
struct MapCache {
    static constexpr int N = 16;
    MapKey key[N];
    CUtensorMap map[N];
    bool used[N] = {};
    int next = 0;
};
static thread_local MapCache t_maps;

static int make_map(CUtensorMap *map, const void *base, CUtensorMapDataType type, int elem_bytes, uint64_t inner, uint64_t outer,
                    uint64_t batches, uint64_t batch_stride, uint32_t box_inner, uint32_t box_rows, uint64_t pitch = 0) {
    if (!pitch) pitch = inner;
    const MapKey key{base, inner, outer, batches, batch_stride, pitch, box_inner, box_rows, (uint32_t)type};
    MapCache &mc = t_maps;
    for (int i = 0; i < MapCache::N; ++i)
        if (mc.used[i] && mc.key[i] == key) {
            *map = mc.map[i];
            return TB200_OK;
        }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return TB200_ERR_DRIVER;
    cuuint64_t dims[3] = {inner, outer, batches};
    // a single matrix: the third dimension has extent 1 and its stride only has to be a valid multiple of 16 bytes
    cuuint64_t strides[2] = {pitch * elem_bytes, (batches > 1 ? batch_stride : pitch * outer) * elem_bytes};
    cuuint32_t box[3] = {box_inner, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, type, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return TB200_ERR_DRIVER;
    const int slot = mc.next;
    mc.next = (mc.next + 1) % MapCache::N;
    mc.key[slot] = key, mc.map[slot] = *map, mc.used[slot] = true;
    return TB200_OK;
}

struct HgProblem {
    int m, n, k, batches;
    const uint16_t *a, *b;
    long long stride_a, stride_b;  // elements between consecutive matrices (batches > 1)
    bool bf16;
};

static int out_elem_bytes(int out_type) { return out_type == TB200_OUT_F32 ? 4 : 2; }

// Floats between the 128-byte line below a tile's first column and that column (hg_epilogue_lines), the same for every
// tile and row when the row pitch and the batch stride are whole lines; -1: that epilogue does not apply.
static int line_shift_of(const HgOut &out, int n, int nshift, int batches) {
    if (out.out_type != TB200_OUT_F32 || out.ndst != 1 || !aligned_to(out.dst[0], 8)) return -1;
    if (out.ld % 32 != 0 || out.col_off % 2 != 0 || n % 2 != 0 || (batches > 1 && out.batch_stride % 32 != 0)) return -1;
    const long long x0 = (long long)(((uintptr_t)out.dst[0] & 127) / 4) + out.col_off - nshift;
    return (int)(((x0 % 32) + 32) % 32);
}

// D = act(alpha * A * B + beta * C + bias) with the tile stores described by `out`.
static int hgemm_launch(const HgProblem &pr, HgOut out, tb200_stream_t stream) {
    const int m = pr.m, n = pr.n, k = pr.k;
    out.xpose = out.ndst >= option_value(TB200_OPT_HGEMM_LINE_STORES);
    if (m < 0 || n < 0 || k < 0 || pr.batches < 1) return TB200_ERR_INVALID_ARG;
    if (m == 0 || n == 0) return TB200_OK;
    if (k > 0 && (!pr.a || !pr.b)) return TB200_ERR_INVALID_ARG;
    if (out.ndst < 1 || out.ndst > HG_MAX_DST || out.ld < n || out.col_off < 0 || out.col_off > out.ld - n) return TB200_ERR_INVALID_ARG;
    if (out.out_type < TB200_OUT_F32 || out.out_type > TB200_OUT_BF16 || out.act < TB200_ACT_NONE || out.act > TB200_ACT_HARDSWISH) return TB200_ERR_INVALID_ARG;
    if (pr.batches > 1 && (pr.stride_a < (long long)m * k || pr.stride_b < (long long)k * n || out.batch_stride < (long long)m * out.ld)) return TB200_ERR_INVALID_ARG;
    if (!aligned_to(pr.a, 2) || !aligned_to(pr.b, 2)) return TB200_ERR_ALIGNMENT;
    const int eb = out_elem_bytes(out.out_type);
    const int per16 = 16 / eb;  // output elements per 16 bytes
    // row pitches keep the 16-byte phase of a destination; the kernel looks at the pointers themselves
    const bool rows_vec = n % per16 == 0 && out.ld % per16 == 0 && out.col_off % per16 == 0 && out.batch_stride % per16 == 0;
    bool dst_aligned = true;
    for (int p = 0; p < out.ndst; ++p) {
        if (!out.dst[p]) return TB200_ERR_INVALID_ARG;
        if (!aligned_to(out.dst[p], eb)) return TB200_ERR_ALIGNMENT;
        dst_aligned = dst_aligned && aligned_to(out.dst[p], 16);
    }
    if ((out.c && !aligned_to(out.c, eb)) || (out.bias && !aligned_to(out.bias, eb))) return TB200_ERR_ALIGNMENT;
    if (out.beta != 0.f && !out.c) return TB200_ERR_INVALID_ARG;
    out.plain = out.alpha == 1.f && out.beta == 0.f && !out.bias && out.act == TB200_ACT_NONE && out.out_type == TB200_OUT_F32;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    cudaStream_t s = (cudaStream_t)stream;
    // tensor-core path: row pitches of 16 bytes and operands at 0 or 8 modulo 16 (an array behind a 16- or a 24-byte
    // header); tiny products are not worth a 128 x 128 tile
    const bool tensor = k >= 32 && k % 8 == 0 && n % 8 == 0 && aligned_to(pr.a, 8) && aligned_to(pr.b, 8) && (long long)m * n >= 64 * 64 &&
                        (pr.batches == 1 || (pr.stride_a % 8 == 0 && pr.stride_b % 8 == 0));
    if (!tensor) {
        // the CUDA-core kernel writes dense fp32 [m][n] matrices without an epilogue
        if (out.ndst != 1 || out.ld != n || !out.plain || pr.bf16) return TB200_ERR_UNSUPPORTED;
        st = ensure_kernel<gemm_generic_kernel<uint16_t>, 0>(di);
        if (st) return st;
        dim3 grid((n + 31) / 32, (m + 31) / 32);
        for (int b = 0; b < pr.batches; ++b) {
            gemm_generic_kernel<uint16_t><<<grid, 1024, 0, s>>>(m, n, k, 1.0f, pr.a + (size_t)b * pr.stride_a, pr.b + (size_t)b * pr.stride_b, 0.0f,
                                                                reinterpret_cast<float *>(out.dst[0]) + (size_t)b * out.batch_stride);
            st = check_launch();
            if (st) return st;
        }
        return TB200_OK;
    }
    // operands off a 128-byte line (arrays behind a 16- or 24-byte header in an aligned buffer): maps over the line
    // boundary below when every row keeps the phase (row pitch and batch stride are whole lines), else over the
    // 16-byte boundary below; the matrices are shifted by that many elements
    auto shift_of = [&](const uint16_t *p, long long row_elems, long long stride_elems) {
        const bool lines = row_elems % 64 == 0 && (pr.batches == 1 || stride_elems % 64 == 0);
        return (int)(((uintptr_t)p & (lines ? 127 : 15)) / 2);
    };
    const int kshift = shift_of(pr.a, k, pr.stride_a), nshift = shift_of(pr.b, n, pr.stride_b);
    const CUtensorMapDataType in_type = pr.bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap map_a, map_b, map_d;
    st = make_map(&map_a, pr.a - kshift, in_type, 2, (uint64_t)(k + kshift), (uint64_t)m, (uint64_t)pr.batches, (uint64_t)pr.stride_a, 64, HG_BM, (uint64_t)k);
    if (st) return st;
    st = make_map(&map_b, pr.b - nshift, in_type, 2, (uint64_t)(n + nshift), (uint64_t)k, (uint64_t)pr.batches, (uint64_t)pr.stride_b, 64, HG_BK, (uint64_t)n);
    if (st) return st;
    // finished fp32 pieces of a single dense, 16-byte aligned destination leave as TMA tensor stores (32 x 32 boxes);
    // shifted columns would start the first store at a negative coordinate
    // -- when the tiles' columns start on the destination's 128-byte lines; off the lines, the stores follow the lines
    out.line_shift = line_shift_of(out, n, nshift, pr.batches);
    out.tma_store = out.out_type == TB200_OUT_F32 && out.ndst == 1 && out.col_off == 0 && rows_vec && dst_aligned && n % 4 == 0 && nshift == 0 &&
                    out.line_shift <= 0;
    if (out.tma_store) {
        st = make_map(&map_d, out.dst[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)n, (uint64_t)m, (uint64_t)pr.batches,
                      (uint64_t)out.batch_stride, 32, 32);
        if (st) out.tma_store = 0;  // e.g. a row pitch the encoder does not take: plain stores
        // a leading dimension other than n is not described by the map
        if (out.ld != n) out.tma_store = 0;
    }
    if (!out.tma_store) map_d = CUtensorMap{};  // unused by the kernel
    if (out.tma_store) out.line_shift = -1;
    if (out.line_shift >= 0 && out.col_off == 0 && out.ld == n) {
        // whole lines of the line-following epilogue as TMA stores: a map over the line boundary below the destination,
        // line_cs floats wider than the row pitch (box columns in front of a row are never stored: such segments are partial)
        out.line_cs = (int)(((uintptr_t)out.dst[0] & 127) / 4);
        out.line_tma = make_map(&map_d, reinterpret_cast<float *>(out.dst[0]) - out.line_cs, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
                                (uint64_t)(n + out.line_cs), (uint64_t)m, (uint64_t)pr.batches, (uint64_t)out.batch_stride, 32, 32, (uint64_t)n) == TB200_OK;
    }
    // tile rows per band: the band's A panels (rows x k halves) should take about 48 MB of the 126 MB L2
    auto band_rows = [&](int tile_m) {
        long long g = (48ll << 20) / ((long long)tile_m * k * 2);
        return (int)(g < 1 ? 1 : (g > 1024 ? 1024 : g));
    };
    const long long tiles256 = (long long)((m + 255) / 256) * ((n + nshift + 255) / 256) * pr.batches;
    // SM pairs pay off once the 256 x 256 tiles fill about 85 % of the pairs (measured: 2048 x 2048 results, 64 tiles
    // on 74 pairs, run alike on both kernels; 3072^3 and 1024 x 8192 x 4096 4 % faster on pairs; 1024^2 results, 16
    // tiles, 13 % slower); smaller products fill the machine better with 128 x 256 or 128 x 128 tiles on single CTAs
    // (and so does an A 8 bytes off a 16-byte boundary, whose clearing of the bytes in front of the rows stays
    // inside one CTA there)
    if (kshift % 8 == 0 && option_value(TB200_OPT_HGEMM_SM_PAIRS) && tiles256 * 20 >= 17 * (di->sm_count / 2)) {
        st = ensure_smem_optin<hgemm_tc2_kernel>(di);
        if (st) return st;
        CUtensorMap map_a0 = map_a;  // first K block of a shifted A: a map over A itself (see the kernel)
        if (kshift) {
            st = make_map(&map_a0, pr.a, in_type, 2, (uint64_t)k, (uint64_t)m, (uint64_t)pr.batches, (uint64_t)pr.stride_a, 64, HG_BM);
            if (st) return st;
        }
        const int pairs = tiles256 < di->sm_count / 2 ? (int)tiles256 : di->sm_count / 2;
        hgemm_tc2_kernel<<<2 * pairs, HG_THREADS, H2_SMEM_BYTES, s>>>(map_a, map_a0, map_b, map_d, out, m, n, k, pr.batches, (int)rows_vec,
                                                                      band_rows(256), hg_idesc(256, 256, pr.bf16), kshift, nshift);
        return check_launch();
    }
    const long long tiles_wide = (long long)((m + HG_BM - 1) / HG_BM) * ((n + nshift + 255) / 256) * pr.batches;
    const long long tiles_narrow = (long long)((m + HG_BM - 1) / HG_BM) * ((n + nshift + 127) / 128) * pr.batches;
    // 128 x 128 tiles read as many operand bytes from shared memory per MMA as 128 x 256 tiles for half the
    // arithmetic and run at about half the rate per SM (2048^3: 602 against 812 TFLOP/s), so they only pay when
    // the wide tiles would leave more than half of the SMs idle
    const bool wide = 2 * tiles_wide >= di->sm_count;
    const long long tiles = wide ? tiles_wide : tiles_narrow;
    const int grid = tiles < di->sm_count ? (int)tiles : di->sm_count;
    const uint32_t idesc = hg_idesc(128, wide ? 256 : 128, pr.bf16);
    const int gm = band_rows(HG_BM);
    if (wide) {
        st = ensure_smem_optin<hgemm_tc_kernel<256>>(di);
        if (st) return st;
        hgemm_tc_kernel<256><<<grid, HG_THREADS, HgTile<256>::SMEM_BYTES, s>>>(map_a, map_b, map_d, out, m, n, k, pr.batches, (int)rows_vec, gm, idesc, kshift, nshift);
    } else {
        st = ensure_smem_optin<hgemm_tc_kernel<128>>(di);
        if (st) return st;
        hgemm_tc_kernel<128><<<grid, HG_THREADS, HgTile<128>::SMEM_BYTES, s>>>(map_a, map_b, map_d, out, m, n, k, pr.batches, (int)rows_vec, gm, idesc, kshift, nshift);
    }
    return check_launch();
}

// ---- int8 and fp8 GEMM ---------------------------------------------------------------------------
// Bt[n][k] = B[k][n], bytes; 32 x 32 tiles through shared memory
// Row n of Bt is `pitch` bytes long and holds column n of B from byte `shift` on; the `shift` bytes in front of it
// are zeros (an A whose rows start `shift` bytes past the base of its tensor map meets them there).
__global__ void __launch_bounds__(256) transpose_bytes_kernel(const int8_t *__restrict__ b, int8_t *__restrict__ bt, int k, int n, int pitch,
                                                              int shift) {
    __shared__ int8_t tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    for (int r = ty; r < 32; r += 8)
        if (k0 + r < k && n0 + tx < n) tile[r][tx] = b[(size_t)(k0 + r) * n + n0 + tx];
    __syncthreads();
    for (int r = ty; r < 32; r += 8)
        if (n0 + r < n && k0 + tx < k) bt[(size_t)(n0 + r) * pitch + shift + k0 + tx] = tile[tx][r];
    if (blockIdx.y == 0)
        for (int r = ty; r < 32; r += 8)
            for (int j = tx; j < shift; j += 32)
                if (n0 + r < n) bt[(size_t)(n0 + r) * pitch + j] = 0;
}

// fp8 byte -> float: E5M2 is the upper byte of an fp16; E4M3 has bias 7, subnormals m * 2^-9 and one NaN (S.1111.111)
__device__ __forceinline__ float fp8_to_float(uint8_t v, int e5m2) {
    if (e5m2) return half_bits_to_float((uint16_t)((uint16_t)v << 8));
    const int sign = v >> 7, e = (v >> 3) & 15, mant = v & 7;
    float r;
    if (e == 0) r = ldexpf((float)mant, -9);
    else if (e == 15 && mant == 7) r = __int_as_float(0x7fc00000);
    else r = ldexpf(1.0f + (float)mant * 0.125f, e - 7);
    return sign ? -r : r;
}

// any shape and alignment: one thread per output (KIND 1: int8 -> int32, 2: fp8 -> fp32 accumulated in k order)
template <int KIND>
__global__ void __launch_bounds__(256) gemm8_generic_kernel(int m, int n, int k, const uint8_t *__restrict__ a, const uint8_t *__restrict__ b,
                                                            void *__restrict__ c, int e5m2) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)m * n) return;
    const int row = (int)(i / n), col = (int)(i - (long long)row * n);
    if (KIND == 1) {
        int acc = 0;
        for (int kk = 0; kk < k; ++kk) acc += (int)(int8_t)a[(size_t)row * k + kk] * (int)(int8_t)b[(size_t)kk * n + col];
        reinterpret_cast<int32_t *>(c)[i] = acc;
    } else {
        float acc = 0.f;
        for (int kk = 0; kk < k; ++kk) acc = fmaf(fp8_to_float(a[(size_t)row * k + kk], e5m2), fp8_to_float(b[(size_t)kk * n + col], e5m2), acc);
        reinterpret_cast<float *>(c)[i] = acc;
    }
}

// KIND 1: int8 x int8 -> int32 (tcgen05.mma.kind::i8); KIND 2: fp8 x fp8 -> fp32 (kind::f8f6f4, format 0 = E4M3, 1 = E5M2)
template <int KIND>
static int gemm8_launch(int m, int n, int k, const uint8_t *a, const uint8_t *b, void *c, int e5m2, void *workspace, size_t workspace_bytes,
                        tb200_stream_t stream) {
    if (m < 0 || n < 0 || k < 0) return TB200_ERR_INVALID_ARG;
    if (m == 0 || n == 0) return TB200_OK;
    if (!c || (k > 0 && (!a || !b))) return TB200_ERR_INVALID_ARG;
    if (!aligned_to(c, 4)) return TB200_ERR_ALIGNMENT;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    cudaStream_t s = (cudaStream_t)stream;
    // A off a 128-byte line (an array behind a 16- or 24-byte header): its map lies over the line boundary below
    // when every row keeps the phase, else over the 16-byte boundary below, and the rows of Bt carry as many zero bytes
    // in front (see hgemm_tc_kernel)
    const int kshift = a ? (int)((uintptr_t)a & (k % 128 == 0 ? 127 : 15)) : 0;
    const int pitch = k + ((kshift + 15) & ~15);
    const bool tensor = k >= 32 && k % 16 == 0 && aligned_to(a, 8) && (long long)m * n >= 64 * 64 && workspace && aligned_to(workspace, 16) &&
                        workspace_bytes >= (size_t)n * pitch;
    if (!tensor) {
        st = ensure_kernel<gemm8_generic_kernel<KIND>, 0>(di);
        if (st) return st;
        const long long total = (long long)m * n;
        gemm8_generic_kernel<KIND><<<(unsigned)((total + 255) / 256), 256, 0, s>>>(m, n, k, a, b, c, e5m2);
        return check_launch();
    }
    st = ensure_kernel<transpose_bytes_kernel, 0>(di);
    if (st) return st;
    int8_t *bt = reinterpret_cast<int8_t *>(workspace);
    transpose_bytes_kernel<<<dim3((n + 31) / 32, (k + 31) / 32), 256, 0, s>>>(reinterpret_cast<const int8_t *>(b), bt, k, n, pitch, kshift);
    st = check_launch();
    if (st) return st;
    HgOut out{};
    out.dst[0] = c, out.ld = n, out.ndst = 1, out.alpha = 1.f, out.out_type = TB200_OUT_F32, out.plain = 1, out.batch_stride = (long long)m * n;
    const bool vec = n % 4 == 0 && aligned_to(c, 16);
    const long long tiles_wide = (long long)((m + HG_BM - 1) / HG_BM) * ((n + 255) / 256);
    const bool wide = 2 * tiles_wide >= di->sm_count;
    const int bn = wide ? 256 : 128;
    CUtensorMap map_a, map_b, map_d{};
    st = make_map(&map_a, a - kshift, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)(k + kshift), (uint64_t)m, 1, 0, 128, HG_BM, (uint64_t)k);
    if (st) return st;
    st = make_map(&map_b, bt, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)(k + kshift), (uint64_t)n, 1, 0, 128, (uint32_t)bn, (uint64_t)pitch);
    if (st) return st;
    out.line_shift = line_shift_of(out, n, 0, 1);
    out.tma_store = vec && out.line_shift <= 0;  // 32-bit results of either kind leave as they are
    if (out.tma_store && make_map(&map_d, c, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, (uint64_t)n, (uint64_t)m, 1, 0, 32, 32) != TB200_OK) out.tma_store = 0;
    if (out.tma_store) out.line_shift = -1;
    if (out.line_shift >= 0) {  // whole lines as TMA stores through a map over the line boundary below c (see hgemm_launch)
        out.line_cs = (int)(((uintptr_t)c & 127) / 4);
        out.line_tma = make_map(&map_d, reinterpret_cast<int32_t *>(c) - out.line_cs, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, (uint64_t)(n + out.line_cs),
                                (uint64_t)m, 1, 0, 32, 32, (uint64_t)n) == TB200_OK;
    }
    // instruction descriptor, both operands K-major: D format at [4,6) (1 = F32, 2 = S32), A and B formats at [7,10) and
    // [10,13) (kind::i8: 1 = signed 8-bit; kind::f8f6f4: 0 = E4M3, 1 = E5M2), N >> 3 at [17,23), M >> 4 at [24,29)
    const uint32_t fmt = KIND == 1 ? 1u : (e5m2 ? 1u : 0u);
    const uint32_t idesc = ((KIND == 1 ? 2u : 1u) << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(HG_BM >> 4) << 24);
    const long long tiles = (long long)((m + HG_BM - 1) / HG_BM) * ((n + bn - 1) / bn);
    const int grid = tiles < di->sm_count ? (int)tiles : di->sm_count;
    long long g = (48ll << 20) / ((long long)HG_BM * k);
    const int gm = (int)(g < 1 ? 1 : (g > 1024 ? 1024 : g));
    if (wide) {
        st = ensure_smem_optin<hgemm_tc_kernel<256, KIND>>(di);
        if (st) return st;
        hgemm_tc_kernel<256, KIND><<<grid, HG_THREADS, HgTile<256>::SMEM_BYTES, s>>>(map_a, map_b, map_d, out, m, n, k, 1, (int)vec, gm, idesc, kshift, 0);
    } else {
        st = ensure_smem_optin<hgemm_tc_kernel<128, KIND>>(di);
        if (st) return st;
        hgemm_tc_kernel<128, KIND><<<grid, HG_THREADS, HgTile<128>::SMEM_BYTES, s>>>(map_a, map_b, map_d, out, m, n, k, 1, (int)vec, gm, idesc, kshift, 0);
    }
    return check_launch();
}

}  // namespace tb200

using namespace tb200;

// room for Bt with up to 128 bytes of zeros in front of every row (an A off a 128-byte line)
extern "C" size_t tb200_igemm_workspace_bytes(int n, int k) { return n > 0 && k > 0 ? (size_t)n * ((size_t)k + 128) : 0; }

extern "C" int tb200_igemm_s32(int m, int n, int k, const int8_t *a, const int8_t *b, int32_t *c, void *workspace, size_t workspace_bytes,
                               tb200_stream_t stream) {
    return gemm8_launch<1>(m, n, k, reinterpret_cast<const uint8_t *>(a), reinterpret_cast<const uint8_t *>(b), c, 0, workspace, workspace_bytes, stream);
}

extern "C" int tb200_fp8gemm_f32(int m, int n, int k, int format, const uint8_t *a, const uint8_t *b, float *c, void *workspace,
                                 size_t workspace_bytes, tb200_stream_t stream) {
    if (format != TB200_FP8_E4M3 && format != TB200_FP8_E5M2) return TB200_ERR_INVALID_ARG;
    return gemm8_launch<2>(m, n, k, a, b, c, format == TB200_FP8_E5M2, workspace, workspace_bytes, stream);
}

extern "C" int tb200_hgemm_f32(int m, int n, int k, const uint16_t *a, const uint16_t *b, float *c, tb200_stream_t stream) {
    if (m < 0 || n < 0 || k < 0) return TB200_ERR_INVALID_ARG;
    if (m == 0 || n == 0) return TB200_OK;
    if (!c) return TB200_ERR_INVALID_ARG;
    HgOut out{};
    out.dst[0] = c, out.ld = n, out.ndst = 1, out.alpha = 1.f, out.out_type = TB200_OUT_F32;
    return hgemm_launch(HgProblem{m, n, k, 1, a, b, 0, 0, false}, out, stream);
}

extern "C" int tb200_hgemm_f32_scatter(int m, int n, int k, const uint16_t *a, const uint16_t *b, float *const *dst, int ndst,
                                       long long ld, long long col_offset, tb200_stream_t stream) {
    if (!dst || ndst < 1 || ndst > HG_MAX_DST) return TB200_ERR_INVALID_ARG;
    HgOut out{};
    for (int p = 0; p < ndst; ++p) out.dst[p] = dst[p];
    out.ld = ld, out.col_off = col_offset, out.ndst = ndst, out.alpha = 1.f, out.out_type = TB200_OUT_F32;
    return hgemm_launch(HgProblem{m, n, k, 1, a, b, 0, 0, false}, out, stream);
}

extern "C" int tb200_gemm_ex(int m, int n, int k, int in_type, const void *a, const void *b, int out_type, void *d, float alpha, float beta,
                             const void *c, const void *bias, int activation, int batch_count, tb200_stream_t stream) {
    if (in_type != TB200_IN_F16 && in_type != TB200_IN_BF16) return TB200_ERR_INVALID_ARG;
    if (m < 0 || n < 0 || k < 0 || batch_count < 0) return TB200_ERR_INVALID_ARG;
    if (m == 0 || n == 0 || batch_count == 0) return TB200_OK;
    if (!d) return TB200_ERR_INVALID_ARG;
    if (bias && batch_count > 1) return TB200_ERR_INVALID_ARG;  // one bias row per call
    HgOut out{};
    out.dst[0] = d, out.ld = n, out.ndst = 1, out.batch_stride = (long long)m * n;
    out.c = beta != 0.f ? (c ? c : d) : nullptr, out.bias = bias, out.alpha = alpha, out.beta = beta;
    out.out_type = out_type, out.act = activation;
    HgProblem pr{m, n, k, batch_count, reinterpret_cast<const uint16_t *>(a), reinterpret_cast<const uint16_t *>(b), (long long)m * k,
                 (long long)k * n, in_type == TB200_IN_BF16};
    return hgemm_launch(pr, out, stream);
}
