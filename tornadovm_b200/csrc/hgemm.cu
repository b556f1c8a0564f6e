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

#define TB200_OP_CLASS TB200_PREPARE_GEMM_F16
#include "common.cuh"
#include "gemm_generic.cuh"

TB200_TU_STATUS(hgemm)

namespace tb200 {

constexpr int HG_BM = 128, HG_BN = 256, HG_BK = 64, HG_STAGES = 4;
constexpr int HG_THREADS = 192;
constexpr int HG_A_BYTES = HG_BM * HG_BK * 2;      // 16 KB
constexpr int HG_B_BYTES = HG_BK * HG_BN * 2;      // 32 KB, four 8 KB boxes of 64 columns
constexpr int HG_STAGE_BYTES = HG_A_BYTES + HG_B_BYTES;
// Each epilogue warp owns a 32 x 32 fp32 transposition buffer (row pitch 36 floats: conflict-free float4 access both ways),
// used when tiles go to several destinations: stores to peer memory should be whole 128-byte lines, not 16-byte pieces
// of 32 different rows.
constexpr int HG_XPOSE_PITCH = 36, HG_XPOSE_BYTES = 4 * 32 * HG_XPOSE_PITCH * 4;
constexpr int HG_SMEM_BYTES = HG_STAGES * HG_STAGE_BYTES + 1024 + HG_XPOSE_BYTES;  // + slack for 1024-byte alignment
constexpr uint32_t HG_TMEM_COLS = 512;

// ---- PTX wrappers ------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void *dst_smem, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

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

// Instruction descriptor, kind::f16: D fp32, A/B fp16, A K-major, B MN-major (N contiguous), M128, N256.
//   [4,6) D format 1 = F32   [7,10) A format 0 = F16   [10,13) B format 0 = F16
//   bit 15 A major (0 = K)   bit 16 B major (1 = MN)   [17,23) N >> 3   [24,29) M >> 4
constexpr uint32_t HG_IDESC = (1u << 4) | (1u << 16) | ((uint32_t)(HG_BN >> 3) << 17) | ((uint32_t)(HG_BM >> 4) << 24);

// Where the epilogue stores a tile: every destination gets C[row][col] at dst[p][row * ld + col_off + col].
// One local destination with ld = N is the plain GEMM; several destinations (this GPU's buffer and
// peer-mapped buffers of other GPUs) with ld = the unsharded N and col_off = the first column of this GPU's
// column block make the all-gather of a column-sharded GEMM part of the epilogue.
constexpr int HG_MAX_DST = 8;
struct HgOut {
    float *dst[HG_MAX_DST];
    long long ld, col_off;
    int ndst;
    int xpose;  // store through the transposition buffer (whole 128-byte lines per row)
};

__global__ void __launch_bounds__(HG_THREADS, 1)
hgemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ HgOut out,
                int M, int N, int K, int c_vec_ok, int gm) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[HG_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[HG_STAGES];
    __shared__ __align__(8) uint64_t acc_full_bar[2];
    __shared__ __align__(8) uint64_t acc_empty_bar[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    // the swizzled tiles need 1024-byte aligned bases
    unsigned char *tiles = reinterpret_cast<unsigned char *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + HG_BM - 1) / HG_BM, tiles_n = (N + HG_BN - 1) / HG_BN;
    const int num_tiles = tiles_m * tiles_n;
    const int k_blocks = (K + HG_BK - 1) / HG_BK;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < HG_STAGES; ++s) {
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
        // whole warp: allocate all 512 tensor-memory columns (two 128 x 256 fp32 accumulators)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(HG_TMEM_COLS)
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
                int tm, tn;
                tile_coords(tile, tiles_m, tiles_n, gm, tm, tn);
                const int m0 = tm * HG_BM, n0 = tn * HG_BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % HG_STAGES;
                    const uint32_t use = it / HG_STAGES;
                    if (use > 0) {
                        ok = mbar_wait_abortable(&empty_bar[s], (use - 1) & 1, abortp);
                        if (!ok) break;
                    }
                    unsigned char *a_dst = tiles + (size_t)s * HG_STAGE_BYTES;
                    unsigned char *b_dst = a_dst + HG_A_BYTES;
                    mbar_expect_tx(&full_bar[s], HG_STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, kb * HG_BK, m0, &full_bar[s]);
#pragma unroll
                    for (int j = 0; j < HG_BN / 64; ++j)
                        tma_load_2d(b_dst + j * (HG_BK * 128), &map_b, n0 + j * 64, kb * HG_BK, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t it = 0, local_tile = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
                const uint32_t acc = local_tile & 1, acc_use = local_tile >> 1;
                if (acc_use > 0) {
                    ok = mbar_wait_abortable(&acc_empty_bar[acc], (acc_use - 1) & 1, abortp);
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t d_tmem = tmem_base + acc * HG_BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % HG_STAGES;
                    ok = mbar_wait_abortable(&full_bar[s], (it / HG_STAGES) & 1, abortp);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + (size_t)s * HG_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + HG_A_BYTES;
                    // A: K-major, rows of 128 bytes, 8-row groups 1024 bytes apart
                    const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024);
                    // B: N contiguous; 64-column boxes HG_BK*128 bytes apart, 8-k-row groups 1024 bytes apart
                    const uint64_t b_desc = make_smem_desc(b_addr, HG_BK * 128, 1024);
#pragma unroll
                    for (int k16 = 0; k16 < HG_BK / 16; ++k16) {
                        // A advances 16 halves = 32 bytes along K; B advances 16 k-rows = 2048 bytes
                        tc_mma_f16(d_tmem, a_desc + (uint64_t)(k16 * 2), b_desc + (uint64_t)(k16 * 128), HG_IDESC,
                                   (kb > 0 || k16 > 0) ? 1u : 0u);
                    }
                    tc_commit(&empty_bar[s]);  // arrives once the MMAs above have read this stage
                }
                if (ok) tc_commit(&acc_full_bar[acc]);  // accumulator complete
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5, TMEM lane quarter = warp % 4 ----------------
        const int quarter = warp & 3;
        uint32_t local_tile = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
            const uint32_t acc = local_tile & 1, acc_use = local_tile >> 1;
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, gm, tm, tn);
            const int m0 = tm * HG_BM, n0 = tn * HG_BN;
            ok = __all_sync(0xffffffffu, mbar_wait_abortable(&acc_full_bar[acc], acc_use & 1, abortp));
            if (!ok) break;
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * HG_BN;
#pragma unroll 1
            for (int c = 0; c < HG_BN / 32; ++c) {
                uint32_t v[32];
                tc_ld_32cols(taddr + c * 32, v);
                tc_wait_ld();
                const int col0 = n0 + c * 32;
                if (out.xpose && c_vec_ok && col0 + 32 <= N) {
                    // through shared memory: lane r wrote row r, now eight lanes store one row's 128 bytes
                    float *stg = reinterpret_cast<float *>(tiles + (size_t)HG_STAGES * HG_STAGE_BYTES) + (warp - 2) * 32 * HG_XPOSE_PITCH;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float4 *>(stg + lane * HG_XPOSE_PITCH + 4 * j) =
                            make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                                        __uint_as_float(v[4 * j + 3]));
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rl = i * 4 + (lane >> 3), c4 = (lane & 7) * 4;
                        const float4 val = *reinterpret_cast<const float4 *>(stg + rl * HG_XPOSE_PITCH + c4);
                        const int grow = row - lane + rl;
                        if (grow < M) {
                            for (int p = 0; p < out.ndst; ++p)  // plain stores, to local or peer-mapped memory
                                *reinterpret_cast<float4 *>(out.dst[p] + (size_t)grow * out.ld + out.col_off + col0 + c4) = val;
                        }
                    }
                    __syncwarp();
                } else if (row < M && col0 < N) {
                    for (int p = 0; p < out.ndst; ++p) {  // plain stores, to local or peer-mapped memory
                        float *dst = out.dst[p] + (size_t)row * out.ld + out.col_off + col0;
                        if (c_vec_ok && col0 + 32 <= N) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                *reinterpret_cast<float4 *>(dst + 4 * j) =
                                    make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < N) dst[j] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(HG_TMEM_COLS) : "memory");
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
constexpr int H2_SMEM_BYTES = H2_STAGES * H2_STAGE_BYTES + 1024 + HG_XPOSE_BYTES;
constexpr uint32_t H2_IDESC = (1u << 4) | (1u << 16) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

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
__device__ __forceinline__ void tma_load_2d_pair(void *dst_smem, const CUtensorMap *map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst_smem)),
        "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
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
hgemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ HgOut out,
                 int M, int N, int K, int c_vec_ok, int gm) {
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
    const int tiles_m = (M + 255) / 256, tiles_n = (N + 255) / 256;
    const int num_tiles = tiles_m * tiles_n;
    const int k_blocks = (K + HG_BK - 1) / HG_BK;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

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
                int tm, tn;
                tile_coords(tile, tiles_m, tiles_n, gm, tm, tn);
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
                    tma_load_2d_pair(a_dst, &map_a, kb * HG_BK, m0, bar);
                    tma_load_2d_pair(b_dst, &map_b, n0, kb * HG_BK, bar);
                    tma_load_2d_pair(b_dst + HG_BK * 128, &map_b, n0 + 64, kb * HG_BK, bar);
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
                        tc2_mma_f16(d_tmem, a_desc + (uint64_t)(k16 * 2), b_desc + (uint64_t)(k16 * 128), H2_IDESC,
                                    (kb > 0 || k16 > 0) ? 1u : 0u);
                    tc2_commit_both(&empty_bar[s]);  // frees this stage in both CTAs
                }
                if (ok) tc2_commit_both(&acc_full_bar[acc]);
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 of each CTA, its own 128 rows ----------------
        const int quarter = warp & 3;
        uint32_t local_tile = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += npairs, ++local_tile) {
            const uint32_t acc = local_tile & 1, acc_use = local_tile >> 1;
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, gm, tm, tn);
            const int m0 = tm * 256 + (int)rank * 128, n0 = tn * 256;
            ok = __all_sync(0xffffffffu, mbar_wait_abortable(&acc_full_bar[acc], acc_use & 1, abortp));
            if (!ok) break;
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * 256;
#pragma unroll 1
            for (int c = 0; c < 8; ++c) {
                uint32_t v[32];
                tc_ld_32cols(taddr + c * 32, v);
                tc_wait_ld();
                const int col0 = n0 + c * 32;
                if (out.xpose && c_vec_ok && col0 + 32 <= N) {
                    // through shared memory: lane r wrote row r, now eight lanes store one row's 128 bytes
                    float *stg = reinterpret_cast<float *>(tiles + (size_t)H2_STAGES * H2_STAGE_BYTES) + (warp - 2) * 32 * HG_XPOSE_PITCH;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float4 *>(stg + lane * HG_XPOSE_PITCH + 4 * j) =
                            make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                                        __uint_as_float(v[4 * j + 3]));
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rl = i * 4 + (lane >> 3), c4 = (lane & 7) * 4;
                        const float4 val = *reinterpret_cast<const float4 *>(stg + rl * HG_XPOSE_PITCH + c4);
                        const int grow = row - lane + rl;
                        if (grow < M) {
                            for (int p = 0; p < out.ndst; ++p)  // plain stores, to local or peer-mapped memory
                                *reinterpret_cast<float4 *>(out.dst[p] + (size_t)grow * out.ld + out.col_off + col0 + c4) = val;
                        }
                    }
                    __syncwarp();
                } else if (row < M && col0 < N) {
                    for (int p = 0; p < out.ndst; ++p) {  // plain stores, to local or peer-mapped memory
                        float *dst = out.dst[p] + (size_t)row * out.ld + out.col_off + col0;
                        if (c_vec_ok && col0 + 32 <= N) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                *reinterpret_cast<float4 *>(dst + 4 * j) =
                                    make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < N) dst[j] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(&acc_empty_bar[acc], 0));
        }
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

// 2-D fp16 tensor map: `inner` contiguous elements per row, `outer` rows, box of 64 x box_rows, 128-byte swizzle.
static int make_map_f16(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer, uint32_t box_rows) {  // box: 64 x box_rows
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return TB200_ERR_DRIVER;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TB200_OK : TB200_ERR_DRIVER;
}

}  // namespace tb200

using namespace tb200;

// C(fp32) = A(fp16) * B(fp16) with the tile stores described by `out`.
static int hgemm_launch(int m, int n, int k, const uint16_t *a, const uint16_t *b, HgOut out, tb200_stream_t stream) {
    out.xpose = out.ndst >= option_value(TB200_OPT_HGEMM_LINE_STORES);
    if (m < 0 || n < 0 || k < 0) return TB200_ERR_INVALID_ARG;
    if (m == 0 || n == 0) return TB200_OK;
    if (k > 0 && (!a || !b)) return TB200_ERR_INVALID_ARG;
    if (out.ndst < 1 || out.ndst > HG_MAX_DST || out.ld < n || out.col_off < 0 || out.col_off > out.ld - n) return TB200_ERR_INVALID_ARG;
    if (!aligned_to(a, 2) || !aligned_to(b, 2)) return TB200_ERR_ALIGNMENT;
    bool vec = n % 4 == 0 && out.ld % 4 == 0 && out.col_off % 4 == 0;
    for (int p = 0; p < out.ndst; ++p) {
        if (!out.dst[p]) return TB200_ERR_INVALID_ARG;
        if (!aligned_to(out.dst[p], 4)) return TB200_ERR_ALIGNMENT;
        vec = vec && aligned_to(out.dst[p], 16);
    }
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    cudaStream_t s = (cudaStream_t)stream;
    // tensor-core path: TMA needs 16-byte aligned bases and row pitches; tiny products are not worth a 128x256 tile
    const bool tensor = k >= 32 && k % 8 == 0 && n % 8 == 0 && aligned_to(a, 16) && aligned_to(b, 16) &&
                        (long long)m * n >= 64 * 64;
    if (!tensor) {
        // the CUDA-core kernel writes one dense [m][n] matrix
        if (out.ndst != 1 || out.ld != n) return TB200_ERR_INVALID_ARG;
        dim3 grid((n + 31) / 32, (m + 31) / 32);
        st = ensure_kernel<gemm_generic_kernel<uint16_t>, 0>(di);
        if (st) return st;
        gemm_generic_kernel<uint16_t><<<grid, 1024, 0, s>>>(m, n, k, 1.0f, a, b, 0.0f, out.dst[0]);
        return check_launch();
    }
    CUtensorMap map_a, map_b;
    st = make_map_f16(&map_a, a, (uint64_t)k, (uint64_t)m, HG_BM);
    if (st) return st;
    st = make_map_f16(&map_b, b, (uint64_t)n, (uint64_t)k, HG_BK);
    if (st) return st;
    const int c_vec_ok = vec;
    // tile rows per band: the band's A panels (rows x k halves) should take about 48 MB of the 126 MB L2
    auto band_rows = [&](int tile_m) {
        long long g = (48ll << 20) / ((long long)tile_m * k * 2);
        return (int)(g < 1 ? 1 : (g > 1024 ? 1024 : g));
    };
    // SM pairs pay off once there are at least two waves of 256 x 256 tiles; smaller products fill the
    // machine better with 128 x 256 tiles on single CTAs
    if (option_value(TB200_OPT_HGEMM_SM_PAIRS) && ((m + 255) / 256) * ((n + 255) / 256) >= 2 * (di->sm_count / 2)) {
        // SM pairs: 256 x 256 tiles, one cluster of two CTAs each
        st = ensure_smem_optin<hgemm_tc2_kernel>(di);
        if (st) return st;
        const int tiles2 = ((m + 255) / 256) * ((n + 255) / 256);
        const int pairs = tiles2 < di->sm_count / 2 ? tiles2 : di->sm_count / 2;
        hgemm_tc2_kernel<<<2 * pairs, HG_THREADS, H2_SMEM_BYTES, s>>>(map_a, map_b, out, m, n, k, c_vec_ok, band_rows(256));
        return check_launch();
    }
    st = ensure_smem_optin<hgemm_tc_kernel>(di);
    if (st) return st;
    const int tiles = ((m + HG_BM - 1) / HG_BM) * ((n + HG_BN - 1) / HG_BN);
    const int grid = tiles < di->sm_count ? tiles : di->sm_count;
    hgemm_tc_kernel<<<grid, HG_THREADS, HG_SMEM_BYTES, s>>>(map_a, map_b, out, m, n, k, c_vec_ok, band_rows(HG_BM));
    return check_launch();
}

extern "C" int tb200_hgemm_f32(int m, int n, int k, const uint16_t *a, const uint16_t *b, float *c, tb200_stream_t stream) {
    if (m > 0 && n > 0 && !c) return TB200_ERR_INVALID_ARG;
    HgOut out{};
    out.dst[0] = c, out.ld = n, out.col_off = 0, out.ndst = 1;
    if (m == 0 || n == 0) return m < 0 || n < 0 || k < 0 ? TB200_ERR_INVALID_ARG : TB200_OK;
    return hgemm_launch(m, n, k, a, b, out, stream);
}

extern "C" int tb200_hgemm_f32_scatter(int m, int n, int k, const uint16_t *a, const uint16_t *b, float *const *dst, int ndst,
                                       long long ld, long long col_offset, tb200_stream_t stream) {
    if (!dst || ndst < 1 || ndst > HG_MAX_DST) return TB200_ERR_INVALID_ARG;
    HgOut out{};
    for (int p = 0; p < ndst; ++p) out.dst[p] = dst[p];
    out.ld = ld, out.col_off = col_offset, out.ndst = ndst;
    return hgemm_launch(m, n, k, a, b, out, stream);
}
