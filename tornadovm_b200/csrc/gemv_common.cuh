// Types and small device helpers shared by the quantised mat-vec translation units
// (gemv_quant.cu: CUDA-core kernels and the dispatcher; gemv_mma.cu / gemv_tc.cu: tensor-core kernels).
#pragma once

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
    int wshift;              // block-layout ring kernels: byte phase of every row chunk (w modulo 128 or modulo 16)
    int xlayout;             // int mode, tensor-core kernel: 0 = xq[batch][cols], xs[batch][cols/32]; 1 = xq[block][batch][32], xs[block][batch]
    int group_rows;          // tensor-core kernel: > 0: the rows are those of rows / group_rows equally shaped matrices that lie
                             // back to back, and y is [matrix][batch][group_rows]
};

// Tensor-core kernel over several matrices that share the column count and the activation vectors: the launch's rows
// are those of all matrices laid end to end (count = 0: one matrix).  Matrix m holds rows row_start[m] ..
// row_start[m + 1] and writes its [batch][rows of m] block at y + y_off[m].
constexpr int kTcMaxGroup = 32;
struct TcGroup {
    int count;
    int row_start[kTcMaxGroup + 1];
    const uint8_t *w[kTcMaxGroup];
    long long y_off[kTcMaxGroup];
};

// Several matrices of one shape sharing the activation vectors, and several destinations for every
// output value (this GPU's buffer and, peer-mapped, the other GPUs' buffers).
// rows a warp of the grouped kernel collects before it stores them (128-byte stores to every destination;
// runs of 8 rows were measured no faster on two GPUs and slightly slower on one)
constexpr int kGroupFlushRows = 32;
constexpr int kMaxGroup = 32;
constexpr int kMaxPeers = 8;
struct QGroupArgs {
    const uint8_t *w[kMaxGroup];   // block arrays; matrix m holds rows row_start[m] .. row_start[m+1] of the launch
    int row_start[kMaxGroup + 1];
    long long out_off[kMaxGroup];  // where matrix m's [batch][ld[m]] output block starts inside a slot (floats)
    int ld[kMaxGroup];             // rows of the whole (unsharded) matrix m
    int row_off[kMaxGroup];        // first row of this launch's share of matrix m
    float *dst[kMaxPeers];         // output buffers, each [slots][...]
    const unsigned *epoch;         // device word whose low bit selects the half (null: half 0)
    long long half_stride;         // floats between the halves
    int count, npeers;
    // In-kernel hand-shake of a multi-GPU step (null flags[0]: none).  sync[0] is this GPU's step counter
    // (the same word as `epoch`), sync[1] counts the CTAs of the running launch that have finished.
    unsigned *flags[kMaxPeers];    // flags[p]: flag array of GPU p, one word per source GPU
    unsigned *sync;
    unsigned long long timeout_ns;
    int rank;
    int handshake;                 // bit 0: wait for the peers before the first store; bit 1: signal them at the end
    int nslots;                    // output slots in rotation (the "halves" above when 2)
};

__device__ __forceinline__ int dp4a_s8(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }
// four unsigned bytes of a times four signed bytes of b
__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// floor(v * inv + 0.5) as the low byte of the result (a signed byte), for |v * inv| <= 127: the rule of
// quantizeKernelContext (MatrixVectorRowMajor.java:349-354) without the conversion unit.  Adding 1.5 * 2^23 with
// rounding toward minus infinity leaves floor(.) in the low mantissa bits.
__device__ __forceinline__ uint32_t quantize_byte(float v, float inv) {
    return (uint32_t)__float_as_int(__fadd_rd(__fadd_rn(__fmul_rn(v, inv), 0.5f), 12582912.0f)) & 0xFFu;
}

__host__ __device__ __forceinline__ int round_up(int v, int m) { return (v + m - 1) / m * m; }

constexpr int MODE_FLOAT = 0;     // fp32 activations
constexpr int MODE_INT = 1;       // int8 activations read from the workspace
constexpr int MODE_INT_FUSED = 2; // int8 activations quantised in the prologue of this kernel

__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void *src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src_gmem) : "memory");
}
// 8-byte form (through L1): for operands that are only 8-byte aligned
__device__ __forceinline__ void cp_async_8(uint32_t dst_smem, const void *src_gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst_smem), "l"(src_gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}


// ---- tensor-core (mma.sync) helpers ----
__device__ __forceinline__ void mma_s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four bytes 0..255 -> two half2 registers holding (byte - bias): the byte is spliced into the mantissa of
// fp16 1024.0 (exponent bits 0x64), which makes 1024 + byte exactly, and the bias is removed with one HSUB2.
__device__ __forceinline__ void u8x4_to_h2x2(uint32_t u, uint32_t bias_h2, uint32_t &lo, uint32_t &hi) {
    const uint32_t l = __byte_perm(u, 0x64646464u, 0x4140);  // bytes 0,1
    const uint32_t h = __byte_perm(u, 0x64646464u, 0x4342);  // bytes 2,3
    __half2 lv = __hsub2(*reinterpret_cast<const __half2 *>(&l), *reinterpret_cast<const __half2 *>(&bias_h2));
    __half2 hv = __hsub2(*reinterpret_cast<const __half2 *>(&h), *reinterpret_cast<const __half2 *>(&bias_h2));
    lo = *reinterpret_cast<uint32_t *>(&lv);
    hi = *reinterpret_cast<uint32_t *>(&hv);
}

// 32-bit read at a byte offset that is 0 or 2 modulo 4
template <int MISALIGNED>
__device__ __forceinline__ uint32_t lds_u32_at(const unsigned char *base, int off) {
    const uint32_t *w = reinterpret_cast<const uint32_t *>(base + (off & ~3));
    if (MISALIGNED) return __funnelshift_r(w[0], w[1], 16);
    return w[0];
}

// ---- entry points of the tensor-core units, called by the dispatcher of gemv_quant.cu ----
// already quantised activations (xq, xs); shapes and alignments the kernels take
bool qmma_eligible(int fmt, const QGemvArgs &a);
int qmma_dispatch(int fmt, const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s);
// fp32 activations split into fp16 pairs, batches of 1..8
bool qmma_float_eligible(int fmt, const QGemvArgs &a, const DeviceInfo *di);
int qmma_float_dispatch(int fmt, const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s, bool overlap);

// gemv_tc.cu: every warp of a CTA owns one 256-column slice of K and keeps the activations of that slice in
// registers.  mode: MODE_FLOAT (a.x), MODE_INT (a.xq / a.xs), MODE_INT_FUSED (a.x, quantised in the prologue);
// a.dots set (batch 1, MODE_INT) writes the int32 block dots instead of y.
bool qtc_eligible(int fmt, int mode, const QGemvArgs &a, const DeviceInfo *di);
int qtc_dispatch(int fmt, int mode, const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s, bool overlap);
// block formats, MODE_INT, 1..16 vectors: a.rows = rows of all matrices of grp, a.w = grp.w[0] (all at one 16-byte phase)
int qtc_dispatch_group(int fmt, const QGemvArgs &a, const TcGroup &grp, const DeviceInfo *di, cudaStream_t s, bool overlap);

// ---- helpers of gemv_quant.cu used by the allocation-free entry point ----
int split_workspace(int cols, int batch, void *workspace, size_t workspace_bytes, int8_t **xq, float **xs);
int quantize_x(int cols, int batch, const float *x, int8_t *xq, float *xs, cudaStream_t s);
int quantize_x_layout(int cols, int batch, const float *x, int8_t *xq, float *xs, cudaStream_t s, bool interleaved);
int q8s_gemv_quantised(const QGemvArgs &a, tb200_stream_t stream);

}  // namespace tb200
