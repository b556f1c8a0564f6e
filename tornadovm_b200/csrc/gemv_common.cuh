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

__host__ __device__ __forceinline__ int round_up(int v, int m) { return (v + m - 1) / m * m; }

constexpr int MODE_FLOAT = 0;     // fp32 activations
constexpr int MODE_INT = 1;       // int8 activations read from the workspace
constexpr int MODE_INT_FUSED = 2; // int8 activations quantised in the prologue of this kernel

__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void *src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src_gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}


// ---- entry points of the tensor-core units, called by the dispatcher of gemv_quant.cu ----
// already quantised activations (xq, xs); shapes and alignments the kernels take
bool qmma_eligible(int fmt, const QGemvArgs &a);
int qmma_dispatch(int fmt, const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s);
// fp32 activations split into fp16 pairs, batches of 1..8
bool qmma_float_eligible(int fmt, const QGemvArgs &a, const DeviceInfo *di);
int qmma_float_dispatch(int fmt, const QGemvArgs &a, const DeviceInfo *di, cudaStream_t s, bool overlap);

// ---- helpers of gemv_quant.cu used by the allocation-free entry point ----
int split_workspace(int cols, int batch, void *workspace, size_t workspace_bytes, int8_t **xq, float **xs);
int quantize_x(int cols, int batch, const float *x, int8_t *xq, float *xs, cudaStream_t s);
int q8s_gemv_quantised(const QGemvArgs &a, tb200_stream_t stream);

}  // namespace tb200
