// FP32 matrix-vector product, HBM-bound.
//
// Replaces the one-thread-per-row README mxv kernel and the work-group-per-row
// KernelContext kernel of the reference (MatrixVectorRowMajor.java:94-158).
// One warp owns a row at a time; the row is streamed with 128-bit loads that
// skip L1, the vector lives in shared memory (staged once per CTA by a bulk
// async copy), partial sums are combined with warp shuffles.
//
// Algorithmic bytes per launch: 4 * (rows*cols + cols + rows).
#define TB200_OP_CLASS TB200_PREPARE_GEMV_F32
#include "common.cuh"

TB200_TU_STATUS(gemv_f32)

namespace tb200 {

constexpr int kSgemvThreads = 256;
constexpr int kSgemvUnroll = 8;

// Requirements of the fast kernel: cols % 4 == 0, so every row has the same
// 16-byte phase `head` (number of floats before the first 16-byte boundary).
__global__ void __launch_bounds__(kSgemvThreads)
sgemv_rows_kernel(const float *__restrict__ m, const float *__restrict__ v, float *__restrict__ out, int rows,
                  int cols, int head, int bulk_ok) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar;
    // xs[j] holds v[j]; shifted so that xs + head is 16-byte aligned.
    float *xs = reinterpret_cast<float *>(smem_raw) + ((4 - head) & 3);

    const int tid = threadIdx.x;
    const int interior = ((cols - head) / 4) * 4;

    if (bulk_ok) {
        if (tid == 0) {
            mbar_init(&bar, 1);
            mbar_fence_init();
        }
        __syncthreads();
        if (tid == 0) {
            // the engine accepts any multiple of 16 bytes; keep single copies modest
            uint32_t total = (uint32_t)interior * 4u;
            mbar_expect_tx(&bar, total);
            uint32_t done = 0;
            while (done < total) {
                uint32_t chunk = min(total - done, 32768u);
                bulk_g2s(reinterpret_cast<unsigned char *>(xs + head) + done,
                         reinterpret_cast<const unsigned char *>(v + head) + done, chunk, &bar);
                done += chunk;
            }
        }
        for (int j = tid; j < head; j += kSgemvThreads) xs[j] = v[j];
        for (int j = head + interior + tid; j < cols; j += kSgemvThreads) xs[j] = v[j];
        mbar_wait(&bar, 0);
    } else {
        for (int j = tid; j < cols; j += kSgemvThreads) xs[j] = v[j];
    }
    __syncthreads();

    const int lane = tid & 31;
    const int warps_per_cta = kSgemvThreads / 32;
    const int nvec = interior / 4;
    const float4 *xs4 = reinterpret_cast<const float4 *>(xs + head);

    for (int row = blockIdx.x * warps_per_cta + (tid >> 5); row < rows; row += gridDim.x * warps_per_cta) {
        const float *rowp = m + (size_t)row * cols;
        const uint4 *p4 = reinterpret_cast<const uint4 *>(rowp + head);
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        if (lane < head) a0 = rowp[lane] * xs[lane];
        int i = lane;
        for (; i + (kSgemvUnroll - 1) * 32 < nvec; i += kSgemvUnroll * 32) {
            uint4 w[kSgemvUnroll];
#pragma unroll
            for (int u = 0; u < kSgemvUnroll; ++u) w[u] = ldg_stream_v4(p4 + i + u * 32);
#pragma unroll
            for (int u = 0; u < kSgemvUnroll; ++u) {
                float4 xv = xs4[i + u * 32];
                a0 = fmaf(__uint_as_float(w[u].x), xv.x, a0);
                a1 = fmaf(__uint_as_float(w[u].y), xv.y, a1);
                a2 = fmaf(__uint_as_float(w[u].z), xv.z, a2);
                a3 = fmaf(__uint_as_float(w[u].w), xv.w, a3);
            }
        }
        for (; i < nvec; i += 32) {
            uint4 w = ldg_stream_v4(p4 + i);
            float4 xv = xs4[i];
            a0 = fmaf(__uint_as_float(w.x), xv.x, a0);
            a1 = fmaf(__uint_as_float(w.y), xv.y, a1);
            a2 = fmaf(__uint_as_float(w.z), xv.z, a2);
            a3 = fmaf(__uint_as_float(w.w), xv.w, a3);
        }
        int t = head + interior + lane;
        if (t < cols) a1 = fmaf(rowp[t], xs[t], a1);
        float s = warp_sum((a0 + a1) + (a2 + a3));
        if (lane == 0) out[row] = s;
    }
}

// Any shape: one warp per row, scalar loads, vector read from global memory.
__global__ void __launch_bounds__(kSgemvThreads)
sgemv_generic_kernel(const float *__restrict__ m, const float *__restrict__ v, float *__restrict__ out, int rows,
                     int cols) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = kSgemvThreads / 32;
    for (int row = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_cta) {
        const float *rowp = m + (size_t)row * cols;
        float a = 0.f;
        for (int j = lane; j < cols; j += 32) a = fmaf(rowp[j], __ldg(v + j), a);
        a = warp_sum(a);
        if (lane == 0) out[row] = a;
    }
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_sgemv(int rows, int cols, const float *m, const float *v, float *out, tb200_stream_t stream) {
    if (rows < 0 || cols < 0) return TB200_ERR_INVALID_ARG;
    if (rows == 0) return TB200_OK;
    if (!m || !v || !out) return TB200_ERR_INVALID_ARG;
    if (!aligned_to(m, 4) || !aligned_to(v, 4) || !aligned_to(out, 4)) return TB200_ERR_ALIGNMENT;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = kSgemvThreads / 32;
    size_t smem = (size_t)(cols + 4) * sizeof(float);
    if (cols > 0 && cols % 4 == 0 && smem + 256 <= (size_t)di->max_smem_optin) {
        int head = (int)(((16 - ((uintptr_t)m & 15)) & 15) >> 2);
        if (head > cols) head = cols;
        int bulk_ok = (((uintptr_t)m & 15) == ((uintptr_t)v & 15)) && (cols - head) >= 4;
        st = ensure_smem_optin<sgemv_rows_kernel>(di);
        if (st) return st;
        int ctas_per_sm = smem > 100 * 1024 ? 1 : (smem > 48 * 1024 ? 2 : 4);
        int grid = di->sm_count * ctas_per_sm;
        int need = (rows + warps - 1) / warps;
        if (grid > need) grid = need;
        sgemv_rows_kernel<<<grid, kSgemvThreads, smem, s>>>(m, v, out, rows, cols, head, bulk_ok);
    } else {
        int grid = di->sm_count * 8;
        int need = (rows + warps - 1) / warps;
        if (grid > need) grid = need;
        st = ensure_kernel<sgemv_generic_kernel, 0>(di);
        if (st) return st;
        sgemv_generic_kernel<<<grid, kSgemvThreads, 0, s>>>(m, v, out, rows, cols);
    }
    return check_launch();
}
