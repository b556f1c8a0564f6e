// FP16 GEMM with fp32 accumulation and output: C[m][n] = A[m][k] * B[k][n].
#include "common.cuh"

using namespace tb200;

extern "C" int tb200_hgemm_f32(int m, int n, int k, const uint16_t *a, const uint16_t *b, float *c,
                               tb200_stream_t stream) {
    if (m < 0 || n < 0 || k < 0) return TB200_ERR_INVALID_ARG;
    if (m == 0 || n == 0) return TB200_OK;
    if (!c || (k > 0 && (!a || !b))) return TB200_ERR_INVALID_ARG;
    if (!aligned_to(a, 2) || !aligned_to(b, 2) || !aligned_to(c, 4)) return TB200_ERR_ALIGNMENT;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((n + 31) / 32, (m + 31) / 32);
    gemm_generic_kernel<uint16_t><<<grid, 1024, 0, s>>>(m, n, k, 1.0f, a, b, 0.0f, c);
    return check_launch();
}
