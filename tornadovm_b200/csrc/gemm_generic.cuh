// CUDA-core GEMM for shapes and alignments the tiled / tensor-core kernels do not take.
#pragma once

#include "common.cuh"

namespace tb200 {

// Any shape and 4-byte alignment: 32x32 tiles, one output per thread.
// TA / TB are float or __half-bit patterns (uint16_t): the FP16 GEMM reuses this
// kernel for shapes its tensor-core path does not take.
template <typename TA>
__device__ __forceinline__ float to_f32(TA v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<uint16_t>(uint16_t v) { return half_bits_to_float(v); }

template <typename TIN>
__global__ void __launch_bounds__(1024)
gemm_generic_kernel(int m, int n, int k, float alpha, const TIN *__restrict__ A, const TIN *__restrict__ B, float beta,
                    float *__restrict__ C) {
    __shared__ float As[32][33];
    __shared__ float Bs[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int row = blockIdx.y * 32 + ty, col = blockIdx.x * 32 + tx;
    float acc = 0.f;
    for (int k0 = 0; k0 < k; k0 += 32) {
        As[ty][tx] = (row < m && k0 + tx < k) ? to_f32<TIN>(A[(size_t)row * k + k0 + tx]) : 0.f;
        Bs[ty][tx] = (k0 + ty < k && col < n) ? to_f32<TIN>(B[(size_t)(k0 + ty) * n + col]) : 0.f;
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 32; ++kk) acc = fmaf(As[ty][kk], Bs[kk][tx], acc);
        __syncthreads();
    }
    if (row < m && col < n) {
        float *cp = C + (size_t)row * n + col;
        *cp = beta != 0.f ? fmaf(beta, *cp, alpha * acc) : alpha * acc;
    }
}

}  // namespace tb200
