// FP32 SGEMM on CUDA cores (FFMA), C = alpha * A * B + beta * C, row-major.
//
// Replaces the naive one-thread-per-element kernel of the reference
// (MatrixMultiplication2D.java:48-58) and its 32x32 shared-memory tiled variant
// (tornado-cublas/.../tests/BenchmarkSgemm.java:75-99).
//
// Fast kernel: 128x128 CTA tile, BK = 16, 256 threads, 8x8 outputs per thread
// held in registers, operands staged through double-buffered shared memory
// with 128-bit global and shared accesses; A is transposed on the way into
// shared memory so that both operands are read as float4 along the output
// dimension.  Roofline: FP32 FFMA peak = SMs * 128 lanes * 2 * clock.
// flops per launch: 2*m*n*k.
#define TB200_OP_CLASS TB200_PREPARE_GEMM_F32
#include "common.cuh"
#include "gemm_generic.cuh"

TB200_TU_STATUS(sgemm)

namespace tb200 {

constexpr int SG_BM = 128, SG_BN = 128, SG_BK = 16, SG_THREADS = 256;
constexpr int SG_APAD = 4;  // row padding of the transposed A tile (bank spread)

// 128-bit global load, or two 64-bit ones for operands that are only 8-byte aligned (a TornadoVM array
// behind a 24-byte header)
template <bool VEC4>
__device__ __forceinline__ float4 sg_load4(const float *p) {
    if (VEC4) return __ldg(reinterpret_cast<const float4 *>(p));
    const float2 lo = __ldg(reinterpret_cast<const float2 *>(p)), hi = __ldg(reinterpret_cast<const float2 *>(p) + 1);
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// Requirements: k % 4 == 0, n % 4 == 0, A and B 16-byte aligned (VEC4) or 8-byte aligned.
template <bool VEC4>
__global__ void __launch_bounds__(SG_THREADS, 2)
sgemm_tiled_kernel(int m, int n, int k, float alpha, const float *__restrict__ A, const float *__restrict__ B,
                   float beta, float *__restrict__ C) {
    __shared__ __align__(16) float As[2][SG_BK][SG_BM + SG_APAD];
    __shared__ __align__(16) float Bs[2][SG_BK][SG_BN];

    const int tid = threadIdx.x;
    const int bm = blockIdx.y * SG_BM, bn = blockIdx.x * SG_BN;

    // global -> register staging coordinates
    const int a_row = tid >> 2;        // 0..63 (+64 for the second load)
    const int a_kq = (tid & 3) * 4;    // 0,4,8,12
    const int b_row = tid >> 5;        // 0..7 (+8)
    const int b_col = (tid & 31) * 4;  // 0..124

    // thread tile: rows ty*4 + {0..3} and 64 + ty*4 + {0..3}; same for columns
    // a warp covers 4 x 8 threads of the 16 x 16 grid: its B reads are 128 contiguous bytes (one shared-memory
    // wavefront), its A reads four broadcast addresses
    const int warp = tid >> 5, lane = tid & 31;
    const int ty = (warp >> 1) * 4 + (lane >> 3), tx = (warp & 1) * 8 + (lane & 7);

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    float4 ra[2], rb[2];
    auto load_global = [&](int k0) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int gr = bm + a_row + 64 * j, gk = k0 + a_kq;
            ra[j] = (gr < m && gk < k) ? sg_load4<VEC4>(A + (size_t)gr * k + gk) : make_float4(0.f, 0.f, 0.f, 0.f);
            const int gkb = k0 + b_row + 8 * j, gc = bn + b_col;
            rb[j] = (gkb < k && gc < n) ? sg_load4<VEC4>(B + (size_t)gkb * n + gc) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto store_shared = [&](int buf) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int r = a_row + 64 * j;
            As[buf][a_kq + 0][r] = ra[j].x;
            As[buf][a_kq + 1][r] = ra[j].y;
            As[buf][a_kq + 2][r] = ra[j].z;
            As[buf][a_kq + 3][r] = ra[j].w;
            *reinterpret_cast<float4 *>(&Bs[buf][b_row + 8 * j][b_col]) = rb[j];
        }
    };

    const int ktiles = (k + SG_BK - 1) / SG_BK;
    load_global(0);
    store_shared(0);
    __syncthreads();

    for (int kt = 0; kt < ktiles; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < ktiles) load_global((kt + 1) * SG_BK);
#pragma unroll
        for (int kk = 0; kk < SG_BK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4 *>(&As[buf][kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4 *>(&As[buf][kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[buf][kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[buf][kk][64 + tx * 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        if (kt + 1 < ktiles) {
            store_shared(buf ^ 1);
            __syncthreads();
        }
    }

    // epilogue: 128-bit stores when C rows allow it
    const bool c_vec = ((uintptr_t)C & 15) == 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int gr = bm + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (gr >= m) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int gc = bn + h * 64 + tx * 4;
            if (gc >= n) continue;  // n % 4 == 0: a quad is either fully inside or outside
            float *cp = C + (size_t)gr * n + gc;
            float4 v = make_float4(alpha * acc[i][h * 4 + 0], alpha * acc[i][h * 4 + 1], alpha * acc[i][h * 4 + 2],
                                   alpha * acc[i][h * 4 + 3]);
            if (c_vec) {
                if (beta != 0.f) {
                    const float4 old = *reinterpret_cast<const float4 *>(cp);
                    v.x = fmaf(beta, old.x, v.x), v.y = fmaf(beta, old.y, v.y);
                    v.z = fmaf(beta, old.z, v.z), v.w = fmaf(beta, old.w, v.w);
                }
                *reinterpret_cast<float4 *>(cp) = v;
            } else {
                if (beta != 0.f) {
                    v.x = fmaf(beta, cp[0], v.x), v.y = fmaf(beta, cp[1], v.y);
                    v.z = fmaf(beta, cp[2], v.z), v.w = fmaf(beta, cp[3], v.w);
                }
                cp[0] = v.x, cp[1] = v.y, cp[2] = v.z, cp[3] = v.w;
            }
        }
    }
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_sgemm(int m, int n, int k, float alpha, const float *a, const float *b, float beta, float *c,
                           tb200_stream_t stream) {
    if (m < 0 || n < 0 || k < 0) return TB200_ERR_INVALID_ARG;
    if (m == 0 || n == 0) return TB200_OK;
    if (!c || (k > 0 && (!a || !b))) return TB200_ERR_INVALID_ARG;
    if (!aligned_to(a, 4) || !aligned_to(b, 4) || !aligned_to(c, 4)) return TB200_ERR_ALIGNMENT;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    cudaStream_t s = (cudaStream_t)stream;
    const bool fast = k > 0 && k % 4 == 0 && n % 4 == 0 && aligned_to(a, 8) && aligned_to(b, 8) && m >= 64 && n >= 64;
    if (fast) {
        dim3 grid((n + SG_BN - 1) / SG_BN, (m + SG_BM - 1) / SG_BM);
        if (aligned_to(a, 16) && aligned_to(b, 16)) {
            st = ensure_kernel<sgemm_tiled_kernel<true>, 0>(di);
            if (st) return st;
            sgemm_tiled_kernel<true><<<grid, SG_THREADS, 0, s>>>(m, n, k, alpha, a, b, beta, c);
        } else {
            st = ensure_kernel<sgemm_tiled_kernel<false>, 0>(di);
            if (st) return st;
            sgemm_tiled_kernel<false><<<grid, SG_THREADS, 0, s>>>(m, n, k, alpha, a, b, beta, c);
        }
    } else {
        dim3 grid((n + 31) / 32, (m + 31) / 32);
        st = ensure_kernel<gemm_generic_kernel<float>, 0>(di);
        if (st) return st;
        gemm_generic_kernel<float><<<grid, 1024, 0, s>>>(m, n, k, alpha, a, b, beta, c);
    }
    return check_launch();
}
