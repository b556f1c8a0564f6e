// Shared helpers of libtornado_b200: status codes, launch checks, and the few
// PTX wrappers (mbarrier, bulk async copy) the GEMV kernels need.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tornado_b200.h"

namespace tb200 {

// Device-wide sticky status word: a kernel that gives up a bounded wait stores
// TB200_ERR_TIMEOUT here instead of trapping, so the context stays usable.
// (The library is built as one translation unit, see libtornado_b200.cu.)
__device__ int g_device_status = 0;

constexpr int kWarp = 32;

static inline int check_launch() {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();  // clear the non-sticky launch error
        return (int)e;
    }
    return TB200_OK;
}

static inline bool aligned_to(const void *p, uintptr_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

// Cached per-device facts (queried once per device, no allocation).
struct DeviceInfo {
    int device;
    int sm_count;
    int cc_major;
    int max_smem_optin;
};
const DeviceInfo *device_info(int *status);

constexpr int kMaxDevices = 64;

// Opt a kernel in to the device's full dynamic shared memory, once per device
// and kernel.  The first call for a kernel should come from a warm-up launch or
// a prepare step, outside any stream capture.
template <auto kernel>
static int ensure_smem_optin(const DeviceInfo *di) {
    static bool done[kMaxDevices];
    if (!done[di->device]) {
        // the opt-in limit covers static + dynamic shared memory of the kernel
        cudaFuncAttributes attr;
        cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 di->max_smem_optin - (int)attr.sharedSizeBytes);
        if (e != cudaSuccess) return (int)e;
        done[di->device] = true;
    }
    return TB200_OK;
}

// Process-wide options (tb200_set_option).
extern int g_overlap_launches;
extern int g_float_tensor_cores;   // float-mode quantised mat-vec on the tensor cores (fp16 hi/lo split of x)
extern int g_float_tc_min_batch;
extern int g_int_tc_min_batch;     // smallest batch of the integer mode that runs on the tensor cores
extern int g_mma_warp_rings;      // tensor-core mat-vec: per-warp rings (1) or the CTA-wide ring (0)   // smallest batch that takes that path

// Launch through cudaLaunchKernelEx so that a kernel can carry the programmatic
// stream serialization attribute: it may then begin while its predecessor in
// the stream is still draining.  Such kernels call pdl_wait() before they touch
// anything the predecessor may have produced.
template <typename... KArgs, typename... Args>
static int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool overlap,
                         Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (overlap) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return (int)e;
    }
    return check_launch();
}

// --------------------------------------------------------------------------
// PTX wrappers
// --------------------------------------------------------------------------
// Programmatic dependent launch: both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: returns false (and records the timeout) instead of spinning
// forever.  try_wait itself blocks for a hardware-defined slice, so the limit
// is generous in wall time but finite.
constexpr uint32_t kMbarSpinLimit = 1u << 22;

__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    for (uint32_t i = 0; i < kMbarSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    g_device_status = TB200_ERR_TIMEOUT;
    return false;
}

// 1-D bulk async copy global -> shared (TMA engine, no tensor map).  Both
// addresses must be 16-byte aligned and `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Same, with an L2 evict-first hint: weights are streamed once and should not
// displace the activation vector.
__device__ __forceinline__ void bulk_g2s_stream(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// Streaming 128-bit / 64-bit / 32-bit global loads that bypass L1 allocation.
__device__ __forceinline__ uint4 ldg_stream_v4(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
__device__ __forceinline__ uint2 ldg_stream_v2(const void *p) {
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// int8 lanes of a 32-bit word -> fp32 without I2F: bias each byte to unsigned,
// splice it into the mantissa of 2^23 and subtract 2^23 + 128.  Exact.
__device__ __forceinline__ void s8x4_to_f32(uint32_t w, float &f0, float &f1, float &f2, float &f3) {
    uint32_t u = w ^ 0x80808080u;
    f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
    f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
    f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
    f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
}

// four unsigned bytes (0..255) + compile-time bias -> fp32
__device__ __forceinline__ void u8x4_to_f32(uint32_t u, float bias, float &f0, float &f1, float &f2, float &f3) {
    f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - bias;
    f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - bias;
    f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - bias;
    f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - bias;
}

__device__ __forceinline__ float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

}  // namespace tb200
