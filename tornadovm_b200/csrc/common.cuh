// Shared helpers of libtornado_b200: status codes, launch checks, and the few
// PTX wrappers (mbarrier, bulk async copy) the GEMV kernels need.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "tornado_b200.h"

namespace tb200 {

// Sticky status word: a kernel that gives up a bounded wait stores
// TB200_ERR_TIMEOUT here instead of trapping, so the context stays usable.
// The library is several translation units without relocatable device code, so
// each unit owns one copy; TB200_TU_STATUS(name) below exports a reader for it
// and tb200_device_status (api.cu) combines them.
static __device__ int g_device_status = 0;

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

// Facts about the CUDA context that is current on the calling thread, cached per
// context (queried once, no allocation).  TornadoVM's NVIDIA backends each create
// their own context per device (cuCtxCreate; cuda-jni/.../CUDAPlatform.cpp:118-146,
// ptx-jni/.../PTXContext.cpp:37-51) next to the primary one, and kernel attributes,
// loaded modules and __device__ symbol addresses all belong to a context, not to a
// device ordinal: every cache of the library is therefore indexed by `slot`.
constexpr int kMaxContexts = 64;
struct DeviceInfo {
    int device;
    int sm_count;
    int cc_major;
    int max_smem_optin;
    int slot;                      // index of the current context in the per-context caches
    unsigned long long context_id; // cuCtxGetId of that context
};
const DeviceInfo *device_info(int *status);

// One entry per __global__ function the library launches.  Entries register themselves when the
// library is loaded, so that tb200_prepare can make every kernel resident and configured in the
// current context before a stream capture begins (the first launch of a kernel otherwise loads its
// module and sets its attributes lazily, which a capture in global mode does not allow).
constexpr int KERNEL_OPTIN_SMEM = 1;     // opt in to the device's full dynamic shared memory
constexpr int KERNEL_MAX_CARVEOUT = 2;   // prefer the largest shared-memory carve-out
struct KernelEntry {
    const void *func;
    int flags;
    int op_class;                              // TB200_PREPARE_* bit of the unit that launches it
    std::atomic<unsigned char> ready[kMaxContexts];
    std::atomic<long long> occupancy[kMaxContexts];  // (dynamic smem bytes << 8 | resident CTAs) of the last query, 0 = none
    KernelEntry *next;
};
bool register_kernel(KernelEntry *e, const void *func, int flags, int op_class);
int prepare_kernel(KernelEntry *e, const DeviceInfo *di);

#ifndef TB200_OP_CLASS
#define TB200_OP_CLASS 0
#endif

template <auto kernel, int FLAGS>
struct KernelReg {
    static KernelEntry entry;
    static const bool registered;
};
template <auto kernel, int FLAGS>
KernelEntry KernelReg<kernel, FLAGS>::entry;
template <auto kernel, int FLAGS>
const bool KernelReg<kernel, FLAGS>::registered =
    register_kernel(&KernelReg<kernel, FLAGS>::entry, reinterpret_cast<const void *>(kernel), FLAGS, TB200_OP_CLASS);

// Makes `kernel` ready in the current context: loaded, and opted in to the full dynamic shared
// memory when FLAGS asks for it.  After tb200_prepare this is one relaxed load.
template <auto kernel, int FLAGS = KERNEL_OPTIN_SMEM>
static inline int ensure_kernel(const DeviceInfo *di) {
    (void)&KernelReg<kernel, FLAGS>::registered;  // instantiates the registration
    KernelEntry *e = &KernelReg<kernel, FLAGS>::entry;
    if (e->ready[di->slot].load(std::memory_order_acquire)) return TB200_OK;
    return prepare_kernel(e, di);
}
template <auto kernel>
static inline int ensure_smem_optin(const DeviceInfo *di) { return ensure_kernel<kernel, KERNEL_OPTIN_SMEM>(di); }

// Resident CTAs per SM of a kernel at a given block size and dynamic shared memory, cached per
// context for the size last asked about (a mat-vec task asks for the same size on every launch).
template <auto kernel, int FLAGS = KERNEL_OPTIN_SMEM>
static inline int resident_ctas(const DeviceInfo *di, int threads, size_t smem) {
    KernelEntry *e = &KernelReg<kernel, FLAGS>::entry;
    const long long cached = e->occupancy[di->slot].load(std::memory_order_relaxed);
    if (cached && (size_t)(cached >> 8) == smem) return (int)(cached & 0xFF);
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem) != cudaSuccess) {
        cudaGetLastError();
        n = 1;
    }
    n = n < 1 ? 1 : (n > 255 ? 255 : n);
    e->occupancy[di->slot].store(((long long)smem << 8) | n, std::memory_order_relaxed);
    return n;
}

// Exports this translation unit's status word (read, and clear when set).
#define TB200_TU_STATUS(name)                                                                   \
    namespace tb200 {                                                                           \
    /* read and clear */                                                                        \
    int tu_status_##name(int *value) {                                                          \
        int v = 0;                                                                              \
        cudaError_t e = cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int));                 \
        if (e != cudaSuccess) return (int)e;                                                    \
        if (v != 0) {                                                                           \
            const int zero = 0;                                                                 \
            e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));                        \
            if (e != cudaSuccess) return (int)e;                                                \
        }                                                                                       \
        *value = v;                                                                             \
        return TB200_OK;                                                                        \
    }                                                                                           \
    /* the same in two steps, so that one synchronisation serves several units: enqueue the read */ \
    /* into pinned memory on the legacy stream, and clear after the caller has synchronised */   \
    int tu_status_read_async_##name(int *pinned) {                                              \
        return (int)cudaMemcpyFromSymbolAsync(pinned, g_device_status, sizeof(int), 0, cudaMemcpyDeviceToHost, 0); \
    }                                                                                           \
    int tu_status_clear_##name() {                                                              \
        const int zero = 0;                                                                     \
        return (int)cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));                    \
    }                                                                                           \
    }

// Options: process-wide defaults (tb200_set_option) that a thread may override for the calls it
// makes (tb200_set_thread_option / tb200_clear_thread_options), which is how a provider applies a
// task's tuning object around one dispatch without touching other plans.
int option_value(int option);

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
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void bulk_g2s_stream(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void bulk_g2s_stream(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    const uint64_t policy = l2_evict_first_policy();
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

// ---- bounded waits on flags that another GPU writes ----
__device__ __forceinline__ unsigned long long qg_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait until the flag word has reached `target` (step numbers wrap, hence the signed difference).
__device__ __forceinline__ void wait_flag_at_least(const unsigned *flag, unsigned target, unsigned long long timeout_ns) {
    const unsigned long long t0 = qg_timer_ns();
    for (unsigned spin = 0;; ++spin) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if ((int)(v - target) >= 0) return;
        if ((spin & 63) == 63 && qg_timer_ns() - t0 > timeout_ns) {
            g_device_status = TB200_ERR_TIMEOUT;
            return;
        }
    }
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
