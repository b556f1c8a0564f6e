// Status strings, version, options, and the per-context bookkeeping of libtornado_b200.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

TB200_TU_STATUS(api)

namespace tb200 {

// status readers of the other translation units (TB200_TU_STATUS in each)
int tu_status_gemv_f32(int *);
int tu_status_gemv_quant(int *);
int tu_status_gemv_mma(int *);
int tu_status_gemv_tc(int *);
int tu_status_sgemm(int *);
int tu_status_hgemm(int *);
int tu_status_peer(int *);
int tu_status_read_async_api(int *);
int tu_status_clear_api();
int tu_status_read_async_gemv_f32(int *);
int tu_status_clear_gemv_f32();
int tu_status_read_async_gemv_quant(int *);
int tu_status_clear_gemv_quant();
int tu_status_read_async_gemv_mma(int *);
int tu_status_clear_gemv_mma();
int tu_status_read_async_gemv_tc(int *);
int tu_status_clear_gemv_tc();
int tu_status_read_async_sgemm(int *);
int tu_status_clear_sgemm();
int tu_status_read_async_hgemm(int *);
int tu_status_clear_hgemm();
int tu_status_read_async_peer(int *);
int tu_status_clear_peer();


// ---- options ---------------------------------------------------------------------------------
constexpr int kNumOptions = 8;  // option ids are 1 .. kNumOptions - 1
static std::atomic<int> g_option[kNumOptions] = {{0}, {0}, {1}, {1}, {1}, {2}, {2}, {1}};
struct ThreadOptions {
    unsigned set_mask = 0;
    int value[kNumOptions] = {};
};
static thread_local ThreadOptions t_options;

static int validate_option(int option, int &value) {
    switch (option) {
        case TB200_OPT_OVERLAP_LAUNCHES:
        case TB200_OPT_HGEMM_SM_PAIRS:
        case TB200_OPT_MMA_WARP_RINGS:
        case TB200_OPT_TC_REGISTER_KERNEL:
            value = value != 0;
            return TB200_OK;
        case TB200_OPT_INT_TENSOR_CORE_MIN_BATCH:
            return value < 1 || value > 17 ? TB200_ERR_INVALID_ARG : TB200_OK;
        case TB200_OPT_HGEMM_LINE_STORES:
            return value < 1 ? TB200_ERR_INVALID_ARG : TB200_OK;
        case TB200_OPT_FLOAT_TENSOR_CORES:
            value = value < 0 ? 0 : (value > 2 ? 2 : value);
            return TB200_OK;
        default:
            return TB200_ERR_INVALID_ARG;
    }
}

int option_value(int option) {
    if (option < 1 || option >= kNumOptions) return 0;
    if (t_options.set_mask & (1u << option)) return t_options.value[option];
    return g_option[option].load(std::memory_order_relaxed);
}

// ---- per-context facts -------------------------------------------------------------------------
typedef CUresult (*CtxGetCurrentFn)(CUcontext *);
typedef CUresult (*CtxGetIdFn)(CUcontext, unsigned long long *);
typedef CUresult (*CtxGetDeviceFn)(CUdevice *);

struct DriverFns {
    CtxGetCurrentFn get_current = nullptr;
    CtxGetIdFn get_id = nullptr;
    CtxGetDeviceFn get_device = nullptr;
    bool ok = false;
};

static const DriverFns &driver_fns() {
    static DriverFns fns = [] {
        DriverFns f;
        cudaDriverEntryPointQueryResult q;
        void *p = nullptr;
        bool ok = true;
        auto get = [&](const char *name) -> void * {
            p = nullptr;
            if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
                cudaGetLastError();
                ok = false;
                return nullptr;
            }
            return p;
        };
        f.get_current = reinterpret_cast<CtxGetCurrentFn>(get("cuCtxGetCurrent"));
        f.get_id = reinterpret_cast<CtxGetIdFn>(get("cuCtxGetId"));
        f.get_device = reinterpret_cast<CtxGetDeviceFn>(get("cuCtxGetDevice"));
        f.ok = ok;
        return f;
    }();
    return fns;
}

static DeviceInfo g_info[kMaxContexts];
static std::atomic<unsigned long long> g_info_id[kMaxContexts];  // context id + 1 of a filled slot, 0 = free
static std::atomic<int> g_info_count{0};
static std::mutex g_info_mutex;

const DeviceInfo *device_info(int *status) {
    const DriverFns &drv = driver_fns();
    if (!drv.ok) {
        *status = TB200_ERR_DRIVER;
        return nullptr;
    }
    CUcontext ctx = nullptr;
    if (drv.get_current(&ctx) != CUDA_SUCCESS || !ctx) {
        // no context bound to this thread yet: the runtime binds the device's primary context on demand
        cudaError_t e = cudaFree(nullptr);
        if (e != cudaSuccess) {
            cudaGetLastError();
            *status = (int)e;
            return nullptr;
        }
        if (drv.get_current(&ctx) != CUDA_SUCCESS || !ctx) {
            *status = TB200_ERR_DRIVER;
            return nullptr;
        }
    }
    unsigned long long id = 0;
    if (drv.get_id(ctx, &id) != CUDA_SUCCESS) {
        *status = TB200_ERR_DRIVER;
        return nullptr;
    }
    const unsigned long long key = id + 1;
    int n = g_info_count.load(std::memory_order_acquire);
    int slot = -1;
    for (int i = 0; i < n; ++i)
        if (g_info_id[i].load(std::memory_order_acquire) == key) {
            slot = i;
            break;
        }
    if (slot < 0) {
        std::lock_guard<std::mutex> lock(g_info_mutex);
        n = g_info_count.load(std::memory_order_acquire);
        for (int i = 0; i < n && slot < 0; ++i)
            if (g_info_id[i].load(std::memory_order_acquire) == key) slot = i;
        if (slot < 0) {
            if (n >= kMaxContexts) {  // more live-and-dead contexts than the caches hold
                *status = TB200_ERR_UNSUPPORTED;
                return nullptr;
            }
            DeviceInfo di{};
            CUdevice dev = 0;
            if (drv.get_device(&dev) != CUDA_SUCCESS) {
                *status = TB200_ERR_DRIVER;
                return nullptr;
            }
            int v = 0;
            cudaError_t e = cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, (int)dev);
            if (e != cudaSuccess) {
                cudaGetLastError();
                *status = (int)e;
                return nullptr;
            }
            di.device = (int)dev, di.sm_count = v;
            cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, (int)dev);
            di.cc_major = v;
            cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, (int)dev);
            di.max_smem_optin = v;
            di.slot = n, di.context_id = id;
            g_info[n] = di;
            g_info_id[n].store(key, std::memory_order_release);
            g_info_count.store(n + 1, std::memory_order_release);
            slot = n;
        }
    }
    if (g_info[slot].cc_major != 10) {
        *status = TB200_ERR_UNSUPPORTED;
        return nullptr;
    }
    *status = TB200_OK;
    return &g_info[slot];
}

// ---- kernel registry -----------------------------------------------------------------------------
static std::atomic<KernelEntry *> &kernel_list() {
    static std::atomic<KernelEntry *> head{nullptr};
    return head;
}

bool register_kernel(KernelEntry *e, const void *func, int flags, int op_class) {
    e->func = func, e->flags = flags, e->op_class = op_class;
    std::atomic<KernelEntry *> &head = kernel_list();
    KernelEntry *old = head.load(std::memory_order_relaxed);
    do {
        e->next = old;
    } while (!head.compare_exchange_weak(old, e, std::memory_order_release, std::memory_order_relaxed));
    return true;
}

int prepare_kernel(KernelEntry *e, const DeviceInfo *di) {
    // the attribute query loads the kernel into the current context
    cudaFuncAttributes attr;
    cudaError_t err = cudaFuncGetAttributes(&attr, e->func);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return (int)err;
    }
    if (e->flags & KERNEL_OPTIN_SMEM) {
        // the opt-in limit covers static + dynamic shared memory of the kernel
        err = cudaFuncSetAttribute(e->func, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin - (int)attr.sharedSizeBytes);
        if (err != cudaSuccess) {
            cudaGetLastError();
            return (int)err;
        }
    }
    if (e->flags & KERNEL_MAX_CARVEOUT) {
        cudaFuncSetAttribute(e->func, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaGetLastError();
    }
    e->ready[di->slot].store(1, std::memory_order_release);
    return TB200_OK;
}

int hgemm_prepare_driver();  // hgemm.cu: resolves the tensor-map encoder

}  // namespace tb200

using namespace tb200;

extern "C" const char *tb200_status_string(int status) {
    switch (status) {
        case TB200_OK: return "TB200_OK";
        case TB200_ERR_INVALID_ARG: return "TB200_ERR_INVALID_ARG";
        case TB200_ERR_ALIGNMENT: return "TB200_ERR_ALIGNMENT";
        case TB200_ERR_WORKSPACE: return "TB200_ERR_WORKSPACE";
        case TB200_ERR_UNSUPPORTED: return "TB200_ERR_UNSUPPORTED";
        case TB200_ERR_DRIVER: return "TB200_ERR_DRIVER";
        case TB200_ERR_TIMEOUT: return "TB200_ERR_TIMEOUT";
        default: break;
    }
    if (status > 0) return cudaGetErrorName((cudaError_t)status);
    return "TB200_ERR_UNKNOWN";
}

extern "C" int tb200_version(void) { return TB200_VERSION; }

extern "C" int tb200_device_status_of(int op_classes, int *status_out) {
    if (!status_out) return TB200_ERR_INVALID_ARG;
    struct Reader {
        int (*read_async)(int *);
        int (*clear)();
        int op_class;
    };
    static const Reader readers[] = {{tu_status_read_async_api, tu_status_clear_api, TB200_PREPARE_ALL},
                                     {tu_status_read_async_gemv_f32, tu_status_clear_gemv_f32, TB200_PREPARE_GEMV_F32},
                                     {tu_status_read_async_gemv_quant, tu_status_clear_gemv_quant, TB200_PREPARE_GEMV_QUANT},
                                     {tu_status_read_async_gemv_mma, tu_status_clear_gemv_mma, TB200_PREPARE_GEMV_QUANT},
                                     {tu_status_read_async_gemv_tc, tu_status_clear_gemv_tc, TB200_PREPARE_GEMV_QUANT},
                                     {tu_status_read_async_sgemm, tu_status_clear_sgemm, TB200_PREPARE_GEMM_F32},
                                     {tu_status_read_async_hgemm, tu_status_clear_hgemm, TB200_PREPARE_GEMM_F16},
                                     {tu_status_read_async_peer, tu_status_clear_peer, TB200_PREPARE_PEER}};
    constexpr int kReaders = sizeof(readers) / sizeof(readers[0]);
    // One word per translation unit: the reads are enqueued together into pinned memory and waited for once (a
    // host class calls this after every step; eight blocking copies cost more than the step's launch).
    static std::mutex mutex;
    static int *pinned = nullptr;
    std::lock_guard<std::mutex> lock(mutex);
    if (!pinned) {
        void *p = nullptr;
        cudaError_t e = cudaHostAlloc(&p, kReaders * sizeof(int), cudaHostAllocPortable);
        if (e != cudaSuccess) return (int)e;
        pinned = static_cast<int *>(p);
    }
    if (op_classes == 0) op_classes = TB200_PREPARE_ALL;
    bool selected[kReaders];
    for (int i = 0; i < kReaders; ++i) {
        const Reader &r = readers[i];
        selected[i] = r.op_class != TB200_PREPARE_ALL ? (r.op_class & op_classes) != 0 : op_classes == TB200_PREPARE_ALL;
        pinned[i] = 0;
        if (selected[i]) {
            const int st = r.read_async(pinned + i);
            if (st) return st;
        }
    }
    cudaError_t e = cudaStreamSynchronize(0);
    if (e != cudaSuccess) return (int)e;
    int combined = 0;
    for (int i = 0; i < kReaders; ++i) {
        if (!selected[i] || pinned[i] == 0) continue;
        if (combined == 0) combined = pinned[i];
        const int st = readers[i].clear();  // read and clear, like cudaGetLastError
        if (st) return st;
    }
    *status_out = combined;
    return TB200_OK;
}

extern "C" int tb200_device_status(int *status_out) { return tb200_device_status_of(TB200_PREPARE_ALL, status_out); }

extern "C" int tb200_prepare(int op_classes) {
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    if (op_classes == 0) op_classes = TB200_PREPARE_ALL;
    for (KernelEntry *e = kernel_list().load(std::memory_order_acquire); e; e = e->next) {
        if (!(e->op_class & op_classes) || e->ready[di->slot].load(std::memory_order_acquire)) continue;
        st = prepare_kernel(e, di);
        if (st) return st;
    }
    if (op_classes & TB200_PREPARE_GEMM_F16) {
        st = hgemm_prepare_driver();
        if (st) return st;
    }
    return TB200_OK;
}

extern "C" int tb200_device_malloc(size_t bytes, void **out) {
    if (!out) return TB200_ERR_INVALID_ARG;
    *out = nullptr;
    if (bytes == 0) return TB200_OK;
    return (int)cudaMalloc(out, bytes);
}

extern "C" int tb200_device_free(void *ptr) {
    if (!ptr) return TB200_OK;
    return (int)cudaFree(ptr);
}

extern "C" int tb200_set_option(int option, int value) {
    const int st = validate_option(option, value);
    if (st) return st;
    g_option[option].store(value, std::memory_order_relaxed);
    return TB200_OK;
}

extern "C" int tb200_get_option(int option, int *value) {
    if (!value || option < 1 || option >= kNumOptions) return TB200_ERR_INVALID_ARG;
    *value = option_value(option);
    return TB200_OK;
}

extern "C" int tb200_set_thread_option(int option, int value) {
    const int st = validate_option(option, value);
    if (st) return st;
    t_options.set_mask |= 1u << option;
    t_options.value[option] = value;
    return TB200_OK;
}

extern "C" int tb200_clear_thread_options(void) {
    t_options.set_mask = 0;
    return TB200_OK;
}
