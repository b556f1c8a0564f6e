// Status strings, version and per-device bookkeeping of libtornado_b200.
#include <mutex>

#include "common.cuh"

namespace tb200 {

int g_overlap_launches = 0;
int g_float_tensor_cores = 1;
int g_mma_warp_rings = 1;
int g_int_tc_min_batch = 4;
int g_float_tc_min_batch = 0;  // 0: per-format default, 1: every eligible call
extern int g_hgemm_pairs;
extern int g_hgemm_xpose_min_dst;

static DeviceInfo g_info[kMaxDevices];
static bool g_info_valid[kMaxDevices];
static std::mutex g_info_mutex;

const DeviceInfo *device_info(int *status) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        *status = (int)e;
        return nullptr;
    }
    if (dev < 0 || dev >= kMaxDevices) {
        *status = TB200_ERR_INVALID_ARG;
        return nullptr;
    }
    if (!g_info_valid[dev]) {
        std::lock_guard<std::mutex> lock(g_info_mutex);
        if (!g_info_valid[dev]) {
            DeviceInfo di{};
            int v = 0;
            if ((e = cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) {
                *status = (int)e;
                return nullptr;
            }
            di.device = dev;
            di.sm_count = v;
            cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, dev);
            di.cc_major = v;
            cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
            di.max_smem_optin = v;
            g_info[dev] = di;
            g_info_valid[dev] = true;
        }
    }
    if (g_info[dev].cc_major != 10) {
        *status = TB200_ERR_UNSUPPORTED;
        return nullptr;
    }
    *status = TB200_OK;
    return &g_info[dev];
}

}  // namespace tb200

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

extern "C" int tb200_device_status(int *status_out) {
    if (!status_out) return TB200_ERR_INVALID_ARG;
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, tb200::g_device_status, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    if (v != 0) {
        // read and clear, like cudaGetLastError
        const int zero = 0;
        e = cudaMemcpyToSymbol(tb200::g_device_status, &zero, sizeof(int));
        if (e != cudaSuccess) return (int)e;
    }
    *status_out = v;
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
    switch (option) {
        case TB200_OPT_OVERLAP_LAUNCHES:
            tb200::g_overlap_launches = value != 0;
            return TB200_OK;
        case TB200_OPT_HGEMM_SM_PAIRS:
            tb200::g_hgemm_pairs = value != 0;
            return TB200_OK;
        case TB200_OPT_MMA_WARP_RINGS:
            tb200::g_mma_warp_rings = value != 0;
            return TB200_OK;
        case TB200_OPT_INT_TENSOR_CORE_MIN_BATCH:
            if (value < 2 || value > 17) return TB200_ERR_INVALID_ARG;
            tb200::g_int_tc_min_batch = value;
            return TB200_OK;
        case TB200_OPT_HGEMM_LINE_STORES:
            if (value < 1) return TB200_ERR_INVALID_ARG;
            tb200::g_hgemm_xpose_min_dst = value;
            return TB200_OK;
        case TB200_OPT_FLOAT_TENSOR_CORES:
            tb200::g_float_tensor_cores = value != 0;
            tb200::g_float_tc_min_batch = value >= 2 ? 1 : 0;
            return TB200_OK;
        default:
            return TB200_ERR_INVALID_ARG;
    }
}

extern "C" int tb200_get_option(int option, int *value) {
    if (!value) return TB200_ERR_INVALID_ARG;
    switch (option) {
        case TB200_OPT_OVERLAP_LAUNCHES:
            *value = tb200::g_overlap_launches;
            return TB200_OK;
        case TB200_OPT_HGEMM_SM_PAIRS:
            *value = tb200::g_hgemm_pairs;
            return TB200_OK;
        case TB200_OPT_MMA_WARP_RINGS:
            *value = tb200::g_mma_warp_rings;
            return TB200_OK;
        case TB200_OPT_INT_TENSOR_CORE_MIN_BATCH:
            *value = tb200::g_int_tc_min_batch;
            return TB200_OK;
        case TB200_OPT_HGEMM_LINE_STORES:
            *value = tb200::g_hgemm_xpose_min_dst;
            return TB200_OK;
        case TB200_OPT_FLOAT_TENSOR_CORES:
            *value = tb200::g_float_tensor_cores ? 1 + tb200::g_float_tc_min_batch : 0;
            return TB200_OK;
        default:
            return TB200_ERR_INVALID_ARG;
    }
}
