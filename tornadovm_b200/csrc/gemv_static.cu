// Allocation-free entry point of the integer-path Q8_0 mat-vec (split layout).
//
// It reuses the quantiser and the mat-vec dispatch of gemv_quant.cu and adds
// only the built-in scratch array and the entry point that uses it.
#define TB200_OP_CLASS TB200_PREPARE_GEMV_QUANT
#include "gemv_common.cuh"

// The quantised activations go to a fixed scratch array that is part of the
// loaded library image in every CUDA context, instead of caller-provided workspace.
namespace tb200 {

static __device__ __align__(256) unsigned char g_static_qx_scratch[TB200_STATIC_SCRATCH_BYTES];

// Device address of the scratch array, resolved once per CUDA context.  The
// array's name is only a host-side handle here; kernels need the address the
// runtime reports for the context that is current.  A __device__ variable is
// instantiated once per context that loads the library (a process may hold
// several contexts on one GPU), so the cache is indexed by the context's slot,
// never by the device ordinal.
static std::atomic<void *> g_static_scratch_ptr[kMaxContexts];

static int static_scratch(const DeviceInfo *di, void **out) {
    void *p = g_static_scratch_ptr[di->slot].load(std::memory_order_acquire);
    if (!p) {
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_qx_scratch);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return (int)e;
        }
        g_static_scratch_ptr[di->slot].store(p, std::memory_order_release);
    }
    *out = p;
    return TB200_OK;
}

}  // namespace tb200

using namespace tb200;

// Test hook: the address the entry point below will hand to its kernels in the current context
// (`in_use`) and what the runtime reports for the array in this context right now (`fresh`).
extern "C" int tb200_static_scratch_address(void **in_use, void **fresh) {
    if (!in_use || !fresh) return TB200_ERR_INVALID_ARG;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    st = static_scratch(di, in_use);
    if (st) return st;
    cudaError_t e = cudaGetSymbolAddress(fresh, g_static_qx_scratch);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return (int)e;
    }
    return TB200_OK;
}

extern "C" int tb200_q8_gemv_i8_static(int rows, int cols, int batch, const int8_t *q, const uint16_t *scales,
                                       const float *x, float *y, tb200_stream_t stream) {
    if (rows < 0 || cols < 0 || cols % 32 != 0 || batch < 1 || batch > kMaxBatch) return TB200_ERR_INVALID_ARG;
    const size_t need = tb200_qx_workspace_bytes(cols, batch);
    if (need > (size_t)TB200_STATIC_SCRATCH_BYTES) return TB200_ERR_WORKSPACE;  // beyond the built-in scratch
    if (rows == 0) return TB200_OK;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    void *scratch = nullptr;
    st = static_scratch(di, &scratch);
    if (st) return st;
    int8_t *xq;
    float *xs;
    st = split_workspace(cols, batch, scratch, TB200_STATIC_SCRATCH_BYTES, &xq, &xs);
    if (st) return st;
    // always the two-kernel form: quantiser into the scratch, then the mat-vec that reads it
    st = quantize_x(cols, batch, x, xq, xs, (cudaStream_t)stream);
    if (st) return st;
    QGemvArgs a{reinterpret_cast<const uint8_t *>(q), scales, nullptr, xq, xs, y, nullptr, rows, cols, batch};
    return q8s_gemv_quantised(a, stream);
}
