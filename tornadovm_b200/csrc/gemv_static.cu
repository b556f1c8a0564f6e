// Allocation-free entry point of the integer-path Q8_0 mat-vec (split layout).
//
// Part of the single translation unit of the library (see libtornado_b200.cu):
// it reuses the quantiser and the mat-vec dispatch of gemv_quant.cu and adds
// only the built-in scratch array and the entry point that uses it.
#include <mutex>

#include "common.cuh"

// The quantised activations go to a fixed scratch array that is part of the
// loaded library image on every device, instead of caller-provided workspace.
namespace tb200 {

static __device__ __align__(256) unsigned char g_static_qx_scratch[TB200_STATIC_SCRATCH_BYTES];

// Device address of the scratch array, resolved once per device.  The array's
// name is only a host-side handle here; kernels need the address the runtime
// reports for the device that is current.
static void *g_static_scratch_ptr[kMaxDevices];
static std::mutex g_static_scratch_mutex;

static int static_scratch(const DeviceInfo *di, void **out) {
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_ptr[di->device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_qx_scratch);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return (int)e;
        }
        g_static_scratch_ptr[di->device] = p;
    }
    *out = g_static_scratch_ptr[di->device];
    return TB200_OK;
}

}  // namespace tb200

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
    return qgemv_dispatch<FMT_Q8S, MODE_INT, false>(a, nullptr, nullptr, stream);
}
