// Hand-off of sharded outputs between the GPUs of one machine, one process per GPU.
//
// The grouped mat-vec kernels store every output value straight into each GPU's gather buffer
// (plain stores to peer-mapped memory over NVLink).  What is left of the all-gather is the
// hand-shake: after its stores a GPU raises its flag on every peer, then waits until every
// peer's flag has reached the same step.  One small kernel per step does both; nothing is copied
// and no collective library is involved.
//
// Buffers are exchanged between the processes as CUDA IPC handles (tb200_ipc_export / _open).
#include <cstring>

#define TB200_OP_CLASS TB200_PREPARE_PEER
#include "common.cuh"

TB200_TU_STATUS(peer)

namespace tb200 {

constexpr int kPeerMax = 8;

struct PeerFlagArgs {
    unsigned *flags[kPeerMax];  // flags[p]: the flag array of GPU p (own one local, the others peer-mapped), kPeerMax words
    unsigned *epoch;            // local step counter, advanced by this kernel
    unsigned long long timeout_ns;
    int rank, npeers;
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(32) peer_signal_wait_kernel(const __grid_constant__ PeerFlagArgs a) {
    const int p = threadIdx.x;
    const unsigned e = *a.epoch + 1;  // every GPU runs the same sequence of steps, so the counters agree
    __syncwarp();
    if (p < a.npeers) {
        // Kernels enqueued before this one have completed; the fence orders their stores to peer memory,
        // as observed from this GPU, before the flag.
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flags[p] + a.rank), "r"(e) : "memory");
        // wait for GPU p's flag in this GPU's own array; the wait is bounded in time
        const unsigned *mine = a.flags[a.rank] + p;
        const unsigned long long t0 = global_timer_ns();
        for (unsigned spin = 0;; ++spin) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int)(v - e) >= 0) break;
            if ((spin & 63) == 63 && global_timer_ns() - t0 > a.timeout_ns) {
                g_device_status = TB200_ERR_TIMEOUT;
                break;
            }
        }
    }
    __syncwarp();
    if (p == 0) *a.epoch = e;
}

// Completion of the steps whose kernels carry the hand-shake themselves: announce this GPU's count of
// finished steps to every GPU, then wait until every GPU has announced at least as many.
__global__ void __launch_bounds__(32) peer_wait_kernel(const __grid_constant__ PeerFlagArgs a) {
    const unsigned e = *reinterpret_cast<const volatile unsigned *>(a.epoch);
    const int p = threadIdx.x;
    if (p < a.npeers) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flags[p] + a.rank), "r"(e) : "memory");
        if (p != a.rank) wait_flag_at_least(a.flags[a.rank] + p, e, a.timeout_ns);
    }
}

}  // namespace tb200

extern "C" int tb200_peer_wait(int rank, int npeers, unsigned *const *flags, const unsigned *sync, unsigned timeout_ms,
                               tb200_stream_t stream) {
    using namespace tb200;
    if (npeers < 1 || npeers > kPeerMax || rank < 0 || rank >= npeers || !flags || !sync) return TB200_ERR_INVALID_ARG;
    PeerFlagArgs a{};
    for (int p = 0; p < npeers; ++p) {
        if (!flags[p]) return TB200_ERR_INVALID_ARG;
        if (!aligned_to(flags[p], 4)) return TB200_ERR_ALIGNMENT;
        a.flags[p] = flags[p];
    }
    if (!aligned_to(sync, 4)) return TB200_ERR_ALIGNMENT;
    a.epoch = const_cast<unsigned *>(sync), a.rank = rank, a.npeers = npeers;
    a.timeout_ns = (unsigned long long)(timeout_ms ? timeout_ms : 2000u) * 1000000ull;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    st = ensure_kernel<peer_wait_kernel, 0>(di);
    if (st) return st;
    // a plain launch: it starts only after everything enqueued before it has completed
    return launch_kernel(peer_wait_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, false, a);
}

extern "C" int tb200_peer_signal_wait(int rank, int npeers, unsigned *const *flags, unsigned *epoch, unsigned timeout_ms,
                                      tb200_stream_t stream) {
    using namespace tb200;
    if (npeers < 1 || npeers > kPeerMax || rank < 0 || rank >= npeers || !flags || !epoch) return TB200_ERR_INVALID_ARG;
    PeerFlagArgs a{};
    for (int p = 0; p < npeers; ++p) {
        if (!flags[p]) return TB200_ERR_INVALID_ARG;
        if (!aligned_to(flags[p], 4)) return TB200_ERR_ALIGNMENT;
        a.flags[p] = flags[p];
    }
    if (!aligned_to(epoch, 4)) return TB200_ERR_ALIGNMENT;
    a.epoch = epoch, a.rank = rank, a.npeers = npeers;
    a.timeout_ns = (unsigned long long)(timeout_ms ? timeout_ms : 2000u) * 1000000ull;
    int st;
    const DeviceInfo *di = device_info(&st);
    if (!di) return st;
    st = ensure_kernel<peer_signal_wait_kernel, 0>(di);
    if (st) return st;
    // a plain launch: it starts only after everything enqueued before it has completed
    return launch_kernel(peer_signal_wait_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, false, a);
}

extern "C" int tb200_ipc_export(const void *device_allocation, void *handle64) {
    if (!device_allocation || !handle64) return TB200_ERR_INVALID_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void *>(device_allocation));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return (int)e;
    }
    std::memcpy(handle64, &h, 64);
    return TB200_OK;
}

extern "C" int tb200_ipc_open(const void *handle64, void **peer_ptr) {
    if (!handle64 || !peer_ptr) return TB200_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, 64);
    cudaError_t e = cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return (int)e;
    }
    return TB200_OK;
}

extern "C" int tb200_ipc_close(void *peer_ptr) {
    if (!peer_ptr) return TB200_OK;
    cudaError_t e = cudaIpcCloseMemHandle(peer_ptr);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return (int)e;
    }
    return TB200_OK;
}
