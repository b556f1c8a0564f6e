"""The C ABI under the reference's context model.

Both NVIDIA backends of TornadoVM run in a context of their own, created with cuCtxCreate (not the
device's primary context) and made current at the top of every native call
(tornado-drivers/cuda-jni/.../CUDAPlatform.cpp:118-146, ptx-jni/.../PTXContext.cpp:37-51); all of a
plan's buffers are cuMemAlloc'ed there.  A process can hold several such contexts on one GPU.  These
tests drive the library from two driver-API contexts on the same device, with buffers and streams
created through the driver API, and check the results against the CPU oracle.
"""
import ctypes as C

import numpy as np
import pytest

import oracle as o

pytestmark = pytest.mark.gpu

CU_CTX_SCHED_YIELD = 0x02
CU_STREAM_NON_BLOCKING = 0x1


class Driver:
    def __init__(self):
        self.cu = C.CDLL("libcuda.so.1")
        for name, args in {
            "cuInit": [C.c_uint], "cuDeviceGet": [C.POINTER(C.c_int), C.c_int],
            "cuCtxCreate_v2": [C.POINTER(C.c_void_p), C.c_uint, C.c_int], "cuCtxDestroy_v2": [C.c_void_p],
            "cuCtxSetCurrent": [C.c_void_p], "cuCtxGetCurrent": [C.POINTER(C.c_void_p)],
            "cuMemAlloc_v2": [C.POINTER(C.c_uint64), C.c_size_t], "cuMemFree_v2": [C.c_uint64],
            "cuMemcpyHtoD_v2": [C.c_uint64, C.c_void_p, C.c_size_t], "cuMemcpyDtoH_v2": [C.c_void_p, C.c_uint64, C.c_size_t],
            "cuMemsetD8_v2": [C.c_uint64, C.c_ubyte, C.c_size_t],
            "cuStreamCreate": [C.POINTER(C.c_void_p), C.c_uint], "cuStreamSynchronize": [C.c_void_p], "cuStreamDestroy_v2": [C.c_void_p],
        }.items():
            fn = getattr(self.cu, name)
            fn.restype, fn.argtypes = C.c_int, args

    def ok(self, rc, what):
        assert rc == 0, f"{what} failed with CUresult {rc}"


class Buf:
    """cuMemAlloc(header + payload); tasks receive base + header (TornadoVMInterpreter.java:1260-1266)."""

    def __init__(self, drv, host: np.ndarray, header: int):
        host = np.ascontiguousarray(host)
        self.drv, self.host, self.header = drv, host, header
        self.base = C.c_uint64()
        drv.ok(drv.cu.cuMemAlloc_v2(C.byref(self.base), header + host.nbytes), "cuMemAlloc")
        drv.ok(drv.cu.cuMemsetD8_v2(self.base.value, 0xA5, header + host.nbytes), "cuMemsetD8")
        drv.ok(drv.cu.cuMemcpyHtoD_v2(self.base.value + header, host.ctypes.data_as(C.c_void_p), host.nbytes), "cuMemcpyHtoD")

    @property
    def ptr(self):
        return C.c_void_p(self.base.value + self.header)

    def read(self):
        out = np.empty_like(self.host)
        self.drv.ok(self.drv.cu.cuMemcpyDtoH_v2(out.ctypes.data_as(C.c_void_p), self.base.value + self.header, out.nbytes), "cuMemcpyDtoH")
        return out

    def free(self):
        self.drv.cu.cuMemFree_v2(self.base.value)


def _run_in_context(lib, drv, header, seed):
    """One pass over the operations of the path inside the context that is current."""
    stream = C.c_void_p()
    drv.ok(drv.cu.cuStreamCreate(C.byref(stream), CU_STREAM_NON_BLOCKING), "cuStreamCreate")
    bufs = []

    def B(a):
        b = Buf(drv, a, header)
        bufs.append(b)
        return b

    def status_ok(st):
        assert st == 0, lib.tb200_status_string(st).decode()

    try:
        status_ok(lib.tb200_prepare(0))
        # FP32 mat-vec
        rows, cols = 300, 2048
        m, v = o.make_sgemv(rows, cols, seed)
        dm, dv, dout = B(m), B(v), B(np.full(rows, np.nan, np.float32))
        status_ok(lib.tb200_sgemv(rows, cols, dm.ptr, dv.ptr, dout.ptr, stream))
        # Q8_0 integer mode, block layout, batch 1 (dp4a kernel) and 8 (tensor-core kernel)
        qr, qc = 257, 4096
        q, s, x = o.make_q8(qr, qc, 8, seed)
        dblk, dx = B(o.q8_pack_blocks(q, s)), B(x)
        nws = lib.tb200_qx_workspace_bytes(qc, 8)
        dws = B(np.zeros(nws + 16, np.uint8))
        ws_ptr = C.c_void_p((dws.ptr.value + 15) & ~15)
        dy1, dy8 = B(np.full(qr, np.nan, np.float32)), B(np.full(8 * qr, np.nan, np.float32))
        status_ok(lib.tb200_q8b_gemv_i8(qr, qc, 1, dblk.ptr, dx.ptr, dy1.ptr, ws_ptr, nws, stream))
        status_ok(lib.tb200_q8b_gemv_i8(qr, qc, 8, dblk.ptr, dx.ptr, dy8.ptr, ws_ptr, nws, stream))
        # FP16 GEMM on the tensor cores and FP32 SGEMM
        n = 256
        ha, hb = o.make_hgemm(n, n, n, seed)
        dha, dhb, dhc = B(ha), B(hb), B(np.full(n * n, np.nan, np.float32))
        status_ok(lib.tb200_hgemm_f32(n, n, n, dha.ptr, dhb.ptr, dhc.ptr, stream))
        fa, fb = o.JavaRandom(seed).uniform_f32(n * n, 0, 1), o.JavaRandom(seed + 1).uniform_f32(n * n, 0, 1)
        dfa, dfb, dfc = B(fa), B(fb), B(np.full(n * n, np.nan, np.float32))
        status_ok(lib.tb200_sgemm(n, n, n, C.c_float(1.0), dfa.ptr, dfb.ptr, C.c_float(0.0), dfc.ptr, stream))
        # the allocation-free entry: the address it will use must be this context's own copy of the array,
        # checked on the host BEFORE anything is launched with it
        in_use, fresh = C.c_void_p(), C.c_void_p()
        status_ok(lib.tb200_static_scratch_address(C.byref(in_use), C.byref(fresh)))
        assert in_use.value == fresh.value and in_use.value, "scratch address cached for another context"
        dq, dsc = B(q), B(s)
        dys = B(np.full(qr, np.nan, np.float32))
        status_ok(lib.tb200_q8_gemv_i8_static(qr, qc, 1, dq.ptr, dsc.ptr, dx.ptr, dys.ptr, stream))
        drv.ok(drv.cu.cuStreamSynchronize(stream), "cuStreamSynchronize")
        st = C.c_int(-1)
        status_ok(lib.tb200_device_status(C.byref(st)))
        assert st.value == 0

        assert o.rel_l2(dout.read(), o.sgemv_f64(m, v, cols, rows)) <= 1e-5
        want = []
        for b in range(8):
            xq, xs = o.quantize_x_block(np.ascontiguousarray(x[b * qc:(b + 1) * qc]))
            want.append(o.blockdots_combine_f64(o.q8_blockdots_i32(q, xq, qc, qr), s, xs, qc // 32, qr))
        assert o.rel_l2(dy1.read(), want[0]) <= 1e-5
        assert o.rel_l2(dy8.read().reshape(8, qr), np.stack(want)) <= 1e-5
        assert o.rel_l2(dys.read(), want[0]) <= 1e-5
        assert o.rel_l2(dhc.read(), o.hgemm_ref(ha, hb, n, n, n)) <= 2e-3
        assert o.rel_l2(dfc.read(), o.sgemm_f64(fa, fb, n, n, n)) <= 1e-5
        return in_use.value
    finally:
        for b in bufs:
            b.free()
        drv.cu.cuStreamDestroy_v2(stream)


@pytest.mark.parametrize("header", [16, 24])
def test_two_driver_contexts_on_one_gpu(lib, header):
    import torch
    torch.cuda.init()
    torch.zeros(1, device="cuda")  # the primary context exists and is current, as in the other tests
    drv = Driver()
    drv.ok(drv.cu.cuInit(0), "cuInit")
    primary = C.c_void_p()
    drv.ok(drv.cu.cuCtxGetCurrent(C.byref(primary)), "cuCtxGetCurrent")
    dev = C.c_int()
    drv.ok(drv.cu.cuDeviceGet(C.byref(dev), 0), "cuDeviceGet")
    created, addresses = [], []
    try:
        for i in range(2):
            ctx = C.c_void_p()
            drv.ok(drv.cu.cuCtxCreate_v2(C.byref(ctx), CU_CTX_SCHED_YIELD, dev.value), "cuCtxCreate")
            created.append(ctx)
        # alternate between the contexts the way two backends of one JVM would
        for rnd in range(2):
            for i, ctx in enumerate(created):
                drv.ok(drv.cu.cuCtxSetCurrent(ctx), "cuCtxSetCurrent")
                addresses.append(_run_in_context(lib, drv, header, 40 + i))
        assert addresses[0] == addresses[2] and addresses[1] == addresses[3]
    finally:
        drv.cu.cuCtxSetCurrent(primary)
        for ctx in created:
            drv.cu.cuCtxDestroy_v2(ctx)
    # and the primary context still works afterwards
    m, v = o.make_sgemv(64, 256)
    tm, tv = torch.from_numpy(m).cuda(), torch.from_numpy(v).cuda()
    out = torch.empty(64, device="cuda")
    st = lib.tb200_sgemv(64, 256, C.c_void_p(tm.data_ptr()), C.c_void_p(tv.data_ptr()), C.c_void_p(out.data_ptr()),
                         C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0
    torch.cuda.synchronize()
    assert o.rel_l2(out.cpu().numpy(), o.sgemv_f64(m, v, 256, 64)) <= 1e-5
