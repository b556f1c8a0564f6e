"""ctypes binding of libtornado_b200.so -- the Python twin of the Java class
``B200Native`` (java.lang.foreign downcalls), which in turn plays the role of
``CutlassNativeLib`` / ``CuBlasNativeLib`` in the reference
(tornado-cublas/.../provider/CuBlasNativeLib.java:35-100).

There is no fallback: if the shared library is missing or a symbol declared in
include/tornado_b200.h is absent, loading fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

from .build import LIB_PATH

_I, _P, _F, _Z = C.c_int, C.c_void_p, C.c_float, C.c_size_t

# name -> (restype, argtypes); mirrors include/tornado_b200.h one to one
SIGNATURES = {
    "tb200_status_string": (C.c_char_p, [_I]),
    "tb200_version": (_I, []),
    "tb200_device_status": (_I, [C.POINTER(_I)]),
    "tb200_device_status_of": (_I, [_I, C.POINTER(_I)]),
    "tb200_prepare": (_I, [_I]),
    "tb200_set_option": (_I, [_I, _I]),
    "tb200_get_option": (_I, [_I, C.POINTER(_I)]),
    "tb200_set_thread_option": (_I, [_I, _I]),
    "tb200_clear_thread_options": (_I, []),
    "tb200_device_malloc": (_I, [_Z, C.POINTER(_P)]),
    "tb200_device_free": (_I, [_P]),
    "tb200_sgemv": (_I, [_I, _I, _P, _P, _P, _P]),
    "tb200_q8_gemv": (_I, [_I, _I, _I, _P, _P, _P, _P, _P]),
    "tb200_q8b_gemv": (_I, [_I, _I, _I, _P, _P, _P, _P]),
    "tb200_q4b_gemv": (_I, [_I, _I, _I, _P, _P, _P, _P]),
    "tb200_qx_workspace_bytes": (_Z, [_I, _I]),
    "tb200_quantize_x": (_I, [_I, _I, _P, _P, _Z, _P]),
    "tb200_q8_gemv_i8": (_I, [_I, _I, _I, _P, _P, _P, _P, _P, _Z, _P]),
    "tb200_q8_gemv_i8_static": (_I, [_I, _I, _I, _P, _P, _P, _P, _P]),
    "tb200_static_scratch_address": (_I, [C.POINTER(_P), C.POINTER(_P)]),
    "tb200_q8b_gemv_i8": (_I, [_I, _I, _I, _P, _P, _P, _P, _Z, _P]),
    "tb200_q4b_gemv_i8": (_I, [_I, _I, _I, _P, _P, _P, _P, _Z, _P]),
    "tb200_q8b_gemv_i8_grouped": (_I, [_I, _I, _I, _I, _P, _P, _P, _I, C.c_longlong, _P, _I, _I, _P, _Z, _P]),
    "tb200_q4b_gemv_i8_grouped": (_I, [_I, _I, _I, _I, _P, _P, _P, _I, C.c_longlong, _P, _I, _I, _P, _Z, _P]),
    "tb200_q8b_gemv_i8_grouped_rows": (_I, [_I, _P, _I, _I, _P, _P, _P, _P, _Z, _P]),
    "tb200_q4b_gemv_i8_grouped_rows": (_I, [_I, _P, _I, _I, _P, _P, _P, _P, _Z, _P]),
    "tb200_q8b_gemv_i8_grouped_sync": (_I, [_I, _I, _I, _I, _P, _P, _P, _I, _I, _I, C.c_longlong, _P, _P, _I, C.c_uint, _I, _I, _P, _Z, _P]),
    "tb200_q4b_gemv_i8_grouped_sync": (_I, [_I, _I, _I, _I, _P, _P, _P, _I, _I, _I, C.c_longlong, _P, _P, _I, C.c_uint, _I, _I, _P, _Z, _P]),
    "tb200_peer_wait": (_I, [_I, _I, _P, _P, C.c_uint, _P]),
    "tb200_peer_signal_wait": (_I, [_I, _I, _P, _P, C.c_uint, _P]),
    "tb200_ipc_export": (_I, [_P, _P]),
    "tb200_ipc_open": (_I, [_P, C.POINTER(_P)]),
    "tb200_ipc_close": (_I, [_P]),
    "tb200_q8_blockdots_i32": (_I, [_I, _I, _P, _P, _P, _P]),
    "tb200_q8b_blockdots_i32": (_I, [_I, _I, _P, _P, _P, _P]),
    "tb200_q4b_blockdots_i32": (_I, [_I, _I, _P, _P, _P, _P]),
    "tb200_blockdots_i32_batched": (_I, [_I, _I, _I, _I, _P, _P, _P, _P]),
    "tb200_sgemm": (_I, [_I, _I, _I, _F, _P, _P, _F, _P, _P]),
    "tb200_hgemm_f32": (_I, [_I, _I, _I, _P, _P, _P, _P]),
    "tb200_gemm_ex": (_I, [_I, _I, _I, _I, _P, _P, _I, _P, _F, _F, _P, _P, _I, _I, _P]),
    "tb200_igemm_workspace_bytes": (_Z, [_I, _I]),
    "tb200_igemm_s32": (_I, [_I, _I, _I, _P, _P, _P, _P, _Z, _P]),
    "tb200_fp8gemm_f32": (_I, [_I, _I, _I, _I, _P, _P, _P, _P, _Z, _P]),
    "tb200_hgemm_f32_scatter": (_I, [_I, _I, _I, _P, _P, _P, _I, C.c_longlong, C.c_longlong, _P]),
}


class TornadoB200Error(RuntimeError):
    """Python stand-in for TornadoRuntimeException raised by checkStatus
    (CuBlasNativeLib.java:96-100): ``[ERROR] <fn> failed with status: <NAME>``."""

    def __init__(self, function: str, status: int, name: str):
        super().__init__(f"[ERROR] {function} failed with status: {name}")
        self.function, self.status, self.status_name = function, status, name


class B200Native:
    _lib = None

    @classmethod
    def load(cls) -> C.CDLL:
        if cls._lib is None:
            if not os.path.exists(LIB_PATH):
                raise OSError(
                    f"[ERROR] Unable to load libtornado_b200.so (expected at {LIB_PATH}); "
                    "build it with `python -m tornadovm_b200.build`")
            lib = C.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)  # AttributeError if the symbol is missing
                fn.restype, fn.argtypes = res, args
            cls._lib = lib
        return cls._lib

    @classmethod
    def status_string(cls, status: int) -> str:
        return cls.load().tb200_status_string(status).decode()

    @classmethod
    def check_status(cls, status: int, function: str) -> None:
        if status != 0:
            raise TornadoB200Error(function, status, cls.status_string(status))

    @classmethod
    def call(cls, function: str, *args) -> None:
        """Invoke an int-status entry point and raise on a non-zero status."""
        cls.check_status(getattr(cls.load(), function)(*args), function)

    @classmethod
    def device_status(cls, op_classes: int = 0) -> int:
        """Read-and-clear the device status of the kernels of ``op_classes`` (tb200_prepare_class bits; 0 = all)."""
        v = C.c_int(0)
        cls.check_status(cls.load().tb200_device_status_of(op_classes, C.byref(v)), "tb200_device_status_of")
        return v.value


def graph_replayer(cuda_graph, torch_stream, synchronize=True):
    """A callable that replays an instantiated ``torch.cuda.CUDAGraph`` on ``torch_stream`` with one
    cudaGraphLaunch (and, with ``synchronize``, one cudaStreamSynchronize) through the CUDA runtime the process has
    already loaded -- the two calls a JVM host makes per execution -- or None when the runtime library or the
    graph's handle cannot be reached (callers then replay through torch, which also selects the device and the
    stream around the launch)."""
    try:
        rt = C.CDLL("libcudart.so.12")
        launch, sync = rt.cudaGraphLaunch, rt.cudaStreamSynchronize
        launch.argtypes, launch.restype = [C.c_void_p, C.c_void_p], C.c_int
        sync.argtypes, sync.restype = [C.c_void_p], C.c_int
        exec_handle = C.c_void_p(cuda_graph.raw_cuda_graph_exec())
    except (OSError, AttributeError, RuntimeError):
        return None
    stream = C.c_void_p(torch_stream.cuda_stream)

    def replay():
        st = launch(exec_handle, stream) or (sync(stream) if synchronize else 0)
        if st:
            raise RuntimeError(f"[ERROR] replay of a captured execution failed with CUDA status {st}")
    return replay

