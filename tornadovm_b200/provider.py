"""``B200LibraryProvider`` -- Python twin of the Java provider of the same name.

Implements the reference's provider SPI method for method
(tornado-runtime/.../library/spi/TornadoLibraryProvider.java:42-85) with the
structure of CutlassLibraryProvider (tornado-cutlass/.../provider/
CutlassLibraryProvider.java:40-169): a per-(device, plan) context that holds
the plan's stream and a grow-only device workspace, ``prepare`` that sizes the
workspace before any launch (and before stream capture), and ``dispatch`` that
marshals positional arguments into one native call and checks its status.
"""
from __future__ import annotations

import ctypes as C
import os
import sys

from .b200 import LIBRARY_NAME, B200Options
from .native import B200Native


class LibraryInvocation:
    """spi/LibraryInvocation.java:54-97."""

    def __init__(self, args, device_pointers, context, tuning=None, device=None, plan_id=0, host_pointers=None):
        self._args, self._ptrs, self._ctx = list(args), list(device_pointers), context
        self._tuning, self._device, self._plan = tuning, device, plan_id
        # An extension of the reference's invocation object: for an argument that the graph copies to the host after
        # every execution, the address of the payload in the array's own host segment, when that segment is pinned
        # and mapped into the device's address space (None otherwise).
        self._host_ptrs = list(host_pointers) if host_pointers is not None else [None] * len(self._args)
        self._host_delivered = set()

    def getHostPointer(self, i):  # noqa: N802
        return self._host_ptrs[i]

    def markHostDelivered(self, i) -> None:  # noqa: N802
        """The dispatch stored argument i's results into the host segment itself: no copy back is needed."""
        self._host_delivered.add(i)

    def hostDelivered(self):  # noqa: N802
        return frozenset(self._host_delivered)

    def getArg(self, i):  # noqa: N802
        return self._args[i]

    def getDevicePointer(self, i):  # noqa: N802
        p = self._ptrs[i]
        if p is None:
            raise RuntimeError(f"[ERROR] argument {i} is not a device reference")
        return p

    def isReference(self, i):  # noqa: N802
        return self._ptrs[i] is not None

    def getContext(self):  # noqa: N802
        return self._ctx

    def getTuning(self):  # noqa: N802
        return self._tuning

    def getDevice(self):  # noqa: N802
        return self._device

    def getExecutionPlanId(self):  # noqa: N802
        return self._plan


class B200Context:
    """LibraryContext: stream of the plan + grow-only workspace."""

    def __init__(self, stream: int):
        self.stream = stream
        self.workspace_ptr = 0
        self.workspace_bytes = 0

    def grow_workspace(self, required: int) -> None:
        if required > self.workspace_bytes:
            if self.workspace_ptr:
                B200Native.call("tb200_device_free", C.c_void_p(self.workspace_ptr))
                self.workspace_ptr, self.workspace_bytes = 0, 0
            out = C.c_void_p()
            B200Native.call("tb200_device_malloc", required, C.byref(out))
            if not out.value:
                raise RuntimeError(f"[ERROR] Unable to allocate B200 workspace of {required} bytes")
            self.workspace_ptr, self.workspace_bytes = out.value, required


TB200_ERR_INVALID_ARG = -1  # include/tornado_b200.h

#: TB200_LOG=1 prints one line per dispatch to stderr (function, scalar arguments, tuning)
_LOG = os.environ.get("TB200_LOG", "") not in ("", "0")

_QUANT_FUNCTIONS = {"q8Gemv", "q8GemvBytes", "q4GemvBytes"}
_GROUPED_FUNCTIONS = {"q8GemvBytesGrouped": "tb200_q8b_gemv_i8_grouped", "q4GemvBytesGrouped": "tb200_q4b_gemv_i8_grouped"}
_BIAS_ACTIVATIONS = {"gemmBiasRelu": 1, "gemmBiasGelu": 2, "gemmBiasSilu": 3, "gemmBiasSigmoid": 4, "gemmBiasTanh": 5, "gemmBiasHardSwish": 6}
_PACKED_FUNCTIONS = {"q8GemvBytesPacked": ("tb200_q8b_gemv_i8_grouped", 34), "q4GemvBytesPacked": ("tb200_q4b_gemv_i8_grouped", 18)}


class B200LibraryProvider:
    def libraryName(self) -> str:  # noqa: N802
        return LIBRARY_NAME

    def canHandle(self, device) -> bool:  # noqa: N802
        # only devices that expose their native stream (TornadoNativeStreamSupport)
        return hasattr(device, "getNativeStream")

    def createContext(self, device, executionPlanId: int) -> B200Context:  # noqa: N802
        B200Native.load()
        return B200Context(device.getNativeStream(executionPlanId))

    # operation classes of tb200_prepare (include/tornado_b200.h)
    _PREPARE_CLASS = {"sgemv": 1, "q8Gemv": 2, "q8GemvBytes": 2, "q4GemvBytes": 2, "q8GemvBytesGrouped": 2,
                      "q4GemvBytesGrouped": 2, "q8GemvBytesPacked": 2, "q4GemvBytesPacked": 2, "sgemm": 4, "hgemmF32": 8, "hgemm": 8, "bgemm": 8, "hgemmBatched": 8,
                      "gemmBiasRelu": 8, "gemmBiasGelu": 8, "gemmBiasSilu": 8, "gemmBiasSigmoid": 8, "gemmBiasTanh": 8,
                      "gemmBiasHardSwish": 8}

    def prepare(self, descriptor, context: B200Context) -> None:
        """Runs in the pre-launch pass, before any capture (TornadoVMInterpreter.java:1036-1055) and possibly
        several times: loads and configures every kernel the task may launch in the plan's CUDA context, so that
        dispatch issues nothing but kernel launches, and sizes the workspace.  Tuning is NOT applied here: it is
        set around each dispatch and reset after it (cf. CuBlasLibraryProvider.java:124-151)."""
        fn = descriptor.getFunctionName()
        tuning = descriptor.getTuning()
        B200Native.call("tb200_prepare", self._PREPARE_CLASS.get(fn, 0))
        if fn in _QUANT_FUNCTIONS and isinstance(tuning, B200Options) and tuning.exact_int:
            p = descriptor.getParameters()
            need = B200Native.load().tb200_qx_workspace_bytes(int(p[1]), int(p[2]))
            context.grow_workspace(int(need))
        if fn in _PACKED_FUNCTIONS:  # (count, rows, cols, batch, blocks, x, y)
            p = descriptor.getParameters()
            context.grow_workspace(int(B200Native.load().tb200_qx_workspace_bytes(int(p[2]), int(p[3]))))
        if fn in _GROUPED_FUNCTIONS:  # (count, rows, cols, batch, x, y, blocks...); integer mode whatever the tuning says
            p = descriptor.getParameters()
            context.grow_workspace(int(B200Native.load().tb200_qx_workspace_bytes(int(p[2]), int(p[3]))))

    def dispatch(self, functionName: str, inv: LibraryInvocation) -> None:  # noqa: N802
        ctx: B200Context = inv.getContext()
        lib = B200Native.load()
        tuning = inv.getTuning()
        exact = isinstance(tuning, B200Options) and tuning.exact_int
        # the task's tuning holds for this call on this thread only
        scoped = isinstance(tuning, B200Options) and tuning.overlap_launches
        if scoped:
            B200Native.call("tb200_set_thread_option", 1, 1)  # TB200_OPT_OVERLAP_LAUNCHES
        if _LOG:
            shape = [inv.getArg(i) for i in range(len(inv._args)) if not inv.isReference(i)]
            sys.stderr.write(f"[tb200] plan {inv.getExecutionPlanId()} dispatch {functionName}{tuple(shape)} exact_int={exact} overlap={scoped}\n")
        try:
            st = self._dispatch(lib, functionName, inv, ctx, exact)
        finally:
            if scoped:
                lib.tb200_clear_thread_options()
        B200Native.check_status(st, functionName)

    @staticmethod
    def _dispatch(lib, functionName, inv, ctx, exact) -> int:  # noqa: N803
        P = inv.getDevicePointer
        A = inv.getArg
        ws = (ctx.workspace_ptr, ctx.workspace_bytes)
        if functionName == "sgemv":  # (rows, cols, m, v, out)
            st = lib.tb200_sgemv(A(0), A(1), P(2), P(3), P(4), ctx.stream)
        elif functionName == "q8Gemv":  # (rows, cols, batch, q, scales, x, y)
            if exact:
                st = lib.tb200_q8_gemv_i8(A(0), A(1), A(2), P(3), P(4), P(5), P(6), *ws, ctx.stream)
            else:
                st = lib.tb200_q8_gemv(A(0), A(1), A(2), P(3), P(4), P(5), P(6), ctx.stream)
        elif functionName == "q8GemvBytes":  # (rows, cols, batch, blocks, x, y)
            if exact:
                st = lib.tb200_q8b_gemv_i8(A(0), A(1), A(2), P(3), P(4), P(5), *ws, ctx.stream)
            else:
                st = lib.tb200_q8b_gemv(A(0), A(1), A(2), P(3), P(4), P(5), ctx.stream)
        elif functionName == "q4GemvBytes":
            if exact:
                st = lib.tb200_q4b_gemv_i8(A(0), A(1), A(2), P(3), P(4), P(5), *ws, ctx.stream)
            else:
                st = lib.tb200_q4b_gemv(A(0), A(1), A(2), P(3), P(4), P(5), ctx.stream)
        elif functionName in _GROUPED_FUNCTIONS:  # (count, rows, cols, batch, x, y, blocks...)
            count = A(0)
            blocks = (C.c_void_p * count)(*[P(6 + m) for m in range(count)])
            st = B200LibraryProvider._grouped(lib, _GROUPED_FUNCTIONS[functionName], inv, ctx, blocks, x_index=4, y_index=5)
        elif functionName in _PACKED_FUNCTIONS:  # (count, rows, cols, batch, blocks, x, y)
            native, block_bytes = _PACKED_FUNCTIONS[functionName]
            count, per = A(0), A(1) * (A(2) // 32) * block_bytes
            blocks = (C.c_void_p * count)(*[P(4) + m * per for m in range(count)])
            st = B200LibraryProvider._grouped(lib, native, inv, ctx, blocks, x_index=5, y_index=6)
        elif functionName == "sgemm":  # (m, n, k, alpha, a, b, beta, c)
            st = lib.tb200_sgemm(A(0), A(1), A(2), A(3), P(4), P(5), A(6), P(7), ctx.stream)
        elif functionName == "hgemmF32":  # (m, n, k, a, b, c)
            st = lib.tb200_hgemm_f32(A(0), A(1), A(2), P(3), P(4), P(5), ctx.stream)
        elif functionName in ("hgemm", "bgemm"):  # (m, n, k, alpha, a, b, beta, d): 16-bit in and out, D in place
            t = 0 if functionName == "hgemm" else 1
            st = lib.tb200_gemm_ex(A(0), A(1), A(2), t, P(4), P(5), 1 + t, P(7), A(3), A(6), None, None, 0, 1, ctx.stream)
        elif functionName == "hgemmBatched":  # (m, n, k, alpha, a, b, beta, d, batchCount)
            st = lib.tb200_gemm_ex(A(0), A(1), A(2), 0, P(4), P(5), 1, P(7), A(3), A(6), None, None, 0, A(8), ctx.stream)
        elif functionName in _BIAS_ACTIVATIONS:  # (m, n, k, a, b, bias, d): fp16 in and out
            st = lib.tb200_gemm_ex(A(0), A(1), A(2), 0, P(3), P(4), 1, P(6), 1.0, 0.0, None, P(5), _BIAS_ACTIVATIONS[functionName], 1,
                                   ctx.stream)
        else:
            raise RuntimeError(f"[ERROR] B200 function not supported: {functionName}")
        return st

    @staticmethod
    def _grouped(lib, native, inv, ctx, blocks, x_index, y_index) -> int:
        """One grouped launch of len(blocks) matrices; arguments 0..3 of the task are count, rows, cols, batch."""
        P, A = inv.getDevicePointer, inv.getArg
        fn, ws = getattr(lib, native), (ctx.workspace_ptr, ctx.workspace_bytes)
        tuning = inv.getTuning()
        host = inv.getHostPointer(y_index) if isinstance(tuning, B200Options) and tuning.host_results and A(3) == 1 else None
        if host:
            # two destinations: the device buffer and the array's host segment (plain stores over PCIe while the
            # launch runs).  One vector only: there the same kernel runs whatever the number of destinations, so
            # the option never changes a result bit.  Shapes that only the one-destination kernels cover are
            # refused before anything is launched and take the call below.
            dst = (C.c_void_p * 2)(P(y_index), host)
            st = fn(A(0), A(1), A(2), A(3), blocks, P(x_index), dst, 2, 0, None, A(1), 0, *ws, ctx.stream)
            if st == 0:
                inv.markHostDelivered(y_index)
            if st != TB200_ERR_INVALID_ARG:
                return st
        dst = (C.c_void_p * 1)(P(y_index))
        return fn(A(0), A(1), A(2), A(3), blocks, P(x_index), dst, 1, 0, None, A(1), 0, *ws, ctx.stream)

    def destroyContext(self, context: B200Context) -> None:  # noqa: N802
        if context.workspace_ptr:
            B200Native.call("tb200_device_free", C.c_void_p(context.workspace_ptr))
            context.workspace_ptr, context.workspace_bytes = 0, 0
