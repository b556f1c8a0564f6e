"""A small stand-in for the part of TornadoVM that surrounds a library task.

No JVM exists where this package is built and tested, so this module plays the
role of ``TaskGraph`` / ``TornadoExecutionPlan`` and of the interpreter's
``executeLibraryLaunch`` (tornado-runtime/.../interpreter/
TornadoVMInterpreter.java:1245-1328) for graphs made of library tasks:

* device buffers are ``header + payload`` bytes and tasks receive
  ``base + header`` (:1260-1266);
* one non-blocking stream per plan (cuda-jni/.../CUDAContext.cpp:83);
* ``prepare`` for every task before the first launch and before capture
  (:1036-1055); ``withCUDAGraph()`` captures the launches of one execution and
  replays them (HYBRID_API_GUIDE.md:317-334);
* contexts are destroyed when the plan closes (TornadoTaskGraph.java:1277).

Device memory, streams and copies are PyTorch's; nothing here computes.
"""
from __future__ import annotations

import ctypes as C
import enum
import itertools

import torch

from .arrays import TornadoNativeArray
from .descriptor import Access
from .native import graph_replayer
from .provider import B200LibraryProvider, LibraryInvocation


class DataTransferMode(enum.Enum):
    FIRST_EXECUTION = 1
    EVERY_EXECUTION = 2


class CudaDevice:
    """What a provider sees of a device: TornadoNativeStreamSupport
    (spi/TornadoNativeStreamSupport.java:34-63)."""

    def __init__(self, index: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("[ERROR] no CUDA device: the b200/linalg tasks have no CPU path")
        self.index = index
        self.torch_device = torch.device("cuda", index)
        self._streams = {}

    def torch_stream(self, plan_id: int) -> torch.cuda.Stream:
        if plan_id not in self._streams:
            with torch.cuda.device(self.index):
                self._streams[plan_id] = torch.cuda.Stream(device=self.torch_device)
        return self._streams[plan_id]

    def getNativeStream(self, plan_id: int) -> int:  # noqa: N802
        return self.torch_stream(plan_id).cuda_stream

    def getNativeContext(self, plan_id: int) -> int:  # noqa: N802
        return 0  # primary context, current once torch has selected the device

    def nvtxRangePush(self, name: str) -> None:  # noqa: N802
        """Host-side NVTX range around a library task (TornadoNativeStreamSupport.nvtxRangePush,
        spi/TornadoNativeStreamSupport.java:48-63); a no-op unless a profiler is attached."""
        torch.cuda.nvtx.range_push(name)

    def nvtxRangePop(self) -> None:  # noqa: N802
        torch.cuda.nvtx.range_pop()


class _LibraryTask:
    def __init__(self, task_id, descriptor):
        self.id, self.descriptor = task_id, descriptor


class TaskGraph:
    def __init__(self, name: str):
        self.name = name
        self.to_device = []  # (mode, array)
        self.to_host = []
        self.tasks = []

    def transferToDevice(self, mode: DataTransferMode, *arrays):  # noqa: N802
        self.to_device += [(mode, a) for a in arrays]
        return self

    def libraryTask(self, task_id: str, factory, *args):  # noqa: N802
        # the factory runs immediately and its descriptor is what the runtime keeps (TaskGraph.java:737-739);
        # the reference has overloads for 1 to 20 arguments and no varargs form (TaskGraph.java:737-893)
        if not 1 <= len(args) <= 20:
            raise TypeError(f"libraryTask takes 1 to 20 task arguments, got {len(args)}")
        self.tasks.append(_LibraryTask(task_id, factory(*args)))
        return self

    def transferToHost(self, mode: DataTransferMode, *arrays):  # noqa: N802
        self.to_host += [(mode, a) for a in arrays]
        return self

    def snapshot(self):
        return self


class TornadoExecutionPlan:
    _ids = itertools.count(1)

    def __init__(self, graph: TaskGraph, device: CudaDevice | None = None, provider=None):
        self.graph = graph
        self.device = device or CudaDevice(0)
        self.provider = provider or B200LibraryProvider()
        if not self.provider.canHandle(self.device):
            raise RuntimeError("[ERROR] device does not expose a native stream")
        self.plan_id = next(self._ids)
        self.stream = self.device.torch_stream(self.plan_id)
        self.context = self.provider.createContext(self.device, self.plan_id)
        self._buffers = {}  # id(array) -> (device uint8 view, pinned host view, offset in the slabs)
        self._executions = 0
        self._use_graph = False
        self._cuda_graph = None
        self._replay = None
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0

    # -- plan options -------------------------------------------------------
    def withCUDAGraph(self):  # noqa: N802
        self._use_graph = True
        return self

    # -- internals ------------------------------------------------------------
    def _layout(self):
        """One device slab and one pinned host slab for every array of the graph.

        TornadoVM's off-heap arrays *are* the host side of a transfer (no staging copy), so each
        array's segment is re-homed into the pinned slab: host<->device copies then move the
        array's own memory.  Arrays copied back on every execution sit next to each other, so
        that their device->host transfers merge into one copy.
        """
        g = self.graph
        ordered, seen = [], set()

        def add(arr):
            if isinstance(arr, TornadoNativeArray) and id(arr) not in seen:
                seen.add(id(arr))
                ordered.append(arr)
        for _, arr in g.to_host:          # outputs first and contiguous
            add(arr)
        for mode, arr in g.to_device:
            if mode is DataTransferMode.EVERY_EXECUTION:
                add(arr)
        for _, arr in g.to_device:
            add(arr)
        for t in g.tasks:
            for p in t.descriptor.getParameters():
                add(p)
        offsets, total = {}, 0
        for arr in ordered:
            offsets[id(arr)] = total
            total += (arr.nbytes_with_header + 255) // 256 * 256  # cuMemAlloc-like 256-byte alignment per buffer
        self._dev_slab = torch.empty(max(total, 256), dtype=torch.uint8, device=self.device.torch_device)
        self._host_slab = torch.empty(max(total, 256), dtype=torch.uint8, pin_memory=True)
        host_np = self._host_slab.numpy()
        for arr in ordered:
            off, n = offsets[id(arr)], arr.nbytes_with_header
            host_np[off:off + n] = arr.segment
            arr.segment = host_np[off:off + n]                      # the array now lives in pinned memory
            arr.data = arr.segment[arr.header:].view(arr.dtype)
            self._buffers[id(arr)] = (self._dev_slab[off:off + n], self._host_slab[off:off + n], off)
        self._arrays = ordered
        self._host_slab_device_base = self._device_view_of_host_slab()

    def _device_view_of_host_slab(self):
        """The address at which kernels on this device reach the pinned host slab (cudaHostGetDevicePointer), or None
        when the runtime does not report one: host segments are then not offered to providers and every output travels
        by copy."""
        try:
            rt = C.CDLL("libcudart.so.12")
            fn = rt.cudaHostGetDevicePointer
            fn.argtypes, fn.restype = [C.POINTER(C.c_void_p), C.c_void_p, C.c_uint], C.c_int
            out = C.c_void_p()
            if fn(C.byref(out), C.c_void_p(self._host_slab.data_ptr()), 0) != 0 or not out.value:
                return None
            return out.value
        except (OSError, AttributeError):
            return None

    def _buffer(self, arr: TornadoNativeArray):
        return self._buffers[id(arr)]

    def _device_pointer(self, arr: TornadoNativeArray) -> int:
        return self._buffer(arr)[0].data_ptr() + arr.header

    @staticmethod
    def _merge(spans):
        """Merge (offset, nbytes) spans that touch (up to the 256-byte padding between buffers)."""
        out = []
        for off, n in sorted(spans):
            if out and off <= out[-1][0] + out[-1][1] + 256:
                out[-1][1] = off + n - out[-1][0]
            else:
                out.append([off, n])
        return out

    def _launch_all(self):
        # arrays copied back after every execution: their host segment (pinned, device-mapped) is offered to the
        # provider, which may let its kernel store the results there itself
        every_out = {id(arr) for mode, arr in self.graph.to_host if mode is DataTransferMode.EVERY_EXECUTION}
        delivered = {}
        for t in self.graph.tasks:
            d = t.descriptor
            params = d.getParameters()
            ptrs = [self._device_pointer(p) if isinstance(p, TornadoNativeArray) else None for p in params]
            base = self._host_slab_device_base
            host = [base + self._buffer(p)[2] + p.header if base is not None and isinstance(p, TornadoNativeArray) and id(p) in every_out
                    else None for p in params]
            inv = LibraryInvocation(params, ptrs, self.context, d.getTuning(), self.device, self.plan_id, host_pointers=host)
            # the interpreter wraps every library dispatch in an NVTX range named library::function
            # (TornadoVMInterpreter.java:1301-1315)
            self.device.nvtxRangePush(f"{d.getLibraryName()}::{d.getFunctionName()}")
            try:
                self.provider.dispatch(d.getFunctionName(), inv)
            finally:
                self.device.nvtxRangePop()
            # the host copy of an array is current only if the LAST task that writes it delivered it
            access = list(d.getAccess())
            for i, p in enumerate(params):
                if isinstance(p, TornadoNativeArray) and (i >= len(access) or access[i] is not Access.READ_ONLY):
                    delivered[id(p)] = i in inv.hostDelivered()
        return {k for k, v in delivered.items() if v}

    def _copy_back(self, delivered):
        """Device->host copies of an execution: every output array whose results no kernel stored on the host."""
        key = frozenset(delivered)
        if key not in self._d2h_cache:
            out = [(self._buffer(arr)[2], arr.nbytes_with_header) for _, arr in self.graph.to_host if id(arr) not in key]
            self._d2h_cache[key] = [(self._host_slab[off:off + n], self._dev_slab[off:off + n]) for off, n in self._merge(out)]
        for dst, src in self._d2h_cache[key]:
            dst.copy_(src, non_blocking=True)

    def _bind_replay(self):
        """Replaying an execution is one cudaGraphLaunch on the plan's stream and one stream synchronisation, as in
        the reference's interpreter (a JNI call each)."""
        return graph_replayer(self._cuda_graph, self.stream)

    def execute(self):
        g = self.graph
        first = self._executions == 0
        if self._replay is not None and torch.cuda.current_device() == self.device.index:
            self._replay()
            self.h2d_bytes_last, self.d2h_bytes_last = self._h2d_bytes, self._d2h_bytes
            self._executions += 1
            return self
        with torch.cuda.device(self.device.index), torch.cuda.stream(self.stream):
            if first:
                self._layout()
                for t in g.tasks:  # the pre-launch prepare pass
                    self.provider.prepare(t.descriptor, self.context)
            if first:
                spans = [(self._buffer(arr)[2], arr.nbytes_with_header) for _, arr in g.to_device]
                # allocation time: every buffer, outputs included, gets its header (element count) on the device
                self._dev_slab.copy_(self._host_slab, non_blocking=True)
                h2d = sum(n for _, n in spans)
                # the transfers of every later execution never change: merged spans as (device view, host view) pairs
                every = [(self._buffer(arr)[2], arr.nbytes_with_header) for mode, arr in g.to_device
                         if mode is DataTransferMode.EVERY_EXECUTION]
                self._h2d_pairs = [(self._dev_slab[off:off + n], self._host_slab[off:off + n]) for off, n in self._merge(every)]
                self._h2d_bytes = sum(n for _, n in every)
                # bytes that reach the host per execution, whether a copy or a kernel's own stores move them
                self._d2h_bytes = sum(arr.nbytes_with_header for _, arr in g.to_host)
                self._d2h_cache = {}
            else:
                h2d = self._h2d_bytes
            if self._use_graph:
                if self._cuda_graph is None:
                    # as in the reference (TornadoVMInterpreter.java:462-476), the capture region spans the whole
                    # bytecode sequence of an execution -- the every-execution transfers in, the FIRST dispatch of
                    # every task and the transfers out; everything capture-unsafe was done by prepare().  The host
                    # side of every transfer is the pinned slab, whose addresses never change.
                    self.stream.synchronize()
                    self._cuda_graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(self._cuda_graph, stream=self.stream):
                        for dst, src in self._h2d_pairs:
                            dst.copy_(src, non_blocking=True)
                        self._copy_back(self._launch_all())
                    self._cuda_graph.replay()
                    self._replay = self._bind_replay()
                else:
                    self._cuda_graph.replay()
            else:
                if not first:
                    for dst, src in self._h2d_pairs:
                        dst.copy_(src, non_blocking=True)
                self._copy_back(self._launch_all())
            d2h = self._d2h_bytes
            self.stream.synchronize()
        self.h2d_bytes_last, self.d2h_bytes_last = h2d, d2h
        self._executions += 1
        return self

    def close(self):
        if self.context is not None:
            with torch.cuda.device(self.device.index):
                self.stream.synchronize()
                self.provider.destroyContext(self.context)
            self.context = None
        self._buffers.clear()
        self._dev_slab = None
        self._replay = None
        self._cuda_graph = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False
