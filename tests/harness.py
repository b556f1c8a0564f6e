"""Test-side stand-in for how TornadoVM hands buffers to a library task.

A device buffer is ``header`` bytes followed by the payload and a task receives
``base + header`` (TornadoVMInterpreter.java:1260-1266); header 16 gives a
16-byte aligned element pointer, header 24 one that is 8 modulo 16.  Every
buffer carries a poisoned guard band behind the payload that is checked after
the call, because compute-sanitizer is not available for these tests.
"""
import ctypes as C

import numpy as np
import torch

GUARD = 256
POISON = 0xA5


class DevBuf:
    def __init__(self, host: np.ndarray, header: int = 16):
        host = np.ascontiguousarray(host)
        self.dtype, self.shape, self.header = host.dtype, host.shape, header
        self.nbytes = host.nbytes
        raw = np.full(header + self.nbytes + GUARD, POISON, np.uint8)
        raw[header:header + self.nbytes] = host.view(np.uint8).ravel()
        self.t = torch.from_numpy(raw).cuda()

    @property
    def ptr(self) -> C.c_void_p:
        return C.c_void_p(self.t.data_ptr() + self.header)

    def numpy(self) -> np.ndarray:
        raw = self.t.cpu().numpy()
        return raw[self.header:self.header + self.nbytes].view(self.dtype).reshape(self.shape).copy()

    def guard_intact(self) -> bool:
        raw = self.t.cpu().numpy()
        return bool((raw[:self.header] == POISON).all() and (raw[self.header + self.nbytes:] == POISON).all())


def out_buf(n, dtype=np.float32, header=16):
    """Output buffer pre-filled with NaN (or a sentinel) so unwritten elements show."""
    if np.dtype(dtype).kind == "f":
        return DevBuf(np.full(n, np.nan, dtype), header)
    sentinel = np.iinfo(dtype).max - 1 if np.dtype(dtype).kind == "u" else -2
    return DevBuf(np.full(n, sentinel, dtype), header)


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def sync_and_check(lib):
    torch.cuda.synchronize()
    st = C.c_int(0)
    assert lib.tb200_device_status(C.byref(st)) == 0
    assert st.value == 0, f"device status {st.value}"
