"""Host mirror of TornadoVM's off-heap arrays for the types on this path.

A TornadoVM array is one memory segment: ARRAY_HEADER bytes (word 0 holds the
element count as int32) followed by the elements; the whole segment is copied
to the device and library tasks receive ``device base + ARRAY_HEADER``
(tornado-api/.../types/arrays/TornadoNativeArray.java:38-55;
tornado-runtime/.../interpreter/TornadoVMInterpreter.java:1260-1266).  The
header is 24 bytes under the launcher's JVM flags and 16 otherwise, so the
element pointer is 8 or 0 modulo 16.
"""
from __future__ import annotations

import numpy as np

#: header size in bytes; override like ``-Dtornado.panama.objectHeader=N``
ARRAY_HEADER = 16


class TornadoNativeArray:
    dtype = np.uint8

    def __init__(self, size_or_data, header: int | None = None):
        self.header = ARRAY_HEADER if header is None else int(header)
        if isinstance(size_or_data, (int, np.integer)):
            n = int(size_or_data)
            data = None
        else:
            data = np.ascontiguousarray(size_or_data, dtype=self.dtype).ravel()
            n = data.size
        self.size = n
        self.segment = np.zeros(self.header + n * np.dtype(self.dtype).itemsize, np.uint8)
        self.segment[:4] = np.frombuffer(np.int32(n).tobytes(), np.uint8)
        self.data = self.segment[self.header:].view(self.dtype)
        if data is not None:
            self.data[:] = data

    def getSize(self) -> int:  # noqa: N802  (reference naming)
        return self.size

    def get(self, i):
        return self.data[i]

    def set(self, i, v) -> None:
        self.data[i] = v

    def numpy(self) -> np.ndarray:
        return self.data

    @property
    def nbytes_with_header(self) -> int:
        return self.segment.size


class FloatArray(TornadoNativeArray):
    dtype = np.float32


class HalfFloatArray(TornadoNativeArray):
    """IEEE binary16 bit patterns in 16-bit words (HalfFloatArray.java:34-58)."""
    dtype = np.uint16

    @classmethod
    def from_float32(cls, values, header=None):
        return cls(np.asarray(values, np.float32).astype(np.float16).view(np.uint16), header)

    def to_float32(self) -> np.ndarray:
        return self.data.view(np.float16).astype(np.float32)


class BFloat16Array(TornadoNativeArray):
    """bfloat16 bit patterns in 16-bit words (tornado-api/.../types/arrays/BFloat16Array.java)."""
    dtype = np.uint16

    @classmethod
    def from_float32(cls, values, header=None):
        u = np.asarray(values, np.float32).view(np.uint32).astype(np.uint64)
        return cls(((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16), header)

    def to_float32(self) -> np.ndarray:
        return (self.data.astype(np.uint32) << 16).view(np.float32)


class Int8Array(TornadoNativeArray):
    dtype = np.int8


class ByteArray(TornadoNativeArray):
    dtype = np.uint8


class IntArray(TornadoNativeArray):
    dtype = np.int32
