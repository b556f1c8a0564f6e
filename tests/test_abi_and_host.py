"""C-ABI surface and host-side logic (no GPU, no compute calls)."""
import os
import re

import numpy as np
import pytest

from tornadovm_b200 import arrays
from tornadovm_b200.arrays import ByteArray, FloatArray, HalfFloatArray, Int8Array
from tornadovm_b200.b200 import B200, B200Options, LIBRARY_NAME
from tornadovm_b200.descriptor import Access
from tornadovm_b200.native import SIGNATURES

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "tornado_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = _declared()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/tornado_b200.h but not exported"
    assert sorted(SIGNATURES) == names, "ctypes signature table out of sync with the header"


def test_status_strings_and_version(lib):
    assert lib.tb200_version() == 100
    assert lib.tb200_status_string(0) == b"TB200_OK"
    assert lib.tb200_status_string(-1) == b"TB200_ERR_INVALID_ARG"
    assert lib.tb200_status_string(-3) == b"TB200_ERR_WORKSPACE"
    assert lib.tb200_status_string(2) == b"cudaErrorMemoryAllocation"
    assert lib.tb200_status_string(-99) == b"TB200_ERR_UNKNOWN"


def test_workspace_size(lib):
    assert lib.tb200_qx_workspace_bytes(4096, 1) == 4096 + 128 * 4
    assert lib.tb200_qx_workspace_bytes(4096, 8) == 8 * 4096 + 8 * 128 * 4
    assert lib.tb200_qx_workspace_bytes(32, 1) == 32 + 4
    assert lib.tb200_qx_workspace_bytes(32, 3) == 96 + 12


def test_array_header_layout():
    a = FloatArray(np.arange(5, dtype=np.float32))
    assert a.header == 16 and a.segment.size == 16 + 20
    assert int(a.segment[:4].view(np.int32)[0]) == 5
    b = HalfFloatArray.from_float32([1.0, -2.0], header=24)
    assert b.segment.size == 24 + 4 and list(b.numpy()) == [0x3C00, 0xC000]
    assert np.array_equal(b.to_float32(), [1.0, -2.0])
    old = arrays.ARRAY_HEADER
    try:
        arrays.ARRAY_HEADER = 24
        assert Int8Array(3).header == 24
    finally:
        arrays.ARRAY_HEADER = old


def test_factories_build_descriptors():
    m, v, out = FloatArray(12), FloatArray(4), FloatArray(3)
    d = B200.sgemv(3, 4, m, v, out)
    assert d.getLibraryName() == LIBRARY_NAME == "b200/linalg" and d.getFunctionName() == "sgemv"
    assert d.getParameters()[:2] == [3, 4] and d.getParameters()[4] is out
    assert d.getAccess() == [Access.READ_ONLY] * 4 + [Access.WRITE_ONLY]
    a, b, c = FloatArray(6), FloatArray(6), FloatArray(4)
    assert B200.sgemm(2, 2, 3, 1.0, a, b, 0.0, c).getAccess()[7] is Access.WRITE_ONLY
    assert B200.sgemm(2, 2, 3, 1.0, a, b, 0.5, c).getAccess()[7] is Access.READ_WRITE  # CuBlas.java:58-63 rule
    q, s, x, y = Int8Array(64), HalfFloatArray(2), FloatArray(32), FloatArray(2)
    d = B200.q8Gemv(2, 32, 1, q, s, x, y, B200Options(exact_int=True))
    assert d.getTuning().exact_int and d.getAccess()[6] is Access.WRITE_ONLY
    assert B200.q8GemvBytes(2, 32, 1, ByteArray(68), x, y).getFunctionName() == "q8GemvBytes"
    assert B200.q4GemvBytes(2, 32, 1, ByteArray(36), x, y).getFunctionName() == "q4GemvBytes"
    assert B200.hgemmF32(2, 2, 2, HalfFloatArray(4), HalfFloatArray(4), FloatArray(4)).getAccess()[5] is Access.WRITE_ONLY


def test_factories_reject_bad_shapes_early():
    x, y = FloatArray(64), FloatArray(4)
    with pytest.raises(RuntimeError, match="multiple of the 32-element block"):
        B200.q8Gemv(2, 33, 1, Int8Array(66), HalfFloatArray(2), x, y)
    with pytest.raises(RuntimeError, match="batch"):
        B200.q8Gemv(2, 32, 17, Int8Array(64), HalfFloatArray(2), FloatArray(17 * 32), FloatArray(34))
    with pytest.raises(RuntimeError, match="weights too small"):
        B200.q4GemvBytes(2, 32, 1, ByteArray(35), x, y)
    with pytest.raises(RuntimeError, match="array smaller"):
        B200.sgemv(3, 4, FloatArray(11), FloatArray(4), FloatArray(3))
    with pytest.raises(RuntimeError, match="non-negative"):
        B200.sgemm(-1, 2, 2, 1.0, FloatArray(4), FloatArray(4), 0.0, FloatArray(4))


def test_provider_rejects_devices_without_native_stream():
    from tornadovm_b200.provider import B200LibraryProvider
    p = B200LibraryProvider()
    assert p.libraryName() == "b200/linalg"
    assert not p.canHandle(object())

    class Dev:
        def getNativeStream(self, plan):  # noqa: N802
            return 0
    assert p.canHandle(Dev())


def test_invocation_host_segments_and_delivery_marks():
    """The extension of LibraryInvocation that B200Options.host_results uses: the device-visible address of an output
    array's host segment (None unless the plan offers one) and the marks a dispatch leaves for the arrays whose
    results its kernel stored on the host itself."""
    from tornadovm_b200.provider import LibraryInvocation
    x, y = FloatArray(8), FloatArray(8)
    inv = LibraryInvocation([4, x, y], [None, 0x1000, 0x2000], context=None)
    assert inv.getHostPointer(1) is None and inv.getHostPointer(2) is None and inv.hostDelivered() == frozenset()
    inv = LibraryInvocation([4, x, y], [None, 0x1000, 0x2000], context=None, host_pointers=[None, None, 0x7F0000002010])
    assert inv.getHostPointer(2) == 0x7F0000002010 and inv.getHostPointer(1) is None
    inv.markHostDelivered(2)
    assert inv.hostDelivered() == frozenset({2})
    assert B200Options().host_results is False and B200Options(host_results=True).host_results is True


def test_graph_replayer_declines_what_is_not_a_captured_graph():
    """Without an instantiated CUDA graph (no GPU here) the replayer reports that it cannot bind, and callers replay
    through torch instead."""
    from tornadovm_b200.native import graph_replayer

    class NoGraph:
        pass
    assert graph_replayer(NoGraph(), NoGraph()) is None


def test_igemm_workspace_covers_the_padded_transpose(lib):
    """B transposed with up to 128 zero bytes in front of every row (an A off a 128-byte line)."""
    assert lib.tb200_igemm_workspace_bytes(264, 144) == 264 * (144 + 128)
    assert lib.tb200_igemm_workspace_bytes(0, 144) == 0
