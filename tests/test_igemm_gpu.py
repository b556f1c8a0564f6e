"""int8 x int8 -> int32 GEMM on tcgen05 (kind::i8): exact equality with the reference loop
(gemmReferenceInt8, TestMatrixMultiplicationMMAInt8.java:160-172; inputs in [-3, 3] from Random(42) as
:397-404, and full-range bytes, whose products still fit an int32 accumulator)."""
import numpy as np
import pytest

import oracle as o
from harness import DevBuf, out_buf, stream_ptr, sync_and_check

pytestmark = pytest.mark.gpu


def _ref(a, b, m, n, k):
    return (a.reshape(m, k).astype(np.int64) @ b.reshape(k, n).astype(np.int64)).astype(np.int32)


@pytest.mark.parametrize("m,n,k", [(32, 16, 32), (128, 128, 128), (256, 512, 384), (300, 264, 144), (1024, 1024, 1024), (64, 64, 48), (17, 19, 23)])
@pytest.mark.parametrize("full_range", [False, True])
def test_igemm_exact(lib, m, n, k, full_range):
    r = o.JavaRandom(42)
    if full_range:
        a, b = (r.ints(m * k, 256) - 128).astype(np.int8), (r.ints(k * n, 256) - 128).astype(np.int8)
    else:
        a, b = (r.ints(m * k, 7) - 3).astype(np.int8), (r.ints(k * n, 7) - 3).astype(np.int8)
    da, db, dc = DevBuf(a), DevBuf(b), out_buf(m * n, np.int32)
    nws = lib.tb200_igemm_workspace_bytes(n, k)
    ws = DevBuf(np.zeros(nws, np.uint8))
    st = lib.tb200_igemm_s32(m, n, k, da.ptr, db.ptr, dc.ptr, ws.ptr, nws, stream_ptr())
    assert st == 0, lib.tb200_status_string(st)
    sync_and_check(lib)
    assert np.array_equal(dc.numpy().reshape(m, n), _ref(a, b, m, n, k))
    assert dc.guard_intact() and ws.guard_intact()


def test_igemm_without_workspace_and_argument_errors(lib):
    m = n = k = 128
    r = o.JavaRandom(1)
    a, b = (r.ints(m * k, 7) - 3).astype(np.int8), (r.ints(k * n, 7) - 3).astype(np.int8)
    da, db, dc = DevBuf(a), DevBuf(b), out_buf(m * n, np.int32)
    assert lib.tb200_igemm_s32(m, n, k, da.ptr, db.ptr, dc.ptr, None, 0, stream_ptr()) == 0  # CUDA-core kernel
    sync_and_check(lib)
    assert np.array_equal(dc.numpy().reshape(m, n), _ref(a, b, m, n, k))
    assert lib.tb200_igemm_s32(-1, n, k, da.ptr, db.ptr, dc.ptr, None, 0, stream_ptr()) == -1
    assert lib.tb200_igemm_s32(m, n, k, None, db.ptr, dc.ptr, None, 0, stream_ptr()) == -1
