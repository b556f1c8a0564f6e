"""int8 x int8 -> int32 GEMM (kind::i8) and fp8 x fp8 -> fp32 GEMM (kind::f8f6f4) on tcgen05: exact equality with the reference loop
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
@pytest.mark.parametrize("header", [16, 24, 128])
def test_igemm_exact(lib, m, n, k, full_range, header):
    r = o.JavaRandom(42)
    if full_range:
        a, b = (r.ints(m * k, 256) - 128).astype(np.int8), (r.ints(k * n, 256) - 128).astype(np.int8)
    else:
        a, b = (r.ints(m * k, 7) - 3).astype(np.int8), (r.ints(k * n, 7) - 3).astype(np.int8)
    # every array behind a 16- or 24-byte header (A's rows then start off a 128-byte line, at 24 also off a 16-byte
    # boundary), or on a line
    da, db, dc = DevBuf(a, header), DevBuf(b, header), out_buf(m * n, np.int32, header)
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


# ---------------------------------------------------------------------------------------------- fp8
FP8_FORMATS = {"e4m3": 0, "e5m2": 1}


def _fp8_case(lib, m, n, k, fmt, a, b, header=16):
    da, db, dc = DevBuf(a, header), DevBuf(b, header), out_buf(m * n, np.float32, header)
    nws = lib.tb200_igemm_workspace_bytes(n, k)
    ws = DevBuf(np.zeros(max(nws, 16), np.uint8))
    st = lib.tb200_fp8gemm_f32(m, n, k, FP8_FORMATS[fmt], da.ptr, db.ptr, dc.ptr, ws.ptr, nws, stream_ptr())
    assert st == 0, lib.tb200_status_string(st)
    sync_and_check(lib)
    assert dc.guard_intact() and ws.guard_intact()
    return dc.numpy().reshape(m, n)


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("m,n,k", [(16, 16, 32), (64, 64, 64), (128, 128, 128), (256, 512, 384), (300, 264, 144), (1024, 1024, 1024), (17, 19, 23)])
@pytest.mark.parametrize("header", [16, 24])
def test_fp8_gemm_reference_inputs_exact(lib, m, n, k, fmt, header):
    """Inputs of TestMatrixMultiplicationMMAFP8 (multiples of 0.25 in [-2, 2) from Random(42), :433-439): every partial
    sum is exact in fp32, so the result equals the reference loop exactly (its own tolerance is 1e-3, :424)."""
    r = o.JavaRandom(42)
    a = o.fp8_encode_exact((r.ints(m * k, 16) - 8) * 0.25, fmt)
    b = o.fp8_encode_exact((r.ints(k * n, 16) - 8) * 0.25, fmt)
    got = _fp8_case(lib, m, n, k, fmt, a, b, header)
    assert np.array_equal(got.astype(np.float64), o.fp8_gemm_ref(a, b, m, n, k, fmt))


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("header", [16, 24, 72])
@pytest.mark.parametrize("k", [128, 144])
def test_fp8_gemm_nothing_in_front_of_a_row_reaches_it(lib, fmt, header, k):
    """A's rows are read from an aligned address below them, so the bytes in front of a row -- the end of the row
    before -- land in shared memory too.  Row 0 ends in NaNs: they belong in row 0's results and nowhere else."""
    m, n = 256, 128
    r = o.JavaRandom(7)
    a = o.fp8_encode_exact((r.ints(m * k, 16) - 8) * 0.25, fmt).copy()
    b = o.fp8_encode_exact((r.ints(k * n, 16) - 8) * 0.25, fmt)
    a.reshape(m, k)[0, k - 16:] = 0x7F  # NaN in both formats
    got = _fp8_case(lib, m, n, k, fmt, a, b, header)
    assert np.isnan(got[0]).all()
    assert np.array_equal(got[1:].astype(np.float64), o.fp8_gemm_ref(a, b, m, n, k, fmt)[1:])


def test_fp8_gemm_identity_and_all_halves(lib):
    """testGemmFP8Identity (:288-309) and testGemmFP8AllHalves (:312-333), at the reference's 16 x 16 x 32 (CUDA-core
    path) and at a tensor-core shape."""
    for m, n, k in [(16, 16, 32), (128, 256, 128)]:
        a = np.zeros(m * k, np.uint8)
        one = o.fp8_encode_exact(np.array([1.0]), "e4m3")[0]
        for i in range(min(m, k)):
            a[i * k + i] = one
        b = o.fp8_encode_exact((np.arange(k * n) % 5) - 2.0, "e4m3")
        got = _fp8_case(lib, m, n, k, "e4m3", a, b)
        assert np.array_equal(got.astype(np.float64), o.fp8_gemm_ref(a, b, m, n, k, "e4m3"))
        half = o.fp8_encode_exact(np.full(max(m * k, k * n), 0.5), "e4m3")
        got = _fp8_case(lib, m, n, k, "e4m3", half[:m * k], half[:k * n])
        assert np.array_equal(got, np.full((m, n), k * 0.25, np.float32))


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_fp8_gemm_all_finite_bytes(lib, fmt):
    """Every finite byte pattern, subnormals included: against the float64 product of the decoded operands."""
    m, n, k = 256, 256, 512
    table = o.fp8_decode_table(fmt)
    finite = np.array([b for b in range(256) if np.isfinite(table[b]) and abs(table[b]) <= 16.0], np.uint8)
    r = o.JavaRandom(5)
    a, b = finite[r.ints(m * k, len(finite))], finite[r.ints(k * n, len(finite))]
    got = _fp8_case(lib, m, n, k, fmt, a, b)
    assert o.rel_l2(got, o.fp8_gemm_ref(a, b, m, n, k, fmt)) <= 1e-6


def test_fp8_gemm_argument_errors(lib):
    d = DevBuf(np.zeros(4096, np.uint8))
    c = out_buf(64 * 64, np.float32)
    assert lib.tb200_fp8gemm_f32(64, 64, 64, 2, d.ptr, d.ptr, c.ptr, None, 0, stream_ptr()) == -1  # unknown format
    assert lib.tb200_fp8gemm_f32(-1, 64, 64, 0, d.ptr, d.ptr, c.ptr, None, 0, stream_ptr()) == -1
    assert lib.tb200_fp8gemm_f32(64, 64, 64, 0, d.ptr, d.ptr, c.ptr, None, 0, stream_ptr()) == 0  # no workspace: CUDA-core kernel
    sync_and_check(lib)
    assert np.array_equal(c.numpy(), np.zeros(64 * 64, np.float32))
