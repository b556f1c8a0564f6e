"""GPU parity: FP32 SGEMM and FP16 GEMM through the C ABI against the CPU oracle."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import oracle as o
from harness import DevBuf, out_buf, stream_ptr, sync_and_check
from kat import build as build_kat

pytestmark = pytest.mark.gpu
GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")))

REL_L2_FP32 = 1e-5   # FP32 SGEMM vs fp64-accumulated oracle
REL_L2_FP16 = 2e-3   # FP16 GEMM vs the fp32-accumulated reference loop


def _ok(st, lib):
    assert st == 0, lib.tb200_status_string(st).decode()


@pytest.mark.parametrize("m,n,k", [(512, 512, 512), (128, 128, 128), (256, 384, 64), (200, 136, 100), (64, 64, 4),
                                   (17, 19, 23), (1, 1, 1), (130, 260, 36)])
@pytest.mark.parametrize("header", [16, 24])
def test_sgemm_matches_oracle(lib, m, n, k, header):
    r = o.JavaRandom(42)
    a, b = r.uniform_f32(m * k, 0, 1), r.uniform_f32(k * n, 0, 1)
    da, db, dc = DevBuf(a, header), DevBuf(b, header), out_buf(m * n, header=header)
    _ok(lib.tb200_sgemm(m, n, k, 1.0, da.ptr, db.ptr, 0.0, dc.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    got = dc.numpy().reshape(m, n)
    c64 = o.sgemm_f64(a, b, m, n, k)
    cref = o.sgemm_seq(a, b, m, n, k)
    err = o.rel_l2(got, c64)
    # "no worse than the reference's own error": the reference loop's error on the same inputs, with 10 %
    # slack because both errors are sums of ~k roundings whose ratio fluctuates from input to input
    assert err <= REL_L2_FP32 and err <= max(1.1 * o.rel_l2(cref, c64), 2e-7)
    assert np.abs(got - cref).max() <= GOLD["tolerances"]["sgemm_abs"]["value"]
    assert dc.guard_intact()


def test_sgemm_alpha_beta_and_identity(lib):
    n = 256
    b = o.JavaRandom(3).uniform_f32(n * n, 0, 1)
    eye = np.eye(n, dtype=np.float32).ravel()
    c0 = o.JavaRandom(4).uniform_f32(n * n, 0, 1)
    da, db, dc = DevBuf(eye), DevBuf(b), DevBuf(c0.copy())
    _ok(lib.tb200_sgemm(n, n, n, 2.0, da.ptr, db.ptr, 0.5, dc.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    assert np.allclose(dc.numpy(), 2.0 * b + 0.5 * c0, rtol=1e-6, atol=1e-6)
    # SgemmTornado.java:116-134: A = identity gives C == B exactly
    dc2 = out_buf(n * n)
    _ok(lib.tb200_sgemm(n, n, n, 1.0, da.ptr, db.ptr, 0.0, dc2.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    assert np.array_equal(dc2.numpy(), b)


def test_sgemm_benchmark_shape_rows_sampled(lib):
    """M=N=K=4096 (MatrixMultiplication2D shape): a band of rows against the oracle, the rest by linearity."""
    import torch
    n = 4096
    a, b = o.make_sgemm(n, n, n)
    ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    tc = torch.full((n, n), float("nan"), device="cuda")
    P = lambda t: C.c_void_p(t.data_ptr())
    _ok(lib.tb200_sgemm(n, n, n, 1.0, P(ta), P(tb), 0.0, P(tc), stream_ptr()), lib)
    sync_and_check(lib)
    c = tc.cpu().numpy()
    assert not np.isnan(c).any()
    for r0 in (0, 2047, 4088):
        want = o.sgemm_f64(a, b, n, n, n, r0, r0 + 8)
        assert o.rel_l2(c[r0:r0 + 8], want) <= REL_L2_FP32
    # checksum of checksums: (1^T A) B 1 == 1^T C 1 in double
    lhs = (a.reshape(n, n).astype(np.float64).sum(0) * b.reshape(n, n).astype(np.float64).sum(1)).sum()
    assert abs(c.astype(np.float64).sum() - lhs) / lhs < 1e-6


@pytest.mark.parametrize("case", GOLD["mma_gemm"], ids=lambda c: c["source"].split()[-1])
@pytest.mark.parametrize("header", [16, 24])
def test_hgemm_reference_known_answers(lib, case, header):
    a, b, exp = build_kat(case)
    m, n, k = case["m"], case["n"], case["k"]
    da, db, dc = DevBuf(a, header), DevBuf(b, header), out_buf(m * n, header=header)
    _ok(lib.tb200_hgemm_f32(m, n, k, da.ptr, db.ptr, dc.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    assert np.abs(dc.numpy().reshape(m, n) - exp).max() <= case["tol"]
    assert dc.guard_intact()


HGEMM_SHAPES = [tuple(s) for s in GOLD["mma_random_shapes"]["shapes"]] + [
    (128, 128, 64), (256, 256, 256), (128, 256, 512), (384, 640, 192), (1024, 1024, 1024),
    (200, 264, 72), (130, 136, 40), (100, 100, 100), (1, 8, 8), (2048, 2048, 2048)]


@pytest.mark.parametrize("m,n,k", HGEMM_SHAPES)
@pytest.mark.parametrize("header", [16, 24])
def test_hgemm_matches_reference_loop(lib, m, n, k, header):
    if m * n * k > 2**28 and header == 24:
        pytest.skip("large case runs once")
    r = o.JavaRandom(42)
    mul = 1.0 / np.sqrt(k)
    a, b = r.gaussian_f16(m * k, mul), r.gaussian_f16(k * n, mul)
    da, db, dc = DevBuf(a, header), DevBuf(b, header), out_buf(m * n, header=header)
    _ok(lib.tb200_hgemm_f32(m, n, k, da.ptr, db.ptr, dc.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    got = dc.numpy().reshape(m, n)
    rows = m if m * n * k <= 2**27 else 64
    ref = o.hgemm_ref(a, b, m, n, k, 0, rows)
    assert o.rel_l2(got[:rows], ref) <= REL_L2_FP16
    # the reference's own acceptance tests: abs 0.01 (unit tests), rel 2e-2 / max(|ref|,1) (example)
    assert np.abs(got[:rows] - ref).max() <= GOLD["mma_random_shapes"]["abs_tol"]
    assert not np.isnan(got).any() and dc.guard_intact()


@pytest.mark.parametrize("ha,hb,hc", [(24, 24, 24), (24, 16, 16), (16, 24, 16), (16, 16, 24), (24, 24, 16)])
@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (200, 264, 72), (384, 1000, 520)])
def test_hgemm_operands_behind_24_byte_headers(lib, m, n, k, ha, hb, hc):
    """Arrays 8 bytes past a 16-byte boundary, in every combination, with NaN bit patterns right in front of A and B
    and an infinity at the end of A's first row: nothing outside a row may leak into its results."""
    import torch
    r = o.JavaRandom(7)
    mul = 1.0 / np.sqrt(k)
    a, b = r.gaussian_f16(m * k, mul), r.gaussian_f16(k * n, mul)
    a = a.copy()
    a[k - 1] = 0x7C00  # +inf as the last element of row 0: row 0 becomes inf / nan, row 1 must not
    da, db, dc = DevBuf(a, ha), DevBuf(b, hb), out_buf(m * n, header=hc)
    da.t[:ha] = 0xFF  # NaN halves in front of the arrays
    db.t[:hb] = 0xFF
    _ok(lib.tb200_hgemm_f32(m, n, k, da.ptr, db.ptr, dc.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    got = dc.numpy().reshape(m, n)
    ref = o.hgemm_ref(np.ascontiguousarray(a[k:]), b, m - 1, n, k)
    assert np.isfinite(got[1:]).all()
    assert o.rel_l2(got[1:], ref) <= REL_L2_FP16
    assert not np.isfinite(got[0]).all()  # the infinity did arrive in its own row
    raw = dc.t.cpu().numpy()
    assert (raw[:hc] == 0xA5).all() and (raw[hc + dc.nbytes:] == 0xA5).all()


@pytest.mark.parametrize("offset", [8, 16, 24, 48, 72, 112])
def test_hgemm_large_at_byte_offsets(lib, offset):
    """4096 x 4096 x 1024 with A, B and C `offset` bytes past a 128-byte line (16 and 24: arrays behind a header in an
    aligned buffer) against an fp32 product of the same halves.  Multiples of 16 run on SM pairs, the others on single
    CTAs.  Everything around the matrices is NaN, and row 0 of A ends in an infinity: what lies in front of a row
    (the end of the row before, or the bytes before the matrix) must not reach any product."""
    import torch
    m, n, k = 4096, 4096, 1024
    g = torch.Generator(device="cuda").manual_seed(5)
    a = (torch.randn((m, k), device="cuda", generator=g) / k**0.5).half()
    b = (torch.randn((k, n), device="cuda", generator=g) / k**0.5).half()
    a[0, k - 1] = float("inf")
    raw = [torch.full((t.numel() * t.element_size() + 512,), 0xFF, dtype=torch.uint8, device="cuda") for t in (a, b)]
    craw = torch.full((m * n * 4 + 512,), 0xFF, dtype=torch.uint8, device="cuda")
    base = [(t.data_ptr() + 127) // 128 * 128 + offset for t in (raw[0], raw[1], craw)]
    offs = [bb - t.data_ptr() for bb, t in zip(base, (raw[0], raw[1], craw))]
    raw[0][offs[0]:offs[0] + a.numel() * 2].copy_(a.view(torch.uint8).reshape(-1))
    raw[1][offs[1]:offs[1] + b.numel() * 2].copy_(b.view(torch.uint8).reshape(-1))
    _ok(lib.tb200_hgemm_f32(m, n, k, C.c_void_p(base[0]), C.c_void_p(base[1]), C.c_void_p(base[2]), stream_ptr()), lib)
    sync_and_check(lib)
    got = craw[offs[2]:offs[2] + m * n * 4].view(torch.float32).reshape(m, n)
    want = a[1:].float() @ b.float()
    assert torch.isfinite(got[1:]).all()
    assert not torch.isfinite(got[0]).all()  # the infinity did arrive in its own row
    assert ((got[1:] - want).norm() / want.norm()).item() <= 1e-4
    assert (craw[:offs[2]] == 0xFF).all() and (craw[offs[2] + m * n * 4:] == 0xFF).all()


def test_gemm_argument_errors(lib):
    d = DevBuf(np.zeros(64, np.float32))
    assert lib.tb200_sgemm(-1, 2, 2, 1.0, d.ptr, d.ptr, 0.0, d.ptr, stream_ptr()) == -1
    assert lib.tb200_sgemm(2, 2, 2, 1.0, None, d.ptr, 0.0, d.ptr, stream_ptr()) == -1
    assert lib.tb200_hgemm_f32(2, 2, 2, C.c_void_p(d.ptr.value + 1), d.ptr, d.ptr, stream_ptr()) == -2
    assert lib.tb200_hgemm_f32(0, 2, 2, d.ptr, d.ptr, d.ptr, stream_ptr()) == 0


@pytest.mark.parametrize("pairs", [0, 1])
@pytest.mark.parametrize("m,n,k", [(4096, 4096, 512), (3000, 4100 // 8 * 8, 264), (2304, 3328, 1024)])
def test_hgemm_both_tensor_core_variants(lib, pairs, m, n, k):
    """Single-CTA 128x256 tiles and SM-pair 256x256 tiles (tcgen05 cta_group::2) give the same product."""
    import torch
    old = C.c_int(0)
    assert lib.tb200_get_option(2, C.byref(old)) == 0
    try:
        assert lib.tb200_set_option(2, pairs) == 0
        g = torch.Generator(device="cuda").manual_seed(m + n + k)
        a = (torch.randn((m, k), device="cuda", generator=g) / k**0.5).half()
        b = (torch.randn((k, n), device="cuda", generator=g) / k**0.5).half()
        c = torch.full((m, n), float("nan"), device="cuda")
        P = lambda t: C.c_void_p(t.data_ptr())
        _ok(lib.tb200_hgemm_f32(m, n, k, P(a), P(b), P(c), stream_ptr()), lib)
        sync_and_check(lib)
        rows = [0, 127, 128, 255, 256, m // 2, m - 1]
        ah = a.cpu().numpy().view(np.uint16)
        bh = b.cpu().numpy().view(np.uint16)
        got = c.cpu().numpy()
        assert not np.isnan(got).any()
        for r in rows:
            ref = o.hgemm_ref(np.ascontiguousarray(ah[r:r + 1]).ravel(), bh.ravel(), 1, n, k)
            assert o.rel_l2(got[r:r + 1], ref) <= REL_L2_FP16
        # every element against an fp32 matmul of the same halves (tolerance of the fp16 path)
        ref_all = (a.float() @ b.float())
        assert ((c - ref_all).norm() / ref_all.norm()).item() <= 1e-4
    finally:
        lib.tb200_set_option(2, old.value)


def test_hgemm_scatter_stores_every_tile_to_every_destination(lib):
    """The column-sharded form on one GPU: two destination buffers (stand-ins for two GPUs' results), the
    shard's columns land at their offset of the wide row-major matrix, nothing else is touched."""
    m, n_local, k, n_total, col_off = 384, 512, 256, 1536, 512
    a16, b16 = o.make_hgemm(m, n_local, k)
    da, db = DevBuf(a16), DevBuf(b16)
    plain = out_buf(m * n_local)
    assert lib.tb200_hgemm_f32(m, n_local, k, da.ptr, db.ptr, plain.ptr, stream_ptr()) == 0
    sentinel = np.float32(-3.0)
    dsts = [DevBuf(np.full(m * n_total, sentinel, np.float32)) for _ in range(2)]
    ptrs = (C.c_void_p * 2)(*[d.ptr.value for d in dsts])
    st = lib.tb200_hgemm_f32_scatter(m, n_local, k, da.ptr, db.ptr, ptrs, 2, n_total, col_off, stream_ptr())
    assert st == 0, lib.tb200_status_string(st)
    sync_and_check(lib)
    want = np.full((m, n_total), sentinel, np.float32)
    want[:, col_off:col_off + n_local] = plain.numpy().reshape(m, n_local)
    for d in dsts:
        assert np.array_equal(d.numpy().reshape(m, n_total), want)
        assert d.guard_intact()
    # argument checks: the block must fit inside the wide matrix
    assert lib.tb200_hgemm_f32_scatter(m, n_local, k, da.ptr, db.ptr, ptrs, 2, n_total, n_total - n_local + 8, stream_ptr()) == -1
    assert lib.tb200_hgemm_f32_scatter(m, n_local, k, da.ptr, db.ptr, ptrs, 9, n_total, 0, stream_ptr()) == -1
