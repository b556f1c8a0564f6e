"""Pins the CPU oracle to the reference's own known answers (no GPU)."""
import json
import os

import numpy as np
import pytest

import oracle as o
from kat import build as build_kat

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")))


def test_java_random_known_answers():
    g = GOLD["java_util_random"]
    r = o.JavaRandom(g["seed"])
    assert [r.next_int() for _ in g["next_int"]] == g["next_int"]
    r = o.JavaRandom(g["seed"])
    assert [r.next_int(10) for _ in g["next_int_10"]] == g["next_int_10"]
    r = o.JavaRandom(g["seed"])
    # nextGaussian goes through StrictMath.log in the JDK and through libm here: the
    # two may differ in the last bit, which only moves a synthetic operand by 1 ulp.
    assert abs(r.next_gaussian() - g["next_gaussian_first"]) <= 2.3e-16


def test_java_random_next_float_matches_next24():
    r1, r2 = o.JavaRandom(7), o.JavaRandom(7)
    for _ in range(100):
        bits = (r1.next_int() >> 8) & 0xFFFFFF  # next(24) is the top 24 of the same 48-bit state
        assert r2.next_float() == np.float32(bits) / np.float32(1 << 24)


def test_fp16_conversion_is_ieee_rne():
    h = np.arange(65536, dtype=np.uint16)
    ref = h.view(np.float16).astype(np.float32)
    got = o.f16_to_f32(h)
    ok = ~np.isnan(ref)
    assert np.array_equal(got.view(np.uint32)[ok], ref.view(np.uint32)[ok])
    assert np.isnan(got[~ok]).all()
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(200000) * rng.choice([1e-8, 6e-8, 1e-5, 1e-3, 1.0, 300.0, 65504.0], 200000)).astype(np.float32)
    # exact halfway cases between neighbouring halves
    mid = ((ref[ok][:-1].astype(np.float64) + ref[ok][1:].astype(np.float64)) / 2).astype(np.float32)
    x = np.concatenate([x, mid[np.isfinite(mid)], got[ok]])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(o.f32_to_f16(x), want)


def test_dp4a_exact():
    # QuantizationTests.testDP4A: 128 four-byte dots of random bytes, exact
    rng = np.random.default_rng(2)
    a = rng.integers(-128, 128, 512).astype(np.int8)
    b = rng.integers(-128, 128, 512).astype(np.int8)
    want = (a.astype(np.int32).reshape(-1, 4) * b.astype(np.int32).reshape(-1, 4)).sum(1)
    assert np.array_equal(o.dp4a_n(a, b), want)
    for i in range(0, 64, 4):
        pa = int(np.frombuffer(a[i:i + 4].tobytes(), np.int32)[0])
        pb = int(np.frombuffer(b[i:i + 4].tobytes(), np.int32)[0])
        assert o.dp4a_packed(pa, pb, 5) == int(want[i // 4]) + 5


def test_q8_quantizer_rules():
    # quantizeWeightsToQ8: scale = max|v|/127 as fp16, q = clamp(round(v/scale)), zero block -> scale 0
    r = o.JavaRandom(42)
    rows, cols = 8, 256
    w = r.uniform_f32(rows * cols, -0.1, 0.1)
    w[32:64] = 0.0
    q, s, blocks = o.q8_quantize(w, rows, cols)
    wb = w.reshape(-1, 32)
    scale = (np.abs(wb).max(1) / np.float32(127.0)).astype(np.float32)
    assert np.array_equal(s, scale.astype(np.float16).view(np.uint16))
    assert s[1] == 0 and not q[32:64].any()
    inv = np.where(scale == 0, np.float32(0), np.float32(1) / np.where(scale == 0, np.float32(1), scale)).astype(np.float32)
    want = np.clip(np.floor((wb * inv[:, None]).astype(np.float32).astype(np.float64) + 0.5), -127, 127).astype(np.int8)
    assert np.array_equal(q.reshape(-1, 32), want)
    assert np.abs(q).max() == 127
    # unified layout carries the same bytes
    bl = blocks.reshape(-1, 34)
    assert np.array_equal(bl[:, :2].copy().view(np.uint16).ravel(), s)
    assert np.array_equal(bl[:, 2:].copy().view(np.int8), q.reshape(-1, 32))
    assert np.array_equal(o.q8_pack_blocks(q, s), blocks)


def test_q8_gemv_orders_agree_and_meet_reference_tolerance():
    # QuantizationTests.java:838-884: abs 0.1 against the UNQUANTISED fp32 product
    r = o.JavaRandom(42)
    n, d = 2048, 256
    x = r.uniform_f32(n, -1, 1)
    w = r.uniform_f32(n * d, -0.1, 0.1)
    q, s, _ = o.q8_quantize(w, d, n)
    plain = o.sgemv_seq(w, x, n, d)
    y_ref = o.q8_gemv_ref(q, s, x, n, d, 32)
    y_seq = o.q8_gemv_seq(q, s, x, n, d)
    y64 = o.q8_gemv_f64(q, s, x, n, d)
    tol = GOLD["tolerances"]["q8_gemv_abs"]["value"]
    assert np.abs(y_ref - plain).max() < tol
    assert o.rel_l2(y_ref, y64) < 1e-6 and o.rel_l2(y_seq, y64) < 1e-5
    assert np.array_equal(o.q8_gemv_seq(q, s, x, n, d, threads=True), y_seq)


def test_x_quantizer_roundtrip():
    # QuantizationTests.testQuantization: |x - q*scale| <= 0.01 for x in [-1,1)
    r = o.JavaRandom(42)
    x = r.uniform_f32(8192, -1, 1)
    xq, scale = o.quantize_x_tensor(x)
    assert np.abs(x - xq.astype(np.float32) * scale).max() <= GOLD["tolerances"]["x_quant_roundtrip_abs"]["value"]
    xq2, xs2 = o.quantize_x_block(x)
    assert np.abs(x - xq2.astype(np.float32) * np.repeat(xs2, 32)).max() <= 0.01
    assert np.abs(xq2).max() <= 127
    z, zs = o.quantize_x_block(np.zeros(64, np.float32))
    assert not z.any() and (zs == 1.0).all()


def test_sgemv_orders():
    m, v = o.make_sgemv(64, 1024)
    y64 = o.sgemv_f64(m, v, 1024, 64)
    assert np.array_equal(o.sgemv_seq(m, v, 1024, 64), (m.reshape(64, 1024).astype(np.float64) @ v.astype(np.float64)).astype(np.float32)) or \
        o.rel_l2(o.sgemv_seq(m, v, 1024, 64), y64) < 1e-6
    assert o.rel_l2(o.sgemv_workgroup(m, v, 1024, 64, 32), y64) < 1e-6
    # one fp32 accumulator, ascending j, no fused multiply-add
    row = m[:1024]
    acc = np.float32(0)
    for j in range(1024):
        acc = np.float32(acc + np.float32(row[j] * v[j]))
    assert o.sgemv_seq(m, v, 1024, 64)[0] == acc
    assert np.array_equal(o.sgemv_seq(m, v, 1024, 64, threads=True), o.sgemv_seq(m, v, 1024, 64))


@pytest.mark.parametrize("case", GOLD["mma_gemm"], ids=lambda c: c["source"].split()[-1])
def test_hgemm_reference_loop_closed_forms(case):
    a, b, exp = build_kat(case)
    got = o.hgemm_ref(a.ravel(), b.ravel(), case["m"], case["n"], case["k"])
    assert np.abs(got - exp).max() <= case["tol"]
    assert np.array_equal(got, exp)  # these cases are exact in fp32


def test_hgemm_ref_matches_numpy_and_f64():
    a, b = o.make_hgemm(64, 64, 64)
    c = o.hgemm_ref(a, b, 64, 64, 64)
    c64 = o.hgemm_f64(a, b, 64, 64, 64)
    assert o.rel_l2(c, c64) < 1e-6
    af = a.view(np.float16).astype(np.float64).reshape(64, 64)
    bf = b.view(np.float16).astype(np.float64).reshape(64, 64)
    assert np.allclose(c64, af @ bf, rtol=1e-12, atol=1e-12)
    # ascending-k fp32 accumulation of element (3, 5)
    acc = np.float32(0)
    for k in range(64):
        acc = np.float32(acc + np.float32(np.float32(af[3, k]) * np.float32(bf[k, 5])))
    assert c[3, 5] == acc


def test_sgemm_seq_and_identity():
    # SgemmTornado.java:116-134 validates with A = identity -> C == B
    n = 64
    b = o.JavaRandom(3).uniform_f32(n * n, 0, 1)
    eye = np.eye(n, dtype=np.float32).ravel()
    assert np.array_equal(o.sgemm_seq(eye, b, n, n, n).ravel(), b)
    a2, b2 = o.make_sgemm(n, n, n)
    c = o.sgemm_seq(a2, b2, n, n, n)
    assert o.rel_l2(c, o.sgemm_f64(a2, b2, n, n, n)) < 1e-6
    assert np.array_equal(o.sgemm_seq(a2, b2, n, n, n, threads=True), c)
    assert np.array_equal(o.sgemm_seq(a2, b2, n, n, n, 8, 24), c[8:24])


def test_q4_block_format_and_dots():
    rows, cols = 4, 256
    blocks, scales, x = o.make_q4(rows, cols)
    bl = blocks.reshape(-1, 18)
    assert np.array_equal(bl[:, :2].copy().view(np.uint16).ravel(), scales)
    nib = np.concatenate([bl[:, 2:] & 0xF, bl[:, 2:] >> 4], axis=1).astype(np.int32) - 8  # elements 0..15, 16..31
    s = scales.view(np.float16).astype(np.float64)
    want = ((nib * x.reshape(-1, 32).astype(np.float64)[np.tile(np.arange(cols // 32), rows)]) .sum(1) * s).reshape(rows, -1).sum(1)
    assert np.allclose(o.q4_gemv_f64(blocks, x, cols, rows), want, rtol=1e-12)
    assert o.rel_l2(o.q4_gemv_seq(blocks, x, cols, rows), want) < 1e-5
    xq, xs = o.quantize_x_block(x)
    dots = o.q4_blockdots_i32(blocks, xq, cols, rows)
    wantd = (nib * xq.reshape(-1, 32).astype(np.int32)[np.tile(np.arange(cols // 32), rows)]).sum(1)
    assert np.array_equal(dots, wantd)


def test_q8_blockdots_and_combine():
    rows, cols = 8, 512
    q, s, x = o.make_q8(rows, cols)
    xq, xs = o.quantize_x_block(x)
    dots = o.q8_blockdots_i32(q, xq, cols, rows)
    want = (q.astype(np.int32).reshape(rows, -1, 32) * xq.astype(np.int32).reshape(1, -1, 32)).sum(2)
    assert np.array_equal(dots.reshape(rows, -1), want)
    y = o.blockdots_combine_f64(dots, s, xs, cols // 32, rows)
    ref = (want * s.view(np.float16).astype(np.float64).reshape(rows, -1) * xs.astype(np.float64)).sum(1)
    assert np.allclose(y, ref, rtol=1e-12)
    # the int path approximates the float path to quantisation accuracy
    assert o.rel_l2(y, o.q8_gemv_f64(q, s, x, cols, rows)) < 2e-2


def test_fp8_tables_match_the_reference_formats():
    """Constants and encodings of tornado-api/.../types/FP8.java:41-43, :52-76."""
    e4, e5 = o.fp8_decode_table("e4m3"), o.fp8_decode_table("e5m2")
    assert e4[0x7E] == 448.0 and e4[0xFE] == -448.0 and np.isnan(e4[0x7F]) and np.isnan(e4[0xFF])  # max normal, the one NaN
    assert e4[0x38] == 1.0 and e4[0x01] == 2.0 ** -9 and e4[0x08] == 2.0 ** -6 and e4[0x00] == 0.0
    assert np.isfinite(e4[:0x7F]).all() and (np.diff(e4[:0x7F]) > 0).all()  # monotonic: no infinity below the NaN
    assert e5[0x7B] == 57344.0 and np.isinf(e5[0x7C]) and np.isnan(e5[0x7D]) and e5[0x3C] == 1.0 and e5[0x01] == 2.0 ** -16
    # E5M2 is the upper byte of an IEEE half
    halves = (np.arange(256, dtype=np.uint16) << 8).view(np.float16).astype(np.float32)
    assert np.array_equal(np.nan_to_num(halves, nan=7.0), np.nan_to_num(e5, nan=7.0))
    # the reference's test values are exact in both formats, and the all-halves case gives K * 0.25
    vals = (np.arange(16) - 8) * 0.25
    for fmt, table in (("e4m3", e4), ("e5m2", e5)):
        assert np.array_equal(table[o.fp8_encode_exact(vals, fmt)], vals.astype(np.float32))
    half = o.fp8_encode_exact(np.full(16 * 32, 0.5), "e4m3")
    assert np.array_equal(o.fp8_gemm_ref(half, half, 16, 16, 32, "e4m3"), np.full((16, 16), 8.0))
