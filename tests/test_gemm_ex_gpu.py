"""GPU parity of the fused-epilogue / typed-output / batched tensor-core GEMM (tb200_gemm_ex) against the
oracle: the fp32-accumulated reference product followed by the epilogue expressions of the reference's own
tests (TestCutlass.java:225-330, :302-545, :556-585; TestCuBlasGemmExFP16.java:102-117)."""
import ctypes as C

import numpy as np
import pytest

import oracle as o
from harness import DevBuf, out_buf, stream_ptr, sync_and_check

pytestmark = pytest.mark.gpu

IN_F16, IN_BF16 = 0, 1
OUT_F32, OUT_F16, OUT_BF16 = 0, 1, 2
ACTS = {"none": 0, "relu": 1, "gelu": 2, "silu": 3, "sigmoid": 4, "tanh": 5, "hardswish": 6}
# relative L2 against the double-precision epilogue on the fp32-accumulated product: fp32 out carries only the
# fp16 operands' product error (2e-3, the FP16 GEMM bound); 16-bit outputs add one rounding of the result
REL_L2 = {OUT_F32: 2e-3, OUT_F16: 2e-3, OUT_BF16: 8e-3}


def _ok(st, lib):
    assert st == 0, lib.tb200_status_string(st).decode()


def _to_out(x, out_type):
    if out_type == OUT_F32:
        return np.asarray(x, np.float32)
    return o.f32_to_f16(np.asarray(x, np.float32).ravel()) if out_type == OUT_F16 else o.f32_to_bf16(np.asarray(x, np.float32).ravel())


def _from_out(raw, out_type):
    if out_type == OUT_F32:
        return raw.astype(np.float64)
    return (o.f16_to_f32(raw) if out_type == OUT_F16 else o.bf16_to_f32(raw)).astype(np.float64)


def _operands(m, n, k, in_type, seed=42, batches=1):
    r = o.JavaRandom(seed)
    mul = 1.0 / np.sqrt(np.float64(k))
    af = r.gaussian_f32(batches * m * k, mul)
    bf = r.gaussian_f32(batches * k * n, mul)
    if in_type == IN_F16:
        a, b = o.f32_to_f16(af), o.f32_to_f16(bf)
        return a, b, o.f16_to_f32(a), o.f16_to_f32(b)
    a, b = o.f32_to_bf16(af), o.f32_to_bf16(bf)
    return a, b, o.bf16_to_f32(a), o.bf16_to_f32(b)


def _product(af, bf, m, n, k):
    """fp32-accumulated reference loop (gemmReference / hgemmJava order: ascending k)."""
    return o.sgemm_seq(np.ascontiguousarray(af), np.ascontiguousarray(bf), m, n, k, threads=True)


@pytest.mark.parametrize("act", list(ACTS))
@pytest.mark.parametrize("out_type", [OUT_F16, OUT_F32])
def test_gemm_bias_activation(lib, act, out_type):
    """cutlassGemmBias{Relu,Gelu,Silu,Sigmoid,Tanh,HardSwish}: act(A*B + bias), the reference's 64^3 case and a
    ragged multi-tile one."""
    for (m, n, k) in [(64, 64, 64), (300, 264, 136)]:
        a, b, af, bf = _operands(m, n, k, IN_F16, 5)
        bias_f = o.JavaRandom(6).uniform_f32(n, -1, 1)
        bias = _to_out(bias_f, out_type)
        want = o.gemm_epilogue_ref(_product(af, bf, m, n, k), act, bias=_from_out(bias, out_type))
        da, db, dbias = DevBuf(a), DevBuf(b), DevBuf(bias)
        dd = out_buf(m * n, np.float32 if out_type == OUT_F32 else np.uint16)
        _ok(lib.tb200_gemm_ex(m, n, k, IN_F16, da.ptr, db.ptr, out_type, dd.ptr, 1.0, 0.0, None, dbias.ptr, ACTS[act], 1, stream_ptr()), lib)
        sync_and_check(lib)
        got = _from_out(dd.numpy(), out_type).reshape(m, n)
        assert np.abs(got - want).max() <= 0.05  # TestCutlass.java:326
        assert o.rel_l2(got, want) <= REL_L2[out_type], (act, o.rel_l2(got, want))
        assert dd.guard_intact()


@pytest.mark.parametrize("in_type,out_type", [(IN_F16, OUT_F16), (IN_BF16, OUT_BF16), (IN_BF16, OUT_F32), (IN_F16, OUT_F32)])
@pytest.mark.parametrize("m,n,k", [(128, 96, 64), (256, 256, 256), (1024, 512, 768), (130, 72, 40)])
def test_gemm_alpha_beta_typed_outputs(lib, in_type, out_type, m, n, k):
    """cutlassHgemm / cutlassBgemm / cublasGemmEx: D = alpha*A*B + beta*C with fp16, bf16 or fp32 results."""
    a, b, af, bf = _operands(m, n, k, in_type, 9)
    c_f = o.JavaRandom(10).uniform_f32(m * n, -1, 1)
    c = _to_out(c_f, out_type)
    prod = _product(af, bf, m, n, k)
    da, db = DevBuf(a), DevBuf(b)
    for alpha, beta, in_place in [(1.0, 0.0, False), (0.5, 2.0, False), (1.5, -1.0, True)]:
        want = o.gemm_epilogue_ref(prod, "none", alpha, beta, _from_out(c, out_type).reshape(m, n))
        dd = DevBuf(c.copy()) if in_place else out_buf(m * n, np.float32 if out_type == OUT_F32 else np.uint16)
        dc = DevBuf(c)
        _ok(lib.tb200_gemm_ex(m, n, k, in_type, da.ptr, db.ptr, out_type, dd.ptr, alpha, beta, None if in_place else dc.ptr, None, 0, 1,
                              stream_ptr()), lib)
        sync_and_check(lib)
        got = _from_out(dd.numpy(), out_type).reshape(m, n)
        tol = 5e-2 if out_type == OUT_BF16 else 2e-2  # TestCutlass.java:298, :246
        assert (np.abs(got - want) <= tol * np.maximum(1.0, np.abs(want))).all()
        assert o.rel_l2(got, want) <= REL_L2[out_type]
        assert dd.guard_intact()


@pytest.mark.parametrize("batches,m,n,k", [(4, 64, 64, 64), (3, 136, 200, 96), (32, 128, 128, 128)])
@pytest.mark.parametrize("out_type", [OUT_F16, OUT_F32])
def test_gemm_batched(lib, batches, m, n, k, out_type):
    """cutlassHgemmBatched: independent products packed back to back (strides m*k, k*n, m*n)."""
    a, b, af, bf = _operands(m, n, k, IN_F16, 21, batches)
    da, db = DevBuf(a), DevBuf(b)
    dd = out_buf(batches * m * n, np.float32 if out_type == OUT_F32 else np.uint16)
    _ok(lib.tb200_gemm_ex(m, n, k, IN_F16, da.ptr, db.ptr, out_type, dd.ptr, 1.0, 0.0, None, None, 0, batches, stream_ptr()), lib)
    sync_and_check(lib)
    got = _from_out(dd.numpy(), out_type).reshape(batches, m, n)
    for i in range(batches):
        want = _product(af[i * m * k:(i + 1) * m * k], bf[i * k * n:(i + 1) * k * n], m, n, k)
        assert np.abs(got[i] - want).max() <= 0.05  # TestCutlass.java:581
        assert o.rel_l2(got[i], want) <= REL_L2[out_type]
    assert dd.guard_intact()


@pytest.mark.parametrize("in_type,out_type", [(IN_F16, OUT_F16), (IN_BF16, OUT_BF16), (IN_F16, OUT_F32)])
@pytest.mark.parametrize("batches,m,n,k", [(1, 300, 264, 136), (1, 256, 512, 256), (3, 136, 200, 96)])
def test_gemm_ex_every_array_behind_a_24_byte_header(lib, in_type, out_type, batches, m, n, k):
    """TornadoVM's default array header: A, B, C, bias and D all 8 bytes past a 16-byte boundary, with the fused
    epilogue act(alpha*A*B + beta*C + bias), typed outputs and batches."""
    a, b, af, bf = _operands(m, n, k, in_type, 33, batches)
    c = _to_out(o.JavaRandom(34).uniform_f32(batches * m * n, -1, 1), out_type)
    bias = _to_out(o.JavaRandom(35).uniform_f32(n, -1, 1), out_type)
    da, db, dc, dbias = DevBuf(a, 24), DevBuf(b, 24), DevBuf(c, 24), DevBuf(bias, 24)
    dd = out_buf(batches * m * n, np.float32 if out_type == OUT_F32 else np.uint16, header=24)
    use_bias = batches == 1  # a batched call takes no bias row
    _ok(lib.tb200_gemm_ex(m, n, k, in_type, da.ptr, db.ptr, out_type, dd.ptr, 0.75, 0.5, dc.ptr, dbias.ptr if use_bias else None, ACTS["silu"], batches,
                          stream_ptr()), lib)
    sync_and_check(lib)
    got = _from_out(dd.numpy(), out_type).reshape(batches, m, n)
    cf = _from_out(c, out_type).reshape(batches, m, n)
    for i in range(batches):
        prod = _product(af[i * m * k:(i + 1) * m * k], bf[i * k * n:(i + 1) * k * n], m, n, k)
        want = o.gemm_epilogue_ref(prod, "silu", 0.75, 0.5, cf[i], bias=_from_out(bias, out_type) if use_bias else None)
        assert o.rel_l2(got[i], want) <= REL_L2[out_type], (i, o.rel_l2(got[i], want))
    assert dd.guard_intact() and dc.guard_intact() and dbias.guard_intact()


@pytest.mark.parametrize("header", [8, 16, 24, 40, 100, 120, 128])
@pytest.mark.parametrize("batches,m,n,k", [(1, 300, 288, 136), (1, 130, 1024, 64), (3, 136, 224, 96), (1, 128, 32, 64)])
def test_fp32_results_at_every_offset_from_a_line(lib, header, batches, m, n, k):
    """fp32 results whose rows are whole 128-byte lines (n % 32 == 0) into a destination `header` bytes past a line:
    the epilogue stores along the destination's lines (whole lines as TMA stores, the first and last segment of a tile
    and the matrix edges as 8-byte pieces).  Fused epilogue with C and bias at the same offset, ragged rows, several
    tile columns, batches; a 4-byte phase (header 100) takes the per-element stores.  Nothing around D is written."""
    a, b, af, bf = _operands(m, n, k, IN_F16, 51, batches)
    c = _to_out(o.JavaRandom(52).uniform_f32(batches * m * n, -1, 1), OUT_F32)
    bias = _to_out(o.JavaRandom(53).uniform_f32(n, -1, 1), OUT_F32)
    da, db, dc, dbias = DevBuf(a, 16), DevBuf(b, 16), DevBuf(c, header), DevBuf(bias, header)
    dd = out_buf(batches * m * n, np.float32, header=header)
    use_bias = batches == 1
    _ok(lib.tb200_gemm_ex(m, n, k, IN_F16, da.ptr, db.ptr, OUT_F32, dd.ptr, 1.25, -0.5, dc.ptr, dbias.ptr if use_bias else None, ACTS["tanh"], batches,
                          stream_ptr()), lib)
    sync_and_check(lib)
    got = dd.numpy().astype(np.float64).reshape(batches, m, n)
    cf = c.astype(np.float64).reshape(batches, m, n)
    for i in range(batches):
        prod = _product(af[i * m * k:(i + 1) * m * k], bf[i * k * n:(i + 1) * k * n], m, n, k)
        want = o.gemm_epilogue_ref(prod, "tanh", 1.25, -0.5, cf[i], bias=bias.astype(np.float64) if use_bias else None)
        assert o.rel_l2(got[i], want) <= REL_L2[OUT_F32], (i, o.rel_l2(got[i], want))
    assert dd.guard_intact() and dc.guard_intact()
    # the plain product into the same place: bit for bit what it is on a line
    if batches == 1:
        plain = [out_buf(m * n, np.float32, header=h) for h in (128, header)]
        for d in plain:
            _ok(lib.tb200_hgemm_f32(m, n, k, da.ptr, db.ptr, d.ptr, stream_ptr()), lib)
        sync_and_check(lib)
        assert np.array_equal(plain[0].numpy(), plain[1].numpy()) and plain[1].guard_intact()


def test_gemm_ex_equals_plain_entry_and_argument_errors(lib):
    m, n, k = 256, 384, 128
    a, b = o.make_hgemm(m, n, k, 3)
    da, db = DevBuf(a), DevBuf(b)
    d1, d2 = out_buf(m * n), out_buf(m * n)
    _ok(lib.tb200_hgemm_f32(m, n, k, da.ptr, db.ptr, d1.ptr, stream_ptr()), lib)
    _ok(lib.tb200_gemm_ex(m, n, k, IN_F16, da.ptr, db.ptr, OUT_F32, d2.ptr, 1.0, 0.0, None, None, 0, 1, stream_ptr()), lib)
    sync_and_check(lib)
    assert np.array_equal(d1.numpy(), d2.numpy())
    assert lib.tb200_gemm_ex(m, n, k, 7, da.ptr, db.ptr, OUT_F32, d2.ptr, 1.0, 0.0, None, None, 0, 1, stream_ptr()) == -1
    assert lib.tb200_gemm_ex(m, n, k, IN_F16, da.ptr, db.ptr, 5, d2.ptr, 1.0, 0.0, None, None, 0, 1, stream_ptr()) == -1
    assert lib.tb200_gemm_ex(m, n, k, IN_F16, da.ptr, db.ptr, OUT_F32, d2.ptr, 1.0, 0.0, None, None, 9, 1, stream_ptr()) == -1
    assert lib.tb200_gemm_ex(m, n, k, IN_F16, da.ptr, db.ptr, OUT_F32, None, 1.0, 0.0, None, None, 0, 1, stream_ptr()) == -1
    # a shape the tensor-core path does not take, with an epilogue the CUDA-core kernel does not have
    assert lib.tb200_gemm_ex(17, 19, 23, IN_F16, da.ptr, db.ptr, OUT_F16, d2.ptr, 1.0, 0.0, None, None, 1, 1, stream_ptr()) == -4
