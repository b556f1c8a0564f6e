"""GPU parity: FP32 / Q8_0 / Q4_0 mat-vec through the C ABI against the CPU oracle."""
import ctypes as C

import numpy as np
import pytest

import oracle as o
from harness import DevBuf, out_buf, stream_ptr, sync_and_check

pytestmark = pytest.mark.gpu

# FP32 results: relative L2 against the fp64-accumulated oracle, and no worse than
# the reference's own kernels (sequential and work-group order) on the same inputs.
REL_L2_FP32 = 1e-5


def _ok(st, lib):
    assert st == 0, lib.tb200_status_string(st).decode()


# --------------------------------------------------------------------------- FP32
@pytest.mark.parametrize("rows,cols", [(2048, 8192), (128, 4096), (7, 1028), (33, 36), (5, 3), (1, 1), (300, 12), (64, 50000)])
@pytest.mark.parametrize("header", [16, 24])
def test_sgemv_matches_oracle(lib, rows, cols, header):
    m, v = o.make_sgemv(rows, cols)
    dm, dv, dout = DevBuf(m, header), DevBuf(v, header), out_buf(rows, header=header)
    _ok(lib.tb200_sgemv(rows, cols, dm.ptr, dv.ptr, dout.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    got = dout.numpy()
    y64 = o.sgemv_f64(m, v, cols, rows)
    err = o.rel_l2(got, y64)
    ref_err = max(o.rel_l2(o.sgemv_seq(m, v, cols, rows), y64), o.rel_l2(o.sgemv_workgroup(m, v, cols, rows, 32), y64))
    assert err <= REL_L2_FP32
    assert err <= max(ref_err, 2e-7), (err, ref_err)
    assert dout.guard_intact() and dm.guard_intact()
    # the reference's own acceptance: abs 1e-4 at |w| <= 0.1 (MatrixVectorRowMajor.java:54) -> scaled by 10 for [-1,1)
    assert np.abs(got - o.sgemv_seq(m, v, cols, rows)).max() <= 1e-3 * max(1.0, np.sqrt(cols / 8192))


def test_sgemv_mixed_phase_and_empty(lib):
    rows, cols = 64, 2048
    m, v = o.make_sgemv(rows, cols)
    dm, dv, dout = DevBuf(m, 16), DevBuf(v, 24), out_buf(rows)  # matrix and vector on different 16-byte phases
    _ok(lib.tb200_sgemv(rows, cols, dm.ptr, dv.ptr, dout.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    assert o.rel_l2(dout.numpy(), o.sgemv_f64(m, v, cols, rows)) <= REL_L2_FP32
    # rows == 0 is a no-op; cols == 0 writes zeros
    _ok(lib.tb200_sgemv(0, cols, dm.ptr, dv.ptr, dout.ptr, stream_ptr()), lib)
    z = out_buf(4)
    _ok(lib.tb200_sgemv(4, 0, dm.ptr, dv.ptr, z.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    assert (z.numpy() == 0).all()


def test_sgemv_argument_errors(lib):
    d = DevBuf(np.zeros(16, np.float32))
    assert lib.tb200_sgemv(-1, 4, d.ptr, d.ptr, d.ptr, stream_ptr()) == -1
    assert lib.tb200_sgemv(2, 2, None, d.ptr, d.ptr, stream_ptr()) == -1
    assert lib.tb200_sgemv(2, 2, C.c_void_p(d.ptr.value + 2), d.ptr, d.ptr, stream_ptr()) == -2


# --------------------------------------------------------------------------- quantised, float mode
def _q8_case(rows, cols, batch, seed=42):
    q, s, x = o.make_q8(rows, cols, batch, seed)
    return q, s, x, o.q8_pack_blocks(q, s)


def _q8_oracle(q, s, x, rows, cols, batch):
    y64 = np.stack([o.q8_gemv_f64(q, s, x[b * cols:(b + 1) * cols], cols, rows) for b in range(batch)])
    yref = np.stack([o.q8_gemv_ref(q, s, x[b * cols:(b + 1) * cols], cols, rows, 32) for b in range(batch)])
    return y64, yref


Q_SHAPES = [(1024, 4096, 1), (257, 4096, 1), (64, 14336, 1), (96, 2048, 2), (40, 4096, 3), (128, 4096, 8),
            (33, 256, 1), (16, 32, 1), (5, 96, 2), (24, 1024, 16), (3, 6400, 5)]


@pytest.mark.parametrize("rows,cols,batch", Q_SHAPES)
@pytest.mark.parametrize("layout", ["split", "blocks"])
@pytest.mark.parametrize("header", [16, 24])
def test_q8_gemv_float_mode(lib, rows, cols, batch, layout, header):
    q, s, x, blocks = _q8_case(rows, cols, batch)
    dx, dy = DevBuf(x, header), out_buf(rows * batch, header=header)
    if layout == "split":
        dq, ds = DevBuf(q, header), DevBuf(s, header)
        st = lib.tb200_q8_gemv(rows, cols, batch, dq.ptr, ds.ptr, dx.ptr, dy.ptr, stream_ptr())
    else:
        dq = DevBuf(blocks, header)
        st = lib.tb200_q8b_gemv(rows, cols, batch, dq.ptr, dx.ptr, dy.ptr, stream_ptr())
    _ok(st, lib)
    sync_and_check(lib)
    got = dy.numpy().reshape(batch, rows)
    y64, yref = _q8_oracle(q, s, x, rows, cols, batch)
    err = o.rel_l2(got, y64)
    assert err <= REL_L2_FP32
    assert err <= max(o.rel_l2(yref, y64), 3e-7), (err, o.rel_l2(yref, y64))
    assert dy.guard_intact() and dq.guard_intact()


@pytest.mark.parametrize("rows,cols,batch", [(512, 4096, 1), (100, 4096, 4), (64, 14336, 1), (9, 14336, 16), (33, 256, 1), (7, 64, 2)])
@pytest.mark.parametrize("header", [16, 24])
def test_q4_gemv_float_mode(lib, rows, cols, batch, header):
    blocks, scales, x = o.make_q4(rows, cols, batch)
    dw, dx, dy = DevBuf(blocks, header), DevBuf(x, header), out_buf(rows * batch, header=header)
    _ok(lib.tb200_q4b_gemv(rows, cols, batch, dw.ptr, dx.ptr, dy.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    got = dy.numpy().reshape(batch, rows)
    y64 = np.stack([o.q4_gemv_f64(blocks, x[b * cols:(b + 1) * cols], cols, rows) for b in range(batch)])
    yseq = np.stack([o.q4_gemv_seq(blocks, x[b * cols:(b + 1) * cols], cols, rows) for b in range(batch)])
    err = o.rel_l2(got, y64)
    assert err <= REL_L2_FP32 and err <= max(o.rel_l2(yseq, y64), 3e-7)
    assert dy.guard_intact() and dw.guard_intact()


TB200_OPT_FLOAT_TENSOR_CORES = 3


@pytest.mark.parametrize("rows,cols,batch", [(257, 4096, 1), (20000, 512, 2), (1024, 4096, 4), (100, 2048, 5), (48, 1024, 8), (31, 768, 16),
                                              (2400, 256, 3)])
@pytest.mark.parametrize("fmt", ["q8", "q8b", "q4b"])
@pytest.mark.parametrize("setting", [0, 2])
def test_float_mode_tensor_core_setting(lib, rows, cols, batch, fmt, setting):
    """Float mode on the CUDA cores (0) and forced onto the tensor cores (2): both within the fp32 bound."""
    if fmt == "q4b":
        blocks, _, x = o.make_q4(rows, cols, batch)
        y64 = np.stack([o.q4_gemv_f64(blocks, x[b * cols:(b + 1) * cols], cols, rows) for b in range(batch)])
        yref = np.stack([o.q4_gemv_seq(blocks, x[b * cols:(b + 1) * cols], cols, rows) for b in range(batch)])
    else:
        q, s, x, blocks = _q8_case(rows, cols, batch)
        y64, yref = _q8_oracle(q, s, x, rows, cols, batch)
    dx, dy = DevBuf(x), out_buf(rows * batch)
    _ok(lib.tb200_set_option(TB200_OPT_FLOAT_TENSOR_CORES, setting), lib)
    try:
        if fmt == "q8":
            dq, ds = DevBuf(q), DevBuf(s)
            st = lib.tb200_q8_gemv(rows, cols, batch, dq.ptr, ds.ptr, dx.ptr, dy.ptr, stream_ptr())
        elif fmt == "q8b":
            dq = DevBuf(blocks)
            st = lib.tb200_q8b_gemv(rows, cols, batch, dq.ptr, dx.ptr, dy.ptr, stream_ptr())
        else:
            dq = DevBuf(blocks)
            st = lib.tb200_q4b_gemv(rows, cols, batch, dq.ptr, dx.ptr, dy.ptr, stream_ptr())
        _ok(st, lib)
        sync_and_check(lib)
    finally:
        lib.tb200_set_option(TB200_OPT_FLOAT_TENSOR_CORES, 1)
    got = dy.numpy().reshape(batch, rows)
    err = o.rel_l2(got, y64)
    assert err <= REL_L2_FP32
    assert err <= max(o.rel_l2(yref, y64), 3e-7), (err, o.rel_l2(yref, y64))
    assert dy.guard_intact() and dq.guard_intact()


# --------------------------------------------------------------------------- integer path
def _workspace(lib, cols, batch):
    n = lib.tb200_qx_workspace_bytes(cols, batch)
    return DevBuf(np.zeros(n, np.uint8)), n


@pytest.mark.parametrize("cols,batch", [(4096, 1), (14336, 3), (32, 1), (256, 16)])
def test_quantize_x_bit_exact(lib, cols, batch):
    x = o.JavaRandom(5).gaussian_f32(cols * batch)
    x[:32] = 0.0  # an all-zero block takes scale 1
    ws, n = _workspace(lib, cols, batch)
    dx = DevBuf(x)
    _ok(lib.tb200_quantize_x(cols, batch, dx.ptr, ws.ptr, n, stream_ptr()), lib)
    sync_and_check(lib)
    raw = ws.numpy()
    xq = raw[:cols * batch].view(np.int8)
    off = (cols * batch + 15) // 16 * 16
    xs = raw[off:off + 4 * (cols // 32) * batch].view(np.float32)
    wq, wsc = o.quantize_x_block(x)
    assert np.array_equal(xq, wq) and np.array_equal(xs, wsc)
    assert ws.guard_intact()


@pytest.mark.parametrize("rows,cols", [(512, 4096), (65, 14336), (33, 256), (16, 32), (7, 6400)])
@pytest.mark.parametrize("fmt", ["q8", "q8b", "q4b"])
@pytest.mark.parametrize("header", [16, 24])
def test_int32_block_dots_bit_exact(lib, rows, cols, fmt, header):
    """Device form of QuantizationTests.testDP4A: every int32 block dot equals the oracle's."""
    rng = o.JavaRandom(11)
    xq = (rng.ints(cols, 255) - 127).astype(np.int8)
    ddots = out_buf(rows * (cols // 32), np.int32, header)
    dxq = DevBuf(xq, 16)
    if fmt == "q4b":
        blocks, _, _ = o.make_q4(rows, cols)
        dw = DevBuf(blocks, header)
        _ok(lib.tb200_q4b_blockdots_i32(rows, cols, dw.ptr, dxq.ptr, ddots.ptr, stream_ptr()), lib)
        want = o.q4_blockdots_i32(blocks, xq, cols, rows)
    else:
        q, s, _ = o.make_q8(rows, cols)
        want = o.q8_blockdots_i32(q, xq, cols, rows)
        if fmt == "q8":
            dw = DevBuf(q, header)
            _ok(lib.tb200_q8_blockdots_i32(rows, cols, dw.ptr, dxq.ptr, ddots.ptr, stream_ptr()), lib)
        else:
            dw = DevBuf(o.q8_pack_blocks(q, s), header)
            _ok(lib.tb200_q8b_blockdots_i32(rows, cols, dw.ptr, dxq.ptr, ddots.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    assert np.array_equal(ddots.numpy(), want)
    assert ddots.guard_intact()


def test_block_dots_unaligned_activations(lib):
    rows, cols = 40, 512
    q, s, _ = o.make_q8(rows, cols)
    xq = (o.JavaRandom(3).ints(cols, 255) - 127).astype(np.int8)
    dxq, dw, dd = DevBuf(xq, 17), DevBuf(q, 16), out_buf(rows * cols // 32, np.int32)
    _ok(lib.tb200_q8_blockdots_i32(rows, cols, dw.ptr, dxq.ptr, dd.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    assert np.array_equal(dd.numpy(), o.q8_blockdots_i32(q, xq, cols, rows))


@pytest.mark.parametrize("rows,cols,batch", [(512, 4096, 1), (96, 4096, 8), (64, 14336, 2), (20, 14336, 16), (33, 256, 1), (5, 96, 3),
                                             (200, 4096, 3), (33, 512, 9), (130, 2048, 16), (2500, 1024, 5)])
@pytest.mark.parametrize("fmt", ["q8", "q8b", "q4b"])
@pytest.mark.parametrize("header", [16, 24])
def test_gemv_int_mode(lib, rows, cols, batch, fmt, header):
    """y = sum_blk (float) dot * wscale * xscale against the same formula in double on the oracle's exact dots."""
    if fmt == "q4b":
        blocks, scales, x = o.make_q4(rows, cols, batch)
    else:
        q, scales, x = o.make_q8(rows, cols, batch)
        blocks = o.q8_pack_blocks(q, scales)
    ws, n = _workspace(lib, cols, batch)
    dx, dy = DevBuf(x, header), out_buf(rows * batch, header=header)
    if fmt == "q8":
        dq, ds = DevBuf(q, header), DevBuf(scales, header)
        st = lib.tb200_q8_gemv_i8(rows, cols, batch, dq.ptr, ds.ptr, dx.ptr, dy.ptr, ws.ptr, n, stream_ptr())
    elif fmt == "q8b":
        dq = DevBuf(blocks, header)
        st = lib.tb200_q8b_gemv_i8(rows, cols, batch, dq.ptr, dx.ptr, dy.ptr, ws.ptr, n, stream_ptr())
    else:
        dq = DevBuf(blocks, header)
        st = lib.tb200_q4b_gemv_i8(rows, cols, batch, dq.ptr, dx.ptr, dy.ptr, ws.ptr, n, stream_ptr())
    _ok(st, lib)
    sync_and_check(lib)
    got = dy.numpy().reshape(batch, rows)
    want = []
    for b in range(batch):
        xq, xs = o.quantize_x_block(x[b * cols:(b + 1) * cols])
        dots = o.q4_blockdots_i32(blocks, xq, cols, rows) if fmt == "q4b" else o.q8_blockdots_i32(q, xq, cols, rows)
        want.append(o.blockdots_combine_f64(dots, scales, xs, cols // 32, rows))
    assert o.rel_l2(got, np.stack(want)) <= REL_L2_FP32
    assert dy.guard_intact() and ws.guard_intact()


def test_int_mode_workspace_errors(lib):
    rows, cols = 8, 64
    q, s, x = o.make_q8(rows, cols)
    dq, ds, dx, dy = DevBuf(q), DevBuf(s), DevBuf(x), out_buf(rows)
    ws, n = _workspace(lib, cols, 1)
    assert lib.tb200_q8_gemv_i8(rows, cols, 1, dq.ptr, ds.ptr, dx.ptr, dy.ptr, ws.ptr, n - 1, stream_ptr()) == -3
    assert lib.tb200_q8_gemv_i8(rows, cols, 1, dq.ptr, ds.ptr, dx.ptr, dy.ptr, None, n, stream_ptr()) == -3
    assert lib.tb200_q8_gemv(rows, 33, 1, dq.ptr, ds.ptr, dx.ptr, dy.ptr, stream_ptr()) == -1
    assert lib.tb200_q8_gemv(rows, cols, 17, dq.ptr, ds.ptr, dx.ptr, dy.ptr, stream_ptr()) == -1


# --------------------------------------------------------------------------- full-size properties
def test_q8_full_size_linearity_and_row_shard_property(lib):
    """At the benchmark size the oracle is only sampled; linearity in x and the
    independence of rows (what row-sharding relies on) are checked on all outputs."""
    import torch
    rows, cols = 14336, 4096
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randint(-127, 128, (rows, cols), dtype=torch.int8, device="cuda", generator=g)
    sc = (torch.randn(rows, cols // 32, device="cuda", generator=g).abs() * 0.02).half()
    x1 = torch.randn(cols, device="cuda", generator=g)
    x2 = torch.randn(cols, device="cuda", generator=g)
    xb = torch.stack([x1, x2, x1 + x2]).contiguous()
    y = torch.full((3, rows), float("nan"), device="cuda")
    P = lambda t: C.c_void_p(t.data_ptr())
    _ok(lib.tb200_q8_gemv(rows, cols, 3, P(q), P(sc), P(xb), P(y), stream_ptr()), lib)
    # the same product on the lower half of the rows only == the lower half of the full product
    yh = torch.full((3, rows // 2), float("nan"), device="cuda")
    _ok(lib.tb200_q8_gemv(rows // 2, cols, 3, P(q[rows // 2:]), P(sc[rows // 2:]), P(xb), P(yh), stream_ptr()), lib)
    sync_and_check(lib)
    assert torch.equal(yh, y[:, rows // 2:])
    lin = (y[0] + y[1] - y[2]).norm() / y[2].norm()
    assert lin.item() < 1e-5
    # sampled rows against the oracle
    idx = np.arange(0, rows, 997)
    qh, sh = q.cpu().numpy(), sc.cpu().numpy().view(np.uint16)
    want = o.q8_gemv_f64(np.ascontiguousarray(qh[idx]).ravel(), np.ascontiguousarray(sh[idx]).ravel(), x1.cpu().numpy(), cols, len(idx))
    assert o.rel_l2(y[0].cpu().numpy()[idx], want) <= REL_L2_FP32
