"""GPU parity at the sizes the benchmark configurations name, and exact int32 block dots of the
tensor-core mat-vec kernel.

The full-size operands are generated on the device from seeded torch generators (synthetic data with
the shapes and value distributions of the configurations); the oracle checks sampled rows, and
size-independent properties cover the rest.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as o
from harness import DevBuf, out_buf, stream_ptr, sync_and_check

pytestmark = pytest.mark.gpu

REL_L2_FP32 = 1e-5   # FP32 results vs the fp64-accumulated oracle
REL_L2_FP16 = 2e-3   # FP16 GEMM vs the fp32-accumulated reference loop
OPT_INT_TC_MIN_BATCH = 6

P = lambda t: C.c_void_p(t.data_ptr())


def _ok(st, lib):
    assert st == 0, lib.tb200_status_string(st).decode()


def _gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


def _q8_blocks(rows, cols, seed):
    """Q8_0 34-byte blocks on the device: int8 U[-127,127], fp16 scale |N(0,1)| * 0.02."""
    g = _gen(seed)
    q = torch.randint(-127, 128, (rows, cols), dtype=torch.int8, device="cuda", generator=g)
    sc = (torch.randn((rows, cols // 32), device="cuda", generator=g).abs() * 0.02).half()
    blocks = torch.empty((rows, cols // 32, 34), dtype=torch.uint8, device="cuda")
    blocks[..., :2] = sc.view(torch.uint8).view(rows, cols // 32, 2)
    blocks[..., 2:] = q.view(torch.uint8).view(rows, cols // 32, 32)
    return q, sc, blocks


def _q4_blocks(rows, cols, seed):
    """Q4_0 18-byte blocks on the device: nibbles U[0,15], fp16 scale |N(0,1)| * 0.02."""
    g = _gen(seed)
    blocks = torch.randint(0, 256, (rows, cols // 32, 18), dtype=torch.uint8, device="cuda", generator=g)
    sc = (torch.randn((rows, cols // 32), device="cuda", generator=g).abs() * 0.02).half()
    blocks[..., :2] = sc.view(torch.uint8).view(rows, cols // 32, 2)
    return blocks


def _int_mode_want(fmt, wrows, x, cols):
    """Integer-mode result of the sampled rows: exact oracle dots combined in double."""
    n = wrows.shape[0]
    out = []
    for xb in x:
        xq, xs = o.quantize_x_block(np.ascontiguousarray(xb))
        if fmt == "q4b":
            flat = np.ascontiguousarray(wrows).ravel()
            dots = o.q4_blockdots_i32(flat, xq, cols, n)
            scales = o.block_scales(flat, n * (cols // 32), 18)
        else:
            flat = np.ascontiguousarray(wrows).ravel()
            scales = o.block_scales(flat, n * (cols // 32), 34)
            q = np.ascontiguousarray(wrows.reshape(n, cols // 32, 34)[..., 2:]).view(np.int8).ravel()
            dots = o.q8_blockdots_i32(q, xq, cols, n)
        out.append(o.blockdots_combine_f64(dots, scales, xs, cols // 32, n))
    return np.stack(out)


# --------------------------------------------------------------------------- exact dots of the tensor-core kernel
@pytest.mark.parametrize("rows,cols,batch", [(512, 4096, 4), (200, 4096, 8), (65, 14336, 16), (33, 256, 1), (100, 2048, 3), (1000, 1024, 16)])
@pytest.mark.parametrize("fmt", [0, 1, 2])
@pytest.mark.parametrize("header", [16, 24])
def test_tensor_core_block_dots_bit_exact(lib, rows, cols, batch, fmt, header):
    """Every int32 block dot that mma.sync.m16n8k32.s8 produces -- all columns of the tiles, i.e. every
    activation vector of a batch -- equals the oracle's dp4a restatement (QuantizationTests.testDP4A)."""
    rng = o.JavaRandom(17)
    xq = (rng.ints(cols * batch, 255) - 127).astype(np.int8)
    if fmt == 2:
        w, _, _ = o.make_q4(rows, cols)
        want = np.stack([o.q4_blockdots_i32(w, xq[b * cols:(b + 1) * cols], cols, rows) for b in range(batch)])
    else:
        q, s, _ = o.make_q8(rows, cols)
        want = np.stack([o.q8_blockdots_i32(q, xq[b * cols:(b + 1) * cols], cols, rows) for b in range(batch)])
        w = q if fmt == 0 else o.q8_pack_blocks(q, s)
    dw, dxq = DevBuf(w, header), DevBuf(xq, 16)
    dd = out_buf(batch * rows * (cols // 32), np.int32, header)
    _ok(lib.tb200_blockdots_i32_batched(fmt, rows, cols, batch, dw.ptr, dxq.ptr, dd.ptr, stream_ptr()), lib)
    sync_and_check(lib)
    assert np.array_equal(dd.numpy().reshape(batch, -1), want)
    assert dd.guard_intact() and dw.guard_intact()


@pytest.mark.parametrize("fmt", ["q8", "q8b", "q4b"])
def test_single_vector_dots_entry_on_tensor_cores(lib, fmt):
    """With the tensor-core threshold at 1 the one-vector block-dot entries run on the same kernel."""
    rows, cols = 300, 4096
    xq = (o.JavaRandom(5).ints(cols, 255) - 127).astype(np.int8)
    dxq, dd = DevBuf(xq), out_buf(rows * (cols // 32), np.int32)
    _ok(lib.tb200_set_thread_option(OPT_INT_TC_MIN_BATCH, 1), lib)
    try:
        if fmt == "q4b":
            w, _, _ = o.make_q4(rows, cols)
            dw = DevBuf(w)
            _ok(lib.tb200_q4b_blockdots_i32(rows, cols, dw.ptr, dxq.ptr, dd.ptr, stream_ptr()), lib)
            want = o.q4_blockdots_i32(w, xq, cols, rows)
        else:
            q, s, _ = o.make_q8(rows, cols)
            want = o.q8_blockdots_i32(q, xq, cols, rows)
            if fmt == "q8":
                dw = DevBuf(q)
                _ok(lib.tb200_q8_blockdots_i32(rows, cols, dw.ptr, dxq.ptr, dd.ptr, stream_ptr()), lib)
            else:
                dw = DevBuf(o.q8_pack_blocks(q, s))
                _ok(lib.tb200_q8b_blockdots_i32(rows, cols, dw.ptr, dxq.ptr, dd.ptr, stream_ptr()), lib)
    finally:
        lib.tb200_clear_thread_options()
    sync_and_check(lib)
    assert np.array_equal(dd.numpy(), want)


# --------------------------------------------------------------------------- FP32 mat-vec, 8192 x 8192
def test_sgemv_8192_full(lib):
    rows = cols = 8192
    m, v = o.make_sgemv(rows, cols)
    tm, tv = torch.from_numpy(m).cuda(), torch.from_numpy(v).cuda()
    out = torch.full((rows,), float("nan"), device="cuda")
    _ok(lib.tb200_sgemv(rows, cols, P(tm), P(tv), P(out), stream_ptr()), lib)
    sync_and_check(lib)
    got = out.cpu().numpy()
    y64 = o.sgemv_f64(m, v, cols, rows)
    err = o.rel_l2(got, y64)
    ref_err = max(o.rel_l2(o.sgemv_seq(m, v, cols, rows, threads=True), y64), o.rel_l2(o.sgemv_workgroup(m, v, cols, rows, 32), y64))
    assert err <= REL_L2_FP32 and err <= max(ref_err, 2e-7), (err, ref_err)


# --------------------------------------------------------------------------- Q8_0 14336 x 4096
@pytest.mark.parametrize("batch", [1, 8])
@pytest.mark.parametrize("mode", ["int", "float"])
def test_q8_14336x4096(lib, batch, mode):
    rows, cols = 14336, 4096
    q, sc, blocks = _q8_blocks(rows, cols, 21)
    x = torch.randn((batch, cols), device="cuda", generator=_gen(22))
    y = torch.full((batch, rows), float("nan"), device="cuda")
    if mode == "int":
        n = lib.tb200_qx_workspace_bytes(cols, batch)
        ws = torch.empty(n, dtype=torch.uint8, device="cuda")
        _ok(lib.tb200_q8b_gemv_i8(rows, cols, batch, P(blocks), P(x), P(y), P(ws), n, stream_ptr()), lib)
    else:
        _ok(lib.tb200_q8b_gemv(rows, cols, batch, P(blocks), P(x), P(y), stream_ptr()), lib)
    sync_and_check(lib)
    got = y.cpu().numpy()
    assert not np.isnan(got).any()
    idx = np.arange(0, rows, 7)  # 2048 rows
    xh = x.cpu().numpy()
    wr = blocks.cpu().numpy().reshape(rows, -1)[idx]
    if mode == "int":
        want = _int_mode_want("q8b", wr, xh, cols)
    else:
        qh = np.ascontiguousarray(q.cpu().numpy()[idx]).ravel()
        sh = np.ascontiguousarray(sc.cpu().numpy().view(np.uint16)[idx]).ravel()
        want = np.stack([o.q8_gemv_f64(qh, sh, xh[b], cols, len(idx)) for b in range(batch)])
    assert o.rel_l2(got[:, idx], want) <= REL_L2_FP32


def test_q8_grouped_32x14336x4096(lib):
    """The benchmark's headline launch: 32 matrices, one grouped integer-mode launch."""
    rows, cols, count = 14336, 4096, 32
    mats = [_q8_blocks(rows, cols, 100 + m)[2] for m in range(count)]
    x = torch.randn((1, cols), device="cuda", generator=_gen(5))
    y = torch.full((count, rows), float("nan"), device="cuda")
    wp = (C.c_void_p * count)(*[t.data_ptr() for t in mats])
    dp = (C.c_void_p * 1)(y.data_ptr())
    _ok(lib.tb200_q8b_gemv_i8_grouped(count, rows, cols, 1, wp, P(x), dp, 1, 0, None, rows, 0, None, 0, stream_ptr()), lib)
    sync_and_check(lib)
    got = y.cpu().numpy()
    assert not np.isnan(got).any()
    xh = x.cpu().numpy()
    idx = np.arange(3, rows, 29)
    for m in (0, 13, 22, 31):
        wr = mats[m].cpu().numpy().reshape(rows, -1)[idx]
        assert o.rel_l2(got[m, idx], _int_mode_want("q8b", wr, xh, cols)[0]) <= REL_L2_FP32
    # every matrix of the group equals its own single launch bit for bit
    n = lib.tb200_qx_workspace_bytes(cols, 1)
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    y1 = torch.empty(rows, device="cuda")
    for m in (1, 30):
        _ok(lib.tb200_q8b_gemv_i8(rows, cols, 1, P(mats[m]), P(x), P(y1), P(ws), n, stream_ptr()), lib)
        sync_and_check(lib)
        assert torch.equal(y1, y[m])


# --------------------------------------------------------------------------- Q4_0 decode layer shapes
Q4_SHAPES = [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336), (128256, 4096)]


@pytest.mark.parametrize("rows,cols", Q4_SHAPES)
@pytest.mark.parametrize("batch", [1, 4, 16])
def test_q4_layer_shapes_int_mode(lib, rows, cols, batch):
    blocks = _q4_blocks(rows, cols, 7 + rows % 97)
    x = torch.randn((batch, cols), device="cuda", generator=_gen(8))
    y = torch.full((batch, rows), float("nan"), device="cuda")
    n = lib.tb200_qx_workspace_bytes(cols, batch)
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    _ok(lib.tb200_q4b_gemv_i8(rows, cols, batch, P(blocks), P(x), P(y), P(ws), n, stream_ptr()), lib)
    sync_and_check(lib)
    got = y.cpu().numpy()
    assert not np.isnan(got).any()
    idx = np.unique(np.concatenate([np.arange(0, rows, max(1, rows // 512)), [rows - 1]]))
    wr = blocks.cpu().numpy().reshape(rows, -1)[idx]
    assert o.rel_l2(got[:, idx], _int_mode_want("q4b", wr, x.cpu().numpy(), cols)) <= REL_L2_FP32


@pytest.mark.parametrize("rows,cols", [(14336, 4096), (4096, 14336), (128256, 4096)])
@pytest.mark.parametrize("batch", [1, 4, 16])
def test_q4_layer_shapes_float_mode(lib, rows, cols, batch):
    blocks = _q4_blocks(rows, cols, 9 + rows % 97)
    x = torch.randn((batch, cols), device="cuda", generator=_gen(10))
    y = torch.full((batch, rows), float("nan"), device="cuda")
    _ok(lib.tb200_q4b_gemv(rows, cols, batch, P(blocks), P(x), P(y), stream_ptr()), lib)
    sync_and_check(lib)
    got = y.cpu().numpy()
    assert not np.isnan(got).any()
    idx = np.unique(np.concatenate([np.arange(0, rows, max(1, rows // 256)), [rows - 1]]))
    wr = np.ascontiguousarray(blocks.cpu().numpy().reshape(rows, -1)[idx]).ravel()
    xh = x.cpu().numpy()
    want = np.stack([o.q4_gemv_f64(wr, xh[b], cols, len(idx)) for b in range(batch)])
    assert o.rel_l2(got[:, idx], want) <= REL_L2_FP32


# --------------------------------------------------------------------------- float mode: range of the activations
@pytest.mark.parametrize("scale", [1e-6, 1e6, 3e-30, 1e30])
@pytest.mark.parametrize("fmt", ["q8", "q8b", "q4b"])
@pytest.mark.parametrize("batch", [1, 3, 8])
def test_float_mode_activation_range(lib, scale, fmt, batch):
    """fp32 activations far outside the fp16 range, and vectors of mixed magnitude in one batch."""
    rows, cols = 96, 4096
    if fmt == "q4b":
        blocks, _, x = o.make_q4(rows, cols, batch)
    else:
        q, s, x = o.make_q8(rows, cols, batch)
        blocks = o.q8_pack_blocks(q, s)
    x = x.reshape(batch, cols).copy()
    x[0] *= np.float32(scale)
    if batch > 1:
        x[1, ::7] *= np.float32(1e-4)  # small entries next to ordinary ones
    x = np.ascontiguousarray(x.ravel())
    dx, dy = DevBuf(x), out_buf(rows * batch)
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
    got = dy.numpy().reshape(batch, rows)
    for b in range(batch):
        xb = x[b * cols:(b + 1) * cols]
        want = o.q4_gemv_f64(blocks, xb, cols, rows) if fmt == "q4b" else o.q8_gemv_f64(q, s, xb, cols, rows)
        assert np.isfinite(got[b]).all()
        assert o.rel_l2(got[b], want) <= REL_L2_FP32, (b, o.rel_l2(got[b], want))


# --------------------------------------------------------------------------- FP16 GEMM sweep sizes
@pytest.mark.parametrize("n", [4096, 8192, 16384])
def test_hgemm_sweep_sizes_rows_sampled(lib, n):
    g = _gen(n)
    a = (torch.randn((n, n), device="cuda", generator=g) / n**0.5).half()
    b = (torch.randn((n, n), device="cuda", generator=g) / n**0.5).half()
    c = torch.full((n, n), float("nan"), device="cuda")
    _ok(lib.tb200_hgemm_f32(n, n, n, P(a), P(b), P(c), stream_ptr()), lib)
    sync_and_check(lib)
    rows = [0, 1, 127, 128, n // 2 + 5, n - 257, n - 129, n - 1]
    ah = np.ascontiguousarray(a[rows].cpu().numpy().view(np.uint16)).ravel()
    bh = b.cpu().numpy().view(np.uint16).ravel()
    want = o.hgemm_ref(ah, bh, len(rows), n, n)
    got = c[rows].cpu().numpy()
    assert o.rel_l2(got, want) <= REL_L2_FP16
    assert np.abs(got - want).max() <= 0.01  # TestMatrixMultiplicationMMA.java:370
    # checksum of checksums over the whole product: (1^T A)(B 1) == 1^T C 1, in double
    lhs = (a.double().sum(0) * b.double().sum(1)).sum().item()
    rhs = c.double().sum().item()
    scale = (a.double().abs().sum(0) * b.double().abs().sum(1)).sum().item()
    assert not torch.isnan(c).any()
    assert abs(lhs - rhs) / scale < 1e-6
