"""Grouped integer-mode mat-vec (one launch for several matrices), multi-destination stores and the
flag hand-shake, on one GPU: the peers of a multi-GPU group are stood in for by further buffers on
the same device."""
import ctypes as C

import numpy as np
import pytest

import oracle as o
from harness import DevBuf, out_buf, stream_ptr, sync_and_check

pytestmark = pytest.mark.gpu

TB200_ERR_TIMEOUT = -6
TB200_OPT_INT_TENSOR_CORE_MIN_BATCH = 6


def _ptr_array(bufs):
    return (C.c_void_p * len(bufs))(*[b.ptr.value for b in bufs])


def _case(fmt, rows, cols, batch, count):
    mats, x = [], None
    for m in range(count):
        if fmt == "q8b":
            q, s, xm = o.make_q8(rows, cols, batch, 100 + m)
            mats.append(o.q8_pack_blocks(q, s))
        else:
            blocks, _, xm = o.make_q4(rows, cols, batch, 100 + m)
            mats.append(blocks)
        x = xm if x is None else x
    return mats, x


def _single(lib, fmt, rows, cols, batch, dw, dx, dp4a=True):
    dy = out_buf(rows * batch)
    n = lib.tb200_qx_workspace_bytes(cols, batch)
    ws = DevBuf(np.zeros(max(n, 16), np.uint8))
    fn = lib.tb200_q8b_gemv_i8 if fmt == "q8b" else lib.tb200_q4b_gemv_i8
    # Bit-for-bit comparisons need the same fp32 summation order, i.e. the same kernel family.  Grouped launches
    # with several destinations or a hand-shake run the dp4a kernel, so the single launch is kept on it for those
    # (dp4a=True; from two vectors on it would otherwise take the tensor-core kernel).  A grouped launch into one
    # local buffer takes the tensor-core kernel itself from two vectors on, like the single launch (dp4a=False).
    if dp4a and batch <= 4:
        assert lib.tb200_set_thread_option(TB200_OPT_INT_TENSOR_CORE_MIN_BATCH, 17) == 0
    try:
        assert fn(rows, cols, batch, dw.ptr, dx.ptr, dy.ptr, ws.ptr, n, stream_ptr()) == 0
        sync_and_check(lib)
    finally:
        lib.tb200_clear_thread_options()
    return dy.numpy().reshape(batch, rows)


@pytest.mark.parametrize("rows,cols,batch,count", [(257, 4096, 1, 3), (64, 1024, 2, 32), (1000, 256, 4, 2), (5, 2048, 3, 7),
                                                   (40, 14336, 1, 2), (33, 96, 2, 3), (16, 4096, 8, 2)])
@pytest.mark.parametrize("fmt", ["q8b", "q4b"])
def test_grouped_equals_one_launch_per_matrix(lib, fmt, rows, cols, batch, count):
    mats, x = _case(fmt, rows, cols, batch, count)
    dws, dx = [DevBuf(m) for m in mats], DevBuf(x)
    dy = out_buf(count * batch * rows)
    n = lib.tb200_qx_workspace_bytes(cols, batch)
    ws = DevBuf(np.zeros(max(n, 16), np.uint8))
    fn = lib.tb200_q8b_gemv_i8_grouped if fmt == "q8b" else lib.tb200_q4b_gemv_i8_grouped
    st = fn(count, rows, cols, batch, _ptr_array(dws), dx.ptr, _ptr_array([dy]), 1, 0, None, rows, 0, ws.ptr, n, stream_ptr())
    assert st == 0, lib.tb200_status_string(st)
    sync_and_check(lib)
    got = dy.numpy().reshape(count, batch, rows)
    for m in range(count):
        want = _single(lib, fmt, rows, cols, batch, dws[m], dx, dp4a=False)
        assert np.array_equal(got[m], want), (m, np.abs(got[m] - want).max())
    assert dy.guard_intact()


@pytest.mark.parametrize("header", [8, 16, 24, 40, 64, 72, 112, 120])
@pytest.mark.parametrize("fmt,cols", [("q8b", 4096), ("q4b", 2048), ("q8b", 6144), ("q4b", 14336), ("q8b", 1280)])
def test_weights_at_every_byte_phase(lib, fmt, cols, header):
    """The ring kernels keep the byte phase of the weights (the offset from the 128-byte line below them) inside their
    ring slots.  Every multiple of 8, in a grouped launch and in one launch per matrix: the same bits as with weights on
    a 128-byte boundary, which the other tests hold against the oracle; nothing outside the matrices is needed (each
    sits in a buffer of its own, so the bytes in front of the first row and behind the last one are poison)."""
    rows, batch, count = 37, 1, 3
    mats, x = _case(fmt, rows, cols, batch, count)
    dx = DevBuf(x)
    fn = lib.tb200_q8b_gemv_i8_grouped if fmt == "q8b" else lib.tb200_q4b_gemv_i8_grouped
    results = []
    for h in (128, header):
        dws, dy = [DevBuf(m, h) for m in mats], out_buf(count * rows)
        assert all(d.ptr.value % 128 == h % 128 for d in dws)
        st = fn(count, rows, cols, batch, _ptr_array(dws), dx.ptr, _ptr_array([dy]), 1, 0, None, rows, 0, None, 0, stream_ptr())
        assert st == 0, lib.tb200_status_string(st)
        sync_and_check(lib)
        one = np.stack([_single(lib, fmt, rows, cols, batch, dws[m], dx)[0] for m in range(count)])
        results.append((dy.numpy().reshape(count, rows), one))
        assert dy.guard_intact()
    assert np.array_equal(results[0][0], results[1][0])
    assert np.array_equal(results[0][1], results[1][1])
    assert np.array_equal(results[0][0], results[0][1])


@pytest.mark.parametrize("header", [16, 24, 128])
def test_widest_rows_that_fit_the_ring(lib, header):
    """Four vectors of 18432 columns fill the shared memory of the ring kernel to the last byte when the weights sit on
    a 128-byte line; off the line the ring slots are 128 bytes longer.  Either way the launch is accepted and equals
    one launch per matrix."""
    rows, cols, batch, count = 9, 18432, 4, 2
    mats, x = _case("q8b", rows, cols, batch, count)
    dws, dx, dy = [DevBuf(m, header) for m in mats], DevBuf(x), out_buf(count * batch * rows)
    n = lib.tb200_qx_workspace_bytes(cols, batch)
    ws = DevBuf(np.zeros(max(n, 16), np.uint8))
    assert lib.tb200_set_thread_option(TB200_OPT_INT_TENSOR_CORE_MIN_BATCH, 17) == 0
    try:
        st = lib.tb200_q8b_gemv_i8_grouped(count, rows, cols, batch, _ptr_array(dws), dx.ptr, _ptr_array([dy]), 1, 0, None, rows, 0,
                                           ws.ptr, n, stream_ptr())
        assert st == 0, lib.tb200_status_string(st)
        sync_and_check(lib)
    finally:
        lib.tb200_clear_thread_options()
    got = dy.numpy().reshape(count, batch, rows)
    for m in range(count):
        assert np.array_equal(got[m], _single(lib, "q8b", rows, cols, batch, dws[m], dx))


def test_grouped_against_oracle(lib):
    rows, cols, count = 96, 4096, 4
    dws, want = [], []
    q0, s0, x = o.make_q8(rows, cols, 1, 7)
    xq, xs = o.quantize_x_block(x)
    for m in range(count):
        q, s, _ = o.make_q8(rows, cols, 1, 7 + m)
        dws.append(DevBuf(o.q8_pack_blocks(q, s)))
        dots = o.q8_blockdots_i32(q, xq, cols, rows)
        want.append(o.blockdots_combine_f64(dots, s, xs, cols // 32, rows))
    dx, dy = DevBuf(x), out_buf(count * rows)
    st = lib.tb200_q8b_gemv_i8_grouped(count, rows, cols, 1, _ptr_array(dws), dx.ptr, _ptr_array([dy]), 1, 0, None, rows, 0, None, 0,
                                       stream_ptr())
    assert st == 0
    sync_and_check(lib)
    got = dy.numpy().reshape(count, rows)
    assert o.rel_l2(got, np.stack(want)) <= 1e-5


@pytest.mark.parametrize("half", [0, 1])
def test_grouped_stores_to_every_destination_at_the_shard_offset(lib, half):
    rows, cols, batch, count, npeers = 120, 2048, 2, 3, 4
    rows_total, row_offset = 500, 260
    mats, x = _case("q8b", rows, cols, batch, count)
    dws, dx = [DevBuf(m) for m in mats], DevBuf(x)
    half_floats = count * batch * rows_total
    sentinel = np.float32(-777.0)
    dsts = [DevBuf(np.full(2 * half_floats, sentinel, np.float32)) for _ in range(npeers)]
    epoch = DevBuf(np.array([half + 4, 0, 0, 0], np.uint32))
    st = lib.tb200_q8b_gemv_i8_grouped(count, rows, cols, batch, _ptr_array(dws), dx.ptr, _ptr_array(dsts), npeers, half_floats,
                                       epoch.ptr, rows_total, row_offset, None, 0, stream_ptr())
    assert st == 0, lib.tb200_status_string(st)
    sync_and_check(lib)
    want = np.full((2, count, batch, rows_total), sentinel, np.float32)
    for m in range(count):
        want[half, m, :, row_offset:row_offset + rows] = _single(lib, "q8b", rows, cols, batch, dws[m], dx)
    for d in dsts:
        assert np.array_equal(d.numpy().reshape(want.shape), want)
        assert d.guard_intact()


def test_grouped_argument_errors(lib):
    rows, cols = 8, 256
    mats, x = _case("q8b", rows, cols, 1, 2)
    dws, dx, dy = [DevBuf(m) for m in mats], DevBuf(x), out_buf(2 * rows)
    f = lib.tb200_q8b_gemv_i8_grouped
    ok = lambda **k: f(k.get("count", 2), rows, cols, 1, _ptr_array(dws), dx.ptr, _ptr_array([dy]), k.get("npeers", 1), 0, None,
                       k.get("rows_total", rows), k.get("row_offset", 0), None, 0, stream_ptr())
    assert ok() == 0
    assert ok(count=0) == -1 and ok(count=33) == -1
    assert ok(npeers=0) == -1 and ok(npeers=9) == -1
    assert ok(rows_total=rows - 1) == -1 and ok(row_offset=1) == -1
    sync_and_check(lib)


def test_signal_wait_raises_flags_everywhere_and_advances_the_epoch(lib):
    npeers, rank = 4, 1
    arrays = [DevBuf(np.zeros(8, np.uint32)) for _ in range(npeers)]
    # the peers of this stand-in group have already signalled step 1 in this rank's array
    mine = np.zeros(8, np.uint32)
    mine[:npeers] = 1
    mine[rank] = 0
    arrays[rank] = DevBuf(mine)
    epoch = DevBuf(np.zeros(4, np.uint32))
    st = lib.tb200_peer_signal_wait(rank, npeers, _ptr_array(arrays), epoch.ptr, 200, stream_ptr())
    assert st == 0
    sync_and_check(lib)
    for a in arrays:
        assert a.numpy()[rank] == 1
    assert epoch.numpy()[0] == 1


def test_signal_wait_gives_up_after_its_time_limit(lib):
    npeers, rank = 2, 0
    arrays = [DevBuf(np.zeros(8, np.uint32)) for _ in range(npeers)]  # nothing ever raises peer 1's flag
    epoch = DevBuf(np.zeros(4, np.uint32))
    assert lib.tb200_peer_signal_wait(rank, npeers, _ptr_array(arrays), epoch.ptr, 20, stream_ptr()) == 0
    import torch
    torch.cuda.synchronize()
    status = C.c_int(0)
    assert lib.tb200_device_status(C.byref(status)) == 0
    assert status.value == TB200_ERR_TIMEOUT
    assert lib.tb200_device_status(C.byref(status)) == 0 and status.value == 0  # reading cleared it
    assert epoch.numpy()[0] == 1 and arrays[1].numpy()[0] == 1


def test_grouped_sync_announces_waits_and_rotates_slots(lib):
    """Three steps of the kernel that carries the hand-shake, as rank 0 of a stand-in group of two (two slots)."""
    import torch
    rows, cols, batch, count, npeers, rank, nslots = 300, 1024, 1, 2, 2, 0, 2
    rows_total = 600
    mats, x = _case("q8b", rows, cols, batch, count)
    dws, dx = [DevBuf(m) for m in mats], DevBuf(x)
    slot_floats = count * batch * rows_total
    dsts = [DevBuf(np.full(nslots * slot_floats, np.float32(-5.0), np.float32)) for _ in range(npeers)]
    flags = [DevBuf(np.zeros(8, np.uint32)) for _ in range(npeers)]
    sync = DevBuf(np.zeros(4, np.uint32))
    want = [_single(lib, "q8b", rows, cols, batch, dws[m], dx) for m in range(count)]

    def set_peer_flag(v):  # what the other rank has announced, in this rank's flag array
        flags[rank].t[flags[rank].header + 4:flags[rank].header + 8] = torch.tensor([v, 0, 0, 0], dtype=torch.uint8)

    def step(timeout_ms=200):
        st = lib.tb200_q8b_gemv_i8_grouped_sync(count, rows, cols, batch, _ptr_array(dws), dx.ptr, _ptr_array(dsts), npeers, rank,
                                                nslots, slot_floats, sync.ptr, _ptr_array(flags), 3, timeout_ms, rows_total, 0, None, 0,
                                                stream_ptr())
        assert st == 0, lib.tb200_status_string(st)
        torch.cuda.synchronize()

    def slots(d):
        return d.numpy().reshape(nslots, count, batch, rows_total)

    step()  # step 0 needs nothing from the peer
    sync_and_check(lib)
    assert sync.numpy()[0] == 1 and sync.numpy()[1] == 0 and all(f.numpy()[rank] == 0 for f in flags)
    for d in dsts:
        assert all(np.array_equal(slots(d)[0, m, :, :rows], want[m]) for m in range(count))
        assert (slots(d)[1] == -5.0).all() and (slots(d)[0, :, :, rows:] == -5.0).all()
    step()  # step 1 announces one finished step and needs the peer to have started step 0: already true
    sync_and_check(lib)
    assert sync.numpy()[0] == 2 and all(f.numpy()[rank] == 1 for f in flags)
    assert all(np.array_equal(slots(dsts[1])[1, m, :, :rows], want[m]) for m in range(count))
    # step 2 overwrites slot 0 and needs the peer to have started its step 1; nothing has announced that,
    # so the bounded wait gives up, records the fact and the kernel carries on
    step(timeout_ms=20)
    status = C.c_int(0)
    assert lib.tb200_device_status(C.byref(status)) == 0 and status.value == TB200_ERR_TIMEOUT
    assert sync.numpy()[0] == 3
    set_peer_flag(2)
    step()
    sync_and_check(lib)
    assert sync.numpy()[0] == 4 and all(f.numpy()[rank] == 3 for f in flags)
    # completion for a consumer: announce 4 finished steps, wait for the peer to announce as many
    assert lib.tb200_peer_wait(rank, npeers, _ptr_array(flags), sync.ptr, 20, stream_ptr()) == 0
    torch.cuda.synchronize()
    assert lib.tb200_device_status(C.byref(status)) == 0 and status.value == TB200_ERR_TIMEOUT  # peer is at 2 < 4
    assert all(f.numpy()[rank] == 4 for f in flags)
    set_peer_flag(4)
    assert lib.tb200_peer_wait(rank, npeers, _ptr_array(flags), sync.ptr, 20, stream_ptr()) == 0
    sync_and_check(lib)


@pytest.mark.parametrize("fmt", ["q8b", "q4b"])
@pytest.mark.parametrize("cols,batch", [(1024, 1), (4096, 2), (96, 1), (14336, 4), (4096, 8), (2048, 16), (4096, 9)])
def test_grouped_rows_of_different_shapes_equal_one_launch_per_matrix(lib, fmt, cols, batch):
    """The projections that read one vector (different row counts, one of them empty), each with its own output array."""
    rows = [300, 64, 0, 64, 1000, 17] if cols < 8192 else [40, 9, 0, 33]
    mats, x = [], None
    for m, r in enumerate(rows):
        ms, xm = _case(fmt, max(r, 1), cols, batch, 1)
        mats.append(ms[0])
        x = xm if x is None else x
    dws, dx = [DevBuf(m) for m in mats], DevBuf(x)
    dys = [out_buf(max(r, 1) * batch) for r in rows]
    n = lib.tb200_qx_workspace_bytes(cols, batch)
    ws = DevBuf(np.zeros(max(n, 16), np.uint8))
    fn = lib.tb200_q8b_gemv_i8_grouped_rows if fmt == "q8b" else lib.tb200_q4b_gemv_i8_grouped_rows
    st = fn(len(rows), (C.c_int * len(rows))(*rows), cols, batch, _ptr_array(dws), dx.ptr, _ptr_array(dys), ws.ptr, n, stream_ptr())
    assert st == 0, lib.tb200_status_string(st)
    sync_and_check(lib)
    for m, r in enumerate(rows):
        if r == 0:
            assert np.isnan(dys[m].numpy()).all()  # untouched
            continue
        want = _single(lib, fmt, r, cols, batch, dws[m], dx, dp4a=False)
        got = dys[m].numpy()[:batch * r].reshape(batch, r)
        assert np.array_equal(got, want), (m, r)
        assert dys[m].guard_intact()


@pytest.mark.parametrize("fmt", ["q8b", "q4b"])
@pytest.mark.parametrize("rows,cols,batch,count", [(144, 4096, 8, 5), (100, 1024, 2, 3), (16, 2048, 5, 32), (264, 256, 8, 2), (80, 4096, 16, 3),
                                                   (24, 1024, 11, 4)])
def test_matrices_back_to_back_run_as_one_tensor_core_launch(lib, fmt, rows, cols, batch, count):
    """Equally shaped matrices that lie back to back (the packed task's array) with two to eight vectors are one matrix
    of count * rows rows to the tensor-core kernel, which writes y[matrix][vector][row].  Bit for bit the results of one
    launch per matrix (a row's sums do not depend on how rows are dealt to CTAs); rows that are no multiple of 16 make
    a 16-row unit span two matrices."""
    mats, x = _case(fmt, rows, cols, batch, count)
    packed = DevBuf(np.concatenate(mats))
    per = mats[0].nbytes
    dx, dy = DevBuf(x), out_buf(count * batch * rows)
    n = lib.tb200_qx_workspace_bytes(cols, batch)
    ws = DevBuf(np.zeros(max(n, 16), np.uint8))
    ptrs = (C.c_void_p * count)(*[packed.ptr.value + m * per for m in range(count)])
    fn = lib.tb200_q8b_gemv_i8_grouped if fmt == "q8b" else lib.tb200_q4b_gemv_i8_grouped
    st = fn(count, rows, cols, batch, ptrs, dx.ptr, _ptr_array([dy]), 1, 0, None, rows, 0, ws.ptr, n, stream_ptr())
    assert st == 0, lib.tb200_status_string(st)
    sync_and_check(lib)
    got = dy.numpy().reshape(count, batch, rows)
    for m in range(count):
        want = _single(lib, fmt, rows, cols, batch, DevBuf(mats[m]), dx, dp4a=False)
        assert np.array_equal(got[m], want), (m, np.abs(got[m] - want).max())
    assert dy.guard_intact() and packed.guard_intact()
