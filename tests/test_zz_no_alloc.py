"""The allocation-free Q8_0 entry point against the workspace-taking one.

Some callers of this library cannot allocate device memory at the point where
they launch: a TornadoVM provider may only enqueue work from ``dispatch`` (the
runtime owns the plan's device memory and a capture may be in progress), and a
program that is already capturing a stream cannot call cudaMalloc at all.
``tb200_q8_gemv_i8_static`` serves them by keeping the quantised activations in
a fixed array inside the library.  This file is collected last on purpose, so a
failure here cannot hide the result of any other test.
"""
import numpy as np
import pytest

import oracle as o
from harness import DevBuf, out_buf, stream_ptr, sync_and_check

pytestmark = pytest.mark.gpu

REL_L2 = 1e-5  # the tolerance of the other integer-path tests


@pytest.mark.parametrize("rows,cols,batch", [(300, 4096, 1), (64, 4096, 8), (40, 14336, 5), (9, 96, 2)])
def test_static_scratch_entry_matches_workspace_entry_twice(lib, rows, cols, batch):
    q, s, _ = o.make_q8(rows, cols, 1)
    dq, ds = DevBuf(q), DevBuf(s)
    n = lib.tb200_qx_workspace_bytes(cols, batch)
    ws = DevBuf(np.zeros(n, np.uint8))
    for call in range(2):  # the second call finds the first call's bytes in the shared array
        x = o.JavaRandom(7 + call).gaussian_f32(cols * batch) * np.float32(1 + 3 * call)
        dx = DevBuf(x)
        y_ws, y_static = out_buf(rows * batch), out_buf(rows * batch)
        st = lib.tb200_q8_gemv_i8(rows, cols, batch, dq.ptr, ds.ptr, dx.ptr, y_ws.ptr, ws.ptr, n, stream_ptr())
        assert st == 0, lib.tb200_status_string(st)
        st = lib.tb200_q8_gemv_i8_static(rows, cols, batch, dq.ptr, ds.ptr, dx.ptr, y_static.ptr, stream_ptr())
        assert st == 0, lib.tb200_status_string(st)
        sync_and_check(lib)
        a, b = y_ws.numpy(), y_static.numpy()
        assert not np.isnan(b).any()
        assert o.rel_l2(b, a) <= REL_L2
        # and both agree with the oracle's exact block dots combined in double
        want = []
        for bb in range(batch):
            xq, xs = o.quantize_x_block(x[bb * cols:(bb + 1) * cols])
            want.append(o.blockdots_combine_f64(o.q8_blockdots_i32(q, xq, cols, rows), s, xs, cols // 32, rows))
        assert o.rel_l2(b.reshape(batch, rows), np.stack(want)) <= REL_L2
        assert y_static.guard_intact()


def test_static_scratch_entry_rejects_oversized_shapes(lib):
    d = DevBuf(np.zeros(64, np.float32))
    # 16384 columns x 16 vectors needs 294912 bytes of scratch: more than the built-in array
    assert lib.tb200_qx_workspace_bytes(16384, 16) > 147456
    assert lib.tb200_q8_gemv_i8_static(4, 16384, 16, d.ptr, d.ptr, d.ptr, d.ptr, stream_ptr()) == -3
    assert lib.tb200_status_string(-3) == b"TB200_ERR_WORKSPACE"
    assert lib.tb200_q8_gemv_i8_static(4, 33, 1, d.ptr, d.ptr, d.ptr, d.ptr, stream_ptr()) == -1
