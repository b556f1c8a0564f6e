"""The multi-GPU host classes in their one-rank form (no process group): same code path as a rank of a
group, with this GPU's slab as the only destination."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as o
from tornadovm_b200.native import B200Native

pytestmark = pytest.mark.gpu


def test_sharded_grouped_gemv_one_rank_matches_single_launches():
    from tornadovm_b200.peer import ShardedGroupedGemv
    rows, cols, count = 200, 2048, 5
    lib = B200Native.load()
    mats = []
    x = None
    for m in range(count):
        q, s, xm = o.make_q8(rows, cols, 1, 400 + m)
        mats.append(torch.from_numpy(o.q8_pack_blocks(q, s)).cuda())
        x = xm if x is None else x
    op = ShardedGroupedGemv(rows, cols, 1, mats, "q8b", per_launch=2)  # three launches per step: 2 + 2 + 1 matrices
    try:
        xh = torch.from_numpy(x).reshape(1, cols).pin_memory()
        for _ in range(3):
            y = op.run(xh).clone()
        # the same step replayed from a CUDA graph gives the same bits
        for _ in range(3):
            yg = op.run(xh, graph=True).clone()
        assert torch.equal(yg, y)
        ws_n = lib.tb200_qx_workspace_bytes(cols, 1)
        ws = torch.empty(ws_n, dtype=torch.uint8, device="cuda")
        xd = xh.cuda()
        one = torch.empty(rows, device="cuda")
        S = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        for m in range(count):
            assert lib.tb200_q8b_gemv_i8(rows, cols, 1, C.c_void_p(mats[m].data_ptr()), C.c_void_p(xd.data_ptr()),
                                         C.c_void_p(one.data_ptr()), C.c_void_p(ws.data_ptr()), ws_n, S) == 0
            torch.cuda.synchronize()
            assert torch.equal(y[m, 0], one.cpu())
        assert B200Native.device_status() == 0
    finally:
        op.close()


def test_sharded_hgemm_one_rank_fused_equals_plain():
    from tornadovm_b200.sharding import ShardedHgemm
    m, n, k = 256, 512, 128
    a16, b16 = o.make_hgemm(m, n, k)
    a = torch.from_numpy(a16.view(np.float16).reshape(m, k)).cuda()
    b = torch.from_numpy(b16.view(np.float16).reshape(k, n)).cuda()
    op = ShardedHgemm(m, n, k, a, b, fused=True)
    try:
        with torch.cuda.stream(op.stream):
            fused = op.launch_fused().clone()
            plain = op.launch(assemble=True).clone()
            best = op.launch_best().clone()
        op.stream.synchronize()
        assert torch.equal(fused, plain) and torch.equal(best, plain)
        assert o.rel_l2(plain.cpu().numpy().ravel(), o.hgemm_ref(a16, b16, m, n, k)) <= 2e-3
        assert B200Native.device_status() == 0
    finally:
        op.close()


def test_expired_device_wait_becomes_an_exception():
    """A bounded wait that ran out (here: a flag that nothing sets, 20 ms limit) must surface in the host
    classes: check() -- called by run() after every step -- raises instead of returning stale outputs."""
    from tornadovm_b200.native import TornadoB200Error
    from tornadovm_b200.peer import ShardedGroupedGemv
    rows, cols = 64, 1024
    lib = B200Native.load()
    q, s, x = o.make_q8(rows, cols, 1, 9)
    op = ShardedGroupedGemv(rows, cols, 1, [torch.from_numpy(o.q8_pack_blocks(q, s)).cuda()], "q8b")
    try:
        flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
        epoch = torch.zeros(4, dtype=torch.int32, device="cuda")
        fp = (C.c_void_p * 2)(*[f.data_ptr() for f in flags])
        S = C.c_void_p(op.stream.cuda_stream)
        assert lib.tb200_peer_signal_wait(0, 2, fp, C.c_void_p(epoch.data_ptr()), 20, S) == 0
        op.stream.synchronize()
        with pytest.raises(TornadoB200Error, match="TB200_ERR_TIMEOUT"):
            op.check()
        op.check()  # reading cleared it
        y = op.run(torch.from_numpy(x).reshape(1, cols).pin_memory())
        assert torch.isfinite(y).all()
    finally:
        op.close()
