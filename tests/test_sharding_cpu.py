"""Host-side sharding logic on CPU: world_size-2 gloo ranks, shard compute done by the oracle."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as o
from tornadovm_b200.sharding import col_range, gather_cols, gather_rows, shard_cols, shard_range, shard_rows, take_cols


def test_shard_ranges_cover_rows_exactly():
    for rows in (14336, 128256, 4096, 1024, 7, 1):
        for world in (1, 2, 4, 8):
            per = shard_rows(rows, world)
            spans = [shard_range(rows, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == rows
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(0 <= b - a <= per for a, b in spans)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, rows, cols, batch, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, s, x = o.make_q8(rows, cols, batch)
        r0, r1 = shard_range(rows, world, rank)
        per = shard_rows(rows, world)
        y_local = torch.zeros((batch, per), dtype=torch.float32)
        for b in range(batch):
            if r1 > r0:
                ys = o.q8_gemv_seq(np.ascontiguousarray(q.reshape(rows, cols)[r0:r1]).ravel(),
                                   np.ascontiguousarray(s.reshape(rows, -1)[r0:r1]).ravel(), x[b * cols:(b + 1) * cols], cols, r1 - r0)
                y_local[b, :r1 - r0] = torch.from_numpy(ys)
        y = gather_rows(y_local, rows)
        full = np.stack([o.q8_gemv_seq(q, s, x[b * cols:(b + 1) * cols], cols, rows) for b in range(batch)])
        ret[rank] = bool(np.array_equal(y.numpy(), full))
    finally:
        dist.destroy_process_group()


def _run(world, rows, cols, batch):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), rows, cols, batch, ret), nprocs=world, join=True)
    assert all(ret[r] for r in range(world)) and len(ret) == world


def test_row_sharded_gemv_gathers_bit_exact_world2():
    _run(2, 64, 256, 2)


def test_row_sharded_gemv_ragged_rows_world2():
    _run(2, 37, 128, 1)  # 19 + 18 rows: the padded tail of the last rank is trimmed


def test_col_ranges_cover_columns_in_multiples_of_eight():
    for n in (16384, 8192, 4096, 2048, 1000, 24, 8):
        for world in (1, 2, 4, 8):
            per = shard_cols(n, world)
            assert per % 8 == 0
            spans = [col_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def _gemm_worker(rank, world, port, m, n, k, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a16, b16 = o.make_hgemm(m, n, k)
        a = torch.from_numpy(a16.view(np.float16).reshape(m, k).astype(np.float32))
        b = torch.from_numpy(b16.view(np.float16).reshape(k, n).astype(np.float32))
        b_local = take_cols(b, n, world, rank)
        c_local = a @ b_local  # the shard's GEMM; on a GPU this is tb200_hgemm_f32 on the same operands
        full = a @ b
        c = gather_cols(c_local, n)
        blocks = gather_cols(c_local, n, assemble=False)
        c0, c1 = col_range(n, world, rank)
        ok = torch.allclose(c, full, rtol=1e-5, atol=1e-5) and c.shape == (m, n)
        ok = ok and torch.equal(blocks[rank][:, :c1 - c0], c_local[:, :c1 - c0]) and blocks.shape[0] == world
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_column_sharded_gemm_gathers_world2():
    for m, n, k in ((32, 64, 48), (16, 40, 24)):  # 40 columns: blocks of 24 + 16, the padded tail is trimmed
        mgr = mp.Manager()
        ret = mgr.dict()
        mp.spawn(_gemm_worker, args=(2, _free_port(), m, n, k, ret), nprocs=2, join=True)
        assert all(ret[r] for r in range(2)) and len(ret) == 2
