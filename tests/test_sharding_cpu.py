"""Host-side sharding logic on CPU: world_size-2 gloo ranks, shard compute done by the oracle."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as o
from tornadovm_b200.sharding import gather_rows, shard_range, shard_rows


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
