"""Worker of tests/test_multi_gpu.py: one process per GPU (launched by torch.distributed.run).

Checks the RESULTS of the multi-GPU paths against the CPU oracle on every rank: the row-sharded grouped
mat-vec whose kernel stores its outputs into every GPU's buffer (consecutive steps with changing
activations, so output slots are reused; ragged row shards), and the column-sharded FP16 GEMM whose epilogue
stores every tile to every GPU.  Plain peer loads and stores only.
"""
import datetime
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import oracle as o  # noqa: E402
from tornadovm_b200.peer import ShardedGroupedGemv  # noqa: E402
from tornadovm_b200.sharding import ShardedHgemm, shard_cols, shard_range, take_cols  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # a short collective time-out: a rank that fails must not keep the others (and the GPUs) waiting for minutes
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    ok = True

    # ---- grouped Q8_0 / Q4_0 mat-vec, rows sharded (the last rank owns fewer rows) ----
    for fmt, rows, cols, batch, count in [("q8b", 1000 + world + 1, 1024, 1, 3), ("q4b", 515, 2048, 2, 2)]:
        mats = []
        for m in range(count):
            if fmt == "q8b":
                q, s, _ = o.make_q8(rows, cols, batch, 700 + m)
                mats.append((o.q8_pack_blocks(q, s), q, s))
            else:
                blocks, s, _ = o.make_q4(rows, cols, batch, 700 + m)
                mats.append((blocks, None, s))
        bb = 34 if fmt == "q8b" else 18
        r0, r1 = shard_range(rows, world, rank)
        row_bytes = cols // 32 * bb
        shards = [torch.from_numpy(np.ascontiguousarray(b[r0 * row_bytes:r1 * row_bytes])).to(dev) for b, _, _ in mats]
        op = ShardedGroupedGemv(rows, cols, batch, shards, fmt, per_launch=2, nslots=2)
        try:
            xh = torch.empty((batch, cols)).pin_memory()  # one pinned buffer: the graph-replayed steps read it in place
            for step in range(8):
                x = o.JavaRandom(900 + step).gaussian_f32(batch * cols)
                xh.copy_(torch.from_numpy(x).reshape(batch, cols))
                # plain steps first, then steps replayed from the per-slot CUDA graphs (captured at steps 3 and 4)
                got = op.run(xh, graph=step >= 3).numpy().copy()
                for m, (blocks, q, s) in enumerate(mats):
                    for b in range(batch):
                        xq, xs = o.quantize_x_block(np.ascontiguousarray(x[b * cols:(b + 1) * cols]))
                        dots = o.q8_blockdots_i32(q, xq, cols, rows) if fmt == "q8b" else o.q4_blockdots_i32(blocks, xq, cols, rows)
                        want = o.blockdots_combine_f64(dots, s, xs, cols // 32, rows)
                        err = o.rel_l2(got[m, b], want)
                        if not err <= 1e-5:
                            print(f"rank {rank}: {fmt} step {step} matrix {m} vector {b}: rel-L2 {err}", flush=True)
                            ok = False
        finally:
            op.close()

    # ---- FP16 GEMM, B and C sharded by columns, gather fused into the epilogue ----
    for layout in ("assembled", "blocks"):
        m, n, k = 384, 256 * world, 192
        a16, b16 = o.make_hgemm(m, n, k, 31)
        a = torch.from_numpy(a16.view(np.float16).reshape(m, k)).to(dev)
        b = torch.from_numpy(b16.view(np.float16).reshape(k, n)).to(dev)
        op = ShardedHgemm(m, n, k, a, take_cols(b, n, world, rank), fused=True, layout=layout)
        try:
            want = o.hgemm_ref(a16, b16, m, n, k)
            for step in range(3):
                with torch.cuda.stream(op.stream):
                    c = op.launch_fused().clone()
                op.stream.synchronize()
                op.check()
                got = c.cpu().numpy()
                if layout == "blocks":  # [world][m][per] -> [m][n]
                    got = got.transpose(1, 0, 2).reshape(m, world * shard_cols(n, world))[:, :n]
                err = o.rel_l2(got, want)
                if not err <= 2e-3:
                    print(f"rank {rank}: hgemm {layout} step {step}: rel-L2 {err}", flush=True)
                    ok = False
        finally:
            op.close()

    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("MULTI_GPU_OK" if flag.item() else "MULTI_GPU_FAILED", flush=True)
    sys.exit(0 if flag.item() else 1)


if __name__ == "__main__":
    main()
