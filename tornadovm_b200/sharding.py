"""Row / column sharding of the mat-vec and mat-mul tasks over the GPUs of one box.

One process per GPU (torch.distributed, NCCL over NVLink).  A GEMV shards by
rows: rank r owns a contiguous block of rows of W (whole Q8_0/Q4_0 block runs,
so any row split is byte-exact), the activation is replicated and the output
shards are all-gathered.  A GEMM shards B and C by N-columns the same way.
The reference has no counterpart: its multi-device mode runs independent tasks
on different devices with host round trips (docs/source/multi-device.rst:9-14).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .native import B200Native


def shard_rows(rows: int, world: int) -> int:
    """Rows per rank: equal blocks of ceil(rows / world); the last ranks may own fewer real rows."""
    return (rows + world - 1) // world


def shard_range(rows: int, world: int, rank: int) -> tuple[int, int]:
    per = shard_rows(rows, world)
    r0 = min(rank * per, rows)
    return r0, min(r0 + per, rows)


def gather_rows(y_local: torch.Tensor, rows: int, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather per-rank output blocks ``[batch][per]`` into ``[batch][rows]``.

    ``y_local`` always has ``per = shard_rows(rows, world)`` columns (ranks that
    own fewer rows leave the tail unused) so that the collective is one
    equal-sized all-gather.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return y_local[:, :rows]
    batch, per = y_local.shape
    if out is None:
        out = torch.empty((world, batch, per), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(out.view(-1), y_local.reshape(-1), group=group)
    # [world][batch][per] -> [batch][world*per] -> trim the padding of the last ranks
    return out.permute(1, 0, 2).reshape(batch, world * per)[:, :rows]


class ShardedQ8Gemv:
    """Q8_0 mat-vec whose weight rows are sharded over the ranks.

    ``weights`` is this rank's row block: 34-byte blocks (``scales=None``) or the
    split layout's int8 quants with ``scales`` its fp16 scales.  ``run(x_host)``
    is the end-to-end call: activation host->device, the local shard's GEMV
    through the C ABI (integer path by default), all-gather of the output shards
    over NCCL, gathered result device->host.
    """

    def __init__(self, rows: int, cols: int, batch: int, weights: torch.Tensor, scales: torch.Tensor | None = None,
                 group=None, exact_int: bool = True):
        self.rows, self.cols, self.batch, self.group = rows, cols, batch, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.per = shard_rows(rows, self.world)
        r0, r1 = shard_range(rows, self.world, self.rank)
        self.local_rows = r1 - r0
        per_row = cols if scales is not None else cols // 32 * 34
        assert weights.is_cuda and weights.numel() == self.local_rows * per_row
        self.w, self.scales, self.exact_int = weights, scales, exact_int
        dev = weights.device
        self.lib = B200Native.load()
        self.stream = torch.cuda.Stream(device=dev)
        self.x_dev = torch.empty((batch, cols), dtype=torch.float32, device=dev)
        self.y_local = torch.zeros((batch, self.per), dtype=torch.float32, device=dev)
        self.y_tmp = torch.empty((batch, max(self.local_rows, 1)), dtype=torch.float32, device=dev)
        self.gather_buf = torch.empty((self.world, batch, self.per), dtype=torch.float32, device=dev) if self.world > 1 else None
        self.y_host = torch.empty((batch, rows), dtype=torch.float32, pin_memory=True)
        self.ws_bytes = self.lib.tb200_qx_workspace_bytes(cols, batch)
        self.ws = torch.empty(max(self.ws_bytes, 16), dtype=torch.uint8, device=dev)

    def _gemv(self, y: torch.Tensor) -> None:
        P = lambda t: C.c_void_p(t.data_ptr())
        S = C.c_void_p(self.stream.cuda_stream)
        n, c, b = self.local_rows, self.cols, self.batch
        if self.scales is None:
            if self.exact_int:
                fn, st = "tb200_q8b_gemv_i8", self.lib.tb200_q8b_gemv_i8(n, c, b, P(self.w), P(self.x_dev), P(y), P(self.ws), self.ws_bytes, S)
            else:
                fn, st = "tb200_q8b_gemv", self.lib.tb200_q8b_gemv(n, c, b, P(self.w), P(self.x_dev), P(y), S)
        elif self.exact_int:
            fn, st = "tb200_q8_gemv_i8", self.lib.tb200_q8_gemv_i8(n, c, b, P(self.w), P(self.scales), P(self.x_dev), P(y), P(self.ws), self.ws_bytes, S)
        else:
            fn, st = "tb200_q8_gemv", self.lib.tb200_q8_gemv(n, c, b, P(self.w), P(self.scales), P(self.x_dev), P(y), S)
        B200Native.check_status(st, fn)

    def launch(self) -> torch.Tensor:
        """Enqueue GEMV + gather on this object's stream; returns the gathered device tensor."""
        with torch.cuda.stream(self.stream):
            if self.local_rows > 0:
                # y of the shard is [batch][local_rows]; it lands in the padded [batch][per] block
                tgt = self.y_local if self.local_rows == self.per else self.y_tmp
                self._gemv(tgt)
                if tgt is self.y_tmp:
                    self.y_local[:, :self.local_rows].copy_(self.y_tmp)
            return gather_rows(self.y_local, self.rows, self.group, self.gather_buf)

    def run(self, x_host: torch.Tensor) -> torch.Tensor:
        with torch.cuda.stream(self.stream):
            self.x_dev.copy_(x_host, non_blocking=True)
            y = self.launch()
            self.y_host.copy_(y, non_blocking=True)
        self.stream.synchronize()
        return self.y_host


# ---------------------------------------------------------------------------------------------
# FP16 GEMM: B and C sharded by N-columns, A replicated
# ---------------------------------------------------------------------------------------------
def shard_cols(n: int, world: int, multiple: int = 8) -> int:
    """Columns per rank: equal blocks, rounded up to ``multiple`` (the tensor-core kernel needs n % 8 == 0)."""
    per = (n + world - 1) // world
    return (per + multiple - 1) // multiple * multiple


def col_range(n: int, world: int, rank: int, multiple: int = 8) -> tuple[int, int]:
    per = shard_cols(n, world, multiple)
    c0 = min(rank * per, n)
    return c0, min(c0 + per, n)


def take_cols(b: torch.Tensor, n: int, world: int, rank: int) -> torch.Tensor:
    """This rank's column block of a row-major ``[k][n]`` matrix as a contiguous ``[k][per]`` matrix
    (zero-padded on the ranks whose block runs past n)."""
    per = shard_cols(n, world)
    c0, c1 = col_range(n, world, rank)
    out = torch.zeros((b.shape[0], per), dtype=b.dtype, device=b.device)
    out[:, :c1 - c0] = b[:, c0:c1]
    return out


def gather_cols(c_local: torch.Tensor, n: int, group=None, out: torch.Tensor | None = None, assemble: bool = True) -> torch.Tensor:
    """All-gather per-rank ``[m][per]`` column blocks.  ``assemble=False`` returns the gathered
    ``[world][m][per]`` buffer as it arrives (layout left to the consumer, no extra pass over C);
    ``assemble=True`` returns the row-major ``[m][n]`` matrix (one strided copy)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    m, per = c_local.shape
    if world == 1:
        return c_local[:, :n] if assemble else c_local.view(1, m, per)
    if out is None:
        out = torch.empty((world, m, per), dtype=c_local.dtype, device=c_local.device)
    dist.all_gather_into_tensor(out.view(-1), c_local.reshape(-1), group=group)
    if not assemble:
        return out
    return out.permute(1, 0, 2).reshape(m, world * per)[:, :n].contiguous()


class ShardedHgemm:
    """``C(fp32)[m][n] = A(fp16)[m][k] * B(fp16)[k][n]`` with B and C sharded by columns over the ranks.

    ``b_local`` is this rank's contiguous ``[k][shard_cols(n, world)]`` block (``take_cols``), ``a`` the
    replicated A.  Two ways to end with all of C on every rank:

    * ``launch()``: the local tcgen05 GEMM, then an NCCL all-gather of the C blocks (the unfused baseline);
    * ``launch_fused()`` (``fused=True``): the GEMM's epilogue stores every finished tile straight into the
      row-major ``[m][n]`` result of every rank (its own and, over NVLink, the peers' CUDA-IPC mapped ones),
      so the transfer overlaps the remaining tiles; one flag hand-shake kernel ends the step.  Needs
      ``n % world == 0`` and a column block that is a multiple of 8.
    """

    def __init__(self, m: int, n: int, k: int, a: torch.Tensor, b_local: torch.Tensor, group=None, fused: bool = False,
                 timeout_ms: int = 2000, layout: str = "auto"):
        # fused result: row-major [m][n] ("assembled"), or [world][m][per] like the all-gather ("blocks"); "auto" takes
        # the assembled matrix on one or two GPUs and blocks beyond: with rows 4*n bytes apart in many peer mappings
        # the stores are far slower than with rows 4*per bytes apart
        assert layout in ("auto", "assembled", "blocks")
        world_now = dist.get_world_size(group) if dist.is_initialized() else 1
        self.layout = layout if layout != "auto" else ("assembled" if world_now <= 2 else "blocks")
        self.m, self.n, self.k, self.group = m, n, k, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.per = shard_cols(n, self.world)
        assert a.is_cuda and a.dtype == torch.float16 and a.shape == (m, k)
        assert b_local.is_cuda and b_local.dtype == torch.float16 and b_local.shape == (k, self.per) and b_local.is_contiguous()
        self.a, self.b = a, b_local
        self.lib = B200Native.load()
        self.stream = torch.cuda.Stream(device=a.device)
        self.c_local = torch.empty((m, self.per), dtype=torch.float32, device=a.device)
        self.gathered = torch.empty((self.world, m, self.per), dtype=torch.float32, device=a.device) if self.world > 1 else None
        self.slab, self.timeout_ms, self.steps = None, timeout_ms, 0
        if fused:
            from .peer import PeerSlab  # local import: peer.py imports this module
            assert self.per * self.world == n, "the fused gather needs equal column blocks"
            self.slab = PeerSlab(2 * m * n * 4, a.device, group)  # two halves: a rank may still read the step before
            if self.layout == "assembled":
                self.halves = self.slab.bytes[:2 * m * n * 4].view(torch.float32).view(2, m, n)
                self._dst = [(C.c_void_p * self.world)(*[p + h * m * n * 4 for p in self.slab.ptrs]) for h in range(2)]
                self._ld, self._col = n, self.rank * self.per
            else:  # every rank's block is a dense [m][per] matrix: a tile's rows are 4 * per bytes apart instead of 4 * n
                self.halves = self.slab.bytes[:2 * m * n * 4].view(torch.float32).view(2, self.world, m, self.per)
                self._dst = [(C.c_void_p * self.world)(*[p + (h * m * n + self.rank * m * self.per) * 4 for p in self.slab.ptrs])
                             for h in range(2)]
                self._ld, self._col = self.per, 0
            self._flags = (C.c_void_p * self.world)(*[p + self.slab.flags_offset for p in self.slab.ptrs])
            self._epoch = C.c_void_p(self.slab.own + self.slab.epoch_offset)

    def compute(self) -> torch.Tensor:
        P = lambda t: C.c_void_p(t.data_ptr())
        st = self.lib.tb200_hgemm_f32(self.m, self.per, self.k, P(self.a), P(self.b), P(self.c_local), C.c_void_p(self.stream.cuda_stream))
        B200Native.check_status(st, "tb200_hgemm_f32")
        return self.c_local

    def launch(self, assemble: bool = False) -> torch.Tensor:
        with torch.cuda.stream(self.stream):
            self.compute()
            return gather_cols(self.c_local, self.n, self.group, self.gathered, assemble)

    def launch_fused(self) -> torch.Tensor:
        """Enqueue GEMM-with-scatter and the hand-shake; returns this rank's complete ``[m][n]`` result of the step."""
        assert self.slab is not None, "construct with fused=True"
        P = lambda t: C.c_void_p(t.data_ptr())
        S = C.c_void_p(self.stream.cuda_stream)
        half = self.steps & 1
        st = self.lib.tb200_hgemm_f32_scatter(self.m, self.per, self.k, P(self.a), P(self.b), self._dst[half], self.world, self._ld,
                                              self._col, S)
        B200Native.check_status(st, "tb200_hgemm_f32_scatter")
        if self.world > 1:
            st = self.lib.tb200_peer_signal_wait(self.rank, self.world, self._flags, self._epoch, self.timeout_ms, S)
            B200Native.check_status(st, "tb200_peer_signal_wait")
        self.steps += 1
        return self.halves[half]

    def check(self) -> None:
        """Raise if a bounded device-side wait has expired since the last check (synchronises the device)."""
        status = B200Native.device_status(8 | 16)  # the FP16 GEMM and the hand-shake kernels
        if status != 0:
            from .native import TornadoB200Error
            raise TornadoB200Error(f"tb200_hgemm_f32_scatter (step {self.steps})", status, B200Native.status_string(status))

    def launch_best(self) -> torch.Tensor:
        """The fused epilogue when the object was built for it, else the NCCL gather.  Returns the result in the
        object's layout: ``[m][n]`` ("assembled") or ``[world][m][per]`` ("blocks")."""
        if self.slab is not None:
            return self.launch_fused()
        return self.launch(assemble=self.layout != "blocks")

    def close(self) -> None:
        self.stream.synchronize()
        if self.slab is not None:
            self.halves = None
            self.slab.close()
            self.slab = None
