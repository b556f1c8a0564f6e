"""Grouped, row-sharded integer-mode mat-vec whose outputs reach every GPU by peer stores.

One process per GPU.  Each rank owns the same row block of ``count`` block-format matrices
(Q8_0 34-byte or Q4_0 18-byte blocks) and runs ONE launch per step for all of them
(``tb200_q8b_gemv_i8_grouped_sync``); the kernel stores every output value into the gather buffer of
every rank (its own and, over NVLink, the peers' CUDA-IPC mapped ones) and carries the hand-shake
that replaces the all-gather: at its start it announces the steps this rank has completed to every
rank and waits until no rank still reads the slot it is about to overwrite; ``wait()`` completes a step
for a consumer.  The reference has
no counterpart: its multi-device mode runs independent tasks with host round trips
(docs/source/multi-device.rst:9-14).

``torch.distributed`` is used at set-up only (exchange of the IPC handles) and for barriers at
tear-down; no collective runs on the data path.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .native import B200Native, TornadoB200Error, graph_replayer
from .sharding import shard_range

FLAG_WORDS = 8  # flag array of one rank: one word per peer


class _RawDeviceMemory:
    """A range of device memory that torch did not allocate, exposed through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def wrap_device_memory(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    """uint8 tensor view of raw device memory (no copy, no ownership)."""
    return torch.as_tensor(_RawDeviceMemory(ptr, nbytes), device=device)


class PeerSlab:
    """One device allocation per rank, mapped into every rank of the group.

    Layout: ``[payload_bytes][flags: FLAG_WORDS x u32][step counter: u32][scratch: u32]``, zero-filled.  ``ptrs[p]`` is rank p's
    slab as addressable from this process.
    """

    def __init__(self, payload_bytes: int, device: torch.device, group=None):
        self.lib = B200Native.load()
        self.group, self.device = group, device
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.payload_bytes = (payload_bytes + 255) // 256 * 256
        self.nbytes = self.payload_bytes + 256
        own = C.c_void_p()
        B200Native.check_status(self.lib.tb200_device_malloc(self.nbytes, C.byref(own)), "tb200_device_malloc")
        self.own = own.value
        self.bytes = wrap_device_memory(self.own, self.nbytes, device)
        self.bytes.zero_()
        torch.cuda.synchronize(device)
        self.ptrs = [0] * self.world
        self.ptrs[self.rank] = self.own
        self._opened: list[int] = []
        if self.world > 1:
            handle = (C.c_ubyte * 64)()
            B200Native.check_status(self.lib.tb200_ipc_export(C.c_void_p(self.own), handle), "tb200_ipc_export")
            handles: list = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            for p, h in enumerate(handles):
                if p == self.rank:
                    continue
                buf, out = (C.c_ubyte * 64).from_buffer_copy(h), C.c_void_p()
                B200Native.check_status(self.lib.tb200_ipc_open(buf, C.byref(out)), "tb200_ipc_open")
                self.ptrs[p] = out.value
                self._opened.append(out.value)
            dist.barrier(group=group)  # every slab is zeroed and mapped before anyone stores into it

    @property
    def flags_offset(self) -> int:
        return self.payload_bytes

    @property
    def epoch_offset(self) -> int:
        return self.payload_bytes + FLAG_WORDS * 4

    def close(self) -> None:
        """Unmap the peers and free the slab; collective (every rank must have stopped launching)."""
        if self.own is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        for ptr in self._opened:
            self.lib.tb200_ipc_close(C.c_void_p(ptr))
        self._opened = []
        if self.world > 1:
            dist.barrier(group=self.group)  # nobody frees memory a peer still has mapped
        self.bytes = None
        self.lib.tb200_device_free(C.c_void_p(self.own))
        self.own = None


class ShardedGroupedGemv:
    """``count`` equally shaped block matrices, rows sharded over the ranks, ``per_launch`` matrices per launch
    (one launch per step and rank by default) and one hand-shake per step.

    ``weights[m]`` is this rank's row block of matrix m (uint8 CUDA tensor of 34- or 18-byte blocks, rows
    ``shard_range(rows, world, rank)``).  ``launch()`` enqueues the step and returns the gathered
    ``[count][batch][rows]`` device tensor of that step; ``run(x_host)`` adds the activation upload and
    the download of the gathered result.
    """

    def __init__(self, rows: int, cols: int, batch: int, weights: list[torch.Tensor], fmt: str = "q8b", group=None,
                 timeout_ms: int = 2000, per_launch: int = 32, nslots: int = 3):
        assert fmt in ("q8b", "q4b") and 1 <= per_launch <= 32 and 2 <= nslots <= 4
        self.nslots = nslots
        self.per_launch = per_launch
        self.lib = B200Native.load()
        self.fn_name = f"tb200_{fmt}_gemv_i8_grouped"
        self.fn = getattr(self.lib, self.fn_name)
        self.rows, self.cols, self.batch, self.count, self.group = rows, cols, batch, len(weights), group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.r0, r1 = shard_range(rows, self.world, self.rank)
        self.local_rows = r1 - self.r0
        block_bytes = 34 if fmt == "q8b" else 18
        for w in weights:
            assert w.is_cuda and w.dtype == torch.uint8 and w.numel() == self.local_rows * (cols // 32) * block_bytes
        self.weights = weights
        dev = weights[0].device
        self.device, self.timeout_ms = dev, timeout_ms
        self.stream = torch.cuda.Stream(device=dev)
        self.half_floats = self.count * batch * rows
        self.slab = PeerSlab(nslots * self.half_floats * 4, dev, group)
        self.halves = self.slab.bytes[:nslots * self.half_floats * 4].view(torch.float32).view(nslots, self.count, batch, rows)
        self.x_dev = torch.empty((batch, cols), dtype=torch.float32, device=dev)
        self.y_host = torch.empty((self.count, batch, rows), dtype=torch.float32, pin_memory=True)
        self.ws_bytes = self.lib.tb200_qx_workspace_bytes(cols, batch)
        self.ws = torch.empty(max(self.ws_bytes, 16), dtype=torch.uint8, device=dev)
        # host arrays of device pointers, kept alive with the object
        self._chunks = []  # (first matrix, matrices, weight pointers, destination pointers) of each launch
        for m0 in range(0, self.count, per_launch):
            n = min(per_launch, self.count - m0)
            w_ptrs = (C.c_void_p * n)(*[w.data_ptr() for w in weights[m0:m0 + n]])
            dst_ptrs = (C.c_void_p * self.world)(*[p + m0 * batch * rows * 4 for p in self.slab.ptrs])
            self._chunks.append((m0, n, w_ptrs, dst_ptrs))
        self._flag_ptrs = (C.c_void_p * self.world)(*[p + self.slab.flags_offset for p in self.slab.ptrs])
        self._flags_local = C.c_void_p(self.slab.own + self.slab.flags_offset)
        self._sync = C.c_void_p(self.slab.own + self.slab.epoch_offset)  # [step counter][finished-CTA counter]
        self.fn_sync = getattr(self.lib, self.fn_name + "_sync")
        assert self.world == 1 or rows >= self.world * 1 and self.local_rows >= 1, "every rank needs at least one row"
        self.steps = 0  # steps enqueued so far; step s writes slot s % nslots
        self._step_graphs = {}  # (slot, download, host pointer) -> (captured step, its output slot)

    def launch(self) -> torch.Tensor:
        """Enqueue one step.  With several ranks the kernels carry the hand-shake: the first launch of the step
        announces the completed steps and waits until no rank reads the slot it is about to overwrite, the last
        one advances the step counter.  The returned slot is complete on this rank once ``wait()`` (enqueued
        after it) has passed."""
        S = C.c_void_p(self.stream.cuda_stream)
        X, W = C.c_void_p(self.x_dev.data_ptr()), C.c_void_p(self.ws.data_ptr())
        with torch.cuda.stream(self.stream):
            last = len(self._chunks) - 1
            for i, (_, n, w_ptrs, dst_ptrs) in enumerate(self._chunks):
                if self.world > 1:
                    handshake = (1 if i == 0 else 0) | (2 if i == last else 0)
                    st = self.fn_sync(n, self.local_rows, self.cols, self.batch, w_ptrs, X, dst_ptrs, self.world, self.rank,
                                      self.nslots, self.half_floats, self._sync, self._flag_ptrs, handshake, self.timeout_ms, self.rows, self.r0,
                                      W, self.ws_bytes, S)
                else:
                    st = self.fn(n, self.local_rows, self.cols, self.batch, w_ptrs, X, dst_ptrs, 1, 0, None, self.rows, 0,
                                 W, self.ws_bytes, S)
                B200Native.check_status(st, self.fn_name)
        half = self.steps % self.nslots if self.world > 1 else 0
        self.steps += 1
        return self.halves[half]

    def wait(self) -> None:
        """Enqueue the completion of the steps launched so far: every rank's outputs have arrived in this rank's buffer."""
        if self.world > 1:
            st = self.lib.tb200_peer_wait(self.rank, self.world, self._flag_ptrs, self._sync, self.timeout_ms, C.c_void_p(self.stream.cuda_stream))
            B200Native.check_status(st, "tb200_peer_wait")

    def check(self) -> None:
        """Raise if a bounded device-side wait of this GPU has expired since the last check: a rank that did not
        arrive in time leaves stale or missing outputs, which must not pass for results.  Synchronises the
        device; ``run()`` calls it after every step, ``launch()`` / ``wait()`` users call it where they consume."""
        status = B200Native.device_status(2 | 16)  # the mat-vec kernels and the hand-shake kernels
        if status != 0:
            raise TornadoB200Error(f"{self.fn_name} (step {self.steps})", status, B200Native.status_string(status))

    def run(self, x_host: torch.Tensor, download: bool = True, graph: bool = False) -> torch.Tensor:
        """One step end to end.  ``download=False`` leaves the gathered result on the device (returned as the
        device tensor): a rank whose consumer reads it there need not copy it to the host.  ``graph=True`` replays
        the step (upload, launches, hand-shake, download) from a CUDA graph captured on first use -- one per output
        slot, because the slot a step writes follows the step count -- the way a TornadoVM plan ``withCUDAGraph()``
        replays its tasks; ``x_host`` must then be the same pinned tensor on every call."""
        if graph:
            slot = self.steps % self.nslots if self.world > 1 else 0
            key = (slot, bool(download), x_host.data_ptr())
            entry = self._step_graphs.get(key)
            if entry is None:
                self.stream.synchronize()
                g = torch.cuda.CUDAGraph()
                steps_before = self.steps
                with torch.cuda.graph(g, stream=self.stream):
                    self.x_dev.copy_(x_host, non_blocking=True)
                    y = self.launch()
                    self.wait()
                    if download:
                        self.y_host.copy_(y, non_blocking=True)
                self.steps = steps_before  # capture enqueued nothing; the replay below is the step
                entry = self._step_graphs[key] = (g, y, graph_replayer(g, self.stream, synchronize=False))
            g, y, replay = entry
            if replay is not None and torch.cuda.current_device() == self.stream.device.index:
                replay()
            else:
                with torch.cuda.stream(self.stream):
                    g.replay()
            self.steps += 1
        else:
            with torch.cuda.stream(self.stream):
                self.x_dev.copy_(x_host, non_blocking=True)
                y = self.launch()
                self.wait()
                if download:
                    self.y_host.copy_(y, non_blocking=True)
        self.stream.synchronize()
        self.check()
        return self.y_host if download else y

    def close(self) -> None:
        self.stream.synchronize()
        self._step_graphs = {}
        self.halves = None
        self.slab.close()
