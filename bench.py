#!/usr/bin/env python
"""Benchmark of the b200/linalg hot path.

Headline workload: Q8_0 quantised GEMV, decode style,
W[14336 x 4096] as 32-element int8 blocks with one fp16 scale each, fp32
activations, batch 1.  One "step" is one decode pass over LAYERS = 32 distinct
weight matrices of that shape, one per decoder layer (2.0 GB > the 126 MB L2, so
every mat-vec streams its weights from HBM).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints one JSON line (rank 0).  `value` is device-resident throughput in GB/s of
algorithmic bytes (34*rows*cols/32 + 4*batch*(cols+rows) per GEMV); `e2e` is the
same metric through the public task-graph API with host buffers (activation
host->device and result device->host inside every step); `roofline` compares
the GEMV kernel with the measured HBM copy bandwidth; `cpu_baseline` times the
CPU restatement of the reference's sequential / multi-core loop on the host.
The step is one grouped launch over the 32 matrices (--group G: G per launch).
With N > 1 the weight rows are sharded over the ranks and the kernel stores every
output into every rank's buffer over NVLink (strong scaling: the total work is
fixed).
"""
from __future__ import annotations

import argparse
import datetime
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, COLS, BATCH = 14336, 4096, 1
LAYERS = 32  # one step = this projection in each of 32 decoder layers (Llama-3-8B depth): 32 distinct matrices, 2.0 GB
# dram__bytes_read.sum + dram__bytes_write.sum per 14336 x 4096 matrix of a grouped integer-mode launch, from an ncu
# capture of 8 matrices per launch (499.3 MB read + 5.2 MB written; the kernel reads every weight byte once, so
# traffic grows in proportion to the matrices of a launch)
NCU_TRAFFIC_BYTES_PER_GEMV = 63_060_000
REF_MATVECS = 8  # mat-vecs per step of the CPU reference arm
METRIC = "q8_0_gemv_hbm_throughput"
UNIT = "GB/s"


def algorithmic_bytes(rows, cols, batch, block_bytes=34):
    return block_bytes * rows * cols // 32 + 4 * batch * (cols + rows)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


# ------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()  # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------- CPU baseline / reference arm
def cpu_reference(seconds_target=8.0, threads=True):
    """Times the CPU restatement of the reference's Q8_0 mat-vec loop
    (MatrixVectorRowMajor.java:530-578 arithmetic, rows split over host threads the
    way TornadoVM's multi-core CPU device splits the outer loop) on the full
    14336 x 4096 matrix.  The only place this benchmark touches oracle/."""
    import numpy as np
    import oracle as o
    rng = np.random.default_rng(42)
    q = rng.integers(-127, 128, ROWS * COLS, dtype=np.int8)
    s = (np.abs(rng.standard_normal(ROWS * COLS // 32)) * 0.02).astype(np.float16).view(np.uint16)
    x = rng.standard_normal(COLS).astype(np.float32)
    o.q8_gemv_seq(q, s, x, COLS, ROWS, threads=threads)  # warm-up
    t0 = time.perf_counter()
    n = 0
    while True:
        o.q8_gemv_seq(q, s, x, COLS, ROWS, threads=threads)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= seconds_target:
            break
    per = dt / n
    cores = o.num_threads() if threads else 1
    return {"value": algorithmic_bytes(ROWS, COLS, 1) / per / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{n} full {ROWS}x{COLS} batch-1 mat-vecs in {dt:.1f} s ({'OpenMP rows over host threads' if threads else 'single thread'})",
            "ms_per_matvec": per * 1e3}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # K steps of LAYERS mat-vecs each would take minutes on a CPU: each step is a bounded sample (one mat-vec)
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its ranks; the CPU arm uses every core it may run on
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    import numpy as np
    import oracle as o
    rng = np.random.default_rng(42)
    q = rng.integers(-127, 128, ROWS * COLS, dtype=np.int8)
    s = (np.abs(rng.standard_normal(ROWS * COLS // 32)) * 0.02).astype(np.float16).view(np.uint16)
    x = rng.standard_normal(COLS).astype(np.float32)
    # one step = REF_MATVECS mat-vecs of the GPU step's 32, so that a run of 20 steps spans more than half a second
    # (a single 3 ms mat-vec per step is dominated by thread wake-up noise)
    for _ in range(max(args.warmup, 1)):
        for _ in range(REF_MATVECS):
            o.q8_gemv_seq(q, s, x, COLS, ROWS, threads=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for _ in range(REF_MATVECS):
            o.q8_gemv_seq(q, s, x, COLS, ROWS, threads=True)
    dt = time.perf_counter() - t0
    per = dt / args.steps
    val = REF_MATVECS * algorithmic_bytes(ROWS, COLS, 1) / per / 1e9
    sample = (f"each step = {REF_MATVECS} full {ROWS}x{COLS} batch-1 mat-vecs (of the {LAYERS} per GPU step) on "
              f"{o.num_threads()} host threads")
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"Q8_0 GEMV {ROWS}x{COLS} batch {BATCH}, CPU restatement of the reference loop"},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": o.num_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------- GPU arm
def make_weights(torch, dev, rows, layers, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    q = torch.randint(-127, 128, (layers, rows, COLS), dtype=torch.int8, device=dev, generator=g)
    sc = (torch.randn((layers, rows, COLS // 32), device=dev, generator=g).abs() * 0.02).half()
    return q, sc


def secondary_metrics(torch, lib, stream, hbm_peak, tensor_peak, sections=("sgemv", "q8", "q8layers", "q4", "sgemm", "hgemm"), hgemm_sizes=(2048, 4096, 8192, 16384)):
    """Short device-resident timings of the other kernels on the path (not the headline)."""
    out = {}
    P = lambda t: C.c_void_p(t.data_ptr())
    S = C.c_void_p(stream.cuda_stream)
    dev = torch.device("cuda", torch.cuda.current_device())
    lib.tb200_set_option(1, 1)  # overlapped launches, as in the headline

    def timeit(fn, reps, period=4):
        """Average seconds per call; `period` consecutive calls (distinct operands) are captured in a CUDA graph."""
        for i in range(period):
            fn(i)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(period):
                fn(i)
        g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        e0.record(stream)
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        stream.synchronize()
        return e0.elapsed_time(e1) / (reps * period) * 1e-3

    with torch.cuda.stream(stream):
        if "sgemv" in sections:
            # FP32 GEMV 8192 x 8192; two matrices alternate (537 MB > L2)
            m = torch.rand((2, 8192, 8192), device=dev) * 2 - 1
            v = torch.rand(8192, device=dev) * 2 - 1
            y = torch.empty(8192, device=dev)
            t = timeit(lambda i: lib.tb200_sgemv(8192, 8192, P(m[i & 1]), P(v), P(y), S), 10)
            b = 4 * (8192 * 8192 + 2 * 8192)
            out["sgemv_8192"] = {"GB/s": b / t / 1e9, "frac_hbm": b / t / 1e9 / hbm_peak, "us": t * 1e6}
            del m
        if "q8" in sections:
            # Q8_0 variants on the headline shape
            q, sc = make_weights(torch, dev, ROWS, 4, 7)
            blocks = torch.empty((4, ROWS, COLS // 32, 34), dtype=torch.uint8, device=dev)
            blocks[..., :2] = sc.view(torch.uint8).view(4, ROWS, COLS // 32, 2)
            blocks[..., 2:] = q.view(torch.uint8).view(4, ROWS, COLS // 32, 32)
            for batch in (1, 4, 8):
                x = torch.randn((batch, COLS), device=dev)
                yb = torch.empty((batch, ROWS), device=dev)
                ws_n = lib.tb200_qx_workspace_bytes(COLS, batch)
                ws = torch.empty(ws_n, dtype=torch.uint8, device=dev)
                by = algorithmic_bytes(ROWS, COLS, batch)
                runs = {
                    f"q8_split_f32_b{batch}": lambda i: lib.tb200_q8_gemv(ROWS, COLS, batch, P(q[i & 3]), P(sc[i & 3]), P(x), P(yb), S),
                    f"q8_blocks_f32_b{batch}": lambda i: lib.tb200_q8b_gemv(ROWS, COLS, batch, P(blocks[i & 3]), P(x), P(yb), S),
                    f"q8_split_int_b{batch}": lambda i: lib.tb200_q8_gemv_i8(ROWS, COLS, batch, P(q[i & 3]), P(sc[i & 3]), P(x), P(yb), P(ws), ws_n, S),
                    f"q8_blocks_int_b{batch}": lambda i: lib.tb200_q8b_gemv_i8(ROWS, COLS, batch, P(blocks[i & 3]), P(x), P(yb), P(ws), ws_n, S),
                }
                for name, fn in runs.items():
                    t = timeit(fn, 10)
                    out[name] = {"GB/s": by / t / 1e9, "frac_hbm": by / t / 1e9 / hbm_peak, "us": t * 1e6}
            # the same block matrices behind a 24-byte array header (the reference launcher's JVM mode) in an aligned
            # buffer: element pointers are 24 modulo 128, i.e. 8 modulo 16
            shifted = torch.empty(blocks.numel() + 32, dtype=torch.uint8, device=dev)
            per = blocks[0].numel()
            for batch in (1, 8):
                x = torch.randn((batch, COLS), device=dev)
                yb = torch.empty((batch, ROWS), device=dev)
                ws_n = lib.tb200_qx_workspace_bytes(COLS, batch)
                ws = torch.empty(ws_n, dtype=torch.uint8, device=dev)
                by = algorithmic_bytes(ROWS, COLS, batch)
                base = shifted.data_ptr() + 24
                for i in range(4):
                    shifted[24 + i * per:24 + (i + 1) * per].copy_(blocks[i].reshape(-1))
                t = timeit(lambda i: lib.tb200_q8b_gemv_i8(ROWS, COLS, batch, C.c_void_p(base + (i & 3) * per), P(x), P(yb), P(ws), ws_n, S), 10)
                out[f"q8_blocks_int_b{batch}_header24"] = {"GB/s": by / t / 1e9, "frac_hbm": by / t / 1e9 / hbm_peak, "us": t * 1e6}
            del q, sc, blocks, shifted
        if "q8layers" in sections:
            # the headline's 32 matrices, one launch per mat-vec (the granularity of the reference's tasks) and in
            # groups of 2 (a layer's gate/up pair reads one vector) and 8
            q, sc = make_weights(torch, dev, ROWS, LAYERS, 11)
            blocks = torch.empty((LAYERS, ROWS, COLS // 32, 34), dtype=torch.uint8, device=dev)
            blocks[..., :2] = sc.view(torch.uint8).view(LAYERS, ROWS, COLS // 32, 2)
            blocks[..., 2:] = q.view(torch.uint8).view(LAYERS, ROWS, COLS // 32, 32)
            del q, sc
            x = torch.randn((1, COLS), device=dev)
            yl = torch.empty((LAYERS, ROWS), device=dev)
            by = algorithmic_bytes(ROWS, COLS, 1)
            ws_n = lib.tb200_qx_workspace_bytes(COLS, 1)
            ws = torch.empty(ws_n, dtype=torch.uint8, device=dev)
            t = timeit(lambda i: lib.tb200_q8b_gemv_i8(ROWS, COLS, 1, P(blocks[i]), P(x), P(yl[i]), P(ws), ws_n, S), 10, period=LAYERS)
            out["q8_blocks_int_b1_one_launch_per_matvec"] = {"GB/s": by / t / 1e9, "frac_hbm": by / t / 1e9 / hbm_peak, "us": t * 1e6}
            # the same with 8 activation vectors (the tensor-core mat-vec behind its quantiser kernel), back to back
            x8 = torch.randn((8, COLS), device=dev)
            y8 = torch.empty((LAYERS, 8, ROWS), device=dev)
            ws8_n = lib.tb200_qx_workspace_bytes(COLS, 8)
            ws8 = torch.empty(ws8_n, dtype=torch.uint8, device=dev)
            by8 = algorithmic_bytes(ROWS, COLS, 8)
            t = timeit(lambda i: lib.tb200_q8b_gemv_i8(ROWS, COLS, 8, P(blocks[i]), P(x8), P(y8[i]), P(ws8), ws8_n, S), 10, period=LAYERS)
            out["q8_blocks_int_b8_one_launch_per_matvec"] = {"GB/s": by8 / t / 1e9, "frac_hbm": by8 / t / 1e9 / hbm_peak, "us": t * 1e6}
            # ... and 8 matrices per grouped launch: one quantiser kernel, then the tensor-core mat-vecs chained to one another
            grp = 8
            wp8 = [(C.c_void_p * grp)(*[blocks[c * grp + m].data_ptr() for m in range(grp)]) for c in range(LAYERS // grp)]
            dp8 = [(C.c_void_p * 1)(y8[c * grp].data_ptr()) for c in range(LAYERS // grp)]
            t = timeit(lambda i: lib.tb200_q8b_gemv_i8_grouped(grp, ROWS, COLS, 8, wp8[i], P(x8), dp8[i], 1, 0, None, ROWS, 0, P(ws8), ws8_n, S),
                       10, period=LAYERS // grp)
            out["q8_blocks_int_b8_8_per_launch"] = {"GB/s": grp * by8 / t / 1e9, "frac_hbm": grp * by8 / t / 1e9 / hbm_peak, "us": t * 1e6}
            # the Q4_0 twin: 8 matrices of 14336 x 4096 back to back, 8 vectors, one grouped launch
            q4per = ROWS * (COLS // 32) * 18
            q4 = torch.randint(0, 256, (LAYERS, q4per), dtype=torch.uint8, device=dev)
            q4.view(-1)[1::18] = 0x20  # scales of ordinary size
            wq4 = [(C.c_void_p * grp)(*[q4[c * grp + m].data_ptr() for m in range(grp)]) for c in range(LAYERS // grp)]
            by4 = algorithmic_bytes(ROWS, COLS, 8, 18)
            t = timeit(lambda i: lib.tb200_q4b_gemv_i8_grouped(grp, ROWS, COLS, 8, wq4[i], P(x8), dp8[i], 1, 0, None, ROWS, 0, P(ws8), ws8_n, S),
                       10, period=LAYERS // grp)
            out["q4_blocks_int_b8_8_per_launch"] = {"GB/s": grp * by4 / t / 1e9, "frac_hbm": grp * by4 / t / 1e9 / hbm_peak, "us": t * 1e6}
            del x8, y8, ws8, q4
            for grp in (2, 8):
                wp = [(C.c_void_p * grp)(*[blocks[c * grp + m].data_ptr() for m in range(grp)]) for c in range(LAYERS // grp)]
                dp = [(C.c_void_p * 1)(yl[c * grp].data_ptr()) for c in range(LAYERS // grp)]
                t = timeit(lambda i: lib.tb200_q8b_gemv_i8_grouped(grp, ROWS, COLS, 1, wp[i], P(x), dp[i], 1, 0, None, ROWS, 0, None, 0, S),
                           10, period=LAYERS // grp)
                out[f"q8_blocks_int_b1_{grp}_per_launch"] = {"GB/s": grp * by / t / 1e9, "frac_hbm": grp * by / t / 1e9 / hbm_peak, "us": t * 1e6}
            # the same 32 matrices as payloads behind the reference's 24-byte array header in 256-byte aligned
            # buffers: every matrix, the vector and the outputs start 24 bytes past a 128-byte line (a matrix is a
            # multiple of 128 bytes long, so all share the phase); one launch per 8 matrices
            mat_bytes = ROWS * (COLS // 32) * 34
            raw = torch.empty(LAYERS * mat_bytes + 256, dtype=torch.uint8, device=dev)
            base = 24 + (-raw.data_ptr()) % 128
            raw[base:base + LAYERS * mat_bytes].copy_(blocks.view(-1))
            del blocks
            xr = torch.empty(COLS + 64, device=dev)
            xo = (24 + (-xr.data_ptr()) % 128) // 4
            xr[xo:xo + COLS].copy_(x.view(-1))
            yr = torch.empty(LAYERS * ROWS + 64, device=dev)
            yo = (24 + (-yr.data_ptr()) % 128) // 4
            grp = 8
            wp = [(C.c_void_p * grp)(*[raw.data_ptr() + base + (c * grp + m) * mat_bytes for m in range(grp)]) for c in range(LAYERS // grp)]
            dp = [(C.c_void_p * 1)(yr.data_ptr() + 4 * (yo + c * grp * ROWS)) for c in range(LAYERS // grp)]
            xp = C.c_void_p(xr.data_ptr() + 4 * xo)
            t = timeit(lambda i: lib.tb200_q8b_gemv_i8_grouped(grp, ROWS, COLS, 1, wp[i], xp, dp[i], 1, 0, None, ROWS, 0, None, 0, S),
                       10, period=LAYERS // grp)
            out["q8_blocks_int_b1_8_per_launch_header24"] = {"GB/s": grp * by / t / 1e9, "frac_hbm": grp * by / t / 1e9 / hbm_peak, "us": t * 1e6}
            same = bool(torch.equal(yr[yo:yo + LAYERS * ROWS].view(LAYERS, ROWS), yl))
            out["q8_blocks_int_b1_8_per_launch_header24"]["same_bits_as_aligned"] = same
            del raw
        if "q4" in sections:
            # Q4_0 Llama-3-8B-shaped layer sweep: 7 projections + the output projection
            shapes = [(4096, 4096)] * 2 + [(1024, 4096)] * 2 + [(14336, 4096)] * 2 + [(4096, 14336), (128256, 4096)]
            g = torch.Generator(device=dev).manual_seed(3)
            # two sets of weights alternate so that a pass never finds its matrices in L2 (2 x 418 MB)
            wsets = [[torch.randint(0, 256, (r * (c // 32) * 18,), dtype=torch.uint8, device=dev, generator=g) for r, c in shapes] for _ in range(2)]
            for batch in (1, 4, 16):
                xs = {c: torch.randn((batch, c), device=dev) for c in (4096, 14336)}
                ys = {r: torch.empty((batch, r), device=dev) for r in (4096, 1024, 14336, 128256)}
                ws_n = lib.tb200_qx_workspace_bytes(14336, batch)
                ws = torch.empty(ws_n, dtype=torch.uint8, device=dev)
                by = sum(algorithmic_bytes(r, c, batch, 18) for r, c in shapes)

                def sweep_f(i):
                    for (r, c), w in zip(shapes, wsets[i & 1]):
                        lib.tb200_q4b_gemv(r, c, batch, P(w), P(xs[c]), P(ys[r]), S)

                def sweep_i(i):
                    for (r, c), w in zip(shapes, wsets[i & 1]):
                        lib.tb200_q4b_gemv_i8(r, c, batch, P(w), P(xs[c]), P(ys[r]), P(ws), ws_n, S)
                # the same sweep with every matrix that reads the 4096-element vector in one launch (7 of the 8)
                idx = [[j for j, (r, c) in enumerate(shapes) if c == cc] for cc in (4096, 14336)]
                ysep = [torch.empty((batch, r), device=dev) for r, c in shapes]  # one output array per matrix
                garg = []
                for k in range(2):
                    garg.append([((C.c_int * len(ix))(*[shapes[j][0] for j in ix]), (C.c_void_p * len(ix))(*[wsets[k][j].data_ptr() for j in ix]),
                                  (C.c_void_p * len(ix))(*[ysep[j].data_ptr() for j in ix]), len(ix), shapes[ix[0]][1]) for ix in idx])

                def sweep_g(i):
                    for rows_a, w_a, y_a, n, c in garg[i & 1]:
                        lib.tb200_q4b_gemv_i8_grouped_rows(n, rows_a, c, batch, w_a, P(xs[c]), y_a, P(ws), ws_n, S)
                runs = [(f"q4_layer_sweep_f32_b{batch}", sweep_f), (f"q4_layer_sweep_int_b{batch}", sweep_i)]
                runs.append((f"q4_layer_sweep_int_grouped_b{batch}", sweep_g))
                for name, fn in runs:
                    t = timeit(fn, 3, period=2)
                    out[name] = {"GB/s": by / t / 1e9, "frac_hbm": by / t / 1e9 / hbm_peak, "us": t * 1e6}
            del wsets
        if "sgemm" in sections:
            # FP32 SGEMM 4096^3
            a = torch.rand((4096, 4096), device=dev)
            bm = torch.rand((4096, 4096), device=dev)
            c = torch.empty((4096, 4096), device=dev)
            run = lambda i: lib.tb200_sgemm(4096, 4096, 4096, C.c_float(1.0), P(a), P(bm), C.c_float(0.0), P(c), S)
            t = timeit(run, 3, period=2)
            # the SM clock under sustained FFMA load decides what the CUDA cores can deliver: sample it over half a second
            with ClockSampler(torch.cuda.current_device()) as ck:
                t_long = timeit(run, 100, period=2)
            mhz = ck.summary()["sm_mhz"]
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            out["sgemm_4096"] = {"TFLOP/s": 2 * 4096**3 / t / 1e12, "ms": t * 1e3, "sustained_TFLOP/s": 2 * 4096**3 / t_long / 1e12,
                                 "sm_mhz_sustained": mhz, "frac_ffma_at_clock": (2 * 4096**3 / t_long / 1e12) / (sms * 128 * 2 * mhz * 1e-6) if mhz else None}
            # operands behind a 24-byte header: 8 modulo 16
            raw = [torch.empty(4096 * 4096 * 4 + 32, dtype=torch.uint8, device=dev) for _ in range(3)]
            pa, pb, pc = (r.data_ptr() + 24 for r in raw)
            raw[0][24:24 + a.numel() * 4].copy_(a.view(torch.uint8).reshape(-1))
            raw[1][24:24 + bm.numel() * 4].copy_(bm.view(torch.uint8).reshape(-1))
            t24 = timeit(lambda i: lib.tb200_sgemm(4096, 4096, 4096, C.c_float(1.0), C.c_void_p(pa), C.c_void_p(pb), C.c_float(0.0), C.c_void_p(pc), S), 3, period=2)
            out["sgemm_4096_header24"] = {"TFLOP/s": 2 * 4096**3 / t24 / 1e12, "ms": t24 * 1e3}
            del raw
        if "hgemm" in sections:
            # FP16 GEMM sweep
            for n in hgemm_sizes:
                ah = (torch.randn((n, n), device=dev) / n**0.5).half()
                bh = (torch.randn((n, n), device=dev) / n**0.5).half()
                ch = torch.empty((n, n), device=dev)
                t = timeit(lambda i: lib.tb200_hgemm_f32(n, n, n, P(ah), P(bh), P(ch), S), 3, period=2)
                t24 = t16 = None
                if n == 8192:
                    # A, B and C behind a 16- and a 24-byte header in aligned buffers (payloads 16 / 24 bytes past a
                    # 128-byte line; 24 is also 8 modulo 16), timed like the aligned product and next to it
                    raw = [torch.empty(n * n * e + 32, dtype=torch.uint8, device=dev) for e in (2, 2, 4)]
                    for hdr in (16, 24):
                        raw[0][hdr:hdr + n * n * 2].copy_(ah.view(torch.uint8).reshape(-1))
                        raw[1][hdr:hdr + n * n * 2].copy_(bh.view(torch.uint8).reshape(-1))
                        pa, pb, pc = (C.c_void_p(r.data_ptr() + hdr) for r in raw)
                        th = timeit(lambda i: lib.tb200_hgemm_f32(n, n, n, pa, pb, pc, S), 3, period=2)
                        if hdr == 16:
                            t16 = th
                        else:
                            t24 = th
                    del raw
                # a longer run (about 100 launches) next to the burst figure: the clock settles under sustained tensor load
                t_long = timeit(lambda i: lib.tb200_hgemm_f32(n, n, n, P(ah), P(bh), P(ch), S), 50 if n <= 8192 else 10, period=2)
                out[f"hgemm_{n}"] = {"TFLOP/s": 2 * n**3 / t / 1e12, "frac_tensor": 2 * n**3 / t / 1e12 / tensor_peak, "ms": t * 1e3,
                                     "sustained_TFLOP/s": 2 * n**3 / t_long / 1e12}
                for hdr, th in ((16, t16), (24, t24)):
                    if th is not None:
                        out[f"hgemm_{n}_header{hdr}"] = {"TFLOP/s": 2 * n**3 / th / 1e12, "frac_tensor": 2 * n**3 / th / 1e12 / tensor_peak, "ms": th * 1e3}
                if n == 4096:
                    # fused epilogue and 16-bit output on the same product: D(fp16) = gelu(A*B + bias)
                    dh = torch.empty((n, n), dtype=torch.float16, device=dev)
                    bias = torch.randn(n, device=dev).half()
                    t = timeit(lambda i: lib.tb200_gemm_ex(n, n, n, 0, P(ah), P(bh), 1, P(dh), C.c_float(1.0), C.c_float(0.0), None, P(bias), 2, 1, S), 3, period=2)
                    out["gemm_bias_gelu_f16_4096"] = {"TFLOP/s": 2 * n**3 / t / 1e12, "frac_tensor": 2 * n**3 / t / 1e12 / tensor_peak, "ms": t * 1e3}
    return out


def verify_sharded_step(torch, dist, lib, op, blocks, lrows, r0, dev):
    """Untimed check of the multi-GPU data path: over several consecutive steps with changing activations (so that
    the output slots rotate and are reused), every rank recomputes its own row shard of every matrix with the
    single-launch kernel, the shards are all-gathered with torch.distributed, and the slot the fused kernel
    filled through peer stores must equal the assembled result bit for bit on every rank."""
    P = lambda t: C.c_void_p(t.data_ptr())
    world = dist.get_world_size()
    S = C.c_void_p(op.stream.cuda_stream)
    n_ws = lib.tb200_qx_workspace_bytes(COLS, BATCH)
    ws = torch.empty(max(n_ws, 16), dtype=torch.uint8, device=dev)
    local = torch.empty((LAYERS, BATCH, lrows), device=dev)
    ok = True
    for step in range(5):
        g = torch.Generator(device=dev).manual_seed(1000 + step)  # the same activations on every rank
        op.x_dev.copy_(torch.randn((BATCH, COLS), device=dev, generator=g))
        torch.cuda.synchronize()
        with torch.cuda.stream(op.stream):
            fused = op.launch()
            op.wait()
            for l in range(LAYERS):
                st = lib.tb200_q8b_gemv_i8(lrows, COLS, BATCH, P(blocks[l]), P(op.x_dev), P(local[l]), P(ws), n_ws, S)
                if st:
                    raise SystemExit(f"tb200_q8b_gemv_i8 failed with status {st}")
        op.stream.synchronize()
        op.check()
        shards = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(shards, local)  # equal shards: ROWS is a multiple of the rank count
        want = torch.cat(shards, dim=2)
        ok = ok and bool(torch.equal(fused, want))
        dist.barrier()  # nobody starts the next step (and overwrites a slot) before everyone has compared
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from tornadovm_b200.native import B200Native
    from tornadovm_b200.peer import ShardedGroupedGemv
    from tornadovm_b200.sharding import shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the b200/linalg kernels have no CPU path")
    group = args.group
    if group < 1 or LAYERS % group:
        raise SystemExit(f"--group must divide {LAYERS}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    lib = B200Native.load()  # raises if libtornado_b200.so is missing
    hbm_peak, tensor_peak, peak_kind = measured_peaks()

    # ---- device-resident workload: rank r owns rows [r0, r1) of every layer -------------------------------
    r0, r1 = shard_range(ROWS, world, rank)
    lrows = r1 - r0
    q, sc = make_weights(torch, dev, lrows, LAYERS, 1234 + rank)
    # the benchmarked operand: 34-byte blocks [fp16 scale][32 x int8], TornadoVM's unified ByteArray layout
    blocks = torch.empty((LAYERS, lrows, COLS // 32, 34), dtype=torch.uint8, device=dev)
    blocks[..., :2] = sc.view(torch.uint8).view(LAYERS, lrows, COLS // 32, 2)
    blocks[..., 2:] = q.view(torch.uint8).view(LAYERS, lrows, COLS // 32, 32)
    del q, sc
    # consecutive mat-vec launches may overlap: each prefetches its weights while its predecessor drains
    B200Native.call("tb200_set_option", 1, 1)
    # The step: LAYERS mat-vecs, `group` matrices per launch.  Every output value is stored by the kernel into the
    # gather buffer of every rank (peer stores over NVLink); with N > 1 one flag hand-shake per step completes it.
    op = ShardedGroupedGemv(ROWS, COLS, BATCH, [blocks[l].view(-1) for l in range(LAYERS)], "q8b", per_launch=group)
    stream = op.stream
    op.x_dev.copy_(torch.randn((BATCH, COLS), device=dev, generator=torch.Generator(device=dev).manual_seed(99)))
    launches_per_step = LAYERS // group

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    barrier()
    verified = None
    if world > 1:
        verified = verify_sharded_step(torch, dist, lib, op, blocks, lrows, r0, dev)
        if not verified:
            raise SystemExit("the gathered outputs of the sharded step differ from the single-launch results")
        # every peer mapping, flag page and output slot has been touched before anything is timed
        with torch.cuda.stream(stream):
            for _ in range(60):
                op.launch()
            op.wait()
        barrier()
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            op.launch()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # N > 1: a step is one launch of 40-170 us, which the Python call sequence cannot enqueue fast enough; the
        # timed steps are therefore captured once into a CUDA graph and replayed (what a TornadoVM plan
        # withCUDAGraph() does with its tasks).  The hand-shake lives in device memory and is the same in a replay.
        step_graph = None
        if world > 1:
            try:
                step_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(step_graph, stream=stream):
                    for _ in range(args.steps):
                        op.launch()
                step_graph.replay()  # one untimed replay: instantiation and upload are not part of a step
                op.wait()
            except Exception as exc:  # noqa: BLE001 - report and fall back to plain launches
                sys.stderr.write(f"[bench] CUDA graph of the sharded steps unavailable ({exc}); timing plain launches\n")
                step_graph = None
            barrier()
        with ClockSampler(local) as clocks:
            if world > 1:
                # The ranks leave the host barrier up to a few hundred microseconds apart, which a 20-step region of
                # about a millisecond would count as step time on the early ranks.  One untimed step and its peer
                # wait in front of the start event align the GPUs themselves: the wait kernel returns on every rank
                # only when every rank has announced that step, and the timed launches are already enqueued behind it.
                op.launch()
                op.wait()
            e0.record(stream)
            if step_graph is not None:
                step_graph.replay()
            else:
                for _ in range(args.steps):
                    op.launch()
            op.wait()  # the last step's outputs from every rank have arrived
            e1.record(stream)
            barrier()
            # nvidia-smi samples every 100 ms and a short timed region can fall between two samples: keep the
            # same load running (untimed, every rank the same number of steps) until a few samples exist
            t_load = time.perf_counter()
            for _ in range(40):
                enough = torch.tensor([1 if (len(clocks.rows) >= 3 or time.perf_counter() - t_load > 2.0) else 0], device=dev)
                if world > 1:
                    dist.all_reduce(enough, op=dist.ReduceOp.MIN)
                if enough.item():
                    break
                for _ in range(200):
                    op.launch()
                op.wait()
                barrier()
        elapsed = e0.elapsed_time(e1) * 1e-3
    gpu_launches = args.steps * launches_per_step + (1 if world > 1 else 0)
    if world > 1:
        t = torch.tensor([elapsed], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed = t.item()
    # kernel-only duration for the roofline: the mat-vec launches of a step without the hand-shake, one rank at a
    # time so that no peer is storing into this GPU meanwhile; events on the launch stream
    kernel_s = None
    if world == 1:
        with torch.cuda.stream(stream):
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(args.steps, 10)
            k0.record(stream)
            for _ in range(reps):
                op.launch()
            k1.record(stream)
            stream.synchronize()
            kernel_s = k0.elapsed_time(k1) * 1e-3 / (reps * (LAYERS // group))
    total_bytes = LAYERS * algorithmic_bytes(ROWS, COLS, BATCH)  # whole job, all ranks
    value = total_bytes * args.steps / elapsed / 1e9
    launch_bytes = group * algorithmic_bytes(lrows, COLS, BATCH)
    if kernel_s is None:  # N > 1: the step without its hand-shake share cannot be separated; use the step
        kernel_s = elapsed / args.steps / (LAYERS // group)
    achieved = launch_bytes / kernel_s / 1e9

    # ---- end to end through the public API, host buffers ---------------------------------------------------
    e2e_steps = args.steps
    if world == 1:
        import numpy as np
        from tornadovm_b200.arrays import ByteArray, FloatArray
        from tornadovm_b200.b200 import B200, B200Options
        from tornadovm_b200.taskgraph import CudaDevice, DataTransferMode, TaskGraph, TornadoExecutionPlan
        # one ByteArray per task holds the task's `group` matrices back to back (7 task arguments whatever the count:
        # a library task carries at most 20, TaskGraph.java:886)
        w_host = [blocks[c * group:(c + 1) * group].cpu().numpy().ravel() for c in range(LAYERS // group)]
        x_host = op.x_dev.cpu().numpy()

        def plan_seconds(host_results, header=16):
            """Seconds per execute() of the step as one task graph; the outputs of the last execution.  `header`: bytes
            in front of every array's payload (16, or 24 as with the reference launcher's default JVM flags)."""
            wa = [ByteArray(w, header) for w in w_host]
            xa = FloatArray(x_host, header)
            ya = [FloatArray(group * ROWS * BATCH, header) for _ in range(LAYERS // group)]
            opts = B200Options(exact_int=True, overlap_launches=True, host_results=host_results)
            tg = TaskGraph("q8decode").transferToDevice(DataTransferMode.FIRST_EXECUTION, *wa) \
                .transferToDevice(DataTransferMode.EVERY_EXECUTION, xa)
            for c in range(LAYERS // group):
                tg.libraryTask(f"g{c}", B200.q8GemvBytesPacked, group, ROWS, COLS, BATCH, wa[c], xa, ya[c], opts)
            tg.transferToHost(DataTransferMode.EVERY_EXECUTION, *ya)
            with TornadoExecutionPlan(tg, CudaDevice(local)).withCUDAGraph() as plan:
                for _ in range(max(args.warmup, 3)):
                    plan.execute()
                torch.cuda.synchronize()
                for y in ya:
                    y.numpy()[:] = float("nan")
                t0 = time.perf_counter()
                for _ in range(e2e_steps):
                    plan.execute()
                torch.cuda.synchronize()
                s = (time.perf_counter() - t0) / e2e_steps
                return s, plan.h2d_bytes_last, plan.d2h_bytes_last, [y.numpy().copy() for y in ya]

        # the plan that copies the outputs back after the launches, then the one whose kernels store every result into
        # the output arrays' pinned host segments themselves (B200Options.host_results); the second is the e2e figure
        copy_s, _, _, copy_out = plan_seconds(False)
        e2e_s, h2d, d2h, host_out = plan_seconds(True)
        h24_s, _, _, h24_out = plan_seconds(True, header=24)
        if not all(np.array_equal(a, b) and np.array_equal(a, c) for a, b, c in zip(copy_out, host_out, h24_out)):
            raise SystemExit("e2e: the host-stored results differ from the copied ones")
        del copy_out, host_out, h24_out, w_host
        e2e_s *= e2e_steps
        api = ("TaskGraph.libraryTask(B200.q8GemvBytesPacked, B200Options(host_results=True)) + "
               "TornadoExecutionPlan.withCUDAGraph().execute()")
    else:
        xh = torch.randn((BATCH, COLS)).pin_memory()
        # the job's result reaches the host once: rank 0 downloads the gathered outputs, the other ranks (whose
        # consumers would read them on the device) only complete the step
        # each step (upload, launch, hand-shake, download) is replayed from a CUDA graph, like the single-GPU plan
        for _ in range(max(args.warmup, 3) + op.nslots):
            op.run(xh, download=rank == 0, graph=True)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            op.run(xh, download=rank == 0, graph=True)
        barrier()
        e2e_s = time.perf_counter() - t0
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = t.item()
        h2d, d2h = BATCH * COLS * 4, LAYERS * BATCH * ROWS * 4
        api = "ShardedGroupedGemv.run(graph=True)"
    gpu_launches += e2e_steps * (launches_per_step + (1 if world > 1 else 0))
    e2e_value = total_bytes * e2e_steps / e2e_s / 1e9
    status = C.c_int(0)
    lib.tb200_device_status(C.byref(status))
    if status.value:
        raise SystemExit(f"a bounded device-side wait expired during the run (status {status.value})")

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "s8", "data": "synthetic",
        "config": {"workload": f"Q8_0 GEMV W[{ROWS}x{COLS}] int8 blocks of 32 + fp16 scale (34-byte blocks), fp32 x, batch {BATCH}",
                   "layers_per_step": LAYERS, "matrices_per_launch": group,
                   "l2_policy": f"{LAYERS} distinct weight matrices per step ({LAYERS * 62.4:.0f} MB > 126 MB L2)",
                   "parallelism": (f"rows sharded over {world} GPUs; the kernel stores each output into every GPU's gather buffer "
                                   "(peer stores over NVLink) and carries the flag hand-shake of the step, no collective library on the data path")
                   if world > 1 else "single GPU",
                   "mode": "int (fp32 activations quantised to int8 per 32-block inside the kernel, exact int32 block dots)",
                   "launch": f"{LAYERS // group} grouped launch(es) per step, programmatic dependent launches" + (", timed steps replayed from one CUDA graph" if world > 1 else "")},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_s / e2e_steps * 1e3, "api": api,
                **({"copy_back_ms_per_step": copy_s * 1e3, "copy_back_value": total_bytes / copy_s / 1e9,
                    "header24_ms_per_step": h24_s * 1e3, "header24_value": total_bytes / h24_s / 1e9} if world == 1 else {})},
        "gpu_launches": gpu_launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": NCU_TRAFFIC_BYTES_PER_GEMV * group if world == 1 else None,
                     "peak_source": f"{peak_kind} copy bandwidth", "kernel": "qblk_gemv_grouped_kernel",
                     "bytes_per_launch": launch_bytes, "us_per_launch": kernel_s * 1e6},
        "clocks": clocks.summary(),
    }
    if verified is not None:
        line["verified"] = verified  # N > 1: fused peer-store gather == all-gathered single launches, bit for bit, on every rank
    op.close()
    if world > 1 and not args.no_secondary:
        # the column-sharded FP16 GEMM of the same run (BASELINE configs[2]), verified like the mat-vec step
        del blocks
        torch.cuda.empty_cache()
        line["secondary"] = {"hgemm_sharded": measure_hgemm_sharded(torch, dist, [4096, 8192], dev, world, rank, tensor_peak)}
        if not all(v["verified"] for v in line["secondary"]["hgemm_sharded"].values()):
            raise SystemExit("the sharded FP16 GEMM failed its verification")
    if rank == 0:
        if world == 1:
            line["cpu_baseline"] = cpu_reference(seconds_target=args.cpu_seconds)
            if not args.no_secondary:
                line["secondary"] = secondary_metrics(torch, lib, torch.cuda.Stream(device=dev), hbm_peak, tensor_peak)
        print(json.dumps(line))
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()


def measure_hgemm_sharded(torch, dist, sizes, dev, world, rank, tensor_peak):
    """FP16 GEMM with B and C sharded by N-columns over the ranks: the local tcgen05 GEMM alone, with the NCCL
    all-gather of the C column blocks, and with the gather fused into the epilogue (peer stores).  Every timing is
    the max over ranks.  `verified`: on every rank the fused result equals the NCCL-gathered one bit for bit, and
    sampled rows of the local block agree with an fp32 product of the same operands (relative L2 <= 2e-3)."""
    from tornadovm_b200.sharding import ShardedHgemm, shard_cols
    out = {}
    for n in sizes:
        g = torch.Generator(device=dev).manual_seed(7)  # the same A on every rank
        a = (torch.randn((n, n), device=dev, generator=g) / n**0.5).half()
        b_local = (torch.randn((n, shard_cols(n, world)), device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank)) / n**0.5).half()
        can_fuse = n % (8 * world) == 0
        op = ShardedHgemm(n, n, n, a, b_local, fused=can_fuse, layout="auto")

        align = torch.zeros(1, device=dev)

        def timed(fn, reps=10):
            for _ in range(3):
                fn()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if world > 1:
                # the ranks leave the host barrier at slightly different times; a tiny collective in front of the
                # start event aligns the GPUs themselves (it completes on a rank only when every rank has entered)
                with torch.cuda.stream(op.stream):
                    dist.all_reduce(align)
            e0.record(op.stream)
            for _ in range(reps):
                fn()
            e1.record(op.stream)
            op.stream.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / reps * 1e-3], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()

        def compute_only():
            with torch.cuda.stream(op.stream):
                op.compute()

        def fused():
            with torch.cuda.stream(op.stream):
                op.launch_fused()
        tc, tg = timed(compute_only), timed(lambda: op.launch(assemble=False))
        res = {"gpus": world, "compute_TFLOP/s": 2 * n**3 / tc / 1e12, "compute_ms": tc * 1e3,
               "compute_plus_nccl_gather_TFLOP/s": 2 * n**3 / tg / 1e12, "compute_plus_nccl_gather_ms": tg * 1e3,
               "frac_tensor_compute": 2 * n**3 / tc / 1e12 / (tensor_peak * world)}
        # the local block against an fp32 product of the same operands (rows sampled)
        rows = torch.tensor([0, 1, 127, n // 2 + 3, n - 129, n - 1], device=dev)
        with torch.cuda.stream(op.stream):
            c_local = op.compute()
        op.stream.synchronize()
        want = a[rows].float() @ b_local.float()
        ok = bool(((c_local[rows] - want).norm() / want.norm()).item() <= 2e-3)
        if op.slab is not None:
            tf = timed(fused)
            with torch.cuda.stream(op.stream):
                cf = op.launch_fused()
                cg = op.launch(assemble=op.layout == "assembled")
            op.stream.synchronize()
            op.check()
            same = bool(torch.equal(cf, cg))
            ok = ok and same
            res.update({"fused_epilogue_gather_TFLOP/s": 2 * n**3 / tf / 1e12, "fused_epilogue_gather_ms": tf * 1e3,
                        "fused_layout": op.layout, "fused_equals_gathered": same})
        flag = torch.tensor([1 if ok else 0], device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        res["verified"] = bool(flag.item())
        out[f"hgemm_{n}"] = res
        op.close()
        del op, a, b_local
    return out


def run_hgemm_sharded(args):
    """--sections hgemm_sharded under torch.distributed.run."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    _, tensor_peak, _ = measured_peaks()
    out = measure_hgemm_sharded(torch, dist, [int(v) for v in args.hgemm_sizes.split(",")], dev, world, rank, tensor_peak)
    if rank == 0:
        print(json.dumps({"sections": out}))
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()


def run_probe(args):
    """--sections probe --probe FMT,MODE,BATCH | hgemm,N: a handful of launches of one kernel on a small footprint
    (four 14336 x 4096 matrices, or one GEMM), for profiler captures."""
    import torch
    from tornadovm_b200.native import B200Native
    lib = B200Native.load()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    P = lambda t: C.c_void_p(t.data_ptr())
    S = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    what = args.probe.split(",")
    off = args.probe_offset  # operands this many bytes past a 128-byte line (16 / 24: behind a TornadoVM array header)

    def placed(t):
        """A copy of t's bytes `off` bytes past a 128-byte line; (keep-alive buffer, pointer)."""
        raw = torch.empty(t.numel() * t.element_size() + 256, dtype=torch.uint8, device=dev)
        at = (-raw.data_ptr()) % 128 + off
        raw[at:at + t.numel() * t.element_size()].copy_(t.contiguous().view(torch.uint8).reshape(-1))
        return raw, C.c_void_p(raw.data_ptr() + at)
    if what[0] == "hgemm":
        n = int(what[1])
        k = int(what[2]) if len(what) > 2 else n  # hgemm,N,K: an N x N result over K (a small K shows the epilogue)
        a = (torch.randn((n, k), device=dev) / k**0.5).half()
        b = (torch.randn((k, n), device=dev) / k**0.5).half()
        c = torch.empty((n, n), device=dev)
        (ka, pa), (kb, pb), (kc, pc) = placed(a), placed(b), placed(c)
        for _ in range(3):
            B200Native.call("tb200_hgemm_f32", n, n, k, pa, pb, pc, S)
    else:
        fmt, mode, batch = what[0], what[1], int(what[2])
        bb = 18 if fmt == "q4b" else 34
        w = torch.randint(0, 256, (4, ROWS * (COLS // 32) * bb), dtype=torch.uint8, device=dev)
        keep, pw = placed(w)
        per = w[0].numel()
        del w
        x = torch.randn((batch, COLS), device=dev)
        y = torch.empty((batch, ROWS), device=dev)
        n_ws = lib.tb200_qx_workspace_bytes(COLS, batch)
        ws = torch.empty(n_ws, dtype=torch.uint8, device=dev)
        for i in range(6):
            if mode == "int":
                B200Native.call(f"tb200_{fmt}_gemv_i8", ROWS, COLS, batch, C.c_void_p(pw.value + (i % 4) * per), P(x), P(y), P(ws), n_ws, S)
            else:
                B200Native.call(f"tb200_{fmt}_gemv", ROWS, COLS, batch, C.c_void_p(pw.value + (i % 4) * per), P(x), P(y), S)
    torch.cuda.synchronize()
    print(json.dumps({"probe": args.probe, "offset": off, "status": B200Native.device_status()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=8.0)
    ap.add_argument("--no-secondary", action="store_true")
    ap.add_argument("--group", type=int, default=LAYERS, help="matrices per launch (a divisor of the 32 per step)")
    ap.add_argument("--sections", default="", help="run only these secondary kernels (comma list of sgemv,q8,q8layers,q4,sgemm,hgemm; or hgemm_sharded under torch.distributed.run) and print their timings; for profiling")
    ap.add_argument("--probe", default="q8b,int,8", help="with --sections probe: FMT,MODE,BATCH (q8b|q4b, int|f32) or hgemm,N[,K]")
    ap.add_argument("--probe-offset", type=int, default=0, help="with --sections probe: bytes between a 128-byte line and the operands (a multiple of 8)")
    ap.add_argument("--hgemm-sizes", default="2048,4096,8192,16384")
    ap.add_argument("--hgemm-variant", default="pairs", choices=["pairs", "single"],
                    help="with --sections: 256x256 tiles on SM pairs (the default of the library) or 128x256 tiles on single SMs")
    args = ap.parse_args()
    if args.sections == "hgemm_sharded":
        run_hgemm_sharded(args)
    elif args.sections == "probe":
        run_probe(args)
    elif args.sections:
        import torch
        from tornadovm_b200.native import B200Native
        torch.cuda.set_device(0)
        hbm_peak, tensor_peak, _ = measured_peaks()
        lib = B200Native.load()
        lib.tb200_set_option(2, 1 if args.hgemm_variant == "pairs" else 0)
        res = secondary_metrics(torch, lib, torch.cuda.Stream(), hbm_peak, tensor_peak,
                                tuple(args.sections.split(",")), tuple(int(v) for v in args.hgemm_sizes.split(",")))
        print(json.dumps({"sections": res}))
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
