"""The library tasks driven the way TornadoVM drives them: TaskGraph -> plan -> provider -> C ABI."""
import functools

import numpy as np
import pytest

import oracle as o
from tornadovm_b200 import arrays
from tornadovm_b200.arrays import ByteArray, FloatArray, HalfFloatArray, Int8Array
from tornadovm_b200.b200 import B200, B200Options
from tornadovm_b200.taskgraph import DataTransferMode, TaskGraph, TornadoExecutionPlan

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("header", [16, 24])
@pytest.mark.parametrize("cuda_graph", [False, True])
def test_readme_mxv_as_library_task(header, cuda_graph):
    """README.md:93-109 host code with the mxv task replaced by B200::sgemv."""
    rows, cols = 512, 2048
    m_h, v_h = o.make_sgemv(rows, cols)
    m, v, out = FloatArray(m_h, header), FloatArray(v_h, header), FloatArray(rows, header)
    tg = (TaskGraph("s0")
          .transferToDevice(DataTransferMode.FIRST_EXECUTION, m, v)
          .libraryTask("mxv", B200.sgemv, rows, cols, m, v, out)
          .transferToHost(DataTransferMode.EVERY_EXECUTION, out))
    with TornadoExecutionPlan(tg.snapshot()) as plan:
        if cuda_graph:
            plan.withCUDAGraph()
        for _ in range(3):
            out.numpy()[:] = np.nan
            plan.execute()
            assert o.rel_l2(out.numpy(), o.sgemv_f64(m_h, v_h, cols, rows)) <= 1e-5


@pytest.mark.parametrize("exact_int", [False, True])
def test_q8_decode_graph_with_changing_activations(exact_int):
    rows, cols, batch = 256, 4096, 2
    q_h, s_h, x_h = o.make_q8(rows, cols, batch)
    q, s, x, y = Int8Array(q_h), HalfFloatArray(s_h), FloatArray(x_h), FloatArray(rows * batch)
    blocks, yb = ByteArray(o.q8_pack_blocks(q_h, s_h)), FloatArray(rows * batch)
    opts = B200Options(exact_int=exact_int)
    tg = (TaskGraph("decode")
          .transferToDevice(DataTransferMode.FIRST_EXECUTION, q, s, blocks)
          .transferToDevice(DataTransferMode.EVERY_EXECUTION, x)
          .libraryTask("split", B200.q8Gemv, rows, cols, batch, q, s, x, y, opts)
          .libraryTask("bytes", B200.q8GemvBytes, rows, cols, batch, blocks, x, yb, opts)
          .transferToHost(DataTransferMode.EVERY_EXECUTION, y, yb))
    with TornadoExecutionPlan(tg).withCUDAGraph() as plan:
        for it in range(3):
            x.numpy()[:] = o.JavaRandom(100 + it).gaussian_f32(cols * batch)
            plan.execute()
            xs = x.numpy()
            want = np.stack([o.q8_gemv_f64(q_h, s_h, np.ascontiguousarray(xs[b * cols:(b + 1) * cols]), cols, rows) for b in range(batch)])
            tol = 2e-2 if exact_int else 1e-5  # int mode carries the activation quantisation error
            assert o.rel_l2(y.numpy().reshape(batch, rows), want) <= tol
            assert o.rel_l2(yb.numpy().reshape(batch, rows), want) <= tol
            if exact_int:
                # both layouts see the same exact block dots and scales; only the fp32 summation order differs
                assert o.rel_l2(y.numpy(), yb.numpy()) <= 1e-6


def test_grouped_q8_task_equals_separate_tasks():
    """One grouped task for the matrices that read the same vector gives the results of one task per matrix."""
    rows, cols, batch, count = 192, 2048, 2, 3
    mats = []
    for m in range(count):
        q_h, s_h, x_h = o.make_q8(rows, cols, batch, 300 + m)
        mats.append(ByteArray(o.q8_pack_blocks(q_h, s_h)))
    x = FloatArray(o.JavaRandom(9).gaussian_f32(cols * batch))
    ys = [FloatArray(rows * batch) for _ in range(count)]
    yg = FloatArray(count * rows * batch)
    opts = B200Options(exact_int=True)
    tg = TaskGraph("layer").transferToDevice(DataTransferMode.FIRST_EXECUTION, *mats).transferToDevice(DataTransferMode.EVERY_EXECUTION, x)
    for m in range(count):
        tg.libraryTask(f"one{m}", B200.q8GemvBytes, rows, cols, batch, mats[m], x, ys[m], opts)
    tg.libraryTask("all", B200.q8GemvBytesGrouped, rows, cols, batch, x, yg, *mats)
    tg.transferToHost(DataTransferMode.EVERY_EXECUTION, yg, *ys)
    with TornadoExecutionPlan(tg).withCUDAGraph() as plan:
        for it in range(2):
            x.numpy()[:] = o.JavaRandom(50 + it).gaussian_f32(cols * batch)
            plan.execute()
            got = yg.numpy().reshape(count, batch * rows)
            for m in range(count):
                # the same exact block dots and scales; the one-matrix tasks of two vectors run on the tensor-core
                # kernel, the grouped task on the dp4a kernel, so only the fp32 summation order differs
                assert o.rel_l2(got[m], ys[m].numpy()) <= 1e-6
    with pytest.raises(RuntimeError, match="1 to 14 matrices"):
        B200.q8GemvBytesGrouped(rows, cols, batch, x, yg)


def test_gemm_tasks_and_header_override():
    old = arrays.ARRAY_HEADER
    try:
        arrays.ARRAY_HEADER = 24  # the launcher's JVM mode: element pointers are 8 modulo 16
        n = 128
        a_h, b_h = o.make_sgemm(n, n, n)
        a, b, c = FloatArray(a_h), FloatArray(b_h), FloatArray(n * n)
        ha_h, hb_h = o.make_hgemm(n, n, n)
        ha, hb, hc = HalfFloatArray(ha_h), HalfFloatArray(hb_h), FloatArray(n * n)
        tg = (TaskGraph("mm")
              .transferToDevice(DataTransferMode.EVERY_EXECUTION, a, b, ha, hb)
              .libraryTask("sgemm", B200.sgemm, n, n, n, 1.0, a, b, 0.0, c)
              .libraryTask("hgemm", B200.hgemmF32, n, n, n, ha, hb, hc)
              .transferToHost(DataTransferMode.EVERY_EXECUTION, c, hc))
        with TornadoExecutionPlan(tg) as plan:
            plan.execute()
        assert o.rel_l2(c.numpy(), o.sgemm_f64(a_h, b_h, n, n, n)) <= 1e-5
        assert o.rel_l2(hc.numpy(), o.hgemm_ref(ha_h, hb_h, n, n, n)) <= 2e-3
    finally:
        arrays.ARRAY_HEADER = old


def test_native_status_becomes_exception():
    from tornadovm_b200.native import TornadoB200Error
    rows, cols = 4, 64
    q, s, x, y = Int8Array(rows * cols), HalfFloatArray(rows * 2), FloatArray(cols), FloatArray(rows)
    tg = TaskGraph("bad").libraryTask("t", B200.q8Gemv, rows, cols, 1, q, s, x, y)
    tg.tasks[0].descriptor.getParameters()[1] = 33  # corrupt cols after the factory's check
    with TornadoExecutionPlan(tg) as plan:
        with pytest.raises(TornadoB200Error, match=r"\[ERROR\] q8Gemv failed with status: TB200_ERR_INVALID_ARG"):
            plan.execute()


def test_in_out_task_under_cuda_graph_runs_once_per_execute():
    """C = A*B + C with withCUDAGraph(): every execute() applies the task exactly once, the first one
    included (its launch is captured, not run twice)."""
    n = 128
    a_h, b_h = o.JavaRandom(1).uniform_f32(n * n, 0, 1), o.JavaRandom(2).uniform_f32(n * n, 0, 1)
    a, b, c = FloatArray(a_h), FloatArray(b_h), FloatArray(np.zeros(n * n, np.float32))
    tg = (TaskGraph("acc")
          .transferToDevice(DataTransferMode.FIRST_EXECUTION, a, b, c)
          .libraryTask("sgemm", B200.sgemm, n, n, n, 1.0, a, b, 1.0, c)
          .transferToHost(DataTransferMode.EVERY_EXECUTION, c))
    ab = o.sgemm_f64(a_h, b_h, n, n, n).ravel()
    with TornadoExecutionPlan(tg).withCUDAGraph() as plan:
        for k in (1, 2, 3):
            plan.execute()
            assert o.rel_l2(c.numpy(), k * ab) <= 1e-5, k


def test_first_dispatch_of_every_factory_is_captured():
    """The reference captures the FIRST execution of a plan (TornadoVMInterpreter.java:462-476): prepare() must
    have made every kernel resident, so a fresh plan with one task of each factory captures and replays."""
    rows, cols, batch, n = 128, 4096, 8, 256
    q_h, s_h, x_h = o.make_q8(rows, cols, batch, 77)
    blk_h = o.q8_pack_blocks(q_h, s_h)
    q4_h, _, _ = o.make_q4(rows, cols, batch, 78)
    m_h, v_h = o.make_sgemv(rows, cols, 79)
    ha_h, hb_h = o.make_hgemm(n, n, n, 80)
    fa_h, fb_h = o.JavaRandom(81).uniform_f32(n * n, 0, 1), o.JavaRandom(82).uniform_f32(n * n, 0, 1)
    q, s, x = Int8Array(q_h), HalfFloatArray(s_h), FloatArray(x_h)
    blk, q4 = ByteArray(blk_h), ByteArray(q4_h)
    packed = ByteArray(np.concatenate([blk_h, blk_h]))
    m, v, out = FloatArray(m_h), FloatArray(v_h), FloatArray(rows)
    ha, hb, hc = HalfFloatArray(ha_h), HalfFloatArray(hb_h), FloatArray(n * n)
    fa, fb, fc = FloatArray(fa_h), FloatArray(fb_h), FloatArray(n * n)
    ys = [FloatArray(rows * batch) for _ in range(6)]
    yp = FloatArray(2 * rows * batch)
    exact, flt = B200Options(exact_int=True, overlap_launches=True), B200Options()
    tg = (TaskGraph("all")
          .transferToDevice(DataTransferMode.FIRST_EXECUTION, q, s, blk, q4, packed, m, v, ha, hb, fa, fb)
          .transferToDevice(DataTransferMode.EVERY_EXECUTION, x)
          .libraryTask("t0", B200.sgemv, rows, cols, m, v, out)
          .libraryTask("t1", B200.q8Gemv, rows, cols, batch, q, s, x, ys[0], flt)
          .libraryTask("t2", B200.q8Gemv, rows, cols, batch, q, s, x, ys[1], exact)
          .libraryTask("t3", B200.q8GemvBytes, rows, cols, batch, blk, x, ys[2], flt)
          .libraryTask("t4", B200.q8GemvBytes, rows, cols, batch, blk, x, ys[3], exact)
          .libraryTask("t5", B200.q4GemvBytes, rows, cols, batch, q4, x, ys[4], flt)
          .libraryTask("t6", B200.q4GemvBytes, rows, cols, batch, q4, x, ys[5], exact)
          .libraryTask("t7", B200.q8GemvBytesPacked, 2, rows, cols, 2, packed, x, yp)
          .libraryTask("t8", B200.sgemm, n, n, n, 1.0, fa, fb, 0.0, fc)
          .libraryTask("t9", B200.hgemmF32, n, n, n, ha, hb, hc)
          .transferToHost(DataTransferMode.EVERY_EXECUTION, out, fc, hc, yp, *ys))
    with TornadoExecutionPlan(tg).withCUDAGraph() as plan:
        for _ in range(2):
            plan.execute()
            xs = np.ascontiguousarray(x.numpy())
            f64 = np.stack([o.q8_gemv_f64(q_h, s_h, xs[b * cols:(b + 1) * cols], cols, rows) for b in range(batch)])
            assert o.rel_l2(out.numpy(), o.sgemv_f64(m_h, v_h, cols, rows)) <= 1e-5
            assert o.rel_l2(ys[0].numpy().reshape(batch, rows), f64) <= 1e-5
            assert o.rel_l2(ys[2].numpy().reshape(batch, rows), f64) <= 1e-5
            assert o.rel_l2(ys[1].numpy().reshape(batch, rows), f64) <= 2e-2
            # same exact block dots, different fp32 summation order (tensor-core kernel vs dp4a kernel)
            assert o.rel_l2(yp.numpy()[:2 * 2 * rows].reshape(2, 2, rows)[0], ys[3].numpy().reshape(batch, rows)[:2]) <= 1e-6
            q4f = np.stack([o.q4_gemv_f64(q4_h, xs[b * cols:(b + 1) * cols], cols, rows) for b in range(batch)])
            assert o.rel_l2(ys[4].numpy().reshape(batch, rows), q4f) <= 1e-5
            assert o.rel_l2(ys[5].numpy().reshape(batch, rows), q4f) <= 2e-2
            assert o.rel_l2(fc.numpy(), o.sgemm_f64(fa_h, fb_h, n, n, n)) <= 1e-5
            assert o.rel_l2(hc.numpy(), o.hgemm_ref(ha_h, hb_h, n, n, n)) <= 2e-3


def test_library_task_argument_limit():
    """A library task carries at most 20 arguments (TaskGraph.java:886); the grouped factory therefore
    stops at 14 matrices and the packed form carries up to 32 in one ByteArray."""
    rows, cols = 4, 256
    x, y = FloatArray(cols), FloatArray(32 * rows)
    mats = [ByteArray(rows * (cols // 32) * 34) for _ in range(16)]
    with pytest.raises(RuntimeError, match="1 to 14 matrices"):
        B200.q8GemvBytesGrouped(rows, cols, 1, x, y, *mats)
    with pytest.raises(TypeError, match="1 to 20 task arguments"):
        TaskGraph("big").libraryTask("t", B200.q8GemvBytesGrouped, rows, cols, 1, x, y, *mats)
    B200.q8GemvBytesPacked(32, rows, cols, 1, ByteArray(32 * rows * (cols // 32) * 34), x, y)


def test_two_layer_mlp_of_fused_gemm_tasks():
    """h = relu(x*W1 + b1), y = gelu(h*W2 + b2) as two fused library tasks in one captured plan
    (TestCutlass.java:727-770), plus a bf16 GEMM and a batched fp16 GEMM task."""
    from tornadovm_b200.arrays import BFloat16Array
    m, n1, n2, k = 64, 128, 64, 64
    r = o.JavaRandom(4)
    x_f, w1_f, w2_f = r.uniform_f32(m * k, -1, 1), r.uniform_f32(k * n1, -1, 1) * 0.2, r.uniform_f32(n1 * n2, -1, 1) * 0.2
    b1_f, b2_f = r.uniform_f32(n1, -1, 1), r.uniform_f32(n2, -1, 1)
    x, w1, w2 = HalfFloatArray.from_float32(x_f), HalfFloatArray.from_float32(w1_f), HalfFloatArray.from_float32(w2_f)
    b1, b2 = HalfFloatArray.from_float32(b1_f), HalfFloatArray.from_float32(b2_f)
    h, y = HalfFloatArray(m * n1), HalfFloatArray(m * n2)
    ba, bb, bc = BFloat16Array.from_float32(x_f), BFloat16Array.from_float32(w1_f), BFloat16Array(m * n1)
    ga, gb, gd = HalfFloatArray.from_float32(np.tile(x_f, 3)), HalfFloatArray.from_float32(np.tile(w1_f, 3)), HalfFloatArray(3 * m * n1)
    tg = (TaskGraph("mlp")
          .transferToDevice(DataTransferMode.EVERY_EXECUTION, x, w1, w2, b1, b2, ba, bb, ga, gb)
          .libraryTask("layer1", B200.gemmBiasRelu, m, n1, k, x, w1, b1, h)
          .libraryTask("layer2", B200.gemmBiasGelu, m, n2, n1, h, w2, b2, y)
          .libraryTask("bf16", B200.bgemm, m, n1, k, 1.0, ba, bb, 0.0, bc)
          .libraryTask("batched", B200.hgemmBatched, m, n1, k, 1.0, ga, gb, 0.0, gd, 3)
          .transferToHost(DataTransferMode.EVERY_EXECUTION, h, y, bc, gd))
    with TornadoExecutionPlan(tg).withCUDAGraph() as plan:
        for _ in range(2):
            plan.execute()
    xh, w1h, w2h = x.to_float32(), w1.to_float32(), w2.to_float32()
    h_ref = o.gemm_epilogue_ref(o.sgemm_seq(xh, w1h, m, n1, k), "relu", bias=b1.to_float32())
    assert np.abs(h.to_float32().reshape(m, n1) - h_ref).max() <= 0.05
    # layer 2 reads the fp16 h the device produced, as the reference's chained tasks do
    y_ref = o.gemm_epilogue_ref(o.sgemm_seq(h.to_float32(), w2h, m, n2, n1), "gelu", bias=b2.to_float32())
    assert np.abs(y.to_float32().reshape(m, n2) - y_ref).max() <= 0.1  # TestCutlass.java:769
    bf_ref = o.sgemm_seq(ba.to_float32(), bb.to_float32(), m, n1, k)
    assert (np.abs(bc.to_float32().reshape(m, n1) - bf_ref) <= 5e-2 * np.maximum(1.0, np.abs(bf_ref))).all()
    g_ref = o.sgemm_seq(xh, w1h, m, n1, k)
    for i in range(3):
        assert np.abs(gd.to_float32().reshape(3, m, n1)[i] - g_ref).max() <= 0.05


@pytest.mark.parametrize("header", [16, 24])
@pytest.mark.parametrize("fmt", ["q8", "q4"])
@pytest.mark.parametrize("batch", [1, 2])
def test_packed_results_stored_on_the_host_by_the_kernel(header, fmt, batch):
    """B200Options(host_results=True): the packed mat-vec stores into the output array's pinned host segment as well
    as into its device buffer, and the plan issues no copy back for that array.  Same bits as the plan that copies,
    over executions with changing activations (the later ones replayed from the captured graph), and the integer
    block dots of the oracle.  Two vectors take a one-destination kernel: there the plan keeps its copy."""
    count, rows, cols = 3, 130, 1024
    mats = []
    for m in range(count):
        if fmt == "q8":
            q, s, _ = o.make_q8(rows, cols, batch, 40 + m)
            mats.append((o.q8_pack_blocks(q, s), q, s))
        else:
            blocks, s, _ = o.make_q4(rows, cols, batch, 40 + m)
            mats.append((blocks, None, s))
    packed_h = np.concatenate([b for b, _, _ in mats])
    factory = B200.q8GemvBytesPacked if fmt == "q8" else B200.q4GemvBytesPacked
    grouped = B200.q8GemvBytesGrouped if fmt == "q8" else B200.q4GemvBytesGrouped
    results = {}
    for host_results in (False, True):
        packed, x = ByteArray(packed_h, header), FloatArray(cols * batch, header)
        y, z, u = FloatArray(count * batch * rows, header), FloatArray(rows, header), FloatArray(2 * batch * rows, header)
        sep = [ByteArray(mats[m][0], header) for m in range(2)]  # the grouped form: one array per matrix
        opts = B200Options(exact_int=True, overlap_launches=True, host_results=host_results)
        tg = (TaskGraph("packed")
              .transferToDevice(DataTransferMode.FIRST_EXECUTION, packed, *sep)
              .transferToDevice(DataTransferMode.EVERY_EXECUTION, x)
              .libraryTask("g", factory, count, rows, cols, batch, packed, x, y, opts)
              .libraryTask("s", functools.partial(grouped, options=opts), rows, cols, batch, x, u, *sep)
              # a second task whose output always travels by copy
              .libraryTask("one", factory, 1, rows, cols, 1, packed, x, z, B200Options(exact_int=True))
              .transferToHost(DataTransferMode.EVERY_EXECUTION, y, z, u))
        got = []
        with TornadoExecutionPlan(tg).withCUDAGraph() as plan:
            for it in range(4):
                x.numpy()[:] = o.JavaRandom(300 + it).gaussian_f32(cols * batch)
                for out in (y, z, u):
                    out.numpy()[:] = np.nan
                plan.execute()
                got.append((y.numpy().copy(), z.numpy().copy(), u.numpy().copy()))
                assert plan.d2h_bytes_last == y.nbytes_with_header + z.nbytes_with_header + u.nbytes_with_header
                # the grouped task multiplies the first two matrices of the packed one
                assert np.array_equal(got[-1][2], got[-1][0][:2 * batch * rows])
            skipped = [key for key in plan._d2h_cache if id(y) in key and id(u) in key]
            assert bool(skipped) == (host_results and batch == 1)
            assert y.getSize() == count * batch * rows  # the header on the host is untouched
        results[host_results] = got
        xs = x.numpy()
        for m, (blocks, q, s) in enumerate(mats):
            for b in range(batch):
                xq, xsc = o.quantize_x_block(np.ascontiguousarray(xs[b * cols:(b + 1) * cols]))
                dots = o.q8_blockdots_i32(q, xq, cols, rows) if fmt == "q8" else o.q4_blockdots_i32(blocks, xq, cols, rows)
                want = o.blockdots_combine_f64(dots, s, xsc, cols // 32, rows)
                assert o.rel_l2(got[-1][0].reshape(count, batch, rows)[m, b], want) <= 1e-5
    for (ya, za, ua), (yb, zb, ub) in zip(results[False], results[True]):
        assert np.array_equal(ya, yb) and np.array_equal(za, zb) and np.array_equal(ua, ub)
