"""The library tasks driven the way TornadoVM drives them: TaskGraph -> plan -> provider -> C ABI."""
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
                assert np.array_equal(got[m], ys[m].numpy())
    with pytest.raises(RuntimeError, match="1 to 32 matrices"):
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
