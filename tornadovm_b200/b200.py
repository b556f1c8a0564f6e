"""Factories of the ``b200/linalg`` library tasks.

Python twin of the Java class ``B200``; same shape as ``Cutlass``
(tornado-cutlass/.../Cutlass.java:44-191) and ``CuBlas``
(tornado-cublas/.../CuBlas.java:97-305): each factory validates shapes early
with a clear message and returns a LibraryTaskDescriptor whose parameter list
is what the provider later receives positionally.
"""
from __future__ import annotations

from dataclasses import dataclass

from .arrays import BFloat16Array, ByteArray, FloatArray, HalfFloatArray, Int8Array
from .descriptor import Access, LibraryTaskDescriptor

LIBRARY_NAME = "b200/linalg"
MAX_BATCH = 16
MAX_GROUP = 32
#: TaskGraph.libraryTask takes at most 20 arguments (TaskGraph.java:886): rows, cols, batch, x, y, options + 14 matrices
MAX_GROUP_TASK_ARGS = 14


@dataclass
class B200Options:
    """Per-call tuning object (LibraryTaskDescriptor.withTuning):
    ``exact_int`` selects the int8-activation / int32 block-dot arithmetic for
    the quantised mat-vec tasks; ``overlap_launches`` lets consecutive mat-vec
    kernels of the plan overlap (each prefetches its weights while the kernel
    before it drains), which requires that no task writes a weight array
    immediately before the mat-vec that reads it; ``host_results`` lets the
    grouped and packed mat-vec kernels store every result into the output array's pinned,
    device-mapped host segment as well as into its device buffer, when the
    graph copies that array to the host after every execution -- the plan
    then has no device-to-host copy left to issue for it."""
    exact_int: bool = False
    overlap_launches: bool = False
    host_results: bool = False


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError("[ERROR] " + msg)


def _desc(function, params, out_index, read_write=False, tuning=None):
    access = [Access.READ_ONLY] * len(params)
    access[out_index] = Access.READ_WRITE if read_write else Access.WRITE_ONLY
    d = LibraryTaskDescriptor().withLibrary(LIBRARY_NAME).withFunction(function).withParameters(params).withAccess(access)
    if tuning is not None:
        d.withTuning(tuning)
    return d


class B200:
    LIBRARY_NAME = LIBRARY_NAME

    @staticmethod
    def sgemv(rows: int, cols: int, m: FloatArray, v: FloatArray, out: FloatArray):
        """out[i] = sum_j m[i*cols+j] * v[j] (README mxv, README.md:35-47)."""
        _check(rows >= 0 and cols >= 0, f"B200 sgemv requires non-negative sizes; got rows={rows}, cols={cols}")
        _check(m.getSize() >= rows * cols and v.getSize() >= cols and out.getSize() >= rows,
               "B200 sgemv: array smaller than rows x cols")
        return _desc("sgemv", [rows, cols, m, v, out], 4)

    @staticmethod
    def _check_q(name, rows, cols, batch, x, y):
        _check(cols % 32 == 0, f"B200 {name} requires cols to be a multiple of the 32-element block; got cols={cols}")
        _check(1 <= batch <= MAX_BATCH, f"B200 {name} requires 1 <= batch <= {MAX_BATCH}; got {batch}")
        _check(x.getSize() >= batch * cols and y.getSize() >= batch * rows, f"B200 {name}: x or y too small")

    @staticmethod
    def q8Gemv(rows, cols, batch, q: Int8Array, scales: HalfFloatArray, x: FloatArray, y: FloatArray, options=None):  # noqa: N802
        """Q8_0 mat-vec, split layout (matrixVectorGenericFinal, MatrixVectorRowMajor.java:409-423)."""
        B200._check_q("q8Gemv", rows, cols, batch, x, y)
        _check(q.getSize() >= rows * cols and scales.getSize() >= rows * cols // 32, "B200 q8Gemv: weights too small")
        return _desc("q8Gemv", [rows, cols, batch, q, scales, x, y], 6, tuning=options)

    @staticmethod
    def q8GemvBytes(rows, cols, batch, blocks: ByteArray, x: FloatArray, y: FloatArray, options=None):  # noqa: N802
        """Q8_0 mat-vec, 34-byte blocks (matrixVectorGenericQ8Byte, MatrixVectorRowMajor.java:428-524)."""
        B200._check_q("q8GemvBytes", rows, cols, batch, x, y)
        _check(blocks.getSize() >= rows * (cols // 32) * 34, "B200 q8GemvBytes: weights too small")
        return _desc("q8GemvBytes", [rows, cols, batch, blocks, x, y], 5, tuning=options)

    @staticmethod
    def q4GemvBytes(rows, cols, batch, blocks: ByteArray, x: FloatArray, y: FloatArray, options=None):  # noqa: N802
        """Q4_0 mat-vec, 18-byte blocks."""
        B200._check_q("q4GemvBytes", rows, cols, batch, x, y)
        _check(blocks.getSize() >= rows * (cols // 32) * 18, "B200 q4GemvBytes: weights too small")
        return _desc("q4GemvBytes", [rows, cols, batch, blocks, x, y], 5, tuning=options)

    @staticmethod
    def _grouped(name, block_bytes, rows, cols, batch, x, y, blocks, options):
        B200._check_q(name, rows, cols, batch, x, y)
        _check(1 <= len(blocks) <= MAX_GROUP_TASK_ARGS,
               f"B200 {name} requires 1 to {MAX_GROUP_TASK_ARGS} matrices (a library task carries 20 arguments); got {len(blocks)}; "
               f"use {name.replace('Grouped', 'Packed')} for up to {MAX_GROUP}")
        _check(y.getSize() >= len(blocks) * batch * rows, f"B200 {name}: y smaller than count x batch x rows")
        for b in blocks:
            _check(b.getSize() >= rows * (cols // 32) * block_bytes, f"B200 {name}: weights too small")
        _check(options is None or options.exact_int, f"B200 {name} computes in integer mode; exact_int must be set")
        return _desc(name, [len(blocks), rows, cols, batch, x, y, *blocks], 5, tuning=options or B200Options(exact_int=True))

    @staticmethod
    def q8GemvBytesGrouped(rows, cols, batch, x: FloatArray, y: FloatArray, *blocks: ByteArray, options=None):  # noqa: N802
        """Integer-mode Q8_0 mat-vec of several equally shaped matrices on the same activations in one launch:
        y[m][b][r] for matrix m.  The reference launches one task per matrix; its batched interfaces are the
        strided GEMMs (CuBlas.cublasSgemmStridedBatched, CuBlas.java:206-228)."""
        return B200._grouped("q8GemvBytesGrouped", 34, rows, cols, batch, x, y, blocks, options)

    @staticmethod
    def q4GemvBytesGrouped(rows, cols, batch, x: FloatArray, y: FloatArray, *blocks: ByteArray, options=None):  # noqa: N802
        """Q4_0 twin of q8GemvBytesGrouped."""
        return B200._grouped("q4GemvBytesGrouped", 18, rows, cols, batch, x, y, blocks, options)

    @staticmethod
    def _packed(name, block_bytes, count, rows, cols, batch, blocks, x, y, options):
        B200._check_q(name, rows, cols, batch, x, y)
        _check(1 <= count <= MAX_GROUP, f"B200 {name} requires 1 to {MAX_GROUP} matrices; got {count}")
        per = rows * (cols // 32) * block_bytes
        _check(count == 1 or per % 16 == 0, f"B200 {name} requires matrices of a multiple of 16 bytes; got {per}")
        _check(blocks.getSize() >= count * per, f"B200 {name}: weights smaller than count x rows x cols/32 x {block_bytes}")
        _check(y.getSize() >= count * batch * rows, f"B200 {name}: y smaller than count x batch x rows")
        _check(options is None or options.exact_int, f"B200 {name} computes in integer mode; exact_int must be set")
        return _desc(name, [count, rows, cols, batch, blocks, x, y], 6, tuning=options or B200Options(exact_int=True))

    @staticmethod
    def q8GemvBytesPacked(count, rows, cols, batch, blocks: ByteArray, x: FloatArray, y: FloatArray, options=None):  # noqa: N802
        """The grouped integer-mode mat-vec with its ``count`` (<= 32) equally shaped matrices back to back in ONE
        ByteArray, matrix m at byte m * rows * cols/32 * 34: seven arguments whatever the count, so that a whole
        decode step fits the 20-argument library-task interface (TaskGraph.java:886).  y is [count][batch][rows]."""
        return B200._packed("q8GemvBytesPacked", 34, count, rows, cols, batch, blocks, x, y, options)

    @staticmethod
    def q4GemvBytesPacked(count, rows, cols, batch, blocks: ByteArray, x: FloatArray, y: FloatArray, options=None):  # noqa: N802
        """Q4_0 twin of q8GemvBytesPacked (18-byte blocks)."""
        return B200._packed("q4GemvBytesPacked", 18, count, rows, cols, batch, blocks, x, y, options)

    @staticmethod
    def sgemm(m, n, k, alpha, a: FloatArray, b: FloatArray, beta, c: FloatArray):
        """C = alpha*A*B + beta*C, row-major; signature of Cutlass.cutlassSgemm (Cutlass.java:57-66)."""
        _check(m >= 0 and n >= 0 and k >= 0, f"B200 sgemm requires non-negative sizes; got m={m}, n={n}, k={k}")
        _check(a.getSize() >= m * k and b.getSize() >= k * n and c.getSize() >= m * n, "B200 sgemm: array too small")
        return _desc("sgemm", [m, n, k, float(alpha), a, b, float(beta), c], 7, read_write=(beta != 0.0))

    @staticmethod
    def hgemmF32(m, n, k, a: HalfFloatArray, b: HalfFloatArray, c: FloatArray):  # noqa: N802
        """C(fp32) = A(fp16) * B(fp16), row-major (operands of CuBlas.cublasGemmExFP16FP32, CuBlas.java:261-279)."""
        _check(m >= 0 and n >= 0 and k >= 0, f"B200 hgemmF32 requires non-negative sizes; got m={m}, n={n}, k={k}")
        _check(a.getSize() >= m * k and b.getSize() >= k * n and c.getSize() >= m * n, "B200 hgemmF32: array too small")
        return _desc("hgemmF32", [m, n, k, a, b, c], 5)

    # ---- fused epilogues, typed outputs, batches (tb200_gemm_ex) ---------------------------------------
    @staticmethod
    def _check_tc(name, m, n, k):
        _check(m >= 0 and n >= 0 and k >= 0, f"B200 {name} requires non-negative sizes; got m={m}, n={n}, k={k}")
        # the tensor-core tiles are fetched by TMA: rows of A and B must be multiples of 16 bytes (cf. Cutlass.java:68-77)
        _check(k % 8 == 0 and n % 8 == 0, f"B200 {name} requires k and n to be multiples of 8; got k={k}, n={n}")

    @staticmethod
    def hgemm(m, n, k, alpha, a: HalfFloatArray, b: HalfFloatArray, beta, d: HalfFloatArray):
        """D(fp16) = alpha*A*B + beta*D, fp32 accumulation; signature of Cutlass.cutlassHgemm (Cutlass.java:83-100)."""
        B200._check_tc("hgemm", m, n, k)
        _check(a.getSize() >= m * k and b.getSize() >= k * n and d.getSize() >= m * n, "B200 hgemm: array too small")
        return _desc("hgemm", [m, n, k, float(alpha), a, b, float(beta), d], 7, read_write=(beta != 0.0))

    @staticmethod
    def bgemm(m, n, k, alpha, a: BFloat16Array, b: BFloat16Array, beta, d: BFloat16Array):
        """bfloat16 twin of hgemm; signature of Cutlass.cutlassBgemm (Cutlass.java:102-117)."""
        B200._check_tc("bgemm", m, n, k)
        _check(a.getSize() >= m * k and b.getSize() >= k * n and d.getSize() >= m * n, "B200 bgemm: array too small")
        return _desc("bgemm", [m, n, k, float(alpha), a, b, float(beta), d], 7, read_write=(beta != 0.0))

    @staticmethod
    def _gemm_bias(act, m, n, k, a, b, bias, d):
        name = "gemmBias" + act
        B200._check_tc(name, m, n, k)
        _check(a.getSize() >= m * k and b.getSize() >= k * n and bias.getSize() >= n and d.getSize() >= m * n,
               f"B200 {name}: array too small")
        return _desc(name, [m, n, k, a, b, bias, d], 6)

    @staticmethod
    def gemmBiasRelu(m, n, k, a: HalfFloatArray, b: HalfFloatArray, bias: HalfFloatArray, d: HalfFloatArray):  # noqa: N802
        """D = relu(A*B + bias), bias broadcast over the rows; Cutlass.cutlassGemmBiasRelu (Cutlass.java:119-125)."""
        return B200._gemm_bias("Relu", m, n, k, a, b, bias, d)

    @staticmethod
    def gemmBiasGelu(m, n, k, a, b, bias, d):  # noqa: N802
        """Cutlass.cutlassGemmBiasGelu (Cutlass.java:127-135), erf form."""
        return B200._gemm_bias("Gelu", m, n, k, a, b, bias, d)

    @staticmethod
    def gemmBiasSilu(m, n, k, a, b, bias, d):  # noqa: N802
        return B200._gemm_bias("Silu", m, n, k, a, b, bias, d)

    @staticmethod
    def gemmBiasSigmoid(m, n, k, a, b, bias, d):  # noqa: N802
        return B200._gemm_bias("Sigmoid", m, n, k, a, b, bias, d)

    @staticmethod
    def gemmBiasTanh(m, n, k, a, b, bias, d):  # noqa: N802
        return B200._gemm_bias("Tanh", m, n, k, a, b, bias, d)

    @staticmethod
    def gemmBiasHardSwish(m, n, k, a, b, bias, d):  # noqa: N802
        return B200._gemm_bias("HardSwish", m, n, k, a, b, bias, d)

    @staticmethod
    def hgemmBatched(m, n, k, alpha, a: HalfFloatArray, b: HalfFloatArray, beta, d: HalfFloatArray, batchCount):  # noqa: N802,N803
        """batchCount independent fp16 GEMMs packed back to back; Cutlass.cutlassHgemmBatched (Cutlass.java:177-191)."""
        B200._check_tc("hgemmBatched", m, n, k)
        _check(batchCount >= 1, f"B200 hgemmBatched requires batchCount >= 1; got {batchCount}")
        _check(a.getSize() >= batchCount * m * k and b.getSize() >= batchCount * k * n and d.getSize() >= batchCount * m * n,
               "B200 hgemmBatched: array too small")
        return _desc("hgemmBatched", [m, n, k, float(alpha), a, b, float(beta), d, batchCount], 7, read_write=(beta != 0.0))
