package uk.ac.manchester.tornado.b200;

import java.util.Arrays;

import uk.ac.manchester.tornado.api.common.Access;
import uk.ac.manchester.tornado.api.common.LibraryTaskDescriptor;
import uk.ac.manchester.tornado.api.exceptions.TornadoRuntimeException;
import uk.ac.manchester.tornado.api.types.arrays.BFloat16Array;
import uk.ac.manchester.tornado.api.types.arrays.ByteArray;
import uk.ac.manchester.tornado.api.types.arrays.FloatArray;
import uk.ac.manchester.tornado.api.types.arrays.HalfFloatArray;
import uk.ac.manchester.tornado.api.types.arrays.Int8Array;

/**
 * Factories of the {@code b200/linalg} library tasks: dense and quantised matrix-vector and
 * matrix-matrix products on hand-written sm_100a kernels. Each factory validates shapes early and
 * returns the descriptor whose parameters the provider later receives positionally.
 */
public final class B200 {

    public static final String LIBRARY_NAME = "b200/linalg";
    public static final int MAX_BATCH = 16;

    private B200() {
    }

    private static void check(boolean ok, String message) {
        if (!ok) {
            throw new TornadoRuntimeException("[ERROR] " + message);
        }
    }

    private static LibraryTaskDescriptor descriptor(String function, Object[] params, int out, boolean readWrite, Object tuning) {
        Access[] access = new Access[params.length];
        Arrays.fill(access, Access.READ_ONLY);
        access[out] = readWrite ? Access.READ_WRITE : Access.WRITE_ONLY;
        LibraryTaskDescriptor d = new LibraryTaskDescriptor().withLibrary(LIBRARY_NAME).withFunction(function).withParameters(params).withAccess(access);
        return tuning == null ? d : d.withTuning(tuning);
    }

    /** {@code out[i] = sum_j m[i*cols+j] * v[j]}: the README mxv kernel as a library task. */
    public static LibraryTaskDescriptor sgemv(int rows, int cols, FloatArray m, FloatArray v, FloatArray out) {
        check(rows >= 0 && cols >= 0, "B200 sgemv requires non-negative sizes; got rows=" + rows + ", cols=" + cols);
        check(m.getSize() >= (long) rows * cols && v.getSize() >= cols && out.getSize() >= rows, "B200 sgemv: array smaller than rows x cols");
        return descriptor("sgemv", new Object[] { rows, cols, m, v, out }, 4, false, null);
    }

    private static void checkQuantised(String name, int rows, int cols, int batch, FloatArray x, FloatArray y) {
        check(cols % 32 == 0, "B200 " + name + " requires cols to be a multiple of the 32-element block; got cols=" + cols);
        check(batch >= 1 && batch <= MAX_BATCH, "B200 " + name + " requires 1 <= batch <= " + MAX_BATCH + "; got " + batch);
        check(x.getSize() >= (long) batch * cols && y.getSize() >= (long) batch * rows, "B200 " + name + ": x or y too small");
    }

    /** Q8_0 mat-vec, split layout: int8 quants + fp16 scales; x is [batch][cols], y is [batch][rows]. */
    public static LibraryTaskDescriptor q8Gemv(int rows, int cols, int batch, Int8Array q, HalfFloatArray scales, FloatArray x, FloatArray y, B200Options options) {
        checkQuantised("q8Gemv", rows, cols, batch, x, y);
        check(q.getSize() >= (long) rows * cols && scales.getSize() >= (long) rows * cols / 32, "B200 q8Gemv: weights too small");
        return descriptor("q8Gemv", new Object[] { rows, cols, batch, q, scales, x, y }, 6, false, options);
    }

    /** Q8_0 mat-vec, unified 34-byte blocks (fp16 scale, 32 x int8). */
    public static LibraryTaskDescriptor q8GemvBytes(int rows, int cols, int batch, ByteArray blocks, FloatArray x, FloatArray y, B200Options options) {
        checkQuantised("q8GemvBytes", rows, cols, batch, x, y);
        check(blocks.getSize() >= (long) rows * (cols / 32) * 34, "B200 q8GemvBytes: weights too small");
        return descriptor("q8GemvBytes", new Object[] { rows, cols, batch, blocks, x, y }, 5, false, options);
    }

    /** Q4_0 mat-vec, 18-byte blocks (fp16 scale, 16 nibble bytes, value = nibble - 8). */
    public static LibraryTaskDescriptor q4GemvBytes(int rows, int cols, int batch, ByteArray blocks, FloatArray x, FloatArray y, B200Options options) {
        checkQuantised("q4GemvBytes", rows, cols, batch, x, y);
        check(blocks.getSize() >= (long) rows * (cols / 32) * 18, "B200 q4GemvBytes: weights too small");
        return descriptor("q4GemvBytes", new Object[] { rows, cols, batch, blocks, x, y }, 5, false, options);
    }

    /**
     * Integer-mode Q8_0 mat-vec of up to 14 equally shaped block matrices that read the same activations, in one launch:
     * {@code y[matrix][batch][rows]}. Parameter list: (count, rows, cols, batch, x, y, blocks...). A library task carries at
     * most 20 arguments (TaskGraph.java:886): rows, cols, batch, x, y, options and 14 matrices; {@link #q8GemvBytesPacked}
     * carries up to 32 in one array.
     */
    public static LibraryTaskDescriptor q8GemvBytesGrouped(int rows, int cols, int batch, FloatArray x, FloatArray y, B200Options options, ByteArray... blocks) {
        return grouped("q8GemvBytesGrouped", 34, rows, cols, batch, x, y, options, blocks);
    }

    /** Q4_0 twin of {@link #q8GemvBytesGrouped}. */
    public static LibraryTaskDescriptor q4GemvBytesGrouped(int rows, int cols, int batch, FloatArray x, FloatArray y, B200Options options, ByteArray... blocks) {
        return grouped("q4GemvBytesGrouped", 18, rows, cols, batch, x, y, options, blocks);
    }

    private static LibraryTaskDescriptor grouped(String name, int blockBytes, int rows, int cols, int batch, FloatArray x, FloatArray y, B200Options options, ByteArray[] blocks) {
        checkQuantised(name, rows, cols, batch, x, y);
        check(blocks.length >= 1 && blocks.length <= 14, "B200 " + name + " requires 1 to 14 matrices (a library task carries 20 arguments); got " + blocks.length);
        check(y.getSize() >= (long) blocks.length * batch * rows, "B200 " + name + ": y smaller than count x batch x rows");
        for (ByteArray b : blocks) {
            check(b.getSize() >= (long) rows * (cols / 32) * blockBytes, "B200 " + name + ": weights too small");
        }
        check(options == null || options.exactInt, "B200 " + name + " computes in integer mode; exactInt must be set");
        Object[] params = new Object[6 + blocks.length];
        params[0] = blocks.length;
        params[1] = rows;
        params[2] = cols;
        params[3] = batch;
        params[4] = x;
        params[5] = y;
        System.arraycopy(blocks, 0, params, 6, blocks.length);
        return descriptor(name, params, 5, false, options != null ? options : new B200Options().exactInt(true));
    }

    /**
     * The grouped integer-mode mat-vec with its {@code count} (at most 32) equally shaped matrices back to back in one
     * ByteArray, matrix m at byte {@code m * rows * cols/32 * 34}: seven arguments whatever the count.
     */
    public static LibraryTaskDescriptor q8GemvBytesPacked(int count, int rows, int cols, int batch, ByteArray blocks, FloatArray x, FloatArray y, B200Options options) {
        return packed("q8GemvBytesPacked", 34, count, rows, cols, batch, blocks, x, y, options);
    }

    /** Q4_0 twin of {@link #q8GemvBytesPacked} (18-byte blocks). */
    public static LibraryTaskDescriptor q4GemvBytesPacked(int count, int rows, int cols, int batch, ByteArray blocks, FloatArray x, FloatArray y, B200Options options) {
        return packed("q4GemvBytesPacked", 18, count, rows, cols, batch, blocks, x, y, options);
    }

    private static LibraryTaskDescriptor packed(String name, int blockBytes, int count, int rows, int cols, int batch, ByteArray blocks, FloatArray x, FloatArray y,
            B200Options options) {
        checkQuantised(name, rows, cols, batch, x, y);
        check(count >= 1 && count <= 32, "B200 " + name + " requires 1 to 32 matrices; got " + count);
        long per = (long) rows * (cols / 32) * blockBytes;
        check(count == 1 || per % 16 == 0, "B200 " + name + " requires matrices of a multiple of 16 bytes; got " + per);
        check(blocks.getSize() >= count * per && y.getSize() >= (long) count * batch * rows, "B200 " + name + ": weights or y too small");
        check(options == null || options.exactInt, "B200 " + name + " computes in integer mode; exactInt must be set");
        return descriptor(name, new Object[] { count, rows, cols, batch, blocks, x, y }, 6, false, options != null ? options : new B200Options().exactInt(true));
    }

    private static void checkTensorCore(String name, int m, int n, int k) {
        check(m >= 0 && n >= 0 && k >= 0, "B200 " + name + " requires non-negative sizes; got m=" + m + ", n=" + n + ", k=" + k);
        check(k % 8 == 0 && n % 8 == 0, "B200 " + name + " requires k and n to be multiples of 8; got k=" + k + ", n=" + n);
    }

    /** {@code D(fp16) = alpha*A*B + beta*D}, fp32 accumulation; signature of {@code Cutlass.cutlassHgemm}. */
    public static LibraryTaskDescriptor hgemm(int m, int n, int k, float alpha, HalfFloatArray a, HalfFloatArray b, float beta, HalfFloatArray d) {
        checkTensorCore("hgemm", m, n, k);
        check(a.getSize() >= (long) m * k && b.getSize() >= (long) k * n && d.getSize() >= (long) m * n, "B200 hgemm: array too small");
        return descriptor("hgemm", new Object[] { m, n, k, alpha, a, b, beta, d }, 7, beta != 0.0f, null);
    }

    /** bfloat16 twin of {@link #hgemm}; signature of {@code Cutlass.cutlassBgemm}. */
    public static LibraryTaskDescriptor bgemm(int m, int n, int k, float alpha, BFloat16Array a, BFloat16Array b, float beta, BFloat16Array d) {
        checkTensorCore("bgemm", m, n, k);
        check(a.getSize() >= (long) m * k && b.getSize() >= (long) k * n && d.getSize() >= (long) m * n, "B200 bgemm: array too small");
        return descriptor("bgemm", new Object[] { m, n, k, alpha, a, b, beta, d }, 7, beta != 0.0f, null);
    }

    /** {@code D = act(A*B + bias)}, bias broadcast over the rows; act is Relu, Gelu, Silu, Sigmoid, Tanh or HardSwish. */
    public static LibraryTaskDescriptor gemmBias(String act, int m, int n, int k, HalfFloatArray a, HalfFloatArray b, HalfFloatArray bias, HalfFloatArray d) {
        checkTensorCore("gemmBias" + act, m, n, k);
        check(a.getSize() >= (long) m * k && b.getSize() >= (long) k * n && bias.getSize() >= n && d.getSize() >= (long) m * n, "B200 gemmBias" + act + ": array too small");
        return descriptor("gemmBias" + act, new Object[] { m, n, k, a, b, bias, d }, 6, false, null);
    }

    public static LibraryTaskDescriptor gemmBiasRelu(int m, int n, int k, HalfFloatArray a, HalfFloatArray b, HalfFloatArray bias, HalfFloatArray d) {
        return gemmBias("Relu", m, n, k, a, b, bias, d);
    }

    public static LibraryTaskDescriptor gemmBiasGelu(int m, int n, int k, HalfFloatArray a, HalfFloatArray b, HalfFloatArray bias, HalfFloatArray d) {
        return gemmBias("Gelu", m, n, k, a, b, bias, d);
    }

    public static LibraryTaskDescriptor gemmBiasSilu(int m, int n, int k, HalfFloatArray a, HalfFloatArray b, HalfFloatArray bias, HalfFloatArray d) {
        return gemmBias("Silu", m, n, k, a, b, bias, d);
    }

    public static LibraryTaskDescriptor gemmBiasSigmoid(int m, int n, int k, HalfFloatArray a, HalfFloatArray b, HalfFloatArray bias, HalfFloatArray d) {
        return gemmBias("Sigmoid", m, n, k, a, b, bias, d);
    }

    public static LibraryTaskDescriptor gemmBiasTanh(int m, int n, int k, HalfFloatArray a, HalfFloatArray b, HalfFloatArray bias, HalfFloatArray d) {
        return gemmBias("Tanh", m, n, k, a, b, bias, d);
    }

    public static LibraryTaskDescriptor gemmBiasHardSwish(int m, int n, int k, HalfFloatArray a, HalfFloatArray b, HalfFloatArray bias, HalfFloatArray d) {
        return gemmBias("HardSwish", m, n, k, a, b, bias, d);
    }

    /** {@code batchCount} independent fp16 GEMMs packed back to back; signature of {@code Cutlass.cutlassHgemmBatched}. */
    public static LibraryTaskDescriptor hgemmBatched(int m, int n, int k, float alpha, HalfFloatArray a, HalfFloatArray b, float beta, HalfFloatArray d, int batchCount) {
        checkTensorCore("hgemmBatched", m, n, k);
        check(batchCount >= 1, "B200 hgemmBatched requires batchCount >= 1; got " + batchCount);
        check(a.getSize() >= (long) batchCount * m * k && b.getSize() >= (long) batchCount * k * n && d.getSize() >= (long) batchCount * m * n, "B200 hgemmBatched: array too small");
        return descriptor("hgemmBatched", new Object[] { m, n, k, alpha, a, b, beta, d, batchCount }, 7, beta != 0.0f, null);
    }

    /** {@code C = alpha*A*B + beta*C}, row-major FP32 on CUDA cores. */
    public static LibraryTaskDescriptor sgemm(int m, int n, int k, float alpha, FloatArray a, FloatArray b, float beta, FloatArray c) {
        check(m >= 0 && n >= 0 && k >= 0, "B200 sgemm requires non-negative sizes; got m=" + m + ", n=" + n + ", k=" + k);
        check(a.getSize() >= (long) m * k && b.getSize() >= (long) k * n && c.getSize() >= (long) m * n, "B200 sgemm: array too small");
        return descriptor("sgemm", new Object[] { m, n, k, alpha, a, b, beta, c }, 7, beta != 0.0f, null);
    }

    /** {@code C(fp32) = A(fp16) * B(fp16)}, row-major, tcgen05 tensor cores with fp32 accumulation. */
    public static LibraryTaskDescriptor hgemmF32(int m, int n, int k, HalfFloatArray a, HalfFloatArray b, FloatArray c) {
        check(m >= 0 && n >= 0 && k >= 0, "B200 hgemmF32 requires non-negative sizes; got m=" + m + ", n=" + n + ", k=" + k);
        check(a.getSize() >= (long) m * k && b.getSize() >= (long) k * n && c.getSize() >= (long) m * n, "B200 hgemmF32: array too small");
        return descriptor("hgemmF32", new Object[] { m, n, k, a, b, c }, 5, false, null);
    }
}
