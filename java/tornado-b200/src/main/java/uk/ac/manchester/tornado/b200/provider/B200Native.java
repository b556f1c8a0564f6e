package uk.ac.manchester.tornado.b200.provider;

import static java.lang.foreign.ValueLayout.ADDRESS;
import static java.lang.foreign.ValueLayout.JAVA_FLOAT;
import static java.lang.foreign.ValueLayout.JAVA_INT;
import static java.lang.foreign.ValueLayout.JAVA_LONG;

import java.lang.foreign.Arena;
import java.lang.foreign.FunctionDescriptor;
import java.lang.foreign.Linker;
import java.lang.foreign.MemorySegment;
import java.lang.foreign.SymbolLookup;
import java.lang.invoke.MethodHandle;

import uk.ac.manchester.tornado.api.exceptions.TornadoRuntimeException;

/**
 * Panama FFM binding of {@code libtornado_b200.so}. Device pointers and the stream are raw 64-bit
 * values (CUdeviceptr / CUstream) and travel as {@code JAVA_LONG}; every entry returns an int status
 * (0 = success, negative = library error, positive = cudaError_t).
 */
public final class B200Native {

    public static final int OPT_OVERLAP_LAUNCHES = 1;
    /** Operation classes of tb200_prepare. */
    public static final int PREPARE_GEMV_F32 = 1;
    public static final int PREPARE_GEMV_QUANT = 2;
    public static final int PREPARE_GEMM_F32 = 4;
    public static final int PREPARE_GEMM_F16 = 8;

    private static final Linker LINKER = Linker.nativeLinker();
    private static SymbolLookup lib;
    private static MethodHandle sgemv;
    private static MethodHandle q8Gemv;
    private static MethodHandle q8GemvI8;
    private static MethodHandle q8bGemv;
    private static MethodHandle q8bGemvI8;
    private static MethodHandle q4bGemv;
    private static MethodHandle q4bGemvI8;
    private static MethodHandle q8bGemvI8Grouped;
    private static MethodHandle q4bGemvI8Grouped;
    private static MethodHandle sgemm;
    private static MethodHandle hgemmF32;
    private static MethodHandle qxWorkspaceBytes;
    private static MethodHandle deviceMalloc;
    private static MethodHandle deviceFree;
    private static MethodHandle statusString;
    private static MethodHandle setOption;
    private static MethodHandle setThreadOption;
    private static MethodHandle clearThreadOptions;
    private static MethodHandle prepare;
    private static MethodHandle gemmEx;

    private B200Native() {
    }

    private static MethodHandle handle(String name, FunctionDescriptor fd) {
        return LINKER.downcallHandle(lib.find(name).orElseThrow(() -> new TornadoRuntimeException("[ERROR] libtornado_b200.so does not export " + name)), fd);
    }

    public static synchronized void load() {
        if (lib != null) {
            return;
        }
        try {
            lib = SymbolLookup.libraryLookup(System.mapLibraryName("tornado_b200"), Arena.global());
        } catch (IllegalArgumentException e) {
            throw new TornadoRuntimeException("[ERROR] Unable to load libtornado_b200.so: " + e.getMessage());
        }
        FunctionDescriptor gemvF = FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG);
        FunctionDescriptor gemvI = FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG);
        sgemv = handle("tb200_sgemv", FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG));
        q8Gemv = handle("tb200_q8_gemv", FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG));
        q8GemvI8 = handle("tb200_q8_gemv_i8", FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG));
        q8bGemv = handle("tb200_q8b_gemv", gemvF);
        q8bGemvI8 = handle("tb200_q8b_gemv_i8", gemvI);
        q4bGemv = handle("tb200_q4b_gemv", gemvF);
        q4bGemvI8 = handle("tb200_q4b_gemv_i8", gemvI);
        // int tb200_q8b_gemv_i8_grouped(count, rows, cols, batch, blocks**, x, dst**, npeers, half_stride, epoch, rows_total, row_offset, ws, ws_bytes, stream)
        FunctionDescriptor grouped = FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_INT,
                JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG);
        q8bGemvI8Grouped = handle("tb200_q8b_gemv_i8_grouped", grouped);
        q4bGemvI8Grouped = handle("tb200_q4b_gemv_i8_grouped", grouped);
        sgemm = handle("tb200_sgemm", FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_FLOAT, JAVA_LONG, JAVA_LONG, JAVA_FLOAT, JAVA_LONG, JAVA_LONG));
        hgemmF32 = handle("tb200_hgemm_f32", FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG));
        qxWorkspaceBytes = handle("tb200_qx_workspace_bytes", FunctionDescriptor.of(JAVA_LONG, JAVA_INT, JAVA_INT));
        deviceMalloc = handle("tb200_device_malloc", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS));
        deviceFree = handle("tb200_device_free", FunctionDescriptor.of(JAVA_INT, JAVA_LONG));
        statusString = handle("tb200_status_string", FunctionDescriptor.of(ADDRESS, JAVA_INT));
        setOption = handle("tb200_set_option", FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT));
        setThreadOption = handle("tb200_set_thread_option", FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT));
        clearThreadOptions = handle("tb200_clear_thread_options", FunctionDescriptor.of(JAVA_INT));
        prepare = handle("tb200_prepare", FunctionDescriptor.of(JAVA_INT, JAVA_INT));
        // int tb200_gemm_ex(m, n, k, in_type, a, b, out_type, d, alpha, beta, c, bias, activation, batch_count, stream)
        gemmEx = handle("tb200_gemm_ex", FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_INT, JAVA_LONG, JAVA_FLOAT,
                JAVA_FLOAT, JAVA_LONG, JAVA_LONG, JAVA_INT, JAVA_INT, JAVA_LONG));
    }

    private static RuntimeException wrap(Throwable t) {
        return new TornadoRuntimeException("[ERROR] libtornado_b200 downcall failed: " + t);
    }

    public static int sgemv(int rows, int cols, long m, long v, long out, long stream) {
        try {
            return (int) sgemv.invokeExact(rows, cols, m, v, out, stream);
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    public static int q8Gemv(int rows, int cols, int batch, long q, long scales, long x, long y, long stream) {
        try {
            return (int) q8Gemv.invokeExact(rows, cols, batch, q, scales, x, y, stream);
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    public static int q8GemvI8(int rows, int cols, int batch, long q, long scales, long x, long y, long workspace, long workspaceBytes, long stream) {
        try {
            return (int) q8GemvI8.invokeExact(rows, cols, batch, q, scales, x, y, workspace, workspaceBytes, stream);
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    /** kind: 0 = Q8_0 34-byte blocks, 1 = Q4_0 18-byte blocks. */
    public static int blockGemv(int kind, int rows, int cols, int batch, long blocks, long x, long y, long stream) {
        try {
            return (int) (kind == 0 ? q8bGemv : q4bGemv).invokeExact(rows, cols, batch, blocks, x, y, stream);
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    public static int blockGemvI8(int kind, int rows, int cols, int batch, long blocks, long x, long y, long workspace, long workspaceBytes, long stream) {
        try {
            return (int) (kind == 0 ? q8bGemvI8 : q4bGemvI8).invokeExact(rows, cols, batch, blocks, x, y, workspace, workspaceBytes, stream);
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    /** One launch for {@code blocks.length} matrices; the pointer arrays live in a confined arena for the duration of the call only. */
    /**
     * yHost: device-visible address of the output array's page-locked host segment, or 0. With it the kernel stores
     * every result to both destinations (one vector only, where the same kernel runs either way).
     */
    public static int blockGemvI8Grouped(int kind, int count, int rows, int cols, int batch, long[] blocks, long x, long y, long yHost, long workspace, long workspaceBytes,
            long stream) {
        try (Arena arena = Arena.ofConfined()) {
            MemorySegment blockPtrs = arena.allocateFrom(JAVA_LONG, blocks);
            boolean both = yHost != 0L && batch == 1;
            MemorySegment dst = both ? arena.allocateFrom(JAVA_LONG, y, yHost) : arena.allocateFrom(JAVA_LONG, y);
            return (int) (kind == 0 ? q8bGemvI8Grouped : q4bGemvI8Grouped).invokeExact(count, rows, cols, batch, blockPtrs, x, dst, both ? 2 : 1, 0L, 0L, rows, 0, workspace,
                    workspaceBytes, stream);
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    public static int sgemm(int m, int n, int k, float alpha, long a, long b, float beta, long c, long stream) {
        try {
            return (int) sgemm.invokeExact(m, n, k, alpha, a, b, beta, c, stream);
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    public static int hgemmF32(int m, int n, int k, long a, long b, long c, long stream) {
        try {
            return (int) hgemmF32.invokeExact(m, n, k, a, b, c, stream);
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    public static long qxWorkspaceBytes(int cols, int batch) {
        try {
            return (long) qxWorkspaceBytes.invokeExact(cols, batch);
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    public static long allocateDeviceMemory(long bytes) {
        try (Arena arena = Arena.ofConfined()) {
            MemorySegment out = arena.allocate(ADDRESS);
            int status = (int) deviceMalloc.invokeExact(bytes, out);
            checkStatus(status, "tb200_device_malloc");
            return out.get(ADDRESS, 0).address();
        } catch (TornadoRuntimeException e) {
            throw e;
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    public static void freeDeviceMemory(long ptr) {
        try {
            checkStatus((int) deviceFree.invokeExact(ptr), "tb200_device_free");
        } catch (TornadoRuntimeException e) {
            throw e;
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    public static void setOption(int option, int value) {
        try {
            checkStatus((int) setOption.invokeExact(option, value), "tb200_set_option");
        } catch (TornadoRuntimeException e) {
            throw e;
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    /** Overrides an option for the calls this thread makes until {@link #clearThreadOptions()}. */
    public static int setThreadOption(int option, int value) {
        try {
            return (int) setThreadOption.invokeExact(option, value);
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    public static void clearThreadOptions() {
        try {
            int ignored = (int) clearThreadOptions.invokeExact();
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    /** Makes the kernels of the given operation classes resident in the CUDA context that is current. */
    public static int prepare(int opClasses) {
        try {
            return (int) prepare.invokeExact(opClasses);
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    /** D = act(alpha*A*B + beta*C + bias); inType 0 fp16, 1 bf16; outType 0 fp32, 1 fp16, 2 bf16; c, bias may be 0. */
    public static int gemmEx(int m, int n, int k, int inType, long a, long b, int outType, long d, float alpha, float beta, long c, long bias, int activation,
            int batchCount, long stream) {
        try {
            return (int) gemmEx.invokeExact(m, n, k, inType, a, b, outType, d, alpha, beta, c, bias, activation, batchCount, stream);
        } catch (Throwable t) {
            throw wrap(t);
        }
    }

    public static String statusName(int status) {
        try {
            MemorySegment s = (MemorySegment) statusString.invokeExact(status);
            return s.reinterpret(64).getUtf8String(0);
        } catch (Throwable t) {
            return Integer.toString(status);
        }
    }

    public static void checkStatus(int status, String function) {
        if (status != 0) {
            throw new TornadoRuntimeException("[ERROR] " + function + " failed with status: " + statusName(status));
        }
    }
}
