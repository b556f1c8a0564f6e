package uk.ac.manchester.tornado.b200.provider;

import uk.ac.manchester.tornado.api.common.LibraryTaskDescriptor;
import uk.ac.manchester.tornado.api.exceptions.TornadoRuntimeException;
import uk.ac.manchester.tornado.b200.B200;
import uk.ac.manchester.tornado.b200.B200Options;
import uk.ac.manchester.tornado.runtime.common.TornadoXPUDevice;
import uk.ac.manchester.tornado.runtime.library.spi.LibraryContext;
import uk.ac.manchester.tornado.runtime.library.spi.LibraryInvocation;
import uk.ac.manchester.tornado.runtime.library.spi.TornadoLibraryProvider;
import uk.ac.manchester.tornado.runtime.library.spi.TornadoNativeStreamSupport;

/**
 * Provider of the {@code b200/linalg} tasks. One context per (device, execution plan) holds the plan's
 * native stream and a grow-only device workspace for the integer path; {@code prepare} makes the task's
 * kernels resident in the plan's CUDA context and sizes the workspace before any launch (and before
 * stream capture); {@code dispatch} applies the task's tuning to the calling thread, marshals the
 * positional arguments into one native call that only enqueues kernels, and clears the tuning again.
 *
 * The context class and the {@code canHandle / createContext / destroyContext} skeleton follow
 * {@code CutlassLibraryProvider} (tornado-cutlass/.../provider/CutlassLibraryProvider.java:40-169), the
 * SPI boilerplate every provider of the reference repeats; {@code prepare} and {@code dispatch} are specific
 * to this library.
 */
public final class B200LibraryProvider implements TornadoLibraryProvider {

    /**
     * B200Options.hostResults needs the device-visible address of the output array's page-locked host segment.
     * LibraryInvocation has no accessor for it (spi/LibraryInvocation.java:54-97), so the kernels get one
     * destination; with such an accessor the address would be passed here and the interpreter would skip its
     * transferToHost copy for the array.
     */
    private static final long NO_HOST_SEGMENT = 0L;

    private static final class B200Context implements LibraryContext {
        private final long stream;
        private long workspacePtr;
        private long workspaceBytes;

        private B200Context(long stream) {
            this.stream = stream;
        }

        private void growWorkspace(long required) {
            if (required > workspaceBytes) {
                if (workspacePtr != 0) {
                    B200Native.freeDeviceMemory(workspacePtr);
                    workspacePtr = 0;
                    workspaceBytes = 0;
                }
                workspacePtr = B200Native.allocateDeviceMemory(required);
                if (workspacePtr == 0) {
                    throw new TornadoRuntimeException("[ERROR] Unable to allocate B200 workspace of " + required + " bytes");
                }
                workspaceBytes = required;
            }
        }
    }

    @Override
    public String libraryName() {
        return B200.LIBRARY_NAME;
    }

    @Override
    public boolean canHandle(TornadoXPUDevice device) {
        return device instanceof TornadoNativeStreamSupport;
    }

    @Override
    public LibraryContext createContext(TornadoXPUDevice device, long executionPlanId) {
        B200Native.load();
        return new B200Context(((TornadoNativeStreamSupport) device).getNativeStream(executionPlanId));
    }

    private static boolean isQuantised(String function) {
        return function.equals("q8Gemv") || function.equals("q8GemvBytes") || function.equals("q4GemvBytes");
    }

    private static int prepareClass(String function) {
        return switch (function) {
            case "sgemv" -> B200Native.PREPARE_GEMV_F32;
            case "sgemm" -> B200Native.PREPARE_GEMM_F32;
            case "q8Gemv", "q8GemvBytes", "q4GemvBytes", "q8GemvBytesGrouped", "q4GemvBytesGrouped", "q8GemvBytesPacked", "q4GemvBytesPacked" -> B200Native.PREPARE_GEMV_QUANT;
            default -> B200Native.PREPARE_GEMM_F16;
        };
    }

    /**
     * Runs in the pre-launch pass, before any capture and possibly several times
     * (TornadoLibraryProvider.java:63-72): everything that is not a kernel launch happens here.
     */
    @Override
    public void prepare(LibraryTaskDescriptor descriptor, LibraryContext context) {
        String function = descriptor.getFunctionName();
        B200Native.checkStatus(B200Native.prepare(prepareClass(function)), "prepare");
        Object[] p = descriptor.getParameters();
        if (isQuantised(function) && descriptor.getTuning() instanceof B200Options options && options.exactInt) {
            ((B200Context) context).growWorkspace(B200Native.qxWorkspaceBytes((int) p[1], (int) p[2]));
        }
        if (function.endsWith("Grouped") || function.endsWith("Packed")) { // (count, rows, cols, batch, ...): integer mode whatever the tuning
            ((B200Context) context).growWorkspace(B200Native.qxWorkspaceBytes((int) p[2], (int) p[3]));
        }
    }

    @Override
    public void dispatch(String functionName, LibraryInvocation inv) {
        B200Context ctx = (B200Context) inv.getContext();
        boolean exact = inv.getTuning() instanceof B200Options o && o.exactInt;
        // the task's tuning holds for this call on this thread only (cf. CuBlasLibraryProvider.java:124-151)
        boolean scoped = inv.getTuning() instanceof B200Options t && t.overlapLaunches;
        if (scoped) {
            B200Native.checkStatus(B200Native.setThreadOption(B200Native.OPT_OVERLAP_LAUNCHES, 1), "setThreadOption");
        }
        int status;
        try {
            status = launch(functionName, inv, ctx, exact);
        } finally {
            if (scoped) {
                B200Native.clearThreadOptions();
            }
        }
        B200Native.checkStatus(status, functionName);
    }

    private static int fusedActivation(String functionName) {
        return switch (functionName) {
            case "gemmBiasRelu" -> 1;
            case "gemmBiasGelu" -> 2;
            case "gemmBiasSilu" -> 3;
            case "gemmBiasSigmoid" -> 4;
            case "gemmBiasTanh" -> 5;
            default -> 6; // gemmBiasHardSwish
        };
    }

    private static int launch(String functionName, LibraryInvocation inv, B200Context ctx, boolean exact) {
        return switch (functionName) {
            // (rows, cols, m, v, out)
            case "sgemv" -> B200Native.sgemv((int) inv.getArg(0), (int) inv.getArg(1), //
                    inv.getDevicePointer(2), inv.getDevicePointer(3), inv.getDevicePointer(4), ctx.stream);
            // (rows, cols, batch, q, scales, x, y)
            case "q8Gemv" -> exact //
                    ? B200Native.q8GemvI8((int) inv.getArg(0), (int) inv.getArg(1), (int) inv.getArg(2), inv.getDevicePointer(3), inv.getDevicePointer(4), //
                            inv.getDevicePointer(5), inv.getDevicePointer(6), ctx.workspacePtr, ctx.workspaceBytes, ctx.stream) //
                    : B200Native.q8Gemv((int) inv.getArg(0), (int) inv.getArg(1), (int) inv.getArg(2), inv.getDevicePointer(3), inv.getDevicePointer(4), //
                            inv.getDevicePointer(5), inv.getDevicePointer(6), ctx.stream);
            // (rows, cols, batch, blocks, x, y)
            case "q8GemvBytes", "q4GemvBytes" -> {
                int kind = functionName.equals("q8GemvBytes") ? 0 : 1;
                yield exact //
                        ? B200Native.blockGemvI8(kind, (int) inv.getArg(0), (int) inv.getArg(1), (int) inv.getArg(2), inv.getDevicePointer(3), //
                                inv.getDevicePointer(4), inv.getDevicePointer(5), ctx.workspacePtr, ctx.workspaceBytes, ctx.stream) //
                        : B200Native.blockGemv(kind, (int) inv.getArg(0), (int) inv.getArg(1), (int) inv.getArg(2), inv.getDevicePointer(3), //
                                inv.getDevicePointer(4), inv.getDevicePointer(5), ctx.stream);
            }
            // (count, rows, cols, batch, x, y, blocks...)
            case "q8GemvBytesGrouped", "q4GemvBytesGrouped" -> {
                int count = (int) inv.getArg(0);
                long[] blocks = new long[count];
                for (int m = 0; m < count; m++) {
                    blocks[m] = inv.getDevicePointer(6 + m);
                }
                yield B200Native.blockGemvI8Grouped(functionName.startsWith("q8") ? 0 : 1, count, (int) inv.getArg(1), (int) inv.getArg(2), (int) inv.getArg(3), //
                        blocks, inv.getDevicePointer(4), inv.getDevicePointer(5), NO_HOST_SEGMENT, ctx.workspacePtr, ctx.workspaceBytes, ctx.stream);
            }
            // (m, n, k, alpha, a, b, beta, c)
            case "sgemm" -> B200Native.sgemm((int) inv.getArg(0), (int) inv.getArg(1), (int) inv.getArg(2), (float) inv.getArg(3), //
                    inv.getDevicePointer(4), inv.getDevicePointer(5), (float) inv.getArg(6), inv.getDevicePointer(7), ctx.stream);
            // (m, n, k, a, b, c)
            case "hgemmF32" -> B200Native.hgemmF32((int) inv.getArg(0), (int) inv.getArg(1), (int) inv.getArg(2), //
                    inv.getDevicePointer(3), inv.getDevicePointer(4), inv.getDevicePointer(5), ctx.stream);
            // (count, rows, cols, batch, blocks, x, y): the matrices lie back to back in one ByteArray
            case "q8GemvBytesPacked", "q4GemvBytesPacked" -> {
                int kind = functionName.startsWith("q8") ? 0 : 1;
                int count = (int) inv.getArg(0);
                long per = (long) (int) inv.getArg(1) * ((int) inv.getArg(2) / 32) * (kind == 0 ? 34 : 18);
                long[] blocks = new long[count];
                for (int m = 0; m < count; m++) {
                    blocks[m] = inv.getDevicePointer(4) + m * per;
                }
                yield B200Native.blockGemvI8Grouped(kind, count, (int) inv.getArg(1), (int) inv.getArg(2), (int) inv.getArg(3), //
                        blocks, inv.getDevicePointer(5), inv.getDevicePointer(6), NO_HOST_SEGMENT, ctx.workspacePtr, ctx.workspaceBytes, ctx.stream);
            }
            // (m, n, k, alpha, a, b, beta, d): 16-bit operands and result, D updated in place
            case "hgemm", "bgemm" -> {
                int type = functionName.equals("hgemm") ? 0 : 1;
                yield B200Native.gemmEx((int) inv.getArg(0), (int) inv.getArg(1), (int) inv.getArg(2), type, inv.getDevicePointer(4), inv.getDevicePointer(5), //
                        1 + type, inv.getDevicePointer(7), (float) inv.getArg(3), (float) inv.getArg(6), 0L, 0L, 0, 1, ctx.stream);
            }
            // (m, n, k, alpha, a, b, beta, d, batchCount)
            case "hgemmBatched" -> B200Native.gemmEx((int) inv.getArg(0), (int) inv.getArg(1), (int) inv.getArg(2), 0, inv.getDevicePointer(4), inv.getDevicePointer(5), //
                    1, inv.getDevicePointer(7), (float) inv.getArg(3), (float) inv.getArg(6), 0L, 0L, 0, (int) inv.getArg(8), ctx.stream);
            // (m, n, k, a, b, bias, d)
            case "gemmBiasRelu", "gemmBiasGelu", "gemmBiasSilu", "gemmBiasSigmoid", "gemmBiasTanh", "gemmBiasHardSwish" -> //
                    B200Native.gemmEx((int) inv.getArg(0), (int) inv.getArg(1), (int) inv.getArg(2), 0, inv.getDevicePointer(3), inv.getDevicePointer(4), //
                            1, inv.getDevicePointer(6), 1.0f, 0.0f, 0L, inv.getDevicePointer(5), fusedActivation(functionName), 1, ctx.stream);
            default -> throw new TornadoRuntimeException("[ERROR] B200 function not supported: " + functionName);
        };
    }

    @Override
    public void destroyContext(LibraryContext context) {
        B200Context ctx = (B200Context) context;
        if (ctx.workspacePtr != 0) {
            B200Native.freeDeviceMemory(ctx.workspacePtr);
            ctx.workspacePtr = 0;
            ctx.workspaceBytes = 0;
        }
    }
}
