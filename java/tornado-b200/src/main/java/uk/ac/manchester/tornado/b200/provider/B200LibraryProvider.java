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
 * native stream and a grow-only device workspace for the integer path; {@code prepare} sizes it before
 * any launch (and before stream capture); {@code dispatch} marshals the positional arguments into one
 * native call that only enqueues kernels.
 */
public final class B200LibraryProvider implements TornadoLibraryProvider {

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

    @Override
    public void prepare(LibraryTaskDescriptor descriptor, LibraryContext context) {
        if (descriptor.getTuning() instanceof B200Options options) {
            if (options.overlapLaunches) {
                B200Native.setOption(B200Native.OPT_OVERLAP_LAUNCHES, 1);
            }
            if (options.exactInt && isQuantised(descriptor.getFunctionName())) {
                Object[] p = descriptor.getParameters();
                ((B200Context) context).growWorkspace(B200Native.qxWorkspaceBytes((int) p[1], (int) p[2]));
            }
            if (descriptor.getFunctionName().endsWith("Grouped")) { // (count, rows, cols, batch, ...)
                Object[] p = descriptor.getParameters();
                ((B200Context) context).growWorkspace(B200Native.qxWorkspaceBytes((int) p[2], (int) p[3]));
            }
        }
    }

    @Override
    public void dispatch(String functionName, LibraryInvocation inv) {
        B200Context ctx = (B200Context) inv.getContext();
        boolean exact = inv.getTuning() instanceof B200Options o && o.exactInt;
        int status = switch (functionName) {
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
                        blocks, inv.getDevicePointer(4), inv.getDevicePointer(5), ctx.workspacePtr, ctx.workspaceBytes, ctx.stream);
            }
            // (m, n, k, alpha, a, b, beta, c)
            case "sgemm" -> B200Native.sgemm((int) inv.getArg(0), (int) inv.getArg(1), (int) inv.getArg(2), (float) inv.getArg(3), //
                    inv.getDevicePointer(4), inv.getDevicePointer(5), (float) inv.getArg(6), inv.getDevicePointer(7), ctx.stream);
            // (m, n, k, a, b, c)
            case "hgemmF32" -> B200Native.hgemmF32((int) inv.getArg(0), (int) inv.getArg(1), (int) inv.getArg(2), //
                    inv.getDevicePointer(3), inv.getDevicePointer(4), inv.getDevicePointer(5), ctx.stream);
            default -> throw new TornadoRuntimeException("[ERROR] B200 function not supported: " + functionName);
        };
        B200Native.checkStatus(status, functionName);
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
