package uk.ac.manchester.tornado.b200;

/**
 * Per-task tuning object handed to {@code LibraryTaskDescriptor.withTuning}; the provider reads it in
 * {@code prepare} and {@code dispatch}.
 */
public final class B200Options {
    /** Quantise activations to int8 per 32-element block and use exact int32 block dots. */
    public boolean exactInt;
    /**
     * Let consecutive mat-vec kernels of the plan overlap: each prefetches its weights while the
     * kernel before it drains. Requires that no task writes a weight array immediately before the
     * mat-vec that reads it.
     */
    public boolean overlapLaunches;
    /**
     * Let the grouped and packed mat-vec kernels store their results into the output array's host segment as
     * well as into its device buffer, so that no device-to-host copy is left for that array. Needs the
     * segment page-locked and mapped ({@code cuMemHostRegister(..., CU_MEMHOSTREGISTER_DEVICEMAP)}) and an
     * accessor for its device-visible address on {@code LibraryInvocation}, which the runtime does not have yet;
     * without them the option is ignored.
     */
    public boolean hostResults;

    public B200Options exactInt(boolean v) {
        this.exactInt = v;
        return this;
    }

    public B200Options overlapLaunches(boolean v) {
        this.overlapLaunches = v;
        return this;
    }

    public B200Options hostResults(boolean v) {
        this.hostResults = v;
        return this;
    }
}
