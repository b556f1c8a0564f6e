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

    public B200Options exactInt(boolean v) {
        this.exactInt = v;
        return this;
    }

    public B200Options overlapLaunches(boolean v) {
        this.overlapLaunches = v;
        return this;
    }
}
