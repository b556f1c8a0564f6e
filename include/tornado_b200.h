/*
 * tornado_b200.h -- C ABI of libtornado_b200.so
 *
 * Hand-written sm_100a kernels for the dense / quantised matrix-vector and
 * matrix-matrix products that TornadoVM runs through its library-task API.
 * The library plays the role that tornado-drivers/cublas-jni and
 * tornado-drivers/cutlass-jni play for cuBLAS and CUTLASS, but exposes a plain
 * C ABI (no jni.h) so that Java binds it with java.lang.foreign downcalls.
 *
 * Calling convention (same discipline as tornado-drivers/cutlass-jni/src/main/
 * cpp/source/tornado-cutlass.cu:176-259 and cublas-jni/.../tornado-cublas.cpp:
 * 131-198):
 *   - every device pointer is a raw CUdeviceptr that already points at element
 *     0 of a TornadoVM off-heap array, i.e. buffer base + array header
 *     (tornado-runtime/.../interpreter/TornadoVMInterpreter.java:1260-1266);
 *     the header is 16 or 24 bytes, so 8-byte alignment is all that is
 *     guaranteed, and a payload normally sits 16 or 24 bytes past a 128-byte
 *     line of its (256-byte aligned) buffer: the block-layout mat-vec kernels
 *     and the tensor-core GEMMs run from the line boundary below their
 *     operands, so that these offsets cost no extra memory transactions;
 *   - scalars are passed by value; `stream` is the CUstream / cudaStream_t of
 *     the execution plan (TornadoNativeStreamSupport.getNativeStream);
 *   - the CUDA context of the plan must be current on the calling thread;
 *   - every call only enqueues work: it never allocates, frees, synchronises
 *     or copies, so it may be issued while the stream is being captured;
 *   - the return value is a status: 0 success, < 0 argument / library error
 *     (tb200_status below), > 0 a cudaError_t.  Nothing throws or aborts.
 *
 * Layouts (all row-major, little-endian):
 *   FloatArray      float32
 *   HalfFloatArray  IEEE binary16 bit patterns in 16-bit words
 *   Int8Array       int8
 *   Q8_0 split      Int8Array q[rows*cols] + HalfFloatArray scale[rows*cols/32]
 *   Q8_0 blocks     ByteArray of 34-byte blocks: fp16 scale, 32 x int8
 *                   (tornado-examples/.../MatrixVectorRowMajor.java:363-407)
 *   Q4_0 blocks     ByteArray of 18-byte blocks: fp16 scale, 16 bytes; byte i
 *                   holds element i in its low nibble and element i+16 in its
 *                   high nibble; value = nibble - 8
 *   batched GEMV    x is [batch][cols], y is [batch][rows]
 */
#ifndef TORNADO_B200_H
#define TORNADO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TB200_VERSION 100

typedef void *tb200_stream_t; /* CUstream / cudaStream_t */

enum tb200_status {
    TB200_OK = 0,
    TB200_ERR_INVALID_ARG = -1,  /* null pointer, non-positive or unsupported shape */
    TB200_ERR_ALIGNMENT = -2,    /* pointer below the guaranteed alignment */
    TB200_ERR_WORKSPACE = -3,    /* workspace missing or too small */
    TB200_ERR_UNSUPPORTED = -4,  /* device is not sm_100 */
    TB200_ERR_DRIVER = -5,       /* a driver entry point could not be resolved */
    TB200_ERR_TIMEOUT = -6       /* a bounded device-side wait expired */
};

/* Replaces Java_..._CutlassNativeLib_statusString
 * (tornado-cutlass.cu:474-478) / CuBlasNativeLib.statusName
 * (tornado-cublas/.../provider/CuBlasNativeLib.java:80-100). */
const char *tb200_status_string(int status);
int tb200_version(void);

/* Non-zero once any kernel of this library on the current device gave up a
 * bounded wait (value = TB200_ERR_TIMEOUT).  Reading it clears it.  Synchronises
 * the device; meant for tests and diagnostics, not for the launch path. */
int tb200_device_status(int *status_out);
/* The same for the kernels of the given operation classes only (tb200_prepare_class bits, 0 = all): fewer
 * device reads for a caller that knows which kernels it ran. */
int tb200_device_status_of(int op_classes, int *status_out);

/* One-time work of the CUDA context that is current on the calling thread: loads every kernel of the
 * selected operation classes into the context, sets their attributes (dynamic shared memory opt-in,
 * carve-out) and resolves the driver entry points the library needs.  A provider calls it from
 * createContext / prepare, i.e. in the reference's pre-compile pass
 * (tornado-runtime/.../interpreter/TornadoVMInterpreter.java:1036-1055,
 * spi/TornadoLibraryProvider.java:63-72), because with withCUDAGraph() the FIRST dispatch of a plan
 * already runs inside a stream capture in global mode (TornadoVMInterpreter.java:462-476), where module
 * loads and attribute calls are not allowed.  Idempotent and cheap when repeated; op_classes = 0 means
 * all.  Without it the same work happens on the first launch of each kernel. */
enum tb200_prepare_class {
    TB200_PREPARE_GEMV_F32 = 1,
    TB200_PREPARE_GEMV_QUANT = 2,
    TB200_PREPARE_GEMM_F32 = 4,
    TB200_PREPARE_GEMM_F16 = 8,
    TB200_PREPARE_PEER = 16,
    TB200_PREPARE_ALL = 31
};
int tb200_prepare(int op_classes);

/* Options.  tb200_set_option changes the process-wide default; tb200_set_thread_option overrides it for
 * the calls the calling thread makes until tb200_clear_thread_options.  A provider applies a task's
 * tuning object (LibraryTaskDescriptor.withTuning, tornado-api/.../common/LibraryTaskDescriptor.java:79-86)
 * by setting thread options before the native call of a dispatch and clearing them after it, the way
 * CuBlasLibraryProvider applies and resets CuBlasOptions around a call (CuBlasLibraryProvider.java:124-151),
 * so one plan's tuning never leaks into another plan or thread.
 *
 * TB200_OPT_OVERLAP_LAUNCHES (default 0): the mat-vec kernels are launched with
 * programmatic stream serialization.  A kernel may then start while the kernel
 * enqueued before it on the same stream is still finishing: it prefetches its
 * WEIGHT operand at once, and waits for the predecessor to complete before it
 * reads activations or writes outputs.  Contract when on: a weight operand must
 * not be written by the kernel enqueued immediately before the mat-vec on the
 * same stream (copies and earlier kernels are fine). */
enum tb200_option { TB200_OPT_OVERLAP_LAUNCHES = 1, TB200_OPT_HGEMM_SM_PAIRS = 2, TB200_OPT_FLOAT_TENSOR_CORES = 3, TB200_OPT_MMA_WARP_RINGS = 4,
                    TB200_OPT_HGEMM_LINE_STORES = 5, TB200_OPT_INT_TENSOR_CORE_MIN_BATCH = 6, TB200_OPT_TC_REGISTER_KERNEL = 7 };
/* TB200_OPT_HGEMM_SM_PAIRS (default 1): the FP16 GEMM runs 256 x 256 tiles on clusters of two CTAs
 * (tcgen05 cta_group::2) instead of 128 x 256 tiles on single CTAs.
 * TB200_OPT_FLOAT_TENSOR_CORES (default 1): the float-mode quantised mat-vecs (tb200_q8_gemv,
 * tb200_q8b_gemv, tb200_q4b_gemv) feed the tensor cores with the fp32 vector split into two fp16
 * halves (relative representation error 2^-22 of the vector's largest element) when shape and alignment
 * allow.  0 keeps them on the CUDA-core kernels; 1 and 2 take the tensor-core kernel for every eligible
 * call (it measured faster from one vector on in every layout; the two values are kept for callers that
 * set them).
 * TB200_OPT_MMA_WARP_RINGS (default 1): diagnostics; 0 selects the older CTA-wide ring of the
 * tensor-core mat-vec kernels.
 * TB200_OPT_HGEMM_LINE_STORES (default 2): the FP16 GEMM's epilogue transposes its tiles through shared memory
 * and stores whole 128-byte lines when a tile goes to at least `value` destinations (1 = always).
 * TB200_OPT_INT_TENSOR_CORE_MIN_BATCH (default 2, 1..17): the integer-mode mat-vecs take the tensor-core kernel from
 * this many activation vectors on (17 = never); smaller batches stay on the dp4a kernels.  With 1 the block-dot
 * test entries (tb200_*_blockdots_i32) run on the tensor-core kernel as well.
 * TB200_OPT_TC_REGISTER_KERNEL (default 1): the tensor-core mat-vecs use the kernel that keeps the activations
 * in registers (one 256-column slice of K per warp); 0 selects the older shared-memory kernels (diagnostics). */
int tb200_set_option(int option, int value);
int tb200_get_option(int option, int *value);
int tb200_set_thread_option(int option, int value);
int tb200_clear_thread_options(void);

/* Device scratch owned by the provider's context (grow-only workspace of the
 * integer path).  Replaces CutlassNativeLib.allocateDeviceMemory /
 * freeDeviceMemory (tornado-cutlass.cu:455-472; CutlassLibraryProvider.java:
 * 51-66).  Called from createContext / prepare / destroyContext only, never
 * between launches. */
int tb200_device_malloc(size_t bytes, void **out);
int tb200_device_free(void *ptr);

/* ---- FP32 matrix-vector ---------------------------------------------------
 * out[i] = sum_j m[i*cols + j] * v[j]
 * Replaces the JIT-compiled README mxv kernel (README.md:35-47),
 * LinearAlgebraArrays.sgemv (tornado-benchmarks/.../LinearAlgebraArrays.java:
 * 34-42) and matrixVectorGeneric (MatrixVectorRowMajor.java:108-158); same
 * operands as CuBlas.cublasSgemv for a row-major matrix
 * (tornado-cublas.cpp:131-140). */
int tb200_sgemv(int rows, int cols, const float *m, const float *v, float *out, tb200_stream_t stream);

/* ---- Q8_0 matrix-vector, fp32 activations ("float mode") -------------------
 * y[b][r] = sum_j ((float) q[r][j] * scale[r][j/32]) * x[b][j]
 * Replaces matrixVectorGenericFinal (MatrixVectorRowMajor.java:409-423,
 * :530-578) for the split layout and matrixVectorGenericQ8Byte (:428-524) for
 * the 34-byte block layout.  cols % 32 == 0, 1 <= batch <= 16. */
int tb200_q8_gemv(int rows, int cols, int batch, const int8_t *q, const uint16_t *scales, const float *x, float *y,
                  tb200_stream_t stream);
int tb200_q8b_gemv(int rows, int cols, int batch, const uint8_t *blocks, const float *x, float *y,
                   tb200_stream_t stream);

/* ---- Q4_0 matrix-vector, fp32 activations ----------------------------------
 * y[b][r] = sum_blk scale[r][blk] * sum_i (nibble[r][blk][i] - 8) * x[b][32 blk + i]
 * No counterpart in the reference (Q4_0 is only on its roadmap,
 * NVIDIA_ROADMAP.md:18); the operand discipline is that of tb200_q8b_gemv. */
int tb200_q4b_gemv(int rows, int cols, int batch, const uint8_t *blocks, const float *x, float *y,
                   tb200_stream_t stream);

/* ---- integer path ("exact-int mode") ----------------------------------------
 * Activations are quantised on the device to int8 with one fp32 scale per
 * 32-element block, scale = max|x|/127 (1 when the block is all zero),
 * q = (int8) floor(x * (1/scale) + 0.5): the rule of reductionCalculateMax +
 * quantizeKernelContext (MatrixVectorRowMajor.java:308-354) applied per block.
 * Each weight block then contributes an exact int32 dot (dp4a, the device form
 * of QuantizationUtils.dp4a, tornado-api/.../utils/QuantizationUtils.java:29-39)
 * and y[b][r] = sum_blk (float) dot * wscale * xscale
 * (dequantizeFusedResult, QuantizationUtils.java:53-55).
 *
 * The quantised activations live in caller-provided scratch memory:
 *   tb200_quantize_x writes  int8 xq[batch][cols], then float xs[batch][cols/32]
 *   (xs starts at the next multiple of 16 bytes after xq); the *_gemv_i8 entries
 *   use the same bytes as scratch in an order of their own.  From two vectors on
 *   (up to eight) they quantise with a small kernel of their own and chain the
 *   mat-vec to it with a programmatic dependent launch. */
size_t tb200_qx_workspace_bytes(int cols, int batch);
int tb200_quantize_x(int cols, int batch, const float *x, void *workspace, size_t workspace_bytes,
                     tb200_stream_t stream);
int tb200_q8_gemv_i8(int rows, int cols, int batch, const int8_t *q, const uint16_t *scales, const float *x,
                     float *y, void *workspace, size_t workspace_bytes, tb200_stream_t stream);
int tb200_q8b_gemv_i8(int rows, int cols, int batch, const uint8_t *blocks, const float *x, float *y,
                      void *workspace, size_t workspace_bytes, tb200_stream_t stream);
int tb200_q4b_gemv_i8(int rows, int cols, int batch, const uint8_t *blocks, const float *x, float *y,
                      void *workspace, size_t workspace_bytes, tb200_stream_t stream);

/* Integer-path Q8_0 mat-vec (split layout) for callers that cannot hand over
 * scratch memory.  It has no counterpart in the reference.
 *
 * Same arithmetic and results as tb200_q8_gemv_i8, but the quantised
 * activations are kept in a fixed TB200_STATIC_SCRATCH_BYTES array inside the
 * library image (present in every CUDA context that loads the library, until the
 * process exits) instead of a workspace argument.  Meant for code that may not allocate
 * device memory where it calls from: a provider whose only hook is the launch
 * itself (TornadoVM owns the plan's device memory and forbids allocation in
 * dispatch), or a caller already inside a stream capture.
 *   - Shapes whose tb200_qx_workspace_bytes(cols, batch) exceeds
 *     TB200_STATIC_SCRATCH_BYTES are rejected with TB200_ERR_WORKSPACE.
 *   - The first call in a CUDA context looks up the array's device address there; make that
 *     first call before any stream capture begins.  No call allocates or frees.
 *   - All calls in a context share the one array and each call overwrites every
 *     byte it later reads, so nothing needs clearing between calls; two calls
 *     whose kernels can run at the same time on one GPU (different streams)
 *     race on it and must be ordered by the caller. */
#define TB200_STATIC_SCRATCH_BYTES 147456 /* enough for cols * batch <= 131072, e.g. 16384 x 8 */
int tb200_q8_gemv_i8_static(int rows, int cols, int batch, const int8_t *q, const uint16_t *scales, const float *x,
                            float *y, tb200_stream_t stream);
/* Test hook: the device address of that array the entry point will use in the CUDA context that is current
 * (`in_use`) and the address the runtime reports for it there (`fresh`); each context that loads the library
 * has its own copy of the array, so the two must agree in every context. */
int tb200_static_scratch_address(void **in_use, void **fresh);

/* ---- Grouped integer-mode mat-vec and the multi-GPU output hand-off ------------
 * `count` (<= 32) block matrices of one shape [rows][cols] that share the same
 * activations are multiplied in ONE launch: the shape of a decoder layer's
 * projections that read the same vector, and of a row shard of several matrices
 * on one GPU of a group.  In the reference every mat-vec is its own task; the
 * nearest interfaces are the batched GEMMs (CuBlas.cublasSgemmStridedBatched,
 * tornado-cublas/.../CuBlas.java:206-228; Cutlass.cutlassHgemmBatched,
 * Cutlass.java:177-191).  Multi-GPU execution has no counterpart in the reference.
 *
 * blocks[m] is matrix m (host array of device pointers).  Every result is stored
 * to each of the `npeers` (<= 8) destination buffers dst[p] (host array of device
 * pointers: this GPU's buffer and, mapped with tb200_ipc_open, its peers'; pinned
 * host memory mapped into the device's address space is a destination like any
 * other -- the kernel's stores then deliver the results to the host while the
 * launch runs, and they are visible there once the stream has been synchronised), at
 *     dst[p][half * half_stride + (m * batch + b) * rows_total + row_offset + r]
 * where `half` is the low bit of *epoch (0 when epoch is NULL): two halves let a
 * GPU fill the next step's outputs while a peer still reads this step's.  With
 * npeers = 1, rows_total = rows, row_offset = 0, epoch = NULL this is a plain
 * grouped mat-vec with y[count][batch][rows].
 * One launch needs batch <= 4, cols % 256 == 0 and matrices that share one
 * 8-byte aligned phase modulo 16 (any offset from a 128-byte line runs at the
 * same rate when rows are whole 128-byte lines, cols % 2048 == 0, and all
 * matrices share it); other cases are accepted only with a single local
 * destination (one launch per matrix).  The workspace is used when batch * cols > 16384 (see above). */
int tb200_q8b_gemv_i8_grouped(int count, int rows, int cols, int batch, const void *const *blocks, const float *x,
                              float *const *dst, int npeers, long long half_stride, const unsigned *epoch, int rows_total,
                              int row_offset, void *workspace, size_t workspace_bytes, tb200_stream_t stream);
int tb200_q4b_gemv_i8_grouped(int count, int rows, int cols, int batch, const void *const *blocks, const float *x,
                              float *const *dst, int npeers, long long half_stride, const unsigned *epoch, int rows_total,
                              int row_offset, void *workspace, size_t workspace_bytes, tb200_stream_t stream);

/* Matrices of different row counts (the Q, K and V projections of a layer, or
 * every matrix of a decode step that reads the same vector): rows[m] rows for
 * matrix m, and y[m] (host array of device pointers) its own [batch][rows[m]]
 * output array on this GPU.  Same shape limits for the one-launch path. */
int tb200_q8b_gemv_i8_grouped_rows(int count, const int *rows, int cols, int batch, const void *const *blocks, const float *x,
                                   float *const *y, void *workspace, size_t workspace_bytes, tb200_stream_t stream);
int tb200_q4b_gemv_i8_grouped_rows(int count, const int *rows, int cols, int batch, const void *const *blocks, const float *x,
                                   float *const *y, void *workspace, size_t workspace_bytes, tb200_stream_t stream);

/* The equally shaped form with the multi-GPU hand-shake inside the kernel (no separate launch
 * between two steps).  The outputs rotate over nslots (2..4) slots of
 * slot_stride floats: step s stores to slot s % nslots.  sync is two local
 * words, zero at start: sync[0] counts this GPU's completed steps, sync[1] is
 * scratch.  flags[p] is GPU p's flag array (8 words, zero at start; flags[rank]
 * local, the others peer-mapped); flags[p][q] is the number of steps GPU q has
 * announced as complete.  handshake bit 0: at its start (the launches before it
 * have completed, so the stores of step s - 1 are performed) the kernel
 * announces sync[0] = s to every GPU, and before its first store it waits until
 * every GPU has announced s - nslots + 1, i.e. has started the step after the
 * one whose outputs are about to be overwritten (two slots keep the GPUs within
 * a step of one another, three give a step of slack); bit 1: the kernel advances
 * sync[0] when its last CTA finishes.  A step made of several launches sets
 * bit 0 on the first and bit 1 on the last.  Consumers of a step's outputs
 * enqueue tb200_peer_wait first.  Needs the one-launch shapes (see above) and
 * rows >= 1 on every GPU; waits are bounded by timeout_ms (0 = 2000), after
 * which TB200_ERR_TIMEOUT is recorded (tb200_device_status) and the kernel
 * carries on. */
int tb200_q8b_gemv_i8_grouped_sync(int count, int rows, int cols, int batch, const void *const *blocks, const float *x,
                                   float *const *dst, int npeers, int rank, int nslots, long long slot_stride, unsigned *sync,
                                   unsigned *const *flags, int handshake, unsigned timeout_ms, int rows_total, int row_offset,
                                   void *workspace, size_t workspace_bytes, tb200_stream_t stream);
int tb200_q4b_gemv_i8_grouped_sync(int count, int rows, int cols, int batch, const void *const *blocks, const float *x,
                                   float *const *dst, int npeers, int rank, int nslots, long long slot_stride, unsigned *sync,
                                   unsigned *const *flags, int handshake, unsigned timeout_ms, int rows_total, int row_offset,
                                   void *workspace, size_t workspace_bytes, tb200_stream_t stream);

/* Announces sync[0] (this GPU's completed steps) to every GPU and waits
 * (bounded) until every GPU has announced at least as many: all outputs of
 * those steps have then arrived in this GPU's buffer.  Same flags / sync as above. */
int tb200_peer_wait(int rank, int npeers, unsigned *const *flags, const unsigned *sync, unsigned timeout_ms,
                    tb200_stream_t stream);

/* Completes a step whose outputs were stored to the peers' buffers: raises this
 * GPU's flag (value *epoch + 1) in every GPU's flag array, waits until all flags
 * of this GPU's own array have reached that value, then stores it to *epoch.
 * flags[p] (host array of device pointers) is GPU p's array of 8 words, zero at
 * start; flags[rank] is local, the others peer-mapped.  Enqueue it on every GPU
 * of the group after the step's kernels.  The wait is bounded: after timeout_ms
 * (0 = 2000) the kernel records TB200_ERR_TIMEOUT (tb200_device_status) and returns. */
int tb200_peer_signal_wait(int rank, int npeers, unsigned *const *flags, unsigned *epoch, unsigned timeout_ms,
                           tb200_stream_t stream);

/* CUDA IPC plumbing for one process per GPU: export a tb200_device_malloc
 * allocation as a 64-byte handle, map a peer's handle, unmap it.  Set-up and
 * tear-down only. */
int tb200_ipc_export(const void *device_allocation, void *handle64);
int tb200_ipc_open(const void *handle64, void **peer_ptr);
int tb200_ipc_close(void *peer_ptr);

/* Test entry points: the raw int32 block dots, dots[r][blk], for one
 * already-quantised activation vector xq[cols].  Device form of the unit test
 * QuantizationTests.testDP4A (tornado-unittests/.../quantization/
 * QuantizationTests.java:517-549). */
int tb200_q8_blockdots_i32(int rows, int cols, const int8_t *q, const int8_t *xq, int32_t *dots,
                           tb200_stream_t stream);
int tb200_q8b_blockdots_i32(int rows, int cols, const uint8_t *blocks, const int8_t *xq, int32_t *dots,
                            tb200_stream_t stream);
int tb200_q4b_blockdots_i32(int rows, int cols, const uint8_t *blocks, const int8_t *xq, int32_t *dots,
                            tb200_stream_t stream);

/* The same check for the tensor-core mat-vec kernel (mma.sync.m16n8k32.s8), which serves the batches:
 * dots[b][r][blk] for `batch` (<= 16) already-quantised vectors xq[batch][cols], every column of the MMA
 * tiles included.  format: 0 = Q8_0 split quants (Int8Array), 1 = Q8_0 34-byte blocks, 2 = Q4_0 18-byte
 * blocks.  Needs cols % 256 == 0 and 8-byte aligned weights.  Pin: TestMatrixMultiplicationMMAInt8
 * (tornado-unittests/.../TestMatrixMultiplicationMMAInt8.java:314-322) demands exact equality of the
 * int8 tile products in the same way. */
int tb200_blockdots_i32_batched(int format, int rows, int cols, int batch, const void *weights, const int8_t *xq,
                                int32_t *dots, tb200_stream_t stream);

/* ---- FP32 SGEMM -------------------------------------------------------------
 * C = alpha * A * B + beta * C, A[m][k], B[k][n], C[m][n] row-major.
 * Replaces MatrixMultiplication2D.matrixMultiplication
 * (tornado-examples/.../MatrixMultiplication2D.java:48-58) and has the
 * signature of Java_..._CutlassNativeLib_sgemm (tornado-cutlass.cu:176-199). */
int tb200_sgemm(int m, int n, int k, float alpha, const float *a, const float *b, float beta, float *c,
                tb200_stream_t stream);

/* ---- FP16 GEMM, fp32 accumulate and output ---------------------------------
 * C(fp32)[m][n] = A(fp16)[m][k] * B(fp16)[k][n], row-major.
 * Replaces the tile-API kernels gemmMMA ... gemmMMASwizzled
 * (tornado-examples/.../MatrixMultiplicationMMA.java:100-613) and the operands
 * of CuBlas.cublasGemmExFP16FP32 (tornado-cublas/.../CuBlas.java:261-279).
 * Runs on tcgen05 tensor cores when k % 8 == 0, n % 8 == 0 and A, B are
 * 16-byte aligned; any other case takes a CUDA-core kernel. */
int tb200_hgemm_f32(int m, int n, int k, const uint16_t *a, const uint16_t *b, float *c, tb200_stream_t stream);

/* The same product with every finished tile stored to ndst (<= 8) destination
 * buffers at dst[p][row * ld + col_offset + col]: this GPU's buffer and, mapped
 * with tb200_ipc_open, its peers'.  With B and C sharded by N-columns over the
 * GPUs (b is this GPU's contiguous [k][n] column block, ld the unsharded N,
 * col_offset the block's first column) the all-gather of C is part of the
 * epilogue; follow it with tb200_peer_signal_wait.  Tensor-core shapes only
 * (see above).  No counterpart in the reference. */
int tb200_hgemm_f32_scatter(int m, int n, int k, const uint16_t *a, const uint16_t *b, float *const *dst, int ndst,
                            long long ld, long long col_offset, tb200_stream_t stream);

/* ---- FP16 / BF16 GEMM with fused epilogue, output type and batches -----------
 *   D[b] = act(alpha * A[b] * B[b] + beta * C[b] + bias),  b = 0 .. batch_count - 1
 * A[m][k], B[k][n] row-major fp16 or bf16 bit patterns (in_type), fp32 accumulation on tcgen05 tensor cores;
 * D, C [m][n] and bias [n] (added to every row) have the element type out_type; the matrices of a batch lie
 * back to back (strides m*k, k*n, m*n).  c == NULL with beta != 0 means C = D (in place); bias may be NULL;
 * bias needs batch_count == 1.  Replaces, with row-major operands of any 8-element-aligned shape:
 *   Cutlass.cutlassHgemm / cutlassBgemm (alpha, beta, fp16 / bf16 out; tornado-cutlass.cu:201-259),
 *   cutlassGemmBias{Relu,Gelu,Silu,Sigmoid,Tanh,HardSwish} (act(A*B + bias); tornado-cutlass.cu:101-140, :279-396),
 *   cutlassHgemmBatched (tornado-cutlass.cu:411-433), CuBlas.cublasGemmExFP16 / BF16 / FP16FP32
 *   (tornado-cublas/.../CuBlas.java:237-305).
 * Tensor-core shapes: k % 8 == 0, n % 8 == 0, 16-byte aligned A and B; other cases return
 * TB200_ERR_UNSUPPORTED unless the call is a plain fp16 -> fp32 product. */
enum tb200_gemm_in { TB200_IN_F16 = 0, TB200_IN_BF16 = 1 };
enum tb200_gemm_out { TB200_OUT_F32 = 0, TB200_OUT_F16 = 1, TB200_OUT_BF16 = 2 };
enum tb200_activation {
    TB200_ACT_NONE = 0,
    TB200_ACT_RELU = 1,
    TB200_ACT_GELU = 2,      /* 0.5 x (1 + erf(x / sqrt 2)) */
    TB200_ACT_SILU = 3,      /* x / (1 + exp(-x)) */
    TB200_ACT_SIGMOID = 4,
    TB200_ACT_TANH = 5,
    TB200_ACT_HARDSWISH = 6  /* x * min(max(x + 3, 0), 6) / 6 */
};
int tb200_gemm_ex(int m, int n, int k, int in_type, const void *a, const void *b, int out_type, void *d, float alpha, float beta,
                  const void *c, const void *bias, int activation, int batch_count, tb200_stream_t stream);

/* ---- int8 GEMM, int32 accumulate and output -----------------------------------
 * C(s32)[m][n] = A(s8)[m][k] * B(s8)[k][n], row-major, exact.
 * Replaces the tile-API int8 kernel (KernelContext.mmaInt8 with MMAShape.M16N8K32,
 * tornado-api/.../KernelContext.java:703-800; kernel and reference loop in
 * tornado-unittests/.../kernelcontext/matrices/TestMatrixMultiplicationMMAInt8.java:70-172) on
 * tcgen05.mma.kind::i8.  Both operands are fed K-major: B is transposed once per call into `workspace`
 * (tb200_igemm_workspace_bytes(n, k) = n * (k + 128) bytes, 16-byte aligned; provider-owned like the mat-vec
 * workspace: an A behind an array header starts off a 128-byte line, its rows are read from the line boundary below,
 * and the rows of the transposed B carry as many zero bytes in front).
 * Tensor-core shapes: k % 16 == 0, 8-byte aligned A, a workspace; other cases run a CUDA-core kernel. */
size_t tb200_igemm_workspace_bytes(int n, int k);
int tb200_igemm_s32(int m, int n, int k, const int8_t *a, const int8_t *b, int32_t *c, void *workspace, size_t workspace_bytes,
                    tb200_stream_t stream);

/* ---- fp8 GEMM, fp32 accumulate and output --------------------------------------
 * C(f32)[m][n] = A(fp8)[m][k] * B(fp8)[k][n], row-major; both operands in the same OCP format.
 * Replaces the tile-API fp8 kernels (KernelContext.mmaFP8E4M3 / mmaFP8E5M2 with MMAShape.M16N8K32; kernels,
 * reference loops and tolerance 1e-3 in
 * tornado-unittests/.../kernelcontext/matrices/TestMatrixMultiplicationMMAFP8.java:80-248, :415-430; byte
 * formats of tornado-api/.../types/FP8.java) on tcgen05.mma.kind::f8f6f4.  Workspace and shape rules as for
 * tb200_igemm_s32. */
enum tb200_fp8_format { TB200_FP8_E4M3 = 0, TB200_FP8_E5M2 = 1 };
int tb200_fp8gemm_f32(int m, int n, int k, int format, const uint8_t *a, const uint8_t *b, float *c, void *workspace,
                      size_t workspace_bytes, tb200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TORNADO_B200_H */
