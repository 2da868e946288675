/*
 * camel_tensor_b200.h - C ABI of libcamel_tensor_b200.so
 *
 * The CUDA (sm_100a) bodies of the dense-tensor operators of OpenCML/Camel's `tensor`
 * module.  The reference module (`tensor.cmo`) is a C++ plugin whose operators have the
 * signature  slot_t op(ArgsView& with, ArgsView& norm, Context& ctx)
 * (include/camel/core/operator.h:63) and compute on host memory; the functions below are what
 * such an operator body calls once its arguments are unpacked: plain pointers, sizes and
 * dtype codes, no C++ types.  Each declaration names the reference function whose loop it
 * replaces (paths are relative to the reference checkout).
 *
 * Conventions
 *  - Every function returns a ct_status.  On a non-zero status ct_last_error() gives a
 *    message for the calling thread; for CT_ERR_DIV_ZERO / CT_ERR_LOG_DOMAIN it is the text
 *    of the exception the reference throws, so a plugin can rethrow it unchanged.
 *  - Pointers named *_dev are device pointers of the current device (ct_set_device); pointers
 *    named *_host are host pointers.  Tensors are dense, row-major, contiguous, exactly as
 *    the reference stores them (modules/tensor/runtime.cpp:482-485).
 *  - dtype codes follow the reference's three storage types (runtime.cpp:553-566).
 *  - Kernels are enqueued on the stream set by ct_set_stream (default: the legacy default
 *    stream).  Functions that return a host value, or that must report a data-dependent
 *    error, synchronise that stream before returning; the others do not.
 *  - There is no CPU fallback: without a usable CUDA device every compute entry point
 *    returns CT_ERR_NO_DEVICE.
 *  - The selected device belongs to the process, not to the calling thread: every entry point
 *    makes it the calling thread's current CUDA device before it does anything else, so worker
 *    threads of a scheduler need no set-up of their own.
 *  - Environment, read once at first use: CAMEL_TENSOR_PRECISION = 3xtf32 | bf16 and
 *    CAMEL_TENSOR_DEVICES = "2" or "0,1,2,3" (the process takes the entry at index LOCAL_RANK,
 *    else CAMEL_TENSOR_RANK, else 0, modulo the list's length); ct_set_precision / ct_set_device
 *    override them, a malformed value makes the first call fail with CT_ERR_INVALID.
 */
#ifndef CAMEL_TENSOR_B200_H
#define CAMEL_TENSOR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ct_status {
    CT_OK             = 0,
    CT_ERR_INVALID    = 1, /* bad shape / dtype / argument (host-side check, nothing launched) */
    CT_ERR_CUDA       = 2, /* a CUDA runtime or driver call failed */
    CT_ERR_DIV_ZERO   = 3, /* "Division by zero", modules/tensor/runtime.cpp:122-124 */
    CT_ERR_LOG_DOMAIN = 4, /* "log: input must be positive", runtime.cpp:1039-1041 */
    CT_ERR_TIMEOUT    = 5, /* a bounded wait inside a kernel ran out; the context stays usable */
    CT_ERR_NO_DEVICE  = 6,
    CT_ERR_TOO_LARGE  = 7  /* size beyond what the entry point supports */
} ct_status;

/* Storage dtypes, modules/tensor/runtime.cpp:553-566 (Float64/Int32 inputs normalise to these). */
typedef enum ct_dtype { CT_F32 = 0, CT_I64 = 1, CT_BOOL = 2 } ct_dtype;

/* enum class BinaryOp / CompareOp, modules/tensor/runtime.h:39-53 (same order). */
typedef enum ct_binary_op { CT_ADD = 0, CT_SUB = 1, CT_MUL = 2, CT_DIV = 3, CT_POW = 4 } ct_binary_op;
typedef enum ct_compare_op { CT_LT = 0, CT_LE = 1, CT_GT = 2, CT_GE = 3, CT_EQ = 4 } ct_compare_op;

/* Fused activation of the dense / conv2d entry points. */
typedef enum ct_activation {
    CT_ACT_NONE    = 0,
    CT_ACT_RELU    = 1, /* x * (x > 0): the idiom of test/run/nn/svm.cml:31 */
    CT_ACT_SOFTMAX = 2  /* row softmax of test/run/nn/mnist.cml:13-25 (dense only) */
} ct_activation;

/* Arithmetic of the tensor-core contractions. */
typedef enum ct_precision {
    CT_PREC_3XTF32 = 0, /* fp32 in, split into two TF32 terms, three MMAs, fp32 accumulate */
    CT_PREC_BF16   = 1  /* inputs rounded to bf16 once, fp32 accumulate (reported separately) */
} ct_precision;

/* ---- library / device --------------------------------------------------------------- */

const char *ct_last_error(void);
const char *ct_version(void);
ct_status ct_device_count(int *count_host);
ct_status ct_set_device(int device);
ct_status ct_get_device(int *device_host);
/* stream is a cudaStream_t passed as void*; NULL selects the legacy default stream. */
ct_status ct_set_stream(void *stream);
ct_status ct_sync(void);
/* Synchronises and reports errors that kernels of earlier asynchronous calls raised on the
 * device (CT_ERR_TIMEOUT: a bounded wait in a contraction kernel ran out; its output is then
 * undefined).  The record is sticky: no entry point clears it on the way in, contraction kernels
 * launched after it return at once without writing, and it stays until ct_check (or a *_host
 * entry point) has reported it once - so a failure between two checks is never lost, however many
 * calls were enqueued after it.  ct_matmul_f32_static keeps its own status word (status_dev) and
 * is not covered by ct_check. */
ct_status ct_check(void);
/* Host-side fault injection for tests of that path: writes device error word `word` (0 division
 * by zero, 1 log domain, 2 kernel timeout) with `value` (1..255) in stream order, as if a kernel
 * had raised it.  Nothing on the GPU waits, traps or faults.  No reference counterpart. */
ct_status ct_inject_status(int word, uint32_t value);
/* Number of kernels this library has launched in this process (all threads). */
uint64_t ct_launch_count(void);
/* Device timing per kernel family: while enabled, each launch is bracketed by CUDA events on
 * the launching stream.  ct_profile_read synchronises, sums and clears the records filed under
 * `kernel` ("gemm_tc", "gemm_prepass", "gemm_skinny", "gemm_splitk_reduce", "weights_pack",
 * "conv_prepass", "conv_small_c", "im2col", "elementwise", "reduce", "softmax", "transpose",
 * "concat", "maxpool"); NULL reads all. */
ct_status ct_profile_enable(int on);
ct_status ct_profile_read(const char *kernel, double *total_ms_host, uint64_t *launches_host);
/* The tensor pipe's own ceiling, measured: every SM issues `mma_groups` x 4 tcgen05.mma of
 * 128 x 256 x (32 bytes of k) back to back on operands already in shared memory (kind::tf32 for
 * CT_PREC_3XTF32, kind::f16 on bf16 for CT_PREC_BF16), `launches` launches in a row, timed with
 * CUDA events.  A short burst (one launch of ~50 us) and a seconds-long run give the two figures
 * a roofline needs: the 3xTF32 contractions spend three such MMAs per product, so their ceiling
 * is the tf32 figure / 3.  No reference counterpart (a measurement, not an operator). */
ct_status ct_measure_mma_peak(
    ct_precision kind, int mma_groups, int launches, double *tflops_host, double *ms_host);
/* The same measurement for another MMA shape: mma_m = 64 or 128 rows, mma_n = 16..256 columns (a
 * multiple of 16).  The rate the pipe gives a narrow shape is what a layer with few output
 * channels can be held against.  No reference counterpart. */
ct_status ct_measure_mma_rate(
    ct_precision kind, int mma_m, int mma_n, int mma_groups, int launches, double *tflops_host,
    double *ms_host);
/* ... and with the B tile read b_row_shift rows (of 128 bytes, 0..16) past a swizzle-aligned
 * start, as the convolution kernels do when they address a filter tap's pixels inside one halo box;
 * b_row_shift + 256 also takes the A operand from tensor memory instead of shared memory (tf32). */
ct_status ct_measure_mma_rate_shifted(
    ct_precision kind, int mma_m, int mma_n, int b_row_shift, int mma_groups, int launches,
    double *tflops_host, double *ms_host);
/* The pipe's rate in its own clock domain, from stamps taken inside the kernel: SM cycles per MMA
 * of the shape (k = 8 for tf32, 16 for bf16) and the SM clock in MHz that the measuring loop
 * really ran at.  flop per clock and SM = 2 * mma_m * mma_n * k / *clocks_per_mma_host.  No
 * reference counterpart. */
ct_status ct_measure_mma_clocks(
    ct_precision kind, int mma_m, int mma_n, double *clocks_per_mma_host, double *sm_mhz_host);
ct_status ct_set_precision(ct_precision precision);
ct_precision ct_get_precision(void);

/* Record-and-replay of a sequence of calls (CUDA graph).  Between ct_graph_begin and
 * ct_graph_end the library's calls are recorded instead of executed; ct_graph_launch then runs
 * the whole sequence with one launch on the current stream.  Recorded calls see the same device
 * pointers at every replay; tensors allocated inside the recording (ct_alloc) are part of it and
 * live from their point in the sequence until ct_free or the next replay.  Calls that return a
 * host value or synchronise (ct_sum, ct_log, ct_binary with CT_DIV, ct_h2d/ct_d2h, ct_check)
 * cannot be recorded, and the sequence must have run once before so that workspaces exist. */
ct_status ct_graph_begin(void);
ct_status ct_graph_end(void **graph_out);
ct_status ct_graph_launch(void *graph);
ct_status ct_graph_destroy(void *graph);

/* ---- device storage: the device side of TensorObject::create,
 *      modules/tensor/runtime.cpp:256-279 (storage gains a device buffer) ---------------- */

ct_status ct_alloc(void **ptr_dev, size_t bytes);
ct_status ct_free(void *ptr_dev);
/* Synchronous copy from host memory of any kind.  A source of 32 MiB or more that is not
 * page-locked is staged by the library itself: a few host threads copy it in chunks into a ring
 * of page-locked buffers while earlier chunks are on their way to the device (about twice the
 * rate of the driver's own staging of pageable memory).  On return src_host may be reused. */
ct_status ct_h2d(void *dst_dev, const void *src_host, size_t bytes);
ct_status ct_d2h(void *dst_host, const void *src_dev, size_t bytes);
/* ct_d2h followed by ct_check in one trip to the device (the copy of the data and of the error
 * record are enqueued together and waited for once): what a host read at a graph boundary needs -
 * a contraction whose bounded wait ran out must not hand its undefined output to the host.  No
 * reference counterpart (the reference's tensors are host memory). */
ct_status ct_d2h_checked(void *dst_host, const void *src_dev, size_t bytes);
ct_status ct_d2d(void *dst_dev, const void *src_dev, size_t bytes);

/* ---- streaming across the graph boundary --------------------------------------------
 * The reference keeps tensors in host memory, so it has no counterpart of these: they exist
 * because the storage moved to the device and a batch now has to cross PCIe on its way in and
 * out.  ct_h2d/ct_d2h above wait for the copy; the _async forms only enqueue it on the current
 * stream and need page-locked host memory (ct_host_alloc) that stays valid until the stream has
 * passed the copy.  With three streams (copy in, compute, copy out) and events between them the
 * copy of batch i+1 overlaps the kernels of batch i and the read-back of batch i-1.
 * A stream handle is what ct_set_stream takes; events are recorded on, and waited for by, the
 * current stream. */
ct_status ct_host_alloc(void **ptr_host, size_t bytes);
ct_status ct_host_free(void *ptr_host);
ct_status ct_h2d_async(void *dst_dev, const void *src_host_pinned, size_t bytes);
ct_status ct_d2h_async(void *dst_host_pinned, const void *src_dev, size_t bytes);
ct_status ct_stream_create(void **stream_out);
ct_status ct_stream_destroy(void *stream);
ct_status ct_event_create(void **event_out);
ct_status ct_event_destroy(void *event);
ct_status ct_event_record(void *event);       /* on the current stream */
ct_status ct_stream_wait_event(void *event);  /* the current stream waits; the host does not */
ct_status ct_event_sync(void *event);         /* the host waits */
ct_status ct_event_elapsed_ms(void *start_event, void *end_event, float *ms_out);

/* Result dtype of a binary operator: promoteTensorTypes (runtime.cpp:570-580) with the
 * Divide/Power -> Float32 override (runtime.cpp:781-784). */
ct_dtype ct_result_dtype(ct_binary_op op, ct_dtype lhs, ct_dtype rhs);

/* ---- elementwise ------------------------------------------------------------------- */

/* tensorBinary, runtime.cpp:775-793.  out has dtype ct_result_dtype(op, lhs, rhs).
 * CT_DIV synchronises and returns CT_ERR_DIV_ZERO when any divisor is 0. */
ct_status ct_binary(
    ct_binary_op op, ct_dtype lhs_dtype, const void *lhs_dev, ct_dtype rhs_dtype,
    const void *rhs_dev, uint64_t numel, void *out_dev);

/* tensorBinaryScalarRight / tensorBinaryScalarLeft, runtime.cpp:795-831.  scalar_dtype is the
 * tensor dtype the scalar's Camel type normalises to (float/double -> CT_F32, int -> CT_I64,
 * bool -> CT_BOOL); the value enters as double (scalarToDouble, runtime.cpp:62-77). */
ct_status ct_binary_scalar(
    ct_binary_op op, ct_dtype tensor_dtype, const void *tensor_dev, double scalar,
    ct_dtype scalar_dtype, int scalar_on_left, uint64_t numel, void *out_dev);

/* tensorCompare, runtime.cpp:863-877: Bool (uint8) output. */
ct_status ct_compare(
    ct_compare_op op, ct_dtype lhs_dtype, const void *lhs_dev, ct_dtype rhs_dtype,
    const void *rhs_dev, uint64_t numel, uint8_t *out_dev);

/* tensorCompareScalarRight / ScalarLeft, runtime.cpp:833-861. */
ct_status ct_compare_scalar(
    ct_compare_op op, ct_dtype tensor_dtype, const void *tensor_dev, double scalar,
    int scalar_on_left, uint64_t numel, uint8_t *out_dev);

/* tensorExp, runtime.cpp:1013-1027. */
ct_status ct_exp(const float *in_dev, uint64_t numel, float *out_dev);
/* tensorLog, runtime.cpp:1029-1045.  Synchronises; CT_ERR_LOG_DOMAIN when any input <= 0. */
ct_status ct_log(const float *in_dev, uint64_t numel, float *out_dev);
/* relu(x) = multiply(x, gt(x, 0)) in one pass; the reference has no such operator, the
 * composition (test/run/nn/svm.cml:31) defines the values, bit patterns included. */
ct_status ct_relu(const float *in_dev, uint64_t numel, float *out_dev);

/* ---- reductions -------------------------------------------------------------------- */

/* tensorSum, runtime.cpp:879-885: float64 sum of all elements, returned to the host. */
ct_status ct_sum(ct_dtype dtype, const void *in_dev, uint64_t numel, double *result_host);
/* tensorSumAxis, runtime.cpp:887-922: rank 2, axis in {0,1,-1,-2}, float32 out. */
ct_status ct_sum_axis(
    ct_dtype dtype, const void *in_dev, int64_t rows, int64_t cols, int64_t axis, float *out_dev);
/* tensorMaxAxis, runtime.cpp:924-963. */
ct_status ct_max_axis(
    ct_dtype dtype, const void *in_dev, int64_t rows, int64_t cols, int64_t axis, float *out_dev);
/* tensorArgmaxAxis, runtime.cpp:965-1011: Int64 out, first maximum wins. */
ct_status ct_argmax_axis(
    ct_dtype dtype, const void *in_dev, int64_t rows, int64_t cols, int64_t axis,
    int64_t *out_dev);
/* Row softmax as one operator: the function `softmax` of test/run/nn/mnist.cml:13-25
 * (max, subtract, exp, sum, divide; each step rounded to float32 like its operator). */
ct_status ct_softmax_rows(const float *in_dev, int64_t rows, int64_t cols, float *out_dev);

/* ---- data movement ----------------------------------------------------------------- */

/* tensorTranspose2D, runtime.cpp:704-720. */
ct_status ct_transpose(ct_dtype dtype, const void *in_dev, int64_t rows, int64_t cols, void *out_dev);
/* tensorConcat, runtime.cpp:722-773, on the (outer, axis, inner) view of the two shapes. */
ct_status ct_concat(
    ct_dtype dtype, const void *lhs_dev, const void *rhs_dev, uint64_t outer, uint64_t lhs_axis,
    uint64_t rhs_axis, uint64_t inner, void *out_dev);
/* tensorReshape, runtime.cpp:692-702, is ct_d2d of the payload. */

/* tensorZeros/Ones/Full, runtime.cpp:614-646: value converted as setFromDouble does. */
ct_status ct_fill(ct_dtype dtype, double value, uint64_t numel, void *out_dev);
/* tensorEye, runtime.cpp:675-690. */
ct_status ct_eye(int64_t size, float *out_dev);
/* tensorArange, runtime.cpp:652-673: count = number of items (host computes it the same way). */
ct_status ct_arange(int64_t start, int64_t step, int64_t count, int64_t *out_dev);

/* ---- contractions ------------------------------------------------------------------ */

/* __tensor_matmul__, modules/tensor/operators.cpp:740-769: C[m,n] = A[m,k] . B[k,n], rank 2,
 * out dtype = promote(a, b).  float32 x float32 runs on the tensor cores (3xTF32 unless
 * ct_set_precision says otherwise); other dtype pairs accumulate in float64 on CUDA cores. */
ct_status ct_matmul(
    ct_dtype a_dtype, const void *a_dev, ct_dtype b_dtype, const void *b_dev, int64_t m,
    int64_t k, int64_t n, void *out_dev);

/* The two fused forms the reference's training loops call for (test/run/nn/mnist.cml:39-40:
 * `transpose(X) @ (probs - y)` and `W - lr * g`), each with the roundings of the operator chain it
 * replaces.  ct_matmul_tn: out[m,n] = A^T . B with A stored [k][m]; identical to ct_transpose
 * followed by ct_matmul, without the transposed copy.  ct_scaled_sub: out = w - float(double(g) * lr)
 * (tensor * scalar, then tensor - tensor).  No single reference function corresponds to either. */
ct_status ct_matmul_tn(const float *a_km_dev, const float *b_dev, int64_t m, int64_t k, int64_t n, float *out_dev);
ct_status ct_scaled_sub(const float *w_dev, const float *g_dev, double lr, uint64_t numel, float *out_dev);

/* dense<w,b>(x) = act(x . w + b): the bias idiom concat(x, ones, 1) @ concat(w, b, 0) of
 * test/run/nn/lr.cml:19-21 with the activation fused into the GEMM epilogue.  bias_dev may be
 * NULL.  With CT_ACT_SOFTMAX, argmax_dev (may be NULL) also receives argmax(logits, 1) as
 * tensorArgmaxAxis defines it. */
ct_status ct_dense(
    const float *x_dev, const float *w_dev, const float *bias_dev, int64_t m, int64_t k,
    int64_t n, ct_activation act, float *out_dev, int64_t *argmax_dev);

/* Weights that are multiplied many times (the layers of a network) can be handed over once in the
 * layout the tensor-core GEMM reads: ct_weights_pack transposes and splits a [k][n] float32 matrix
 * under the current precision and returns a handle; ct_dense_packed is ct_dense with that handle
 * and skips the per-call pre-pass over the weights (packed == NULL: exactly ct_dense).  The
 * handle must come from the same w_dev, k, n, precision and device, else CT_ERR_INVALID; the
 * caller keeps w_dev unchanged and alive (shapes with n <= 32 read w_dev itself).  Tensors of the
 * reference are immutable values (every operator returns a new tensor), which is what makes
 * caching by tensor sound; the reference itself has no counterpart of these two calls.
 * ct_weights_pack cannot be recorded into a graph. */
ct_status ct_weights_pack(const float *w_dev, int64_t k, int64_t n, void **packed_out);
ct_status ct_weights_free(void *packed);

/* The left operand packed as well, for a product whose rows are computed in several calls (the row
 * panels of a sharded product, each sent on its way while the next is computed).  ct_rows_pack
 * splits a [m][k] float32 matrix into planes of its own on the current stream; *packed_inout is
 * NULL on the first call and the returned handle afterwards, whose buffers are then refilled (same
 * shape and precision) without allocating.  ct_matmul_packed_rows computes
 * out[rows][n] = A[row0 .. row0+rows) . W from two packed operands; it touches none of the
 * library's cached workspaces, so calls made under different ct_set_stream streams may run at the
 * same time (the caller orders them after the ct_rows_pack with events).  Same arithmetic as
 * ct_dense_packed without bias, and the same bytes wherever that call does not slice k over CTAs
 * (few output tiles and a long k), which this one never does.  No reference counterpart (operators.cpp:757-766 is the
 * product itself). */
ct_status ct_rows_pack(const float *a_dev, int64_t m, int64_t k, void **packed_inout);
ct_status ct_rows_free(void *packed);
ct_status ct_matmul_packed_rows(
    const void *a_packed, int64_t row0, int64_t rows, const void *w_packed, float *out_dev);
/* The same product with all row bands in ONE launch, for a caller that sends each band on its way
 * as soon as it is complete (the all-gather of a row-sharded product): band b is band_rows_host[b]
 * consecutive rows of the packed left operand (all but the last a multiple of 128) and is written to
 * band_out_host[b] (row-major, n columns; the bands need not be adjacent in the result).  The tiles
 * are computed band by band; band_done_dev[b] (device words that the CALLER clears before the call,
 * and before the waiting stream may look at them: an event between the clear and the waits) counts
 * the finished tiles of band b and reaches band_tiles_host[b] when the band is complete - a second
 * stream waits for that with ct_stream_wait_value while the launch goes on with the later bands.  Separate launches per band would each end in a partly filled wave of tiles; this has one.
 * Same arithmetic and bytes as ct_matmul_packed_rows.  No reference counterpart. */
ct_status ct_matmul_packed_bands(
    const void *a_packed, const void *w_packed, int nbands, const int64_t *band_rows_host,
    float *const *band_out_host, uint32_t *band_done_dev, uint32_t *band_tiles_host);
/* The current stream (ct_set_stream) waits until the 32-bit device word at addr_dev is >= value;
 * the host does not wait.  The word must lie in memory from cudaMalloc (a stream wait does not
 * accept the stream-ordered pool that ct_alloc draws from).  No reference counterpart. */
ct_status ct_stream_wait_value(const uint32_t *addr_dev, uint32_t value);
ct_status ct_dense_packed(
    const float *x_dev, const float *w_dev, const void *packed, const float *bias_dev, int64_t m,
    int64_t k, int64_t n, ct_activation act, float *out_dev, int64_t *argmax_dev);

/* conv2d, NCHW input [n,c,h,w], OIHW weights [k_out,c,kh,kw], zero padding, then + bias and
 * activation (NONE or RELU).  No reference counterpart (the reference has no conv operator);
 * arithmetic follows the reference's style: one accumulation per output over (c,kh,kw). */
ct_status ct_conv2d(
    const float *x_dev, const float *w_dev, const float *bias_dev, int64_t n, int64_t c,
    int64_t h, int64_t w, int64_t k_out, int64_t kh, int64_t kw, int64_t stride, int64_t pad,
    ct_activation act, float *out_dev);
/* conv2d followed by a 2x2 max-pool (window == stride == 2), as one call: the same values as
 * ct_conv2d then ct_maxpool2d.  For stride-1 layers with at most 64 filters the pooling happens in
 * the convolution's epilogue and the full-resolution activation is never written; other shapes run
 * the two steps.  out_dev is [n][k_out][h_out/2][w_out/2]. */
ct_status ct_conv2d_maxpool2(
    const float *x_dev, const float *w_dev, const float *bias_dev, int64_t n, int64_t c, int64_t h,
    int64_t w, int64_t k_out, int64_t kh, int64_t kw, int64_t stride, int64_t pad, ct_activation act,
    float *out_dev);

/* maxpool2d, NCHW, window == stride, no padding.  No reference counterpart; strict '>' from
 * the window's first element, like tensorMaxAxis. */
ct_status ct_maxpool2d(
    const float *x_dev, int64_t n, int64_t c, int64_t h, int64_t w, int64_t window,
    float *out_dev);

/* float32 matmul for callers that must not allocate.  No counterpart in the reference: it is
 * ct_matmul (float32 x float32, 3xTF32) with the kernel's operand planes held in a fixed
 * 16 MiB array inside the library instead of a workspace that grows on demand.  It is meant for
 * a host that calls into the library where device allocation is off limits - under a fixed
 * memory budget, while other threads have work in flight that a cudaMalloc would stall, or in
 * a latency-bound loop - and it calls no cudaMalloc / cudaFree / allocating routine itself.
 *  - Limit: 8 * (m + n) * roundup(k, 32) bytes (planes rounded up to 1 KiB each) must fit in
 *    16 MiB, e.g. m = n = k = 1024; larger shapes return CT_ERR_TOO_LARGE and a message.
 *  - The array is shared by all calls and keeps the previous call's bytes; each call rewrites
 *    everything it later reads.  Calls that overlap on the GPU (different streams or threads)
 *    race on it: serialise them.
 *  - The first call on a device looks up the array's device address (once per device); make
 *    that first call outside any stream capture.
 *  - Asynchronous like ct_matmul.  status_dev (may be NULL) is a device word that receives 0,
 *    or a non-zero value if a bounded wait inside the kernel ran out (output then undefined);
 *    it is written in stream order, read it after synchronising. */
ct_status ct_matmul_f32_static(
    const float *a_dev, const float *b_dev, int64_t m, int64_t k, int64_t n, float *out_dev,
    uint32_t *status_dev);

/* ---- host-buffer forms: what an operator body calls at a graph boundary, where operands
 *      live in TensorObject host storage.  Copies in, computes, copies out, synchronises. ---- */

ct_status ct_matmul_host(
    const float *a_host, const float *b_host, int64_t m, int64_t k, int64_t n, float *out_host);
ct_status ct_binary_host(
    ct_binary_op op, const float *lhs_host, const float *rhs_host, uint64_t numel,
    float *out_host);

#ifdef __cplusplus
}
#endif
#endif /* CAMEL_TENSOR_B200_H */
