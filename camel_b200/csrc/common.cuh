// Shared host/device plumbing of libcamel_tensor_b200.so: per-thread error text, the current
// device/stream, the launch counter, the device-side error words and cached workspaces.
#pragma once

#include "camel_tensor_b200.h"

#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <utility>

namespace ct {

// Device-side error words, read back by the entry points that must report them.
//   words 0-1  data-dependent exceptions of one call: cleared by the entry point that checks them,
//              read back (with a synchronisation) before it returns.
//   word 2     sticky: written by a contraction kernel whose bounded wait ran out and by nothing
//              else; only ct_check() (or a *_host entry point that reports it) clears it.  While it
//              is set every later contraction kernel returns at once, so that a failed launch is
//              not followed by products of its undefined output; no entry point clears it on the
//              way in, and the failure is therefore still there when the host next looks.
enum FlagWord : int {
    FLAG_DIV_ZERO   = 0, // a divisor was 0 (reference: "Division by zero")
    FLAG_LOG_DOMAIN = 1, // an input of log was <= 0
    FLAG_TIMEOUT    = 2, // a bounded in-kernel wait ran out (value = 1 + the block that gave up)
    FLAG_COUNT      = 8
};

struct DeviceState {
    bool ready           = false;
    int device           = -1;
    int sm_count         = 0;
    uint32_t *flags_dev  = nullptr; // FLAG_COUNT words
    uint32_t *flags_host = nullptr; // pinned mirror
    void *reduce_ws      = nullptr; // partials of the two-pass reductions
    size_t reduce_ws_bytes = 0;
    void *gemm_ws        = nullptr; // split operand planes of the tensor-core GEMM
    size_t gemm_ws_bytes = 0;
    void *splitk_ws      = nullptr; // partial outputs of the split-K GEMM
    size_t splitk_ws_bytes = 0;
    void *stage_ws[3]    = {nullptr, nullptr, nullptr}; // device staging of the *_host forms
    size_t stage_ws_bytes[3] = {0, 0, 0};
};

void set_error(const char *fmt, ...);
ct_status fail(ct_status code, const char *fmt, ...);
ct_status cuda_fail(cudaError_t e, const char *what);

// The reference's Taskflow scheduler calls operators from up to 32 threads at once
// (src/passes/sched/taskflow/taskflow.h:79-80).  An entry point may enqueue several kernels that
// share a cached workspace or the device error words; those sequences must not interleave on the
// stream, so every compute entry point holds this lock (recursive: entry points call each other)
// while it enqueues.  Device work itself stays asynchronous.
class OpLock {
  public:
    OpLock();
    ~OpLock();
    OpLock(const OpLock &)            = delete;
    OpLock &operator=(const OpLock &) = delete;
};

// Current device state (initialised on first use) and stream of the calling process.
ct_status current(DeviceState **out);
cudaStream_t stream();
void count_launch(unsigned n = 1);

// Grows a cached workspace (never shrinks); contents are undefined after the call.
ct_status ensure_ws(void **ptr, size_t *cap, size_t bytes);

// Clears the per-call error words (FLAG_DIV_ZERO, FLAG_LOG_DOMAIN) on the stream; the sticky
// FLAG_TIMEOUT word is left alone.
ct_status clear_data_flags(DeviceState *st);
// Synchronises the stream and copies the error words to st->flags_host.
ct_status fetch_flags(DeviceState *st);
// After fetch_flags: reports (and clears) a recorded kernel timeout; CT_OK if there is none.
ct_status report_timeout(DeviceState *st, const char *what);

#define CT_CUDA(call)                                                                              \
    do {                                                                                           \
        cudaError_t e__ = (call);                                                                  \
        if (e__ != cudaSuccess)                                                                    \
            return ::ct::cuda_fail(e__, #call);                                                    \
    } while (0)

#define CT_TRY(call)                                                                               \
    do {                                                                                           \
        ct_status s__ = (call);                                                                    \
        if (s__ != CT_OK)                                                                          \
            return s__;                                                                            \
    } while (0)

#define CT_LAUNCH_CHECK(name)                                                                      \
    do {                                                                                           \
        ::ct::count_launch();                                                                      \
        cudaError_t e__ = cudaGetLastError();                                                      \
        if (e__ != cudaSuccess)                                                                    \
            return ::ct::cuda_fail(e__, name);                                                     \
    } while (0)

// Programmatic dependent launch.  A chain of short kernels (the layers of an MLP: 8-40 us each)
// otherwise pays, at every boundary, the drain of one grid, the launch of the next and its set-up.
// A kernel launched with launch_dependent() may be scheduled while its predecessor in the stream
// is still running; it must execute griddep_wait() before it touches any global memory (the wait
// returns once the predecessor grid has completed and its writes are visible), so only its set-up
// (barrier initialisation, TMEM allocation, descriptor prefetch, index arithmetic) overlaps.  A
// kernel lets its successor start early with griddep_launch_dependents(); without that call the
// successor starts when the grid ends, as usual.  CAMEL_TENSOR_NO_PDL=1 turns the attribute off.
// While per-kernel event brackets are on (ct_profile_enable) kernels are launched the ordinary way,
// so that a bracket times one kernel alone and not its overlap with the neighbours.
bool profiling_enabled();

#ifdef __CUDACC__
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(
    void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args &&...args) {
    static const bool enabled = getenv("CAMEL_TENSOR_NO_PDL") == nullptr;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = grid;
    cfg.blockDim         = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream           = s;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs    = attr;
    cfg.numAttrs = enabled && !profiling_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#endif

// When profiling is on (ct_profile_enable), brackets the launches made in its scope with CUDA
// events on the launching stream, filed under `name` (a string literal).
class ProfScope {
  public:
    explicit ProfScope(const char *name);
    ~ProfScope();
    ProfScope(const ProfScope &)            = delete;
    ProfScope &operator=(const ProfScope &) = delete;

  private:
    const char *name_;
    cudaEvent_t e0_, e1_;
};

inline size_t dtype_size(int dt) { return dt == CT_F32 ? 4 : (dt == CT_I64 ? 8 : 1); }
inline bool valid_dtype(int dt) { return dt == CT_F32 || dt == CT_I64 || dt == CT_BOOL; }

// Entry points of the other translation units used across files.
// The B operand of a float32 GEMM already in the layout the tensor-core kernel reads: transposed
// [n][kp] hi/lo planes (3xTF32) or one bf16 plane, built once from a [k][n] weight matrix.
struct PackedWeights {
    uint32_t magic;
    int mode;
    int device;
    int64_t k, n, kp;
    const float *src; // the matrix the planes were built from
    void *base;       // one device allocation holding the planes
    void *hi, *lo;
};
constexpr uint32_t kPackedMagic = 0x43545057u; // "CTPW"

ct_status gemm_f32_tc(
    DeviceState *st, const float *a, const float *b, const float *bias, int64_t m, int64_t k,
    int64_t n, int act, float *out, const PackedWeights *packed = nullptr, bool a_is_km = false);
// Geometry of a stride-1 convolution run as an implicit GEMM over NHWC input planes.
struct ConvGeom {
    int c_pad;  // channels rounded up to the k-block
    int h, w;   // input height / width
    int ho, wo; // output height / width
    int kh, kw, pad;
    int th;     // output rows per tile (th * wo <= 256, multiple of 16)
    int pool = 0; // 2: store the 2x2 max-pool of the activated output (pixels-on-rows kernel only)
};

// mode: 0 = 3xTF32 (float32 hi/lo planes), 1 = bf16 (one plane).  With conv != nullptr the B
// planes are NHWC input planes [batch][h][w][c_pad] and n = ho*wo output pixels per image.
ct_status gemm_planes(
    DeviceState *st, int mode, const void *a_hi, const void *a_lo, const void *b_hi,
    const void *b_lo, int64_t m, int64_t n, int64_t kp, const float *bias, int act, float *out,
    int batch, int64_t out_batch_stride, int bias_per_row, const ConvGeom *conv = nullptr);
// x [batch][c][h*w] float32 -> NHWC planes [batch][h*w][c_pad] (transpose + split per image)
ct_status nhwc_planes(
    DeviceState *st, int mode, const float *x, int64_t batch, int64_t c, int64_t hw, int64_t c_pad,
    void *hi, void *lo);
ct_status split_rows_planes(
    DeviceState *st, int mode, const float *in, int64_t rows, int64_t k, int64_t kp, void *hi,
    void *lo);
ct_status gemm_f32_skinny(
    DeviceState *st, const float *a, const float *b, const float *bias, int64_t m, int64_t k,
    int64_t n, int act, float *out, int64_t *argmax);
// out[m][n] = A^T . B with A stored [k][m], n <= 32 (float64 accumulation, two launches)
ct_status gemm_f32_tn_skinny(
    DeviceState *st, const float *a_km, const float *b, int64_t m, int64_t k, int64_t n, float *out);
ct_status matmul_generic(
    int adt, const void *a, int bdt, const void *b, int64_t m, int64_t k, int64_t n, void *out);

} // namespace ct
