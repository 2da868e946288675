// Reductions and data movement: full sum, rank-2 axis reductions (sum / max / argmax),
// row softmax, transpose, concat.  All HBM-bound; accumulation is in float64 like the
// reference (modules/tensor/runtime.cpp:879-1011), combined by warp shuffles and a fixed
// block tree so that results do not depend on scheduling.
#include "common.cuh"
#include "fastmath.cuh"

#include <cfloat>
#include <cmath>

namespace ct {
namespace {

__device__ __forceinline__ double as_double(float v) { return (double)v; }
__device__ __forceinline__ double as_double(int64_t v) { return (double)v; }
__device__ __forceinline__ double as_double(uint8_t v) { return v != 0 ? 1.0 : 0.0; }

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- full sum ---------------------------------------------------------------------------

constexpr int kSumThreads = 512;

template <typename T> __device__ __forceinline__ double block_sum_double(double v) {
    __shared__ double warp_part[kSumThreads / 32];
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0)
        warp_part[threadIdx.x >> 5] = v;
    __syncthreads();
    double total = 0.0;
    if (threadIdx.x < 32) {
        total = threadIdx.x < kSumThreads / 32 ? warp_part[threadIdx.x] : 0.0;
        total = warp_sum(total);
    }
    return total; // valid in warp 0
}

// Pass 1: every block strides over the input and leaves one float64 partial.
template <typename T>
__global__ void __launch_bounds__(kSumThreads) sum_partial_kernel(const T *in, uint64_t n, double *partials) {
    double acc      = 0.0;
    uint64_t stride = (uint64_t)gridDim.x * kSumThreads;
    uint64_t i      = (uint64_t)blockIdx.x * kSumThreads + threadIdx.x;
    for (; i < n; i += stride)
        acc += as_double(in[i]);
    double total = block_sum_double<T>(acc);
    if (threadIdx.x == 0)
        partials[blockIdx.x] = total;
}

// float32 specialisation of pass 1: 128-bit loads, four independent accumulators.
__global__ void __launch_bounds__(kSumThreads)
    sum_partial_f32x4_kernel(const float4 *in, uint64_t nvec, double *partials) {
    double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
    uint64_t stride = (uint64_t)gridDim.x * kSumThreads;
    uint64_t i      = (uint64_t)blockIdx.x * kSumThreads + threadIdx.x;
    for (; i + stride < nvec; i += 2 * stride) {
        float4 p = __ldcs(in + i);
        float4 q = __ldcs(in + i + stride);
        a0 += (double)p.x + (double)q.x;
        a1 += (double)p.y + (double)q.y;
        a2 += (double)p.z + (double)q.z;
        a3 += (double)p.w + (double)q.w;
    }
    if (i < nvec) {
        float4 p = __ldcs(in + i);
        a0 += (double)p.x;
        a1 += (double)p.y;
        a2 += (double)p.z;
        a3 += (double)p.w;
    }
    double total = block_sum_double<float>((a0 + a1) + (a2 + a3));
    if (threadIdx.x == 0)
        partials[blockIdx.x] = total;
}

// Pass 2: one block folds the partials (plus a short unvectorised tail) in a fixed order.
template <typename T>
__global__ void __launch_bounds__(kSumThreads)
    sum_final_kernel(const double *partials, int count, const T *tail, uint64_t tail_n, double *out) {
    double acc = 0.0;
    for (int i = threadIdx.x; i < count; i += kSumThreads)
        acc += partials[i];
    for (uint64_t i = threadIdx.x; i < tail_n; i += kSumThreads)
        acc += as_double(tail[i]);
    double total = block_sum_double<T>(acc);
    if (threadIdx.x == 0)
        *out = total;
}

template <typename T> ct_status sum_typed(DeviceState *st, const T *in, uint64_t n, double *result) {
    int blocks = st->sm_count * 4;
    CT_TRY(ensure_ws(&st->reduce_ws, &st->reduce_ws_bytes, (size_t)(blocks + 1) * sizeof(double)));
    double *partials = static_cast<double *>(st->reduce_ws);
    double *out      = partials + blocks;
    const T *tail    = in;
    uint64_t tail_n  = 0;
    int used         = blocks;
    ProfScope prof("reduce");
    if (sizeof(T) == 4 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0 && n >= 4096) {
        uint64_t nvec = n / 4;
        sum_partial_f32x4_kernel<<<blocks, kSumThreads, 0, stream()>>>(
            reinterpret_cast<const float4 *>(in), nvec, partials);
        CT_LAUNCH_CHECK("sum(pass 1)");
        tail   = in + nvec * 4;
        tail_n = n - nvec * 4;
    } else {
        uint64_t want = (n + kSumThreads - 1) / kSumThreads;
        if (want < (uint64_t)blocks)
            used = (int)(want ? want : 1);
        sum_partial_kernel<T><<<used, kSumThreads, 0, stream()>>>(in, n, partials);
        CT_LAUNCH_CHECK("sum(pass 1)");
    }
    sum_final_kernel<T><<<1, kSumThreads, 0, stream()>>>(partials, used, tail, tail_n, out);
    CT_LAUNCH_CHECK("sum(pass 2)");
    CT_CUDA(cudaMemcpyAsync(result, out, sizeof(double), cudaMemcpyDeviceToHost, stream()));
    CT_CUDA(cudaStreamSynchronize(stream()));
    return CT_OK;
}

// ---- rank-2 axis reductions -----------------------------------------------------------

enum { RED_SUM = 0, RED_MAX = 1, RED_ARGMAX = 2 };

// Running state of one reduction: sum, or (best value, its first index).
struct Acc {
    double v;
    int64_t idx;
};

template <int KIND> __device__ __forceinline__ Acc acc_init() { return Acc{0.0, -1}; }

// Fold element (x, i) in.  For max/argmax, idx < 0 means "empty": the reference seeds with
// element 0 and then replaces on strict '>' (runtime.cpp:940-946, 983-991), so a NaN seed
// is never replaced and a later NaN never wins.
template <int KIND> __device__ __forceinline__ void acc_push(Acc &a, double x, int64_t i) {
    if (KIND == RED_SUM) {
        a.v += x;
    } else {
        if (a.idx < 0 || x > a.v) {
            a.v   = x;
            a.idx = i;
        }
    }
}

// Merge b into a where every index in a precedes every index in b... unless swapped: the
// merge keeps the reference's left-to-right semantics by ordering on idx.
template <int KIND> __device__ __forceinline__ void acc_merge(Acc &a, const Acc &b) {
    if (KIND == RED_SUM) {
        a.v += b.v;
        return;
    }
    if (b.idx < 0)
        return;
    if (a.idx < 0) {
        a = b;
        return;
    }
    // Sequential scan over [first ..., second ...]: second wins only if strictly greater,
    // and never when first's best is the scan's NaN seed.
    const Acc &first  = a.idx < b.idx ? a : b;
    const Acc &second = a.idx < b.idx ? b : a;
    Acc r             = first;
    if (second.v > first.v)
        r = second;
    a = r;
}

// A partial whose first element is NaN must stay NaN-seeded only if that element is global
// index 0; elsewhere a NaN is skipped by the reference's strict '>'.  So partials that do not
// start at index 0 must not seed with NaN: push treats NaN as "not greater" but seeding needs
// care.  seed_ok tells push whether x may seed an empty accumulator.
template <int KIND>
__device__ __forceinline__ void acc_push_checked(Acc &a, double x, int64_t i) {
    if (KIND == RED_SUM) {
        a.v += x;
        return;
    }
    if (a.idx < 0) {
        if (i == 0 || x == x) { // NaN may seed only as the very first element
            a.v   = x;
            a.idx = i;
        }
        return;
    }
    if (x > a.v) {
        a.v   = x;
        a.idx = i;
    }
}

template <int KIND> __device__ __forceinline__ Acc warp_merge(Acc a) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Acc b;
        b.v   = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.idx = __shfl_xor_sync(0xffffffffu, a.idx, o);
        acc_merge<KIND>(a, b);
    }
    return a;
}

template <int KIND, typename OT> __device__ __forceinline__ void acc_store(OT *out, int64_t at, const Acc &a);
template <> __device__ __forceinline__ void acc_store<RED_SUM, float>(float *out, int64_t at, const Acc &a) {
    out[at] = (float)a.v;
}
template <> __device__ __forceinline__ void acc_store<RED_MAX, float>(float *out, int64_t at, const Acc &a) {
    out[at] = (float)a.v;
}
template <> __device__ __forceinline__ void acc_store<RED_ARGMAX, int64_t>(int64_t *out, int64_t at, const Acc &a) {
    out[at] = a.idx < 0 ? 0 : a.idx;
}

// axis = 1: one warp per row (cols <= 2048) - lanes stride over the columns.
template <int KIND, typename T, typename OT>
__global__ void __launch_bounds__(256) reduce_rows_warp_kernel(const T *in, int64_t rows, int64_t cols, OT *out) {
    int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows)
        return;
    int lane   = threadIdx.x & 31;
    const T *r = in + row * cols;
    Acc a      = acc_init<KIND>();
    for (int64_t j = lane; j < cols; j += 32)
        acc_push_checked<KIND>(a, as_double(r[j]), j);
    a = warp_merge<KIND>(a);
    if (lane == 0)
        acc_store<KIND, OT>(out, row, a);
}

// axis = 1, wide rows: one block per row.
template <int KIND, typename T, typename OT>
__global__ void __launch_bounds__(256) reduce_rows_block_kernel(const T *in, int64_t rows, int64_t cols, OT *out) {
    __shared__ double sv[8];
    __shared__ long long si[8];
    int64_t row = blockIdx.x;
    const T *r  = in + row * cols;
    Acc a       = acc_init<KIND>();
    for (int64_t j = threadIdx.x; j < cols; j += 256)
        acc_push_checked<KIND>(a, as_double(r[j]), j);
    a = warp_merge<KIND>(a);
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = a.v;
        si[threadIdx.x >> 5] = a.idx;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        Acc t = Acc{sv[0], si[0]};
        for (int w = 1; w < 8; ++w)
            acc_merge<KIND>(t, Acc{sv[w], si[w]});
        acc_store<KIND, OT>(out, row, t);
    }
}

// axis = 0: a 32x8 block owns 32 columns; the 8 row-lanes stride over the rows (coalesced
// 128-byte reads per warp), then merge through shared memory in a fixed order.
template <int KIND, typename T, typename OT>
__global__ void __launch_bounds__(256) reduce_cols_kernel(const T *in, int64_t rows, int64_t cols, OT *out) {
    __shared__ double sv[8][33];
    __shared__ long long si[8][33];
    int tx      = threadIdx.x & 31;
    int ty      = threadIdx.x >> 5;
    int64_t col = (int64_t)blockIdx.x * 32 + tx;
    Acc a       = acc_init<KIND>();
    if (col < cols) {
        for (int64_t i = ty; i < rows; i += 8)
            acc_push_checked<KIND>(a, as_double(in[i * cols + col]), i);
    }
    sv[ty][tx] = a.v;
    si[ty][tx] = a.idx;
    __syncthreads();
    if (ty == 0 && col < cols) {
        Acc t = Acc{sv[0][tx], si[0][tx]};
        for (int w = 1; w < 8; ++w)
            acc_merge<KIND>(t, Acc{sv[w][tx], si[w][tx]});
        acc_store<KIND, OT>(out, col, t);
    }
}

template <int KIND, typename T, typename OT>
ct_status reduce_axis_typed(const T *in, int64_t rows, int64_t cols, int axis, OT *out) {
    ProfScope prof("reduce");
    if (axis == 1) {
        if (rows == 0)
            return CT_OK;
        if (cols <= 2048) {
            unsigned blocks = (unsigned)((rows + 7) / 8);
            reduce_rows_warp_kernel<KIND, T, OT><<<blocks, 256, 0, stream()>>>(in, rows, cols, out);
        } else {
            reduce_rows_block_kernel<KIND, T, OT><<<(unsigned)rows, 256, 0, stream()>>>(in, rows, cols, out);
        }
        CT_LAUNCH_CHECK("reduce(axis=1)");
    } else {
        if (cols == 0)
            return CT_OK;
        unsigned blocks = (unsigned)((cols + 31) / 32);
        reduce_cols_kernel<KIND, T, OT><<<blocks, 256, 0, stream()>>>(in, rows, cols, out);
        CT_LAUNCH_CHECK("reduce(axis=0)");
    }
    return CT_OK;
}


// ---- float32 fast paths of the axis reductions ------------------------------------------------
//
// The generic kernels above fold one element at a time through float64 and a (value, index) pair
// with a seed test: right for every dtype, but far from HBM speed.  For float32 the reference's
// scan (runtime.cpp:940-946, 983-991: element 0 seeds, a later element replaces on strict '>')
// has a closed form that needs no seed state inside the loop:
//     if x[0] is NaN          -> (NaN, 0): nothing is ever greater than a NaN seed
//     else                    -> (largest non-NaN value, the first index that holds it); a NaN
//                                elsewhere never wins because 'NaN > best' is false
// so a thread keeps (best = -inf, idx = none), takes x when x > best (comparisons of floats are
// the comparisons of their float64 values), partial results merge by "greater value, then smaller
// index", and an empty result (every element -inf or NaN) falls back to element 0.  Sums still
// accumulate in float64.

struct BestF {
    float v;
    int64_t idx; // INT64_MAX: nothing taken yet
};
constexpr int64_t kNoIndex = 0x7fffffffffffffffll;

__device__ __forceinline__ void best_take(BestF &b, float x, int64_t i) {
    if (x > b.v) {
        b.v   = x;
        b.idx = i;
    }
}
__device__ __forceinline__ void best_merge(BestF &a, float v, int64_t idx) {
    if (v > a.v || (v == a.v && idx < a.idx)) {
        a.v   = v;
        a.idx = idx;
    }
}
__device__ __forceinline__ BestF warp_best(BestF a) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float v     = __shfl_xor_sync(0xffffffffu, a.v, o);
        int64_t idx = __shfl_xor_sync(0xffffffffu, a.idx, o);
        best_merge(a, v, idx);
    }
    return a;
}
// The reference's result from the merged state and the line's first element.
template <int KIND, typename OT> __device__ __forceinline__ void best_store(OT *out, int64_t at, BestF b, float first) {
    if (first != first || b.idx == kNoIndex) { // NaN seed, or nothing ever exceeded -inf
        b.v   = first;
        b.idx = 0;
    }
    if (KIND == RED_MAX)
        out[at] = (OT)b.v;
    else
        out[at] = (OT)b.idx;
}

// axis = 1, rows of at most 32 columns (a classifier's logits: 10): a block stages 256 * RPT whole
// rows in shared memory with coalesced 128-bit loads (all of them in flight before the first is
// used), then every thread scans RPT rows in order.
template <int KIND, typename OT, int RPT>
__global__ void __launch_bounds__(256) reduce_rows_narrow_f32_kernel(
    const float *__restrict__ in, int64_t rows, int cols, OT *__restrict__ out) {
    extern __shared__ float stage[];
    constexpr int kRows = 256 * RPT;
    const int64_t row0  = (int64_t)blockIdx.x * kRows;
    const int64_t left  = rows - row0;
    const int nrows     = left < kRows ? (int)left : kRows;
    const int count     = nrows * cols;
    const float *src    = in + row0 * cols;
    if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
        const int nvec = count >> 2;
        for (int i = threadIdx.x; i < nvec; i += 256)
            reinterpret_cast<float4 *>(stage)[i] = __ldcs(reinterpret_cast<const float4 *>(src) + i);
        for (int i = (nvec << 2) + threadIdx.x; i < count; i += 256)
            stage[i] = src[i];
    } else {
        for (int i = threadIdx.x; i < count; i += 256)
            stage[i] = src[i];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < RPT; ++k) {
        const int row = threadIdx.x + 256 * k; // consecutive threads, consecutive rows: coalesced results
        if (row >= nrows)
            break;
        const float *r = stage + row * cols;
        if (KIND == RED_SUM) {
            double acc = 0.0;
            for (int j = 0; j < cols; ++j)
                acc += (double)r[j];
            out[row0 + row] = (OT)(float)acc;
        } else {
            BestF b{-INFINITY, kNoIndex};
            for (int j = 0; j < cols; ++j)
                best_take(b, r[j], j);
            best_store<KIND, OT>(out, row0 + row, b, r[0]);
        }
    }
}

// axis = 1, very many rows of a few columns (a classifier's logits over a large batch): a thread
// reads its own row with 64-bit loads straight from global memory - a warp's 32 rows are one
// contiguous piece, so every fetched line is used completely (by several of the warp's loads, out
// of L1) - and scans it in order; no staging, no barrier, results coalesced.
template <int KIND, typename OT>
__global__ void __launch_bounds__(256) reduce_rows_direct_f32_kernel(
    const float *__restrict__ in, int64_t rows, int cols, OT *__restrict__ out) {
    const int64_t row = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (row >= rows)
        return;
    const float2 *r = reinterpret_cast<const float2 *>(in + row * cols); // cols even, base 8-byte aligned
    const int pairs = cols >> 1;
    float first     = 0.0f;
    double acc      = 0.0;
    BestF b{-INFINITY, kNoIndex};
#pragma unroll 8
    for (int j = 0; j < pairs; ++j) {
        const float2 q = __ldg(r + j);
        if (j == 0)
            first = q.x;
        if (KIND == RED_SUM) {
            acc += (double)q.x;
            acc += (double)q.y;
        } else {
            best_take(b, q.x, 2 * j);
            best_take(b, q.y, 2 * j + 1);
        }
    }
    if (KIND == RED_SUM)
        out[row] = (OT)(float)acc;
    else
        best_store<KIND, OT>(out, row, b, first);
}

// axis = 1, wider rows: GROUP threads per row (a warp, or the whole block), 128-bit loads.
template <int KIND, typename OT, int GROUP>
__global__ void __launch_bounds__(256) reduce_rows_f32_kernel(
    const float *__restrict__ in, int64_t rows, int64_t cols, OT *__restrict__ out) {
    constexpr int kGroupsPerBlock = 256 / GROUP;
    __shared__ double s_sum[8];
    __shared__ float s_v[8];
    __shared__ long long s_i[8];
    const int64_t row = (int64_t)blockIdx.x * kGroupsPerBlock + (GROUP == 256 ? 0 : (int)(threadIdx.x / GROUP));
    if (row >= rows)
        return; // GROUP == 256: never taken (one row per block); a warp leaves as a whole
    const int t    = threadIdx.x % GROUP;
    const float *r = in + row * cols;
    double acc     = 0.0;
    BestF b{-INFINITY, kNoIndex};
    const bool vec = (cols & 3) == 0 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0;
    if (vec) {
        const float4 *r4   = reinterpret_cast<const float4 *>(r);
        const int64_t nvec = cols >> 2;
#pragma unroll 4
        for (int64_t j = t; j < nvec; j += GROUP) {
            const float4 q = __ldcs(r4 + j);
            if (KIND == RED_SUM) {
                acc += ((double)q.x + (double)q.y) + ((double)q.z + (double)q.w);
            } else {
                best_take(b, q.x, 4 * j);
                best_take(b, q.y, 4 * j + 1);
                best_take(b, q.z, 4 * j + 2);
                best_take(b, q.w, 4 * j + 3);
            }
        }
    } else {
        for (int64_t j = t; j < cols; j += GROUP) {
            const float x = r[j];
            if (KIND == RED_SUM)
                acc += (double)x;
            else
                best_take(b, x, j);
        }
    }
    if (KIND == RED_SUM) {
        acc = warp_sum(acc);
        if (GROUP == 256) {
            if ((threadIdx.x & 31) == 0)
                s_sum[threadIdx.x >> 5] = acc;
            __syncthreads();
            if (threadIdx.x == 0) {
                double total = 0.0;
                for (int w = 0; w < 8; ++w)
                    total += s_sum[w];
                out[row] = (OT)(float)total;
            }
        } else if (t == 0) {
            out[row] = (OT)(float)acc;
        }
    } else {
        b = warp_best(b);
        if (GROUP == 256) {
            if ((threadIdx.x & 31) == 0) {
                s_v[threadIdx.x >> 5] = b.v;
                s_i[threadIdx.x >> 5] = b.idx;
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int w = 1; w < 8; ++w)
                    best_merge(b, s_v[w], s_i[w]);
                best_store<KIND, OT>(out, row, b, r[0]);
            }
        } else if (t == 0) {
            best_store<KIND, OT>(out, row, b, r[0]);
        }
    }
}

// axis = 0: a block owns 128 columns (a thread 4 of them: one 128-bit load per row) and a slice
// of the rows; its 8 row-lanes stride over the slice with four loads in flight.  Slices leave
// partial results in a workspace [slices][cols]; a second kernel folds them in slice order, so the
// result does not depend on how the rows were cut.
struct ColPartial {
    double sum;
    float v;
    int64_t idx;
};

template <int KIND>
__global__ void __launch_bounds__(256) reduce_cols_f32_kernel(
    const float *__restrict__ in, int64_t rows, int64_t cols, int64_t rows_per_slice, double *__restrict__ psum,
    float *__restrict__ pv, int64_t *__restrict__ pidx) {
    __shared__ double s_sum[8][129];
    __shared__ float s_v[8][129];
    __shared__ long long s_i[8][129];
    const int tx       = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t col  = ((int64_t)blockIdx.x * 32 + tx) * 4;
    const int64_t r0   = (int64_t)blockIdx.y * rows_per_slice;
    const int64_t r1   = r0 + rows_per_slice < rows ? r0 + rows_per_slice : rows;
    double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
    BestF b0{-INFINITY, kNoIndex}, b1 = b0, b2 = b0, b3 = b0;
    if (col < cols) { // cols is a multiple of 4 on this path
#pragma unroll 4
        for (int64_t i = r0 + ty; i < r1; i += 8) {
            const float4 q = __ldcs(reinterpret_cast<const float4 *>(in + i * cols + col));
            if (KIND == RED_SUM) {
                a0 += (double)q.x, a1 += (double)q.y, a2 += (double)q.z, a3 += (double)q.w;
            } else {
                best_take(b0, q.x, i), best_take(b1, q.y, i), best_take(b2, q.z, i), best_take(b3, q.w, i);
            }
        }
    }
    if (KIND == RED_SUM) {
        s_sum[ty][tx * 4] = a0, s_sum[ty][tx * 4 + 1] = a1, s_sum[ty][tx * 4 + 2] = a2, s_sum[ty][tx * 4 + 3] = a3;
    } else {
        s_v[ty][tx * 4] = b0.v, s_v[ty][tx * 4 + 1] = b1.v, s_v[ty][tx * 4 + 2] = b2.v, s_v[ty][tx * 4 + 3] = b3.v;
        s_i[ty][tx * 4] = b0.idx, s_i[ty][tx * 4 + 1] = b1.idx, s_i[ty][tx * 4 + 2] = b2.idx, s_i[ty][tx * 4 + 3] = b3.idx;
    }
    __syncthreads();
    if (threadIdx.x < 128) {
        const int64_t c = (int64_t)blockIdx.x * 128 + threadIdx.x;
        if (c < cols) {
            const int64_t at = (int64_t)blockIdx.y * cols + c;
            if (KIND == RED_SUM) {
                double total = 0.0;
                for (int w = 0; w < 8; ++w)
                    total += s_sum[w][threadIdx.x];
                psum[at] = total;
            } else {
                BestF b{s_v[0][threadIdx.x], s_i[0][threadIdx.x]};
                for (int w = 1; w < 8; ++w)
                    best_merge(b, s_v[w][threadIdx.x], s_i[w][threadIdx.x]);
                pv[at]   = b.v;
                pidx[at] = b.idx;
            }
        }
    }
}

template <int KIND, typename OT>
__global__ void __launch_bounds__(256) reduce_cols_finish_f32_kernel(
    const float *__restrict__ in, int64_t cols, int slices, const double *__restrict__ psum,
    const float *__restrict__ pv, const int64_t *__restrict__ pidx, OT *__restrict__ out) {
    const int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (c >= cols)
        return;
    if (KIND == RED_SUM) {
        double total = 0.0;
        for (int s = 0; s < slices; ++s)
            total += psum[(int64_t)s * cols + c];
        out[c] = (OT)(float)total;
    } else {
        BestF b{-INFINITY, kNoIndex};
        for (int s = 0; s < slices; ++s)
            best_merge(b, pv[(int64_t)s * cols + c], pidx[(int64_t)s * cols + c]);
        best_store<KIND, OT>(out, c, b, in[c]);
    }
}

template <int KIND, typename OT>
ct_status reduce_axis_f32(DeviceState *st, const float *in, int64_t rows, int64_t cols, int axis, OT *out) {
    ProfScope prof("reduce");
    if (axis == 1) {
        if (rows == 0)
            return CT_OK;
        if (cols >= 2 && cols <= 32 && (cols & 1) == 0 && rows >= 256 * (int64_t)st->sm_count &&
            (reinterpret_cast<uintptr_t>(in) & 7u) == 0) {
            reduce_rows_direct_f32_kernel<KIND, OT><<<(unsigned)((rows + 255) / 256), 256, 0, stream()>>>(in, rows, (int)cols, out);
        } else if (cols <= 32 && rows >= 1024 * (int64_t)st->sm_count && cols <= 11) {
            // many short rows: four rows per thread (up to 44 KB of a block's rows in flight)
            const unsigned blocks = (unsigned)((rows + 1023) / 1024);
            reduce_rows_narrow_f32_kernel<KIND, OT, 4>
                <<<blocks, 256, (size_t)1024 * cols * sizeof(float), stream()>>>(in, rows, (int)cols, out);
        } else if (cols <= 32) {
            const unsigned blocks = (unsigned)((rows + 255) / 256);
            reduce_rows_narrow_f32_kernel<KIND, OT, 1>
                <<<blocks, 256, (size_t)256 * cols * sizeof(float), stream()>>>(in, rows, (int)cols, out);
        } else if (cols <= 1024) {
            reduce_rows_f32_kernel<KIND, OT, 32><<<(unsigned)((rows + 7) / 8), 256, 0, stream()>>>(in, rows, cols, out);
        } else {
            reduce_rows_f32_kernel<KIND, OT, 256><<<(unsigned)rows, 256, 0, stream()>>>(in, rows, cols, out);
        }
        CT_LAUNCH_CHECK("reduce(axis=1)");
        return CT_OK;
    }
    if (cols == 0)
        return CT_OK;
    // axis = 0: enough row slices that the grid covers the machine a few times over
    const int64_t col_blocks = (cols + 127) / 128;
    int64_t slices           = ((int64_t)st->sm_count * 4 + col_blocks - 1) / col_blocks;
    if (slices > rows / 64)
        slices = rows / 64;
    if (slices < 1)
        slices = 1;
    if (slices > 1024)
        slices = 1024;
    const int64_t rows_per_slice = (rows + slices - 1) / slices;
    slices                       = rows_per_slice > 0 ? (rows + rows_per_slice - 1) / rows_per_slice : 1;
    const size_t per = (size_t)slices * cols;
    CT_TRY(ensure_ws(&st->reduce_ws, &st->reduce_ws_bytes, per * (sizeof(double) + sizeof(float) + sizeof(int64_t)) + 64));
    double *psum  = static_cast<double *>(st->reduce_ws);
    int64_t *pidx = reinterpret_cast<int64_t *>(psum + per);
    float *pv     = reinterpret_cast<float *>(pidx + per);
    dim3 grid((unsigned)col_blocks, (unsigned)slices);
    reduce_cols_f32_kernel<KIND><<<grid, 256, 0, stream()>>>(in, rows, cols, rows_per_slice, psum, pv, pidx);
    CT_LAUNCH_CHECK("reduce(axis=0)");
    reduce_cols_finish_f32_kernel<KIND, OT>
        <<<(unsigned)((cols + 255) / 256), 256, 0, stream()>>>(in, cols, (int)slices, psum, pv, pidx, out);
    CT_LAUNCH_CHECK("reduce(axis=0, finish)");
    return CT_OK;
}

template <int KIND, typename OT>
ct_status reduce_axis(int dt, const void *in, int64_t rows, int64_t cols, int64_t axis, OT *out, const char *name) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (!valid_dtype(dt))
        return fail(CT_ERR_INVALID, "%s: bad dtype", name);
    if (rows < 0 || cols < 0)
        return fail(CT_ERR_INVALID, "%s: negative dimension", name);
    if (axis < 0)
        axis += 2;
    if (axis != 0 && axis != 1)
        return fail(CT_ERR_INVALID, "%s(axis): axis must be 0 or 1 for rank-2 tensors", name);
    // max/argmax read element 0 of every line unconditionally in the reference; an empty
    // reduced dimension has no defined result there, so reject it here.
    if (KIND != RED_SUM && ((axis == 0 && rows == 0 && cols > 0) || (axis == 1 && cols == 0 && rows > 0)))
        return fail(CT_ERR_INVALID, "%s(axis): empty reduction", name);
    if (rows > 0x7fffffffll * 8 || cols > 0x7fffffffll * 32)
        return fail(CT_ERR_TOO_LARGE, "%s: dimension too large", name);
    if (dt == CT_F32 && rows > 0 && cols > 0 && cols <= 0x7fffffffll &&
        (axis == 1 || ((cols & 3) == 0 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0 && rows >= 64)))
        return reduce_axis_f32<KIND, OT>(st, static_cast<const float *>(in), rows, cols, (int)axis, out);
    switch (dt) {
    case CT_F32:
        return reduce_axis_typed<KIND, float, OT>(static_cast<const float *>(in), rows, cols, (int)axis, out);
    case CT_I64:
        return reduce_axis_typed<KIND, int64_t, OT>(static_cast<const int64_t *>(in), rows, cols, (int)axis, out);
    default:
        return reduce_axis_typed<KIND, uint8_t, OT>(static_cast<const uint8_t *>(in), rows, cols, (int)axis, out);
    }
}

// ---- row softmax ------------------------------------------------------------------------
//
// softmax(x)[i,:] per test/run/nn/mnist.cml:13-25:  m = max_j x;  s = fl32(x - m);
// e = fl32(exp(double(s)));  d = fl32(sum_j double(e));  out = fl32(e / d).
// One warp (cols <= 1024) or one block (cols <= 8192) keeps the row in registers, so the
// input is read once and the output written once: 8 bytes per element.

template <int PER_LANE, int THREADS>
__global__ void __launch_bounds__(THREADS) softmax_rows_kernel(const float *in, int64_t rows, int64_t cols, float *out) {
    constexpr int WARPS         = THREADS / 32;
    constexpr bool kWarpPerRow  = PER_LANE <= 32 && THREADS == 256 && false;
    (void)kWarpPerRow;
    __shared__ float s_max[WARPS];
    __shared__ double s_sum[WARPS];
    int64_t row = blockIdx.x;
    if (row >= rows)
        return;
    const float *r = in + row * cols;
    float *o       = out + row * cols;
    float v[PER_LANE];
    // max with the reference's scan semantics: element 0 seeds (NaN sticks), strict '>'.
    float best   = -INFINITY;
    bool has_any = false;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
        int64_t j = (int64_t)k * THREADS + threadIdx.x;
        v[k]      = j < cols ? r[j] : -INFINITY;
        if (j < cols && v[k] > best)
            best = v[k];
        has_any |= j < cols;
    }
    (void)has_any;
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1)
        best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o2));
    if ((threadIdx.x & 31) == 0)
        s_max[threadIdx.x >> 5] = best;
    __syncthreads();
    float m = s_max[0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w)
        m = fmaxf(m, s_max[w]);
    float first = r[0];
    if (first != first)
        m = first; // a NaN seed is never replaced (runtime.cpp:940-946)
    double acc = 0.0;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
        int64_t j = (int64_t)k * THREADS + threadIdx.x;
        if (j < cols) {
            float s = __fsub_rn(v[k], m);
            v[k]    = exp_f32(s);
            acc += (double)v[k];
        }
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0)
        s_sum[threadIdx.x >> 5] = acc;
    __syncthreads();
    double total = 0.0;
#pragma unroll
    for (int w = 0; w < WARPS; ++w)
        total += s_sum[w];
    float d = (float)total;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
        int64_t j = (int64_t)k * THREADS + threadIdx.x;
        if (j < cols)
            o[j] = __fdiv_rn(v[k], d);
    }
}

// Wide rows (cols a multiple of 4, 16-byte aligned rows, cols <= 4 * V4 * THREADS): the same
// three phases with 128-bit loads and stores, and register use capped so that at least two
// blocks share an SM - while one block sits in a reduction the other streams.
template <int V4, int THREADS, int MIN_BLOCKS = 2>
__global__ void __launch_bounds__(THREADS, MIN_BLOCKS)
    softmax_rows_wide_kernel(const float *__restrict__ in, int64_t rows, int64_t cols, float *__restrict__ out) {
    constexpr int WARPS = THREADS / 32;
    __shared__ float s_max[WARPS];
    __shared__ double s_sum[WARPS];
    const int64_t row = blockIdx.x;
    const float4 *r   = reinterpret_cast<const float4 *>(in + row * cols);
    float4 *o         = reinterpret_cast<float4 *>(out + row * cols);
    const int nvec    = (int)(cols >> 2);
    float4 v[V4];
    float best = -INFINITY;
#pragma unroll
    for (int k = 0; k < V4; ++k) {
        int j = k * THREADS + threadIdx.x;
        v[k]  = j < nvec ? __ldcs(r + j) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        best  = fmaxf(best, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
    }
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1)
        best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o2));
    if ((threadIdx.x & 31) == 0)
        s_max[threadIdx.x >> 5] = best;
    __syncthreads();
    float m = s_max[threadIdx.x & (WARPS - 1)];
#pragma unroll
    for (int o2 = WARPS / 2; o2 > 0; o2 >>= 1)
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o2));
    float first = in[row * cols];
    if (first != first)
        m = first; // a NaN first element seeds the reference's scan and is never replaced
    double acc = 0.0;
#pragma unroll
    for (int k = 0; k < V4; ++k) {
        int j = k * THREADS + threadIdx.x;
        if (j < nvec) {
            // one branch per four elements: all four in the range of the plain form (a NaN fails it)
            const float d0 = __fsub_rn(v[k].x, m), d1 = __fsub_rn(v[k].y, m);
            const float d2 = __fsub_rn(v[k].z, m), d3 = __fsub_rn(v[k].w, m);
            if ((d0 >= -87.0f) & (d1 >= -87.0f) & (d2 >= -87.0f) & (d3 >= -87.0f)) {
                // two elements per instruction: the kernel is bound by instruction issue
                unpack2(exp_f32_plain2(pack2(d0, d1)), v[k].x, v[k].y);
                unpack2(exp_f32_plain2(pack2(d2, d3)), v[k].z, v[k].w);
            } else {
                v[k].x = exp_f32_nonpos(d0);
                v[k].y = exp_f32_nonpos(d1);
                v[k].z = exp_f32_nonpos(d2);
                v[k].w = exp_f32_nonpos(d3);
            }
            acc += ((double)v[k].x + (double)v[k].y) + ((double)v[k].z + (double)v[k].w);
        }
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0)
        s_sum[threadIdx.x >> 5] = acc;
    __syncthreads();
    double total = s_sum[threadIdx.x & (WARPS - 1)];
#pragma unroll
    for (int o2 = WARPS / 2; o2 > 0; o2 >>= 1)
        total += __shfl_xor_sync(0xffffffffu, total, o2);
    const float d  = (float)total;
    const float rd = __frcp_rn(d);
    const f32x2 rd2 = pack2(rd, rd), nd2 = pack2(-d, -d);
#pragma unroll
    for (int k = 0; k < V4; ++k) {
        int j = k * THREADS + threadIdx.x;
        if (j < nvec)
        {
            const f32x2 e01 = pack2(v[k].x, v[k].y), e23 = pack2(v[k].z, v[k].w);
            const f32x2 q01 = mul2(e01, rd2), q23 = mul2(e23, rd2);
            float q0, q1, q2, q3;
            unpack2(q01, q0, q1);
            unpack2(q23, q2, q3);
            float4 res;
            if ((q0 >= 1e-30f) & (q1 >= 1e-30f) & (q2 >= 1e-30f) & (q3 >= 1e-30f)) {
                // quotient = q + (e - q d) r, the correctly rounded one for normal results
                unpack2(fma2(fma2(q01, nd2, e01), rd2, q01), res.x, res.y);
                unpack2(fma2(fma2(q23, nd2, e23), rd2, q23), res.z, res.w);
            } else {
                res = make_float4(div_small_by(v[k].x, d, rd), div_small_by(v[k].y, d, rd),
                                  div_small_by(v[k].z, d, rd), div_small_by(v[k].w, d, rd));
            }
            __stcs(o + j, res);
        }
    }
}

// Several short rows per block: one warp per row, row kept in registers.
template <int PER_LANE>
__global__ void __launch_bounds__(256) softmax_rows_warp_kernel(const float *in, int64_t rows, int64_t cols, float *out) {
    int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows)
        return;
    int lane       = threadIdx.x & 31;
    const float *r = in + row * cols;
    float *o       = out + row * cols;
    float v[PER_LANE];
    float best = -INFINITY;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
        int64_t j = (int64_t)k * 32 + lane;
        v[k]      = j < cols ? r[j] : -INFINITY;
        if (j < cols && v[k] > best)
            best = v[k];
    }
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1)
        best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o2));
    float first = __shfl_sync(0xffffffffu, v[0], 0);
    if (first != first)
        best = first;
    double acc = 0.0;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
        int64_t j = (int64_t)k * 32 + lane;
        if (j < cols) {
            float s = __fsub_rn(v[k], best);
            v[k]    = exp_f32(s);
            acc += (double)v[k];
        }
    }
    acc     = warp_sum(acc);
    float d = (float)acc;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
        int64_t j = (int64_t)k * 32 + lane;
        if (j < cols)
            o[j] = __fdiv_rn(v[k], d);
    }
}

// Rows too long for registers: three passes over global memory, one block per row.
__global__ void __launch_bounds__(256) softmax_rows_stream_kernel(const float *in, int64_t rows, int64_t cols, float *out) {
    __shared__ float s_max[8];
    __shared__ double s_sum[8];
    int64_t row    = blockIdx.x;
    const float *r = in + row * cols;
    float *o       = out + row * cols;
    float best     = -INFINITY;
    for (int64_t j = threadIdx.x; j < cols; j += 256)
        if (r[j] > best)
            best = r[j];
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1)
        best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o2));
    if ((threadIdx.x & 31) == 0)
        s_max[threadIdx.x >> 5] = best;
    __syncthreads();
    float m = s_max[0];
    for (int w = 1; w < 8; ++w)
        m = fmaxf(m, s_max[w]);
    if (r[0] != r[0])
        m = r[0];
    double acc = 0.0;
    for (int64_t j = threadIdx.x; j < cols; j += 256) {
        float e = exp_f32(__fsub_rn(r[j], m));
        o[j]    = e;
        acc += (double)e;
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0)
        s_sum[threadIdx.x >> 5] = acc;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < 8; ++w)
        total += s_sum[w];
    float d = (float)total;
    for (int64_t j = threadIdx.x; j < cols; j += 256)
        o[j] = __fdiv_rn(o[j], d);
}

// ---- transpose / concat -----------------------------------------------------------------

template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T *in, int64_t rows, int64_t cols, T *out) {
    __shared__ T tile[32][33];
    int tx      = threadIdx.x & 31;
    int ty      = threadIdx.x >> 5;
    int64_t c0  = (int64_t)blockIdx.x * 32;
    int64_t r0  = (int64_t)blockIdx.y * 32;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        int64_t r = r0 + ty + k * 8, c = c0 + tx;
        if (r < rows && c < cols)
            tile[ty + k * 8][tx] = in[r * cols + c];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        int64_t c = c0 + ty + k * 8, r = r0 + tx; // out[c][r]
        if (r < rows && c < cols)
            out[c * rows + r] = tile[tx][ty + k * 8];
    }
}

// float32 with both extents multiples of four: 64 x 64 tiles, 128-bit loads along the input rows
// and 128-bit stores along the output rows (four times the bytes in flight per thread of the
// element-wise kernel above).
__global__ void __launch_bounds__(256) transpose_f32x4_kernel(
    const float *__restrict__ in, int64_t rows, int64_t cols, float *__restrict__ out) {
    __shared__ float tile[64][65];
    const int q      = threadIdx.x & 15;  // which group of four along the contiguous direction
    const int lane_r = threadIdx.x >> 4;  // 0..15
    const int64_t c0 = (int64_t)blockIdx.x * 64, r0 = (int64_t)blockIdx.y * 64;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int r      = lane_r + 16 * k;
        const int64_t gr = r0 + r, gc = c0 + q * 4;
        if (gr < rows && gc < cols) {
            const float4 v = __ldcs(reinterpret_cast<const float4 *>(in + gr * cols + gc));
            tile[r][q * 4] = v.x, tile[r][q * 4 + 1] = v.y, tile[r][q * 4 + 2] = v.z, tile[r][q * 4 + 3] = v.w;
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int c      = lane_r + 16 * k; // input column = output row
        const int64_t gc = c0 + c, gr = r0 + q * 4;
        if (gc < cols && gr < rows) {
            const float4 v = make_float4(tile[q * 4][c], tile[q * 4 + 1][c], tile[q * 4 + 2][c], tile[q * 4 + 3][c]);
            __stcs(reinterpret_cast<float4 *>(out + gc * rows + gr), v);
        }
    }
}

// out viewed as [outer][lhs_len + rhs_len] bytes-items of `unit` bytes each.
template <typename U>
__global__ void __launch_bounds__(256) concat_kernel(
    const U *lhs, const U *rhs, uint64_t outer, uint64_t lhs_len, uint64_t rhs_len, U *out) {
    uint64_t row_len = lhs_len + rhs_len;
    uint64_t total   = outer * row_len;
    uint64_t stride  = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
        uint64_t o = i / row_len, j = i - o * row_len;
        out[i] = j < lhs_len ? lhs[o * lhs_len + j] : rhs[o * rhs_len + (j - lhs_len)];
    }
}

template <typename U>
ct_status concat_typed(
    DeviceState *st, const void *l, const void *r, uint64_t outer, uint64_t ll, uint64_t rl, void *o) {
    uint64_t total  = outer * (ll + rl);
    uint64_t blocks = (total + 255) / 256;
    uint64_t cap    = (uint64_t)st->sm_count * 16;
    if (blocks > cap)
        blocks = cap;
    ProfScope prof("concat");
    concat_kernel<U><<<(unsigned)blocks, 256, 0, stream()>>>(
        static_cast<const U *>(l), static_cast<const U *>(r), outer, ll, rl, static_cast<U *>(o));
    CT_LAUNCH_CHECK("concat");
    return CT_OK;
}

} // namespace
} // namespace ct

using namespace ct;

extern "C" {

ct_status ct_sum(ct_dtype dt, const void *in, uint64_t n, double *result) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (!valid_dtype(dt) || !result)
        return fail(CT_ERR_INVALID, "ct_sum: bad dtype or null result");
    if (n == 0) {
        *result = 0.0;
        return CT_OK;
    }
    if (!in)
        return fail(CT_ERR_INVALID, "ct_sum: null pointer");
    switch (dt) {
    case CT_F32:
        return sum_typed<float>(st, static_cast<const float *>(in), n, result);
    case CT_I64:
        return sum_typed<int64_t>(st, static_cast<const int64_t *>(in), n, result);
    default:
        return sum_typed<uint8_t>(st, static_cast<const uint8_t *>(in), n, result);
    }
}

ct_status ct_sum_axis(ct_dtype dt, const void *in, int64_t rows, int64_t cols, int64_t axis, float *out) {
    return reduce_axis<RED_SUM, float>(dt, in, rows, cols, axis, out, "sum");
}

ct_status ct_max_axis(ct_dtype dt, const void *in, int64_t rows, int64_t cols, int64_t axis, float *out) {
    return reduce_axis<RED_MAX, float>(dt, in, rows, cols, axis, out, "max");
}

ct_status ct_argmax_axis(ct_dtype dt, const void *in, int64_t rows, int64_t cols, int64_t axis, int64_t *out) {
    return reduce_axis<RED_ARGMAX, int64_t>(dt, in, rows, cols, axis, out, "argmax");
}

ct_status ct_softmax_rows(const float *in, int64_t rows, int64_t cols, float *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (rows < 0 || cols < 0)
        return fail(CT_ERR_INVALID, "softmax: negative dimension");
    if (rows == 0 || cols == 0)
        return CT_OK;
    if (!in || !out)
        return fail(CT_ERR_INVALID, "softmax: null pointer");
    if (rows > 0x7fffffffll)
        return fail(CT_ERR_TOO_LARGE, "softmax: too many rows");
    unsigned wblocks = (unsigned)((rows + 7) / 8);
    ProfScope prof("softmax");
    if (cols <= 32)
        softmax_rows_warp_kernel<1><<<wblocks, 256, 0, stream()>>>(in, rows, cols, out);
    else if (cols <= 128)
        softmax_rows_warp_kernel<4><<<wblocks, 256, 0, stream()>>>(in, rows, cols, out);
    else if (cols <= 512)
        softmax_rows_warp_kernel<16><<<wblocks, 256, 0, stream()>>>(in, rows, cols, out);
    else if (cols <= 8192 && (cols & 3) == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0) {
        if (cols <= 2048)
            softmax_rows_wide_kernel<1, 512><<<(unsigned)rows, 512, 0, stream()>>>(in, rows, cols, out);
        else if (cols <= 4096)
            softmax_rows_wide_kernel<2, 512><<<(unsigned)rows, 512, 0, stream()>>>(in, rows, cols, out);
        else
            softmax_rows_wide_kernel<4, 512><<<(unsigned)rows, 512, 0, stream()>>>(in, rows, cols, out);
    } else if (cols <= 2048)
        softmax_rows_kernel<8, 256><<<(unsigned)rows, 256, 0, stream()>>>(in, rows, cols, out);
    else if (cols <= 8192)
        softmax_rows_kernel<8, 1024><<<(unsigned)rows, 1024, 0, stream()>>>(in, rows, cols, out);
    else
        softmax_rows_stream_kernel<<<(unsigned)rows, 256, 0, stream()>>>(in, rows, cols, out);
    CT_LAUNCH_CHECK("softmax_rows");
    return CT_OK;
}

ct_status ct_transpose(ct_dtype dt, const void *in, int64_t rows, int64_t cols, void *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (!valid_dtype(dt) || rows < 0 || cols < 0)
        return fail(CT_ERR_INVALID, "transpose: bad dtype or dimension");
    if (rows == 0 || cols == 0)
        return CT_OK;
    dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
    if ((rows + 31) / 32 > 65535)
        return fail(CT_ERR_TOO_LARGE, "transpose: too many rows");
    ProfScope prof("transpose");
    if (dt == CT_F32 && (rows & 3) == 0 && (cols & 3) == 0 && (rows + 63) / 64 <= 65535 &&
        ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0) {
        dim3 grid64((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64));
        transpose_f32x4_kernel<<<grid64, 256, 0, stream()>>>(
            static_cast<const float *>(in), rows, cols, static_cast<float *>(out));
        CT_LAUNCH_CHECK("transpose");
        return CT_OK;
    }
    switch (dt) {
    case CT_F32:
        transpose_kernel<float><<<grid, 256, 0, stream()>>>(
            static_cast<const float *>(in), rows, cols, static_cast<float *>(out));
        break;
    case CT_I64:
        transpose_kernel<int64_t><<<grid, 256, 0, stream()>>>(
            static_cast<const int64_t *>(in), rows, cols, static_cast<int64_t *>(out));
        break;
    default:
        transpose_kernel<uint8_t><<<grid, 256, 0, stream()>>>(
            static_cast<const uint8_t *>(in), rows, cols, static_cast<uint8_t *>(out));
        break;
    }
    CT_LAUNCH_CHECK("transpose");
    return CT_OK;
}

ct_status ct_concat(
    ct_dtype dt, const void *lhs, const void *rhs, uint64_t outer, uint64_t lhs_axis,
    uint64_t rhs_axis, uint64_t inner, void *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (!valid_dtype(dt))
        return fail(CT_ERR_INVALID, "concat: bad dtype");
    uint64_t ll = lhs_axis * inner, rl = rhs_axis * inner;
    if (outer == 0 || ll + rl == 0)
        return CT_OK;
    size_t item = dtype_size(dt);
    // Move the widest unit that divides both row segments and respects the alignment.
    uintptr_t bits = reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs) |
                     reinterpret_cast<uintptr_t>(out) | (ll * item) | (rl * item);
    if ((bits & 15u) == 0)
        return concat_typed<uint4>(st, lhs, rhs, outer, ll * item / 16, rl * item / 16, out);
    if ((bits & 7u) == 0)
        return concat_typed<uint64_t>(st, lhs, rhs, outer, ll * item / 8, rl * item / 8, out);
    if ((bits & 3u) == 0)
        return concat_typed<uint32_t>(st, lhs, rhs, outer, ll * item / 4, rl * item / 4, out);
    return concat_typed<uint8_t>(st, lhs, rhs, outer, ll * item, rl * item, out);
}

} // extern "C"
