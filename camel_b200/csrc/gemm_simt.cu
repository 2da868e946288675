// CUDA-core contractions for the shapes and dtypes the tensor-core kernel does not take:
//  - matmul_generic: any dtype pair, float64 accumulation per output element, exactly the
//    reference loop (modules/tensor/operators.cpp:757-766); used for int64/bool operands and
//    for tiny problems.
//  - gemm_f32_skinny: float32 x float32 with n <= 32 output columns (the classifier layer of
//    an MLP): one warp per output row, float64 accumulation, with bias / relu / row-softmax /
//    argmax fused, so the logits never round-trip through HBM.
#include "common.cuh"
#include "fastmath.cuh"

#include <cmath>

namespace ct {
namespace {

__device__ __forceinline__ double ld_as_double(int dt, const void *p, int64_t i) {
    switch (dt) {
    case CT_F32:
        return (double)static_cast<const float *>(p)[i];
    case CT_I64:
        return (double)static_cast<const int64_t *>(p)[i];
    default:
        return static_cast<const uint8_t *>(p)[i] != 0 ? 1.0 : 0.0;
    }
}

__device__ __forceinline__ void st_from_double(int dt, void *p, int64_t i, double v) {
    switch (dt) {
    case CT_F32:
        static_cast<float *>(p)[i] = (float)v;
        break;
    case CT_I64:
        static_cast<int64_t *>(p)[i] = (int64_t)v;
        break;
    default:
        static_cast<uint8_t *>(p)[i] = v != 0.0 ? 1 : 0;
        break;
    }
}

// 16x16 outputs per block, operands staged through shared memory as float64.
__global__ void __launch_bounds__(256) matmul_generic_kernel(
    int adt, const void *a, int bdt, const void *b, int64_t m, int64_t k, int64_t n, int odt,
    void *out) {
    __shared__ double sa[16][17];
    __shared__ double sb[16][17];
    int tx      = threadIdx.x & 15;
    int ty      = threadIdx.x >> 4;
    int64_t row = (int64_t)blockIdx.y * 16 + ty;
    int64_t col = (int64_t)blockIdx.x * 16 + tx;
    double acc  = 0.0;
    for (int64_t k0 = 0; k0 < k; k0 += 16) {
        int64_t ka = k0 + tx, kb = k0 + ty;
        sa[ty][tx] = (row < m && ka < k) ? ld_as_double(adt, a, row * k + ka) : 0.0;
        sb[ty][tx] = (kb < k && col < n) ? ld_as_double(bdt, b, kb * n + col) : 0.0;
        __syncthreads();
        int lim = (int)((k - k0) < 16 ? (k - k0) : 16);
        for (int kk = 0; kk < lim; ++kk)
            acc += sa[ty][kk] * sb[kk][tx]; // k ascending, like the reference
        __syncthreads();
    }
    if (row < m && col < n)
        st_from_double(odt, out, row * n + col, acc);
}

// One warp per output row; lanes split k.  N_MAX bounds the register accumulators.
template <int N_MAX>
__global__ void __launch_bounds__(256) gemm_skinny_kernel(
    const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
    int64_t m, int64_t k, int n, int act, float *__restrict__ out, int64_t *__restrict__ argmax) {
    int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= m)
        return;
    int lane        = threadIdx.x & 31;
    const float *xr = x + row * k;
    double acc[N_MAX];
#pragma unroll
    for (int j = 0; j < N_MAX; ++j)
        acc[j] = 0.0;
    for (int64_t kk = lane; kk < k; kk += 32) {
        double xv       = (double)xr[kk];
        const float *wr = w + kk * n;
#pragma unroll
        for (int j = 0; j < N_MAX; ++j)
            if (j < n)
                acc[j] = __fma_rn(xv, (double)__ldg(wr + j), acc[j]); // float32 x float32 is exact in float64: same bits as mul, add
    }
#pragma unroll
    for (int j = 0; j < N_MAX; ++j) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    }
    // Every lane now holds all n sums; lane j finishes column j.
    float logit = 0.0f;
#pragma unroll
    for (int j = 0; j < N_MAX; ++j) {
        if (j == lane && j < n) {
            double v = acc[j];
            if (bias)
                v += (double)bias[j]; // the bias is the last term of the float64 sum
            logit = (float)v;
        }
    }
    bool live = lane < n;
    if (act == CT_ACT_RELU) {
        logit = __fmul_rn(logit, logit > 0.0f ? 1.0f : 0.0f);
    }
    if (act != CT_ACT_SOFTMAX) {
        if (live)
            out[row * n + lane] = logit;
        return;
    }
    // Row softmax and argmax across the first n lanes, with the reference's scan semantics:
    // element 0 seeds, a later element wins only on strict '>'.
    float best   = __shfl_sync(0xffffffffu, logit, 0);
    int best_idx = 0;
    for (int j = 1; j < n; ++j) {
        float v = __shfl_sync(0xffffffffu, logit, j);
        if (v > best) {
            best     = v;
            best_idx = j;
        }
    }
    float e  = live ? exp_f32(__fsub_rn(logit, best)) : 0.0f;
    double s = 0.0;
    for (int j = 0; j < n; ++j)
        s += (double)__shfl_sync(0xffffffffu, e, j);
    float d = (float)s;
    if (live)
        out[row * n + lane] = __fdiv_rn(e, d);
    if (argmax && lane == 0)
        argmax[row] = best_idx;
}

// Lane j < n holds the rounded logit of column j of one row: activation, and for softmax the
// row softmax / argmax with the reference's scan semantics (element 0 seeds, a later element
// wins only on strict '>').  Called by a whole warp.
__device__ __forceinline__ void skinny_finish_logit(
    float logit, int64_t row, int n, int act, int lane, float *__restrict__ out,
    int64_t *__restrict__ argmax) {
    bool live = lane < n;
    if (act == CT_ACT_RELU)
        logit = __fmul_rn(logit, logit > 0.0f ? 1.0f : 0.0f);
    if (act != CT_ACT_SOFTMAX) {
        if (live)
            out[row * n + lane] = logit;
        return;
    }
    float best   = __shfl_sync(0xffffffffu, logit, 0);
    int best_idx = 0;
    for (int j = 1; j < n; ++j) {
        float v = __shfl_sync(0xffffffffu, logit, j);
        if (v > best) {
            best     = v;
            best_idx = j;
        }
    }
    float e  = live ? exp_f32(__fsub_rn(logit, best)) : 0.0f;
    double s = 0.0;
    for (int j = 0; j < n; ++j)
        s += (double)__shfl_sync(0xffffffffu, e, j);
    float d = (float)s;
    if (live)
        out[row * n + lane] = __fdiv_rn(e, d);
    if (argmax && lane == 0)
        argmax[row] = best_idx;
}

// The same for two rows at once, one per half-warp: `sub` is the lane within its half.
__device__ __forceinline__ void skinny_finish_logit_half(
    float logit, int64_t row, bool row_valid, int n, int act, int sub, float *__restrict__ out,
    int64_t *__restrict__ argmax) {
    bool live = sub < n && row_valid;
    if (act == CT_ACT_RELU)
        logit = __fmul_rn(logit, logit > 0.0f ? 1.0f : 0.0f);
    if (act != CT_ACT_SOFTMAX) {
        if (live)
            out[row * n + sub] = logit;
        return;
    }
    float best   = __shfl_sync(0xffffffffu, logit, 0, 16);
    int best_idx = 0;
    for (int j = 1; j < n; ++j) {
        float v = __shfl_sync(0xffffffffu, logit, j, 16);
        if (v > best) {
            best     = v;
            best_idx = j;
        }
    }
    float e  = sub < n ? exp_f32(__fsub_rn(logit, best)) : 0.0f;
    double s = 0.0;
    for (int j = 0; j < n; ++j)
        s += (double)__shfl_sync(0xffffffffu, e, j, 16);
    float d = (float)s;
    if (live)
        out[row * n + sub] = __fdiv_rn(e, d);
    if (argmax && sub == 0 && row_valid)
        argmax[row] = best_idx;
}

// Finishes one output row held as per-lane partial sums: butterfly reduction, then bias,
// activation, and (for softmax) the row softmax / argmax across the first n lanes.
template <int N_MAX>
__device__ __forceinline__ void skinny_finish_row(
    double (&acc)[N_MAX], const float *__restrict__ bias, int64_t row, int n, int act, int lane,
    float *__restrict__ out, int64_t *__restrict__ argmax) {
#pragma unroll
    for (int j = 0; j < N_MAX; ++j) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    }
    float logit = 0.0f;
#pragma unroll
    for (int j = 0; j < N_MAX; ++j) {
        if (j == lane && j < n) {
            double v = acc[j];
            if (bias)
                v += (double)bias[j]; // the bias is the last term of the float64 sum
            logit = (float)v;
        }
    }
    skinny_finish_logit(logit, row, n, act, lane, out, argmax);
}

// Same contraction with the whole weight matrix [k][n] staged once per block in shared memory
// (k*n*4 bytes <= 200 KB): the weight reads that made the kernel above latency-bound become
// shared-memory reads, the activations stream in with 128-bit loads, and a persistent grid
// of 2 blocks per SM walks the rows.
template <int N_MAX>
__global__ void __launch_bounds__(256) gemm_skinny_smem_kernel(
    const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
    int64_t m, int64_t k, int n, int act, float *__restrict__ out, int64_t *__restrict__ argmax) {
    extern __shared__ __align__(16) double w_s[];
    // staged transposed [n][k] and already widened to float64: the float32 -> float64
    // conversions run on the slow special-function pipe, so they are paid once per weight
    // and block here instead of once per multiply-add
    const int total = (int)(k * n); // <= 25600 by the dispatch condition
    for (int base = threadIdx.x; base < total; base += 256 * 8) {
        float tmp[8]; // eight independent loads in flight per thread, then the scattered stores
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            int i  = base + u * 256;
            tmp[u] = i < total ? __ldg(w + i) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            int i = base + u * 256;
            if (i < total) {
                int kk = i / n, j = i - kk * n;
                w_s[(int64_t)j * k + kk] = (double)tmp[u];
            }
        }
    }
    __syncthreads();
    const int lane     = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t step = (int64_t)gridDim.x * 8;
    const bool vec     = (k & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    for (int64_t row = warp; row < m; row += step) {
        const float *xr = x + row * k;
        double acc[N_MAX];
#pragma unroll
        for (int j = 0; j < N_MAX; ++j)
            acc[j] = 0.0;
        if (vec) {
            // eight 128-bit loads in flight per lane before any arithmetic: with few resident warps
            // the row would otherwise be one load-latency per 128 values of k
            constexpr int kChunk = 8;
            for (int64_t kk0 = (int64_t)lane * 4; kk0 < k; kk0 += 128 * kChunk) {
                float4 q[kChunk];
#pragma unroll
                for (int c = 0; c < kChunk; ++c) {
                    int64_t kk = kk0 + (int64_t)c * 128;
                    q[c]       = kk < k ? __ldcs(reinterpret_cast<const float4 *>(xr + kk)) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int c = 0; c < kChunk; ++c) {
                    int64_t kk = kk0 + (int64_t)c * 128;
                    if (kk >= k)
                        break;
                    double x0 = (double)q[c].x, x1 = (double)q[c].y, x2 = (double)q[c].z, x3 = (double)q[c].w;
#pragma unroll
                    for (int j = 0; j < N_MAX; ++j)
                        if (j < n) {
                            const double2 *wp = reinterpret_cast<const double2 *>(w_s + (int64_t)j * k + kk);
                            double2 wa = wp[0], wb = wp[1];
                            acc[j] = __fma_rn(x0, wa.x, acc[j]);
                            acc[j] = __fma_rn(x1, wa.y, acc[j]);
                            acc[j] = __fma_rn(x2, wb.x, acc[j]);
                            acc[j] = __fma_rn(x3, wb.y, acc[j]);
                        }
                }
            }
        } else {
            for (int64_t kk = lane; kk < k; kk += 32) {
                double xd = (double)xr[kk];
#pragma unroll
                for (int j = 0; j < N_MAX; ++j)
                    if (j < n)
                        acc[j] = __fma_rn(xd, w_s[(int64_t)j * k + kk], acc[j]);
            }
        }
        skinny_finish_row<N_MAX>(acc, bias, row, n, act, lane, out, argmax);
    }
}

template <int N_MAX>
ct_status launch_skinny_smem(
    DeviceState *st, const float *a, const float *b, const float *bias, int64_t m, int64_t k, int n,
    int act, float *out, int64_t *argmax) {
    size_t smem = (size_t)k * n * sizeof(double);
    if (smem > 48 * 1024)
        CT_CUDA(cudaFuncSetAttribute(
            gemm_skinny_smem_kernel<N_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    int64_t blocks = (m + 7) / 8;
    int64_t cap    = (int64_t)st->sm_count * (smem > 100 * 1024 ? 1 : 2);
    if (blocks > cap)
        blocks = cap;
    gemm_skinny_smem_kernel<N_MAX><<<(unsigned)blocks, 256, smem, stream()>>>(a, b, bias, m, k, n, act, out, argmax);
    CT_LAUNCH_CHECK("gemm_skinny_smem");
    return CT_OK;
}

__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gmem_src) {
    uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_src) : "memory");
}

__device__ __forceinline__ void cp_async_4(void *smem_dst, const void *gmem_src) {
    unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gmem_src) : "memory");
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

// Waits until at most `pending` of this thread's committed copy groups are still in flight.
__device__ __forceinline__ void cp_async_wait_pending(int pending) {
    switch (pending) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
    }
}

// Row-tiled variant for the classifier layer of a large batch.  A block owns 32 rows; warp s owns
// the k-slice [s*ks, (s+1)*ks) and lane r owns row r, so every weight read is one broadcast
// shared-memory wavefront for 32 rows (the warp-per-row kernel above re-reads the whole weight
// matrix from shared memory for every row, which bounds it).  The activations of a slice arrive
// by 16-byte asynchronous copies in 32-wide k chunks, each its own commit group, so arithmetic on
// chunk c overlaps the arrival of the later chunks; the weights of the slice are widened to
// float64 once per block.  NP = ceil(n/2) column pairs; the float64 partial sums of the sixteen
// slices are added in slice order, then bias, activation and softmax / argmax as above.
constexpr int kSkinnyWarps = 16; // k-slices per block

#ifdef CT_GEMM_TRACE
__device__ unsigned long long g_skinny_trace[1024 * 8];
#define SK_STAMP(slot)                                                                     \
    do {                                                                                   \
        if (threadIdx.x == 0 && blockIdx.x < 1024)                                         \
            g_skinny_trace[blockIdx.x * 8 + (slot)] = (unsigned long long)clock64();       \
    } while (0)
#else
#define SK_STAMP(slot) do { } while (0)
#endif

template <int NP>
__global__ void __launch_bounds__(32 * kSkinnyWarps, 1) gemm_skinny_tile_kernel(
    const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
    int64_t m, int k, int n, int ks, int x_aligned, int act, float *__restrict__ out,
    int64_t *__restrict__ argmax) {
    constexpr int NE = 2 * NP;
    extern __shared__ __align__(16) unsigned char skinny_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int xs_stride = ks + 4; // floats; (ks + 4) / 4 is odd, so 128-bit row reads spread over the banks
    float *xs           = reinterpret_cast<float *>(skinny_smem) + (size_t)warp * 32 * xs_stride;
    double *ws = reinterpret_cast<double *>(skinny_smem + (size_t)kSkinnyWarps * 32 * xs_stride * sizeof(float)) +
                 (size_t)warp * ks * NE;
    const int64_t row0 = (int64_t)blockIdx.x * 32;
    const int k0       = warp * ks;
    int klen           = k - k0;
    klen               = klen < 0 ? 0 : (klen > ks ? ks : klen);
    const int nchunks  = (klen + 31) >> 5;
    griddep_launch_dependents();
    griddep_wait(); // activations (and possibly weights) come from the previous kernel
    SK_STAMP(0);
    // weights of the slice, w[(k0 + kk) * n + j] -> ws[kk * NE + j], widened once.  The first round of
    // loads is issued before the activation copies so that its latency passes while those are issued.
    const float *wsrc    = w + (int64_t)k0 * n;
    const int total      = klen * n;
    constexpr int kLoads = 20; // independent loads in flight per lane: one round for 64 x 10 weights
    float tmp[kLoads];
    auto load_round = [&](int base) {
#pragma unroll
        for (int u = 0; u < kLoads; ++u) {
            int i  = base + u * 32;
            tmp[u] = i < total ? __ldg(wsrc + i) : 0.0f;
        }
    };
    auto store_round = [&](int base) {
#pragma unroll
        for (int u = 0; u < kLoads; ++u) {
            int i = base + u * 32;
            if (i < total) {
                // n is NE or NE - 1: divisions by constants instead of one by a run-time value
                int kk = n == NE ? i / NE : i / (NE > 1 ? NE - 1 : 1);
                int j  = i - kk * n;
                ws[kk * NE + j] = (double)tmp[u];
            }
        }
    };
    load_round(lane);
    // activations: chunk c covers k0 + [32c, 32c+32) of the block's 32 rows; eight lanes copy one row's 128 bytes
    for (int c = 0; c < nchunks; ++c) {
        if (x_aligned) {
            for (int idx = lane; idx < 256; idx += 32) {
                int r = idx >> 3, kk = c * 32 + (idx & 7) * 4;
                if (kk < klen && row0 + r < m)
                    cp_async_16(xs + r * xs_stride + kk, x + (row0 + r) * k + k0 + kk);
            }
        } else {
            // k is not a multiple of four (784 features and a bias column): rows start at any
            // 4-byte address, so a warp copies the 32 floats of a row's chunk one per lane
            const int kk = c * 32 + lane;
            if (kk < klen) {
                const float *src = x + row0 * k + k0 + kk;
                float *dst       = xs + kk;
                const int rows   = m - row0 < 32 ? (int)(m - row0) : 32;
#pragma unroll 4
                for (int r = 0; r < rows; ++r, src += k, dst += xs_stride)
                    cp_async_4(dst, src);
            }
        }
        cp_async_commit();
    }
    // the arithmetic walks k in fours: zero what lies between the end of the slice and the next four
    const int kpad = (klen + 3) & ~3;
    if (kpad > klen) {
        const int extra = kpad - klen;
        for (int idx = lane; idx < 32 * extra; idx += 32)
            xs[(idx / extra) * xs_stride + klen + idx % extra] = 0.0f;
        for (int idx = lane; idx < extra * NE; idx += 32)
            ws[klen * NE + idx] = 0.0;
    }
    SK_STAMP(1);
    store_round(lane);
    for (int base = lane + 32 * kLoads; base < total; base += 32 * kLoads) {
        load_round(base);
        store_round(base);
    }
    if (n < NE)
        for (int kk = lane; kk < klen; kk += 32)
            ws[kk * NE + n] = 0.0;
    __syncwarp();
    SK_STAMP(2);
    double acc[NE];
#pragma unroll
    for (int j = 0; j < NE; ++j)
        acc[j] = 0.0;
    const float *xrow = xs + lane * xs_stride;
    for (int c = 0; c < nchunks; ++c) {
        cp_async_wait_pending(nchunks - 1 - c);
        __syncwarp();
        if (c == 0)
            SK_STAMP(3);
        int kend = (c + 1) * 32 < klen ? (c + 1) * 32 : klen;
#pragma unroll 4
        for (int kk = c * 32; kk < kend; kk += 4) {
            float4 q     = *reinterpret_cast<const float4 *>(xrow + kk);
            double xd[4] = {(double)q.x, (double)q.y, (double)q.z, (double)q.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const double2 *wp = reinterpret_cast<const double2 *>(ws + (kk + u) * NE);
#pragma unroll
                for (int j = 0; j < NP; ++j) {
                    double2 wv = wp[j];
                    // float32 x float32 is exact in float64, so the fused form rounds like mul, add
                    acc[2 * j]     = __fma_rn(xd[u], wv.x, acc[2 * j]);
                    acc[2 * j + 1] = __fma_rn(xd[u], wv.y, acc[2 * j + 1]);
                }
            }
        }
    }
    SK_STAMP(4);
    __syncthreads(); // every warp is done with its activations: the region becomes the partial sums
    double *red = reinterpret_cast<double *>(skinny_smem);
#pragma unroll
    for (int j = 0; j < NE; ++j)
        red[((size_t)warp * 32 + lane) * NE + j] = acc[j];
    __syncthreads();
    SK_STAMP(5);
    // two rows per warp, one per half-warp; lane (sub) j < n of a half finishes column j
    static_assert(kSkinnyWarps == 16, "the finish phase maps one row to each half-warp");
    {
        const int sub = lane & 15;
        const int r   = warp * 2 + (lane >> 4);
        float logit   = 0.0f;
        if (sub < n) {
            double part[kSkinnyWarps];
#pragma unroll
            for (int s = 0; s < kSkinnyWarps; ++s)
                part[s] = red[((size_t)s * 32 + r) * NE + sub];
            double v = 0.0;
#pragma unroll
            for (int s = 0; s < kSkinnyWarps; ++s)
                v += part[s];
            if (bias)
                v += (double)bias[sub];
            logit = (float)v;
        }
        skinny_finish_logit_half(logit, row0 + r, row0 + r < m, n, act, sub, out, argmax);
    }
    SK_STAMP(6);
}

// Slice length of the tiled kernel: a multiple of 8 so that (ks + 4) / 4 is odd.
inline int skinny_tile_slice(int64_t k) { return (int)((((k + kSkinnyWarps - 1) / kSkinnyWarps) + 7) / 8 * 8); }

inline size_t skinny_tile_smem(int64_t k, int np) {
    int ks    = skinny_tile_slice(k);
    size_t xs = (size_t)kSkinnyWarps * 32 * (ks + 4) * sizeof(float);
    size_t ws = (size_t)kSkinnyWarps * ks * 2 * np * sizeof(double);
    size_t rd = (size_t)kSkinnyWarps * 32 * 2 * np * sizeof(double);
    return (xs > rd ? xs : rd) + ws;
}

template <int NP>
ct_status launch_skinny_tile(
    const float *a, const float *b, const float *bias, int64_t m, int64_t k, int n, int act, float *out,
    int64_t *argmax) {
    size_t smem = skinny_tile_smem(k, NP);
    if (smem > 48 * 1024)
        CT_CUDA(cudaFuncSetAttribute(
            gemm_skinny_tile_kernel<NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CT_CUDA(launch_dependent(
        gemm_skinny_tile_kernel<NP>, dim3((unsigned)((m + 31) / 32)), dim3(32 * kSkinnyWarps), smem, stream(), a, b, bias,
        m, (int)k, n, skinny_tile_slice(k), (int)((k & 3) == 0 && (reinterpret_cast<uintptr_t>(a) & 15u) == 0), act, out,
        argmax));
    CT_LAUNCH_CHECK("gemm_skinny_tile");
    return CT_OK;
}

} // namespace

ct_status matmul_generic(
    int adt, const void *a, int bdt, const void *b, int64_t m, int64_t k, int64_t n, void *out) {
    if (m == 0 || n == 0)
        return CT_OK;
    int odt = ct_result_dtype(CT_ADD, (ct_dtype)adt, (ct_dtype)bdt);
    if ((m + 15) / 16 > 65535)
        return fail(CT_ERR_TOO_LARGE, "matmul: too many rows for the generic kernel");
    dim3 grid((unsigned)((n + 15) / 16), (unsigned)((m + 15) / 16));
    matmul_generic_kernel<<<grid, 256, 0, stream()>>>(adt, a, bdt, b, m, k, n, odt, out);
    CT_LAUNCH_CHECK("matmul_generic");
    return CT_OK;
}

// ---- transposed left operand, few output columns --------------------------------------------
//
// out[i][j] = sum_k a_km[k][i] * b[k][j], n <= 32: the gradient of a classifier,
// `transpose(X) @ (probs - y)` (test/run/nn/mnist.cml:39; k = samples, m = features, n = classes).
// Both operands are read in their own row-major order, X exactly once: a thread owns R output rows
// (columns of X, so a warp's loads are contiguous), the rows of b are widened to float64 in shared
// memory once per block and read as broadcasts, and every product is an exact float64 FMA as in
// the reference (operators.cpp:757-766).  The long dimension is cut into slices over the grid;
// the slices' float64 sums are added in slice order by gemm_tn_skinny_finish_kernel, so the result
// does not depend on scheduling.  Bound by the float64 pipe and the read of X, which are about
// equal at n = 10.
constexpr int kTnThreads = 128;
constexpr int kTnChunk   = 32; // rows of b staged per step
constexpr int kTnGroup   = 4;  // k steps whose operands are fetched together, one group ahead

template <int V> struct TnCount {
    static constexpr int value = V;
};

// A read-only load that stays where it is written: the compiler may otherwise move a plain load
// down to its first use, which undoes fetching the operands a group ahead.  0 where !ok.
__device__ __forceinline__ float tn_load_early(const float *p, bool ok) {
    float v;
    asm volatile(
        "{ .reg .pred q; setp.ne.u32 q, %2, 0; mov.f32 %0, 0f00000000; @q ld.global.nc.f32 %0, [%1]; }"
        : "=f"(v)
        : "l"(p), "r"((unsigned)ok));
    return v;
}

__device__ __forceinline__ void tn_block_barrier() {
    // a named barrier counts arriving threads, wherever in the code they arrive from: the warps of a
    // block run differently specialised copies of the loop below
    asm volatile("bar.sync 1, %0;" ::"n"(kTnThreads) : "memory");
}

template <int NMAX, int R>
__global__ void __launch_bounds__(kTnThreads, 2) gemm_tn_skinny_kernel(
    const float *__restrict__ a_km, const float *__restrict__ b, int64_t m, int64_t k, int n, int64_t k_per_slice,
    double *__restrict__ partial) {
    constexpr int G  = kTnGroup;
    constexpr int BL = (kTnChunk * NMAX + kTnThreads - 1) / kTnThreads; // staged b values per thread
    __shared__ double bs[2][kTnChunk][NMAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t warp_row = ((int64_t)blockIdx.x * (kTnThreads / 32) + warp) * (32 * R);
    const int64_t row0     = warp_row + lane;
    // 32-row groups of this warp that hold rows at all: the others cost no loads and no arithmetic
    const int64_t left = m - warp_row;
    const int ractive  = left <= 0 ? 0 : (left >= 32 * R ? R : (int)((left + 31) / 32));
    const int64_t k0   = (int64_t)blockIdx.y * k_per_slice;
    const int64_t k1   = k0 + k_per_slice < k ? k0 + k_per_slice : k;

    float bnext[BL];
    auto fetch_b = [&](int64_t kc) {
#pragma unroll
        for (int u = 0; u < BL; ++u) {
            int idx = threadIdx.x + u * kTnThreads;
            int kk = idx / NMAX, j = idx - kk * NMAX;
            bnext[u] = (idx < kTnChunk * NMAX && kc + kk < k1 && j < n) ? __ldg(b + (kc + kk) * n + j) : 0.0f;
        }
    };
    auto store_b = [&](int buf) {
#pragma unroll
        for (int u = 0; u < BL; ++u) {
            int idx = threadIdx.x + u * kTnThreads;
            if (idx < kTnChunk * NMAX)
                (&bs[buf][0][0])[idx] = (double)bnext[u];
        }
    };

    auto run = [&](auto count) {
        constexpr int RA = decltype(count)::value; // 32-row groups this warp computes
        constexpr int RN = RA > 0 ? RA : 1;
        double acc[RN][NMAX];
#pragma unroll
        for (int r = 0; r < RN; ++r)
#pragma unroll
            for (int j = 0; j < NMAX; ++j)
                acc[r][j] = 0.0;
        bool rowok[RN];
#pragma unroll
        for (int r = 0; r < RN; ++r)
            rowok[r] = row0 + 32 * r < m;
        // operands of G k steps are fetched one group ahead of their use, into two register sets
        float abuf[2][G][RN];
        const float *pa = a_km + k0 * m + row0; // row `next` of the operand, this lane's first column
        int64_t next    = k0;
        auto fetch_a    = [&](float(&dst)[G][RN]) {
            if (RA > 0) {
#pragma unroll
                for (int u = 0; u < G; ++u)
#pragma unroll
                    for (int r = 0; r < RN; ++r)
                        dst[u][r] = tn_load_early(pa + u * m + 32 * r, next + u < k1 && rowok[r]);
                pa += G * m;
                next += G;
            }
        };
        auto compute = [&](const float(&src)[G][RN], int buf, int g) {
            if (RA > 0) {
#pragma unroll
                for (int u = 0; u < G; ++u) {
                    double av[RN];
#pragma unroll
                    for (int r = 0; r < RN; ++r)
                        av[r] = (double)src[u][r];
#pragma unroll
                    for (int j = 0; j < NMAX; ++j) {
                        double bj = bs[buf][g + u][j];
#pragma unroll
                        for (int r = 0; r < RN; ++r)
                            acc[r][j] = fma(av[r], bj, acc[r][j]);
                    }
                }
            }
        };
        fetch_b(k0);
        fetch_a(abuf[0]);
        store_b(0);
        tn_block_barrier();
        int buf = 0;
        for (int64_t kc = k0; kc < k1; kc += kTnChunk, buf ^= 1) {
            const bool more = kc + kTnChunk < k1;
            if (more)
                fetch_b(kc + kTnChunk);
#pragma unroll 1
            for (int g = 0; g < kTnChunk; g += 2 * G) {
                fetch_a(abuf[1]);
                compute(abuf[0], buf, g);
                fetch_a(abuf[0]); // may already belong to the next chunk; zeros past the slice
                compute(abuf[1], buf, g + G);
            }
            if (more)
                store_b(buf ^ 1); // nobody reads that buffer any more: all warps passed the last barrier
            tn_block_barrier();
        }
        if (RA > 0) {
#pragma unroll
            for (int r = 0; r < RN; ++r) {
                if (rowok[r]) {
                    double *dst = partial + ((int64_t)blockIdx.y * m + row0 + 32 * r) * n;
#pragma unroll
                    for (int j = 0; j < NMAX; ++j)
                        if (j < n)
                            dst[j] = acc[r][j];
                }
            }
        }
    };
    static_assert(R == 1 || R == 2 || R == 4, "row groups per warp");
    if (ractive == R)
        run(TnCount<R>{});
    else if (ractive == 0)
        run(TnCount<0>{});
    else if (R == 4 && ractive == 3)
        run(TnCount<(R == 4 ? 3 : 1)>{});
    else if (R == 4 && ractive == 2)
        run(TnCount<(R == 4 ? 2 : 1)>{});
    else
        run(TnCount<1>{});
}

// One warp per output element: lane l adds the slices l, l + 32, ... in that order, then the lanes'
// sums are added in a fixed butterfly - the same order on every run.
__global__ void __launch_bounds__(256) gemm_tn_skinny_finish_kernel(
    const double *__restrict__ partial, int64_t mn, int slices, float *__restrict__ out) {
    const int lane  = threadIdx.x & 31;
    const int64_t i = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 5;
    if (i >= mn)
        return;
    double sum = 0.0;
    for (int s = lane; s < slices; s += 32)
        sum += partial[(int64_t)s * mn + i];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1)
        sum += __shfl_xor_sync(0xffffffffu, sum, d);
    if (lane == 0)
        out[i] = (float)sum;
}

template <int NMAX, int R>
static ct_status launch_tn_skinny(
    DeviceState *st, const float *a_km, const float *b, int64_t m, int64_t k, int n, float *out) {
    const int64_t rows_per_block = (int64_t)(kTnThreads / 32) * 32 * R;
    const int64_t mblocks        = (m + rows_per_block - 1) / rows_per_block;
    // one wave: two blocks fit an SM, and rounding the slice length up only takes blocks away
    int64_t slices = 2 * (int64_t)st->sm_count / mblocks;
    const int64_t most           = (k + 4 * kTnChunk - 1) / (4 * kTnChunk); // at least four chunks per slice
    if (slices > most)
        slices = most;
    if (slices < 1)
        slices = 1;
    if (slices > 65535)
        slices = 65535;
    int64_t k_per_slice = (k + slices - 1) / slices;
    k_per_slice         = (k_per_slice + kTnChunk - 1) / kTnChunk * kTnChunk;
    if (k_per_slice < kTnChunk)
        k_per_slice = kTnChunk;
    slices = k > 0 ? (k + k_per_slice - 1) / k_per_slice : 1;
    CT_TRY(ensure_ws(&st->splitk_ws, &st->splitk_ws_bytes, (size_t)slices * m * n * sizeof(double)));
    auto *partial = static_cast<double *>(st->splitk_ws);
    dim3 grid((unsigned)mblocks, (unsigned)slices);
    gemm_tn_skinny_kernel<NMAX, R><<<grid, kTnThreads, 0, stream()>>>(a_km, b, m, k, n, k_per_slice, partial);
    CT_LAUNCH_CHECK("gemm_tn_skinny");
    const int64_t mn = m * n;
    gemm_tn_skinny_finish_kernel<<<(unsigned)((mn * 32 + 255) / 256), 256, 0, stream()>>>(partial, mn, (int)slices, out);
    CT_LAUNCH_CHECK("gemm_tn_skinny_finish");
    return CT_OK;
}

ct_status gemm_f32_tn_skinny(
    DeviceState *st, const float *a_km, const float *b, int64_t m, int64_t k, int64_t n, float *out) {
    if (m == 0 || n == 0)
        return CT_OK;
    if (n > 32 || m > 0x7fffffffll * 64)
        return fail(CT_ERR_INVALID, "transposed skinny GEMM takes at most 32 output columns");
    ProfScope prof("gemm_skinny");
    switch ((n + 1) / 2) {
    case 1: return launch_tn_skinny<2, 4>(st, a_km, b, m, k, (int)n, out);
    case 2: return launch_tn_skinny<4, 4>(st, a_km, b, m, k, (int)n, out);
    case 3: return launch_tn_skinny<6, 4>(st, a_km, b, m, k, (int)n, out);
    case 4: return launch_tn_skinny<8, 4>(st, a_km, b, m, k, (int)n, out);
    case 5: return launch_tn_skinny<10, 4>(st, a_km, b, m, k, (int)n, out);
    case 6: return launch_tn_skinny<12, 2>(st, a_km, b, m, k, (int)n, out);
    case 7: return launch_tn_skinny<14, 2>(st, a_km, b, m, k, (int)n, out);
    case 8: return launch_tn_skinny<16, 2>(st, a_km, b, m, k, (int)n, out);
    default: break;
    }
    if (n <= 24)
        return launch_tn_skinny<24, 1>(st, a_km, b, m, k, (int)n, out);
    return launch_tn_skinny<32, 1>(st, a_km, b, m, k, (int)n, out);
}

ct_status gemm_f32_skinny(
    DeviceState *st, const float *a, const float *b, const float *bias, int64_t m, int64_t k,
    int64_t n, int act, float *out, int64_t *argmax) {
    if (m == 0 || n == 0)
        return CT_OK;
    if (n > 32)
        return fail(CT_ERR_INVALID, "skinny GEMM takes at most 32 output columns");
    unsigned blocks = (unsigned)((m + 7) / 8);
    ProfScope prof("gemm_skinny");
    const int np = (int)((n + 1) / 2);
    if (m >= 256 && n <= 16 && k >= 32 && k <= (1 << 20) && skinny_tile_smem(k, np) <= 220 * 1024) {
        switch (np) {
        case 1: return launch_skinny_tile<1>(a, b, bias, m, k, (int)n, act, out, argmax);
        case 2: return launch_skinny_tile<2>(a, b, bias, m, k, (int)n, act, out, argmax);
        case 3: return launch_skinny_tile<3>(a, b, bias, m, k, (int)n, act, out, argmax);
        case 4: return launch_skinny_tile<4>(a, b, bias, m, k, (int)n, act, out, argmax);
        case 5: return launch_skinny_tile<5>(a, b, bias, m, k, (int)n, act, out, argmax);
        case 6: return launch_skinny_tile<6>(a, b, bias, m, k, (int)n, act, out, argmax);
        case 7: return launch_skinny_tile<7>(a, b, bias, m, k, (int)n, act, out, argmax);
        default: return launch_skinny_tile<8>(a, b, bias, m, k, (int)n, act, out, argmax);
        }
    }
    if ((size_t)k * n * sizeof(double) <= 200 * 1024 && k > 0) {
        if (n <= 8)
            return launch_skinny_smem<8>(st, a, b, bias, m, k, (int)n, act, out, argmax);
        if (n <= 16)
            return launch_skinny_smem<16>(st, a, b, bias, m, k, (int)n, act, out, argmax);
        return launch_skinny_smem<32>(st, a, b, bias, m, k, (int)n, act, out, argmax);
    }
    if (n <= 8)
        gemm_skinny_kernel<8><<<blocks, 256, 0, stream()>>>(a, b, bias, m, k, (int)n, act, out, argmax);
    else if (n <= 16)
        gemm_skinny_kernel<16><<<blocks, 256, 0, stream()>>>(a, b, bias, m, k, (int)n, act, out, argmax);
    else
        gemm_skinny_kernel<32><<<blocks, 256, 0, stream()>>>(a, b, bias, m, k, (int)n, act, out, argmax);
    CT_LAUNCH_CHECK("gemm_skinny");
    return CT_OK;
}

} // namespace ct

#ifdef CT_GEMM_TRACE
extern "C" int ct_debug_skinny_trace(unsigned long long *host, int count) {
    return (int)cudaMemcpyFromSymbol(host, ct::g_skinny_trace, sizeof(unsigned long long) * (size_t)count);
}
#endif
