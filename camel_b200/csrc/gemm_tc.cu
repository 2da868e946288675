// Tensor-core GEMM for sm_100a: C[m,n] = act(A[m,k] . B[k,n] + bias), float32 in and out.
//
// Precision modes
//   3xTF32 (default): every operand value v is split as v = hi + lo with hi = tf32(v) and
//   lo = tf32(v - hi); the kernel issues hi*hi + hi*lo + lo*hi on the tf32 tensor pipe
//   (the dropped lo*lo term is ~2^-22 relative).  The tensor core adds into float32
//   accumulators in tensor memory; to keep the rounding error of a long k loop at float32
//   level the accumulator is drained every `chunk` k-blocks into registers and summed there
//   with round-to-nearest adds, while the next chunk accumulates into the second TMEM buffer.
//   BF16: operands rounded to bf16 once, one MMA per k-step, same pipeline.
//
// Data layout in HBM
//   A pre-pass writes operand "planes": A -> [m][kp] (hi and lo), B -> transposed [n][kp]
//   (hi and lo), kp = k rounded up to the k-block, zero padded.  Both operands are then
//   K-major, so one TMA box of 128-byte rows with the 128-byte swizzle is exactly the
//   canonical shared-memory layout tcgen05.mma reads.  The pre-pass moves 12 bytes per operand
//   element once; the GEMM then reads planes only.
//
// Kernel structure (one CTA per 128 x BN output tile, one CTA per SM)
//   warp 0   : TMA producer - fills a ring of STAGES stages (A hi/lo + B hi/lo per k-block)
//   warp 1   : allocates TMEM, one elected lane issues tcgen05.mma and commits barriers
//   warps 2+ : epilogue - drain TMEM chunks into registers, then bias/activation and store
// Every barrier wait is bounded; on a timeout the kernel raises an error word, unwinds and
// frees its TMEM, and the host reports CT_ERR_TIMEOUT.
//
// Variants in this file
//   gemm_tc_kernel          one CTA per tile; long k ranges are accumulated in chunks (see above);
//                           few tiles with a long k are sliced along k (split-K + reduce kernel)
//   gemm_tc_stream_kernel   many tiles with k <= 1024: one CTA per SM walks the tiles, the store of
//                           tile i overlaps the MMAs of tile i+1 (conv2d, batched layers)
//   conv_swap_stream_kernel conv2d with <= 64 output channels: pixels on the accumulator rows
//   ct_weights_pack         the B planes of a weight matrix built once and reused
//   ct_matmul_f32_static    the GEMM for callers that may not allocate device memory
#include "common.cuh"
#include "tc_ptx.cuh"
#include "split.cuh"
#include "tmap.cuh"

#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdlib>
#include <mutex>

namespace ct {
namespace {

using namespace ptx;

constexpr int BM       = 128;
constexpr int ROW_B    = 128; // bytes of one operand row per k-block (= swizzle span)
constexpr int MODE_3X  = 0;
constexpr int MODE_BF  = 1;

// RB = bytes of one operand row per k-block = swizzle span of the shared-memory tiles (128 or
// 64).  A k-block of 64-byte rows halves the stage, so twice as many stages fit: with 96 KB
// stages (BN = 256, 3xTF32, RB = 128) only two fit and the MMA warp waits on every TMA round
// trip; four 48 KB stages cover that latency.
template <int BN, int MODE, int RB = ROW_B> struct Cfg {
    static constexpr int kRowB       = RB;
    static constexpr int kKSteps     = RB / 32; // MMAs along k per k-block (32 bytes of k each)
    static constexpr int kElem       = MODE == MODE_3X ? 4 : 2;
    static constexpr int kBlockK     = RB / kElem; // elements of k per k-block
    static constexpr int kPlanes     = MODE == MODE_3X ? 2 : 1;
    static constexpr int kABytes     = BM * RB;
    static constexpr int kBBytes     = BN * RB;
    static constexpr int kStageBytes = kPlanes * (kABytes + kBBytes);
    static constexpr int kStages     = (200 * 1024) / kStageBytes > 8 ? 8 : (200 * 1024) / kStageBytes;
    static constexpr int kEpiWarps   = BN / 32; // 128 accumulator columns per thread
    static constexpr int kThreads    = 64 + 32 * kEpiWarps;
    static constexpr int kTmemCols   = 2 * BN;
    static constexpr int kSmemBytes  = kStages * kStageBytes + 1024;
    static constexpr uint32_t kIdesc = make_idesc(MODE == MODE_3X ? 2u : 1u, BM, BN);
    // epilogue staging in the idle pipeline stages: 32 rows of 128 floats per warp, rows padded by 16 bytes
    static constexpr int kEpiRowBytes   = 128 * 4 + 16;
    static constexpr int kEpiStageBytes = 32 * kEpiRowBytes;
    static_assert(kEpiWarps * kEpiStageBytes <= kStages * kStageBytes, "epilogue staging must fit in the stages");
};

struct GemmParams {
    int64_t m, n;
    int num_k_blocks;
    int chunk_blocks;
    int tiles_m, tiles_n;
    const float *bias;
    int act;
    float *out;
    int64_t ldc;
    int batch;                // B planes and the output carry a leading batch dimension
    int64_t out_batch_stride; // elements between consecutive outputs of the batch
    int bias_per_row;         // bias indexed by output row (conv: one per output channel)
    uint32_t *flags;
    int kb_per_split;         // > 0: split-K, k-blocks per slice (slices take the batch index)
    int tile_n;               // output columns per tile: BN, or th*wo for the implicit-GEMM conv
    // implicit-GEMM convolution (conv != 0): the B operand is the NHWC input itself, fetched by
    // 4-D TMA boxes shifted by the filter tap, instead of a materialised patch matrix
    int conv;
    int conv_cblocks; // channel blocks of 32 per filter tap
    int conv_kw;      // filter width (taps are numbered r * kw + s)
    int conv_pad;
    int conv_th;      // output rows per tile
    // Row bands (bands > 0): the row tiles are dealt out band by band - band b holds the row tiles
    // [band_first[b], band_first[b + 1]) - and every CTA adds one to band_done[b] after its tile's
    // stores: a stream that waits for band_done[b] to reach the band's tile count (ct_stream_wait_value)
    // may then read the band, while later bands are still being computed by the same launch.
    int bands;
    int band_first[9];
    int64_t band_out_off[8]; // elements added to `out` for the tiles of band b (bands need not be adjacent in C)
    uint32_t *band_done;
};

// The band plan of the product being enqueued (set under the entry point's lock by
// ct_matmul_packed_bands, read by launch_gemm); bands == 0: none.
struct BandPlan {
    int bands = 0;
    int first[9];
    int64_t out_off[8];
    uint32_t *done = nullptr;
};
BandPlan g_band_plan;

// ---- operand pre-pass ---------------------------------------------------------------------

// in [rows][k] row-major  ->  hi/lo (or bf16) planes [rows][kp]
template <int MODE>
__global__ void __launch_bounds__(256) split_rows_kernel(
    const float *__restrict__ in, int64_t rows, int64_t k, int64_t kp, void *__restrict__ p_hi,
    void *__restrict__ p_lo) {
    int64_t total  = rows * kp;
    int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
        int64_t r = i / kp, c = i - r * kp;
        float v   = c < k ? in[r * k + c] : 0.0f;
        if (MODE == MODE_3X) {
            float hi, lo;
            split_tf32(v, hi, lo);
            static_cast<float *>(p_hi)[i] = hi;
            static_cast<float *>(p_lo)[i] = lo;
        } else {
            static_cast<__nv_bfloat16 *>(p_hi)[i] = __float2bfloat16_rn(v);
        }
    }
}

// Same result, four consecutive k per thread: 128-bit loads and stores, rows on blockIdx.y, no
// integer division.  kp is a multiple of 32 and the planes are 1 KiB aligned.  A thread takes
// kSplitRows rows at a time and issues all their loads before the first store: with one row per
// thread the kernel was a chain of one load and two stores per thread, i.e. latency, for the
// 4096 x 1024 activations of an MLP layer (8.5 us for 50 MB that mostly sit in L2).
constexpr int kSplitRows = 4;
template <int MODE>
__global__ void __launch_bounds__(256) split_rows_vec_kernel(
    const float *__restrict__ in, int64_t rows, int64_t k, int64_t kp, void *__restrict__ p_hi,
    void *__restrict__ p_lo, int in_vec_ok) {
    griddep_launch_dependents();
    griddep_wait(); // the input may be the previous kernel's output, the planes its operands
    const int64_t c = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 4;
    if (c >= kp)
        return;
    const bool vec = in_vec_ok && c + 3 < k;
    for (int64_t r0 = (int64_t)blockIdx.y * kSplitRows; r0 < rows; r0 += (int64_t)gridDim.y * kSplitRows) {
        float v[kSplitRows][4];
#pragma unroll
        for (int j = 0; j < kSplitRows; ++j) {
            const int64_t r = r0 + j;
            if (r < rows) {
                const float *src = in + r * k + c;
                if (vec) {
                    float4 q = __ldcs(reinterpret_cast<const float4 *>(src));
                    v[j][0] = q.x, v[j][1] = q.y, v[j][2] = q.z, v[j][3] = q.w;
                } else {
#pragma unroll
                    for (int t = 0; t < 4; ++t)
                        v[j][t] = c + t < k ? src[t] : 0.0f;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kSplitRows; ++j) {
            const int64_t r = r0 + j;
            if (r >= rows)
                break;
            const int64_t at = r * kp + c;
            if (MODE == MODE_3X) {
                float hi[4], lo[4];
#pragma unroll
                for (int t = 0; t < 4; ++t)
                    split_tf32(v[j][t], hi[t], lo[t]);
                *reinterpret_cast<float4 *>(static_cast<float *>(p_hi) + at) = make_float4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<float4 *>(static_cast<float *>(p_lo) + at) = make_float4(lo[0], lo[1], lo[2], lo[3]);
            } else {
                __nv_bfloat162 a = __floats2bfloat162_rn(v[j][0], v[j][1]);
                __nv_bfloat162 b = __floats2bfloat162_rn(v[j][2], v[j][3]);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t *>(&a);
                packed.y = *reinterpret_cast<uint32_t *>(&b);
                *reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(p_hi) + at) = packed;
            }
        }
    }
}

// in [k][n] row-major  ->  transposed planes [n][kp]
template <int MODE>
__global__ void __launch_bounds__(256) split_transpose_kernel(
    const float *__restrict__ in, int64_t k, int64_t n, int64_t kp, void *__restrict__ p_hi,
    void *__restrict__ p_lo, int64_t in_batch_stride = 0, int64_t out_batch_stride = 0) {
    __shared__ float tile[32][33];
    int tx     = threadIdx.x & 31;
    int ty     = threadIdx.x >> 5;
    int64_t n0 = (int64_t)blockIdx.x * 32;
    int64_t k0 = (int64_t)blockIdx.y * 32;
    // blockIdx.z walks a batch of [k][n] matrices (conv: one [c][h*w] image each)
    in += (int64_t)blockIdx.z * in_batch_stride;
    const int64_t out_base = (int64_t)blockIdx.z * out_batch_stride;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int64_t kk = k0 + ty + j * 8, nn = n0 + tx;
        tile[ty + j * 8][tx] = (kk < k && nn < n) ? in[kk * n + nn] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int64_t nn = n0 + ty + j * 8, kk = k0 + tx;
        if (nn < n && kk < kp) {
            float v     = tile[tx][ty + j * 8];
            int64_t at  = out_base + nn * kp + kk;
            if (MODE == MODE_3X) {
                float hi, lo;
                split_tf32(v, hi, lo);
                static_cast<float *>(p_hi)[at] = hi;
                static_cast<float *>(p_lo)[at] = lo;
            } else {
                static_cast<__nv_bfloat16 *>(p_hi)[at] = __float2bfloat16_rn(v);
            }
        }
    }
}

// ---- main kernel ------------------------------------------------------------------------

// Optional per-CTA timeline (SM clock stamps) for tuning; compiled in only with -DCT_GEMM_TRACE.
#ifdef CT_GEMM_TRACE
__device__ unsigned long long g_gemm_trace[1024 * 16];
#define CT_STAMP(slot)                                                        \
    do {                                                                      \
        if (blockIdx.x < 1024)                                                \
            g_gemm_trace[blockIdx.x * 16 + (slot)] = (unsigned long long)clock64(); \
    } while (0)
#define CT_STAMP_NS(slot)                                                     \
    do {                                                                      \
        if (blockIdx.x < 1024)                                                \
            g_gemm_trace[blockIdx.x * 16 + (slot)] = globaltimer_ns();        \
    } while (0)
#define CT_CLOCK() clock64()
#define CT_ACCUM(slot, cycles)                                                \
    do {                                                                      \
        if (blockIdx.x < 1024)                                                \
            g_gemm_trace[blockIdx.x * 16 + (slot)] += (unsigned long long)(cycles); \
    } while (0)
#else
#define CT_STAMP(slot) do { } while (0)
#define CT_STAMP_NS(slot) do { } while (0)
#define CT_CLOCK() 0ll
#define CT_ACCUM(slot, cycles) do { } while (0)
#endif

template <int BN, int MODE, int RB = ROW_B>
__global__ void __launch_bounds__(Cfg<BN, MODE, RB>::kThreads, 1) gemm_tc_kernel(
    const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
    const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
    const GemmParams p) {
    using C = Cfg<BN, MODE, RB>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[C::kStages];
    __shared__ uint64_t bar_empty[C::kStages];
    __shared__ uint64_t bar_tmem_full[2];
    __shared__ uint64_t bar_tmem_empty[2];
    __shared__ uint64_t bar_done;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag_s;
    volatile int *abort_flag = &abort_flag_s;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    griddep_launch_dependents();

    // If an earlier CTA of this launch already timed out, do not start: the launch has failed
    // and the remaining CTAs should drain at once instead of each waiting out its own budget.
    if (threadIdx.x == 0) {
        CT_STAMP(0);
        CT_STAMP_NS(8);
        abort_flag_s = *reinterpret_cast<volatile uint32_t *>(p.flags + FLAG_TIMEOUT) != 0 ? 1 : 0;
    }
    __syncthreads();

    // tile coordinates: groups of 16 row-tiles sweep the column tiles, so that the CTAs
    // running at the same time share operand tiles in L2
    int tm, tn, tz, band = 0;
    if (p.bands > 0) {
        // band by band; inside a band its row tiles sweep the column tiles together
        tz      = 0;
        int bid = blockIdx.x;
        while (band + 1 < p.bands && bid >= (p.band_first[band + 1] - p.band_first[band]) * p.tiles_n) {
            bid -= (p.band_first[band + 1] - p.band_first[band]) * p.tiles_n;
            ++band;
        }
        const int gm = p.band_first[band + 1] - p.band_first[band];
        tm           = p.band_first[band] + bid % gm;
        tn           = bid / gm;
    } else {
        int per_batch  = p.tiles_m * p.tiles_n;
        tz             = blockIdx.x / per_batch;
        int bid        = blockIdx.x - tz * per_batch;
        int group_size = 16 * p.tiles_n;
        int g          = bid / group_size;
        int first_m    = g * 16;
        int gm         = p.tiles_m - first_m < 16 ? p.tiles_m - first_m : 16;
        int in_group   = bid - g * group_size;
        tm             = first_m + in_group % gm;
        tn             = in_group / gm;
    }
    if (abort_flag_s) {
        // a waiting stream is released also when the launch has failed; the failure is on record
        if (threadIdx.x == 0 && p.bands > 0)
            atomicAdd(p.band_done + band, 1u);
        return;
    }

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    auto stage_addr          = [&](int s) { return smem_base + (uint32_t)s * C::kStageBytes; };

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bar_tmem_full[b]), 1);
            mbar_init(smem_u32(&bar_tmem_empty[b]), C::kEpiWarps);
        }
        mbar_init(smem_u32(&bar_done), 1);
        mbar_fence_init();
        prefetch_tensormap(&map_a_hi);
        prefetch_tensormap(&map_b_hi);
        if (MODE == MODE_3X) {
            prefetch_tensormap(&map_a_lo);
            prefetch_tensormap(&map_b_lo);
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    if (threadIdx.x == 0)
        CT_STAMP(1);
    // everything above is set-up that does not depend on earlier kernels; the operands and the
    // output may
    griddep_wait();

    // split-K (kb_per_split > 0): the leading block index selects a slice of the k-blocks instead
    // of a batch entry; every slice writes its own partial output, summed by a second kernel
    const int kb_first = p.kb_per_split > 0 ? tz * p.kb_per_split : 0;
    const int kb_left  = p.num_k_blocks - kb_first;
    const int nkb      = p.kb_per_split > 0 ? (kb_left < p.kb_per_split ? kb_left : p.kb_per_split) : p.num_k_blocks;
    const int bz       = p.kb_per_split > 0 ? 0 : tz; // batch coordinate of the B operand
    const int chunk      = p.chunk_blocks;
    const int num_chunks = (nkb + chunk - 1) / chunk;

    if (warp == 0) {
        // ===== TMA producer =====
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < nkb; ++kb) {
                int s       = kb % C::kStages;
                uint32_t ph = (uint32_t)(kb / C::kStages) & 1u;
                if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_flag))
                    break;
                uint32_t full = smem_u32(&bar_full[s]);
                uint32_t dst  = stage_addr(s);
                mbar_expect_tx(full, (uint32_t)(C::kPlanes * (C::kABytes + p.tile_n * C::kRowB)));
                int32_t kc = (kb_first + kb) * C::kBlockK;
                tma_load_2d(dst, &map_a_hi, full, kc, tm * BM);
                dst += C::kABytes;
                if (MODE == MODE_3X) {
                    tma_load_2d(dst, &map_a_lo, full, kc, tm * BM);
                    dst += C::kABytes;
                }
                if (p.conv) {
                    // k-block = (filter tap rs, channel block cb); the box covers th output rows
                    // by wo columns of 32 channels, shifted by the tap; the halo reads as zero
                    int rs = kb / p.conv_cblocks, cb = kb - rs * p.conv_cblocks;
                    int r = rs / p.conv_kw, sx = rs - r * p.conv_kw;
                    int32_t c0 = cb * C::kBlockK, w0 = sx - p.conv_pad, h0 = tn * p.conv_th + r - p.conv_pad;
                    tma_load_4d(dst, &map_b_hi, full, c0, w0, h0, tz);
                    dst += C::kBBytes;
                    if (MODE == MODE_3X)
                        tma_load_4d(dst, &map_b_lo, full, c0, w0, h0, tz);
                } else {
                    tma_load_3d(dst, &map_b_hi, full, kc, tn * BN, bz);
                    dst += C::kBBytes;
                    if (MODE == MODE_3X)
                        tma_load_3d(dst, &map_b_lo, full, kc, tn * BN, bz);
                }
                issued = kb + 1;
            }
            if (*abort_flag) {
                // unwind: let the copies still in flight land before the CTA goes away
                int first = issued - C::kStages < 0 ? 0 : issued - C::kStages;
                for (int kb = first; kb < issued; ++kb) {
                    uint32_t bar = smem_u32(&bar_full[kb % C::kStages]);
                    uint32_t ph  = (uint32_t)(kb / C::kStages) & 1u;
                    uint64_t t0  = globaltimer_ns();
                    while (!mbar_try_wait(bar, ph) && globaltimer_ns() - t0 < kWaitBudgetNs) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer =====
        if (lane == 0) {
            // MMA shape 128 x tile_n x (32 bytes of k): tile_n == BN except for conv tiles
            const uint32_t idesc = make_idesc(MODE == MODE_3X ? 2u : 1u, BM, (uint32_t)p.tile_n);
            int kb = 0;
            bool ok = true;
            for (int c = 0; c < num_chunks && ok; ++c) {
                int buf = c & 1;
                if (!mbar_wait(smem_u32(&bar_tmem_empty[buf]), (((uint32_t)c >> 1) & 1u) ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                uint32_t d_tmem = tmem_base + (uint32_t)buf * BN;
                int kb_end      = kb + chunk < nkb ? kb + chunk : nkb;
                bool first      = true;
                for (; kb < kb_end; ++kb) {
                    int s       = kb % C::kStages;
                    uint32_t ph = (uint32_t)(kb / C::kStages) & 1u;
                    if (!mbar_wait(smem_u32(&bar_full[s]), ph, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    if (kb == 0)
                        CT_STAMP(2);
                    uint32_t a_hi = stage_addr(s);
                    uint32_t a_lo = a_hi + C::kABytes;
                    uint32_t b_hi = a_hi + C::kPlanes * C::kABytes;
                    uint32_t b_lo = b_hi + C::kBBytes;
                    uint64_t da_hi = smem_desc_k<RB>(a_hi), db_hi = smem_desc_k<RB>(b_hi);
                    uint64_t da_lo = smem_desc_k<RB>(a_lo), db_lo = smem_desc_k<RB>(b_lo);
#pragma unroll
                    for (int kk = 0; kk < C::kKSteps; ++kk) {
                        uint64_t adv = (uint64_t)(kk * 32 >> 4);
                        if (MODE == MODE_3X) {
                            // small terms first, then the leading term
                            mma_tf32(d_tmem, da_lo + adv, db_hi + adv, idesc,first ? 0u : 1u);
                            mma_tf32(d_tmem, da_hi + adv, db_lo + adv, idesc,1u);
                            mma_tf32(d_tmem, da_hi + adv, db_hi + adv, idesc,1u);
                        } else {
                            mma_f16(d_tmem, da_hi + adv, db_hi + adv, idesc,first ? 0u : 1u);
                        }
                        first = false;
                    }
                    tc_commit(smem_u32(&bar_empty[s])); // stage reusable once these MMAs retire
                }
                if (ok)
                    tc_commit(smem_u32(&bar_tmem_full[buf]));
            }
            CT_STAMP(3);
            if (!ok || *abort_flag) {
                // unwind: wait until every MMA issued so far has retired
                tc_commit(smem_u32(&bar_done));
                uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(smem_u32(&bar_done), 0) && globaltimer_ns() - t0 < kWaitBudgetNs) {
                }
            }
        }
    } else {
        // ===== epilogue =====
        const int ew      = warp - 2;
        const int quarter = warp & 3;      // TMEM lanes this warp may read: 32*quarter ..
        const int half    = ew >> 2;       // which 128-column half of the tile (BN = 256)
        float acc[128];
#pragma unroll
        for (int j = 0; j < 128; ++j)
            acc[j] = 0.0f;
        bool ok = true;
        for (int c = 0; c < num_chunks; ++c) {
            int buf  = c & 1;
            bool got = mbar_wait(smem_u32(&bar_tmem_full[buf]), ((uint32_t)c >> 1) & 1u, abort_flag);
            ok       = __all_sync(0xffffffffu, got);
            if (!ok)
                break;
            if (c == num_chunks - 1 && warp == 2 && lane == 0)
                CT_STAMP(4);
            tc_fence_after_sync();
            uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + half * 128);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + g * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    acc[g * 32 + j] = __fadd_rn(acc[g * 32 + j], __uint_as_float(r[j]));
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&bar_tmem_empty[buf]));
        }
        if (warp == 2 && lane == 0)
            CT_STAMP(5);
        if (ok) {
            int64_t row  = (int64_t)tm * BM + quarter * 32 + lane;
            int64_t col0 = (int64_t)tn * p.tile_n + half * 128;
            int64_t lim  = (int64_t)(tn + 1) * p.tile_n < p.n ? (int64_t)(tn + 1) * p.tile_n : p.n;
            float *out_z = p.out + (int64_t)tz * p.out_batch_stride + (p.bands > 0 ? p.band_out_off[band] : 0);
            if ((p.ldc & 3) == 0 && (col0 & 3) == 0 && (reinterpret_cast<uintptr_t>(out_z) & 15u) == 0) {
                // A thread holds 128 consecutive columns of one row, so storing straight from the
                // registers writes 32 scattered 16-byte pieces per instruction, and the tile's store
                // then takes longer than 300 k-steps of the main loop.  The pipeline stages are idle by
                // now (every MMA has retired): each warp parks its 32 x 128 block there, rows padded to
                // 528 bytes so that neither phase has bank conflicts, and writes it out with one row
                // (512 contiguous bytes) per instruction.  Lane l owns columns 4l..4l+3 in that phase,
                // so the column bias is read once per lane.
                uint8_t *stg = smem_raw + (smem_base - smem_u32(smem_raw)) + (uint32_t)ew * C::kEpiStageBytes;
                float4 *mine = reinterpret_cast<float4 *>(stg + lane * C::kEpiRowBytes);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    mine[j] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
                __syncwarp();
                const int64_t col = col0 + lane * 4;
                float b4[4]       = {0.0f, 0.0f, 0.0f, 0.0f};
                if (p.bias && !p.bias_per_row) {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (col + q < lim)
                            b4[q] = p.bias[col + q];
                }
                const int64_t row0 = (int64_t)tm * BM + quarter * 32;
#pragma unroll 4
                for (int i = 0; i < 32; ++i) {
                    if (row0 + i >= p.m)
                        break;
                    float4 q4 = *reinterpret_cast<const float4 *>(stg + i * C::kEpiRowBytes + lane * 16);
                    float v[4] = {q4.x, q4.y, q4.z, q4.w};
                    const float rb = (p.bias && p.bias_per_row) ? p.bias[row0 + i] : 0.0f;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float x = v[q];
                        if (p.bias)
                            x = __fadd_rn(x, p.bias_per_row ? rb : b4[q]);
                        if (p.act == CT_ACT_RELU)
                            x = __fmul_rn(x, x > 0.0f ? 1.0f : 0.0f);
                        v[q] = x;
                    }
                    float *dst = out_z + (row0 + i) * p.ldc;
                    if (col + 3 < lim) {
                        *reinterpret_cast<float4 *>(dst + col) = make_float4(v[0], v[1], v[2], v[3]);
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (col + q < lim)
                                dst[col + q] = v[q];
                    }
                }
            } else if (row < p.m) {
                float *dst      = out_z + row * p.ldc;
                const float rb  = (p.bias && p.bias_per_row) ? p.bias[row] : 0.0f;
                const bool vec4 = (p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
#pragma unroll
                for (int j = 0; j < 128; j += 4) {
                    int64_t col = col0 + j;
                    float v[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float x = acc[j + q];
                        if (p.bias_per_row)
                            x = __fadd_rn(x, rb);
                        else if (p.bias && col + q < lim)
                            x = __fadd_rn(x, p.bias[col + q]);
                        if (p.act == CT_ACT_RELU)
                            x = __fmul_rn(x, x > 0.0f ? 1.0f : 0.0f);
                        v[q] = x;
                    }
                    if (vec4 && col + 3 < lim) {
                        *reinterpret_cast<float4 *>(dst + col) = make_float4(v[0], v[1], v[2], v[3]);
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (col + q < lim)
                                dst[col + q] = v[q];
                    }
                }
            }
        }
    }

    if (warp == 2 && lane == 0)
        CT_STAMP(6);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
    if (threadIdx.x == 0) {
        CT_STAMP(7);
        CT_STAMP_NS(9);
    }
    if (threadIdx.x == 0 && *abort_flag)
        atomicExch(p.flags + FLAG_TIMEOUT, 1u + (uint32_t)blockIdx.x);
    if (threadIdx.x == 0 && p.bands > 0) {
        // every store of this tile was issued before the __syncthreads above: make them visible to
        // the device before the band's count moves (also on the failure path, so that a waiting
        // stream is always released; the failure itself is on record in the error word)
        __threadfence();
        atomicAdd(p.band_done + band, 1u);
    }
}

// ---- the same pipeline, many short tiles per CTA ------------------------------------------
//
// When a tile's whole k range fits one accumulation (k <= 1024: conv2d with a few hundred
// channel-taps, batched layers), the kernel above spends as long before and after the main loop
// (barrier and TMEM set-up, first operands, final store: ~7 us) as in it.  Here one CTA per SM
// walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...: the TMA ring and the two TMEM accumulators
// carry on across tiles, so the producer is already fetching tile i+1 while tile i computes, and
// the epilogue warps drain and store tile i (from registers, through their own staging area)
// while the MMA warp fills the other accumulator with tile i+1.
template <int BN, int MODE> struct StreamCfg {
    using C = Cfg<BN, MODE, 64>;
    static constexpr int kEpiCols      = 64; // columns staged at a time
    static constexpr int kEpiRowBytes  = kEpiCols * 4 + 16;
    static constexpr int kEpiWarpBytes = 32 * kEpiRowBytes;
    static constexpr int kEpiBytes     = C::kEpiWarps * kEpiWarpBytes;
    static constexpr int kStagesFit    = (226 * 1024 - 1024 - kEpiBytes) / C::kStageBytes;
    static constexpr int kStages       = kStagesFit > 8 ? 8 : kStagesFit;
    static constexpr int kSmemBytes    = kStages * C::kStageBytes + kEpiBytes + 1024;
    static_assert(kStages >= 2, "at least two pipeline stages");
};

__device__ __forceinline__ void tile_coords(const GemmParams &p, int tile, int &tm, int &tn, int &tz) {
    int per_batch  = p.tiles_m * p.tiles_n;
    tz             = tile / per_batch;
    int bid        = tile - tz * per_batch;
    int group_size = 16 * p.tiles_n;
    int g          = bid / group_size;
    int first_m    = g * 16;
    int gm         = p.tiles_m - first_m < 16 ? p.tiles_m - first_m : 16;
    int in_group   = bid - g * group_size;
    tm             = first_m + in_group % gm;
    tn             = in_group / gm;
}

template <int BN, int MODE>
__global__ void __launch_bounds__(Cfg<BN, MODE, 64>::kThreads, 1) gemm_tc_stream_kernel(
    const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
    const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
    const GemmParams p, const int total_tiles) {
    constexpr int RB = 64;
    using C          = Cfg<BN, MODE, RB>;
    using S          = StreamCfg<BN, MODE>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[S::kStages];
    __shared__ uint64_t bar_empty[S::kStages];
    __shared__ uint64_t bar_tmem_full[2];
    __shared__ uint64_t bar_tmem_empty[2];
    __shared__ uint64_t bar_done;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag_s;
    volatile int *abort_flag = &abort_flag_s;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0)
        abort_flag_s = *reinterpret_cast<volatile uint32_t *>(p.flags + FLAG_TIMEOUT) != 0 ? 1 : 0;
    __syncthreads();
    if (abort_flag_s)
        return;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    auto stage_addr          = [&](int s) { return smem_base + (uint32_t)s * C::kStageBytes; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bar_tmem_full[b]), 1);
            mbar_init(smem_u32(&bar_tmem_empty[b]), C::kEpiWarps);
        }
        mbar_init(smem_u32(&bar_done), 1);
        mbar_fence_init();
        prefetch_tensormap(&map_a_hi);
        prefetch_tensormap(&map_b_hi);
        if (MODE == MODE_3X) {
            prefetch_tensormap(&map_a_lo);
            prefetch_tensormap(&map_b_lo);
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    const int nkb            = p.num_k_blocks;

    if (warp == 0) {
        // ===== TMA producer: k-blocks numbered across tiles =====
        if (lane == 0) {
            int kbg = 0; // k-blocks issued so far
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                int tm, tn, tz;
                tile_coords(p, tile, tm, tn, tz);
                for (int kb = 0; kb < nkb; ++kb, ++kbg) {
                    int s       = kbg % S::kStages;
                    uint32_t ph = (uint32_t)(kbg / S::kStages) & 1u;
                    if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint32_t full = smem_u32(&bar_full[s]);
                    uint32_t dst  = stage_addr(s);
                    mbar_expect_tx(full, (uint32_t)(C::kPlanes * (C::kABytes + p.tile_n * C::kRowB)));
                    int32_t kc = kb * C::kBlockK;
                    tma_load_2d(dst, &map_a_hi, full, kc, tm * BM);
                    dst += C::kABytes;
                    if (MODE == MODE_3X) {
                        tma_load_2d(dst, &map_a_lo, full, kc, tm * BM);
                        dst += C::kABytes;
                    }
                    if (p.conv) {
                        int rs = kb / p.conv_cblocks, cb = kb - rs * p.conv_cblocks;
                        int r = rs / p.conv_kw, sx = rs - r * p.conv_kw;
                        int32_t c0 = cb * C::kBlockK, w0 = sx - p.conv_pad, h0 = tn * p.conv_th + r - p.conv_pad;
                        tma_load_4d(dst, &map_b_hi, full, c0, w0, h0, tz);
                        dst += C::kBBytes;
                        if (MODE == MODE_3X)
                            tma_load_4d(dst, &map_b_lo, full, c0, w0, h0, tz);
                    } else {
                        tma_load_3d(dst, &map_b_hi, full, kc, tn * BN, tz);
                        dst += C::kBBytes;
                        if (MODE == MODE_3X)
                            tma_load_3d(dst, &map_b_lo, full, kc, tn * BN, tz);
                    }
                }
            }
            if (*abort_flag) {
                // unwind: let the copies still in flight land before the CTA goes away
                int first = kbg - S::kStages < 0 ? 0 : kbg - S::kStages;
                for (int k2 = first; k2 < kbg; ++k2) {
                    uint32_t bar = smem_u32(&bar_full[k2 % S::kStages]);
                    uint32_t ph  = (uint32_t)(k2 / S::kStages) & 1u;
                    uint64_t t0  = globaltimer_ns();
                    while (!mbar_try_wait(bar, ph) && globaltimer_ns() - t0 < kWaitBudgetNs) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: accumulator buffer i & 1 for the CTA's i-th tile =====
        if (lane == 0) {
            const uint32_t idesc = make_idesc(MODE == MODE_3X ? 2u : 1u, BM, (uint32_t)p.tile_n);
            int kbg = 0, i = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++i) {
                int buf = i & 1;
                if (!mbar_wait(smem_u32(&bar_tmem_empty[buf]), (((uint32_t)i >> 1) & 1u) ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                uint32_t d_tmem = tmem_base + (uint32_t)buf * BN;
                bool first      = true;
                for (int kb = 0; kb < nkb; ++kb, ++kbg) {
                    int s       = kbg % S::kStages;
                    uint32_t ph = (uint32_t)(kbg / S::kStages) & 1u;
                    if (!mbar_wait(smem_u32(&bar_full[s]), ph, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    uint32_t a_hi = stage_addr(s);
                    uint32_t a_lo = a_hi + C::kABytes;
                    uint32_t b_hi = a_hi + C::kPlanes * C::kABytes;
                    uint32_t b_lo = b_hi + C::kBBytes;
                    uint64_t da_hi = smem_desc_k<RB>(a_hi), db_hi = smem_desc_k<RB>(b_hi);
                    uint64_t da_lo = smem_desc_k<RB>(a_lo), db_lo = smem_desc_k<RB>(b_lo);
#pragma unroll
                    for (int kk = 0; kk < C::kKSteps; ++kk) {
                        uint64_t adv = (uint64_t)(kk * 32 >> 4);
                        if (MODE == MODE_3X) {
                            mma_tf32(d_tmem, da_lo + adv, db_hi + adv, idesc, first ? 0u : 1u);
                            mma_tf32(d_tmem, da_hi + adv, db_lo + adv, idesc, 1u);
                            mma_tf32(d_tmem, da_hi + adv, db_hi + adv, idesc, 1u);
                        } else {
                            mma_f16(d_tmem, da_hi + adv, db_hi + adv, idesc, first ? 0u : 1u);
                        }
                        first = false;
                    }
                    tc_commit(smem_u32(&bar_empty[s]));
                }
                if (ok)
                    tc_commit(smem_u32(&bar_tmem_full[buf]));
            }
            if (!ok || *abort_flag) {
                tc_commit(smem_u32(&bar_done));
                uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(smem_u32(&bar_done), 0) && globaltimer_ns() - t0 < kWaitBudgetNs) {
                }
            }
        }
    } else {
        // ===== epilogue: drain tile i to registers, release the accumulator, then store =====
        const int ew      = warp - 2;
        const int quarter = warp & 3;
        const int half    = ew >> 2;
        uint8_t *stg = smem_raw + (smem_base - smem_u32(smem_raw)) + (uint32_t)S::kStages * C::kStageBytes +
                       (uint32_t)ew * S::kEpiWarpBytes;
        int i = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++i) {
            int tm, tn, tz;
            tile_coords(p, tile, tm, tn, tz);
            const int buf = i & 1;
            bool got = mbar_wait(smem_u32(&bar_tmem_full[buf]), ((uint32_t)i >> 1) & 1u, abort_flag);
            if (!__all_sync(0xffffffffu, got))
                break;
            tc_fence_after_sync();
            float acc[128];
            uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + half * 128);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + g * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    acc[g * 32 + j] = __uint_as_float(r[j]);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&bar_tmem_empty[buf]));

            const int64_t row0 = (int64_t)tm * BM + quarter * 32;
            const int64_t col0 = (int64_t)tn * p.tile_n + half * 128;
            const int64_t lim  = (int64_t)(tn + 1) * p.tile_n < p.n ? (int64_t)(tn + 1) * p.tile_n : p.n;
            float *out_z       = p.out + (int64_t)tz * p.out_batch_stride;
            if ((p.ldc & 3) == 0 && (col0 & 3) == 0 && (reinterpret_cast<uintptr_t>(out_z) & 15u) == 0) {
                // 64 columns at a time through the warp's staging block (rows padded to 272 bytes);
                // written out two rows (2 x 256 contiguous bytes) per instruction
                const int sub = lane & 15, rr = lane >> 4;
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    if (col0 + h2 * 64 >= lim)
                        break;
                    float4 *mine = reinterpret_cast<float4 *>(stg + lane * S::kEpiRowBytes);
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        mine[j] = make_float4(acc[h2 * 64 + 4 * j], acc[h2 * 64 + 4 * j + 1], acc[h2 * 64 + 4 * j + 2],
                                              acc[h2 * 64 + 4 * j + 3]);
                    __syncwarp();
                    const int64_t col = col0 + h2 * 64 + sub * 4;
                    float b4[4]       = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (p.bias && !p.bias_per_row) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (col + q < lim)
                                b4[q] = p.bias[col + q];
                    }
#pragma unroll 4
                    for (int it = 0; it < 16; ++it) {
                        const int r_in = it * 2 + rr;
                        if (row0 + r_in < p.m) {
                            float4 q4 = *reinterpret_cast<const float4 *>(stg + r_in * S::kEpiRowBytes + sub * 16);
                            float v[4] = {q4.x, q4.y, q4.z, q4.w};
                            const float rb = (p.bias && p.bias_per_row) ? p.bias[row0 + r_in] : 0.0f;
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                float x = v[q];
                                if (p.bias)
                                    x = __fadd_rn(x, p.bias_per_row ? rb : b4[q]);
                                if (p.act == CT_ACT_RELU)
                                    x = __fmul_rn(x, x > 0.0f ? 1.0f : 0.0f);
                                v[q] = x;
                            }
                            float *dst = out_z + (row0 + r_in) * p.ldc;
                            if (col + 3 < lim) {
                                *reinterpret_cast<float4 *>(dst + col) = make_float4(v[0], v[1], v[2], v[3]);
                            } else {
#pragma unroll
                                for (int q = 0; q < 4; ++q)
                                    if (col + q < lim)
                                        dst[col + q] = v[q];
                            }
                        }
                    }
                    __syncwarp(); // the block is rewritten by the next half / tile
                }
            } else if (row0 + lane < p.m) {
                const int64_t row = row0 + lane;
                float *dst        = out_z + row * p.ldc;
                const float rb    = (p.bias && p.bias_per_row) ? p.bias[row] : 0.0f;
#pragma unroll
                for (int j = 0; j < 128; ++j) {
                    int64_t col = col0 + j;
                    if (col < lim) {
                        float x = acc[j];
                        if (p.bias)
                            x = __fadd_rn(x, p.bias_per_row ? rb : p.bias[col]);
                        if (p.act == CT_ACT_RELU)
                            x = __fmul_rn(x, x > 0.0f ? 1.0f : 0.0f);
                        dst[col] = x;
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag)
        atomicExch(p.flags + FLAG_TIMEOUT, 1u + (uint32_t)blockIdx.x);
}

// ---- conv2d with at most 64 output channels: pixels on the rows ----------------------------
//
// With the output channels on the 128 accumulator rows, a layer of 64 (or 32) filters spends half
// (or three quarters) of every MMA on zero rows.  Here the operands trade places: the A tile is a
// block of th*wo <= 128 output pixels (the shifted NHWC box, one per filter tap and channel block),
// the B tile the 64 filter rows of the weight planes, N = 64.  The accumulator then holds
// [pixel][channel]; a thread owns one pixel, and for a fixed channel the 32 lanes of a warp write 32
// consecutive pixels of that channel's NCHW plane: coalesced without any staging.  Same streaming
// structure as above (one CTA per SM walks the tiles, two TMEM accumulators).
struct ConvSwapParams {
    int ko;            // output channels (<= 64)
    int n_mma;         // ko rounded up to 16: the MMA's N
    int num_k_blocks;  // taps * channel blocks
    int cblocks, kw, pad, th, wo;
    int rows;          // th * wo pixels per tile (<= 128)
    int tiles_y;       // ceil(ho / th)
    int64_t pix;       // ho * wo
    const float *bias;
    int act;
    float *out;        // [batch][ko][pix], or [batch][ko][ho/2][wo/2] with pool
    uint32_t *flags;
    int pool;          // 2: a 2x2 max-pool of the activated output is what gets stored
    int ho;
};

template <int MODE> struct SwapCfg {
    // 128-byte operand rows (32 float32 channels per k-block).  Measured on the 32 -> 64 channel
    // layer of the CNN: 64-byte rows (twice as many, half as large copies) are a third slower, also
    // with the filter planes kept resident in shared memory, so neither variant is kept.
    static constexpr int kRowB       = 128;
    static constexpr int kKSteps     = kRowB / 32;
    static constexpr int kBN         = 64;
    static constexpr int kElem       = MODE == MODE_3X ? 4 : 2;
    static constexpr int kBlockK     = kRowB / kElem;
    static constexpr int kPlanes     = MODE == MODE_3X ? 2 : 1;
    static constexpr int kABytes     = BM * kRowB;
    static constexpr int kBBytes     = kBN * kRowB;
    static constexpr int kStageBytes = kPlanes * (kABytes + kBBytes);
    static constexpr int kStages     = (200 * 1024) / kStageBytes > 8 ? 8 : (200 * 1024) / kStageBytes;
    static constexpr int kThreads    = 64 + 4 * 32;
    static constexpr int kTmemCols   = 2 * kBN;
    // pooled epilogue: the tile's [pixel][channel] values, rows padded to 65 floats
    static constexpr int kPoolRowF   = 65;
    static constexpr int kPoolBytes  = BM * kPoolRowF * 4;
    static constexpr int kSmemBytes  = kStages * kStageBytes + kPoolBytes + 1024;
};

template <int MODE>
__global__ void __launch_bounds__(SwapCfg<MODE>::kThreads, 1) conv_swap_stream_kernel(
    const __grid_constant__ CUtensorMap map_x_hi, const __grid_constant__ CUtensorMap map_x_lo,
    const __grid_constant__ CUtensorMap map_w_hi, const __grid_constant__ CUtensorMap map_w_lo,
    const ConvSwapParams p, const int total_tiles) {
    using S = SwapCfg<MODE>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[S::kStages];
    __shared__ uint64_t bar_empty[S::kStages];
    __shared__ uint64_t bar_tmem_full[2];
    __shared__ uint64_t bar_tmem_empty[2];
    __shared__ uint64_t bar_done;
    __shared__ uint64_t bar_epi; // the four epilogue warps meet here (bounded, unlike bar.sync)
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag_s;
    volatile int *abort_flag = &abort_flag_s;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0)
        abort_flag_s = *reinterpret_cast<volatile uint32_t *>(p.flags + FLAG_TIMEOUT) != 0 ? 1 : 0;
    __syncthreads();
    if (abort_flag_s)
        return;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    auto stage_addr          = [&](int s) { return smem_base + (uint32_t)s * S::kStageBytes; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bar_tmem_full[b]), 1);
            mbar_init(smem_u32(&bar_tmem_empty[b]), 4);
        }
        mbar_init(smem_u32(&bar_done), 1);
        mbar_init(smem_u32(&bar_epi), 4);
        mbar_fence_init();
        prefetch_tensormap(&map_x_hi);
        prefetch_tensormap(&map_w_hi);
        if (MODE == MODE_3X) {
            prefetch_tensormap(&map_x_lo);
            prefetch_tensormap(&map_w_lo);
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), S::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    const int nkb            = p.num_k_blocks;

    if (warp == 0) {
        // ===== TMA producer =====
        if (lane == 0) {
            int kbg = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int img = tile / p.tiles_y, ty = tile - img * p.tiles_y;
                for (int kb = 0; kb < nkb; ++kb, ++kbg) {
                    int s       = kbg % S::kStages;
                    uint32_t ph = (uint32_t)(kbg / S::kStages) & 1u;
                    if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint32_t full = smem_u32(&bar_full[s]);
                    uint32_t dst  = stage_addr(s);
                    mbar_expect_tx(full, (uint32_t)(S::kPlanes * (p.rows * S::kRowB + S::kBBytes)));
                    // k-block = (filter tap rs, channel block cb): pixels of th rows by wo columns,
                    // shifted by the tap, the halo read as zero
                    int rs = kb / p.cblocks, cb = kb - rs * p.cblocks;
                    int r = rs / p.kw, sx = rs - r * p.kw;
                    int32_t c0 = cb * S::kBlockK, w0 = sx - p.pad, h0 = ty * p.th + r - p.pad;
                    tma_load_4d(dst, &map_x_hi, full, c0, w0, h0, img);
                    dst += S::kABytes;
                    if (MODE == MODE_3X) {
                        tma_load_4d(dst, &map_x_lo, full, c0, w0, h0, img);
                        dst += S::kABytes;
                    }
                    int32_t kc = kb * S::kBlockK;
                    tma_load_2d(dst, &map_w_hi, full, kc, 0);
                    dst += S::kBBytes;
                    if (MODE == MODE_3X)
                        tma_load_2d(dst, &map_w_lo, full, kc, 0);
                }
            }
            if (*abort_flag) {
                int first = kbg - S::kStages < 0 ? 0 : kbg - S::kStages;
                for (int k2 = first; k2 < kbg; ++k2) {
                    uint32_t bar = smem_u32(&bar_full[k2 % S::kStages]);
                    uint32_t ph  = (uint32_t)(k2 / S::kStages) & 1u;
                    uint64_t t0  = globaltimer_ns();
                    while (!mbar_try_wait(bar, ph) && globaltimer_ns() - t0 < kWaitBudgetNs) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer =====
        if (lane == 0) {
            const uint32_t idesc = make_idesc(MODE == MODE_3X ? 2u : 1u, BM, (uint32_t)p.n_mma);
            int kbg = 0, i = 0;
            bool ok = true;
            long long c_start = CT_CLOCK();
            (void)c_start;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++i) {
                int buf = i & 1;
                long long c0 = CT_CLOCK();
                if (!mbar_wait(smem_u32(&bar_tmem_empty[buf]), (((uint32_t)i >> 1) & 1u) ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                CT_ACCUM(11, CT_CLOCK() - c0);
                tc_fence_after_sync();
                uint32_t d_tmem = tmem_base + (uint32_t)buf * S::kBN;
                bool first      = true;
                for (int kb = 0; kb < nkb; ++kb, ++kbg) {
                    int s       = kbg % S::kStages;
                    uint32_t ph = (uint32_t)(kbg / S::kStages) & 1u;
                    long long c1 = CT_CLOCK();
                    if (!mbar_wait(smem_u32(&bar_full[s]), ph, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    CT_ACCUM(10, CT_CLOCK() - c1);
                    uint32_t a_hi = stage_addr(s);
                    uint32_t a_lo = a_hi + S::kABytes;
                    uint32_t b_hi = a_hi + S::kPlanes * S::kABytes;
                    uint32_t b_lo = b_hi + S::kBBytes;
                    uint64_t da_hi = smem_desc_k<S::kRowB>(a_hi), db_hi = smem_desc_k<S::kRowB>(b_hi);
                    uint64_t da_lo = smem_desc_k<S::kRowB>(a_lo), db_lo = smem_desc_k<S::kRowB>(b_lo);
#pragma unroll
                    for (int kk = 0; kk < S::kKSteps; ++kk) {
                        uint64_t adv = (uint64_t)(kk * 32 >> 4);
                        if (MODE == MODE_3X) {
                            mma_tf32(d_tmem, da_lo + adv, db_hi + adv, idesc, first ? 0u : 1u);
                            mma_tf32(d_tmem, da_hi + adv, db_lo + adv, idesc, 1u);
                            mma_tf32(d_tmem, da_hi + adv, db_hi + adv, idesc, 1u);
                        } else {
                            mma_f16(d_tmem, da_hi + adv, db_hi + adv, idesc, first ? 0u : 1u);
                        }
                        first = false;
                    }
                    tc_commit(smem_u32(&bar_empty[s]));
                }
                if (ok)
                    tc_commit(smem_u32(&bar_tmem_full[buf]));
            }
            CT_ACCUM(12, CT_CLOCK() - c_start);
            CT_ACCUM(13, i);
            if (!ok || *abort_flag) {
                tc_commit(smem_u32(&bar_done));
                uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(smem_u32(&bar_done), 0) && globaltimer_ns() - t0 < kWaitBudgetNs) {
                }
            }
        }
    } else {
        // ===== epilogue: one pixel per thread, 64 channels =====
        const int quarter = warp & 3;
        int i             = 0;
        uint32_t epi_phase = 0;
        float *pool_st = reinterpret_cast<float *>(smem_raw + (smem_base - smem_u32(smem_raw)) +
                                                    (uint32_t)S::kStages * S::kStageBytes);
        // all four epilogue warps arrive, then wait (bounded); false when the launch is aborting
        auto epi_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&bar_epi));
            bool ok = mbar_wait(smem_u32(&bar_epi), epi_phase, abort_flag);
            epi_phase ^= 1u;
            return __all_sync(0xffffffffu, ok);
        };
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++i) {
            const int img = tile / p.tiles_y, ty = tile - img * p.tiles_y;
            const int buf = i & 1;
            long long c2 = CT_CLOCK();
            bool got = mbar_wait(smem_u32(&bar_tmem_full[buf]), ((uint32_t)i >> 1) & 1u, abort_flag);
            if (warp == 2 && lane == 0)
                CT_ACCUM(14, CT_CLOCK() - c2);
            if (!__all_sync(0xffffffffu, got))
                break;
            tc_fence_after_sync();
            float acc[64];
            uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * S::kBN);
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + g * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    acc[g * 32 + j] = __uint_as_float(r[j]);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&bar_tmem_empty[buf]));

            const int row     = quarter * 32 + lane;                       // pixel within the tile
            const int64_t pix = (int64_t)ty * p.th * p.wo + row;           // pixel within the image
            if (p.pool) {
                // activated values of the tile to shared memory as [pixel][channel]; then each warp
                // takes every fourth channel and its lanes the tile's (th/2) x (wo/2) <= 32 pooled
                // pixels: a store instruction writes consecutive pooled pixels of one channel plane.
                // Window order and strict '>' as in maxpool2d (first element seeds, NaN never wins).
#pragma unroll
                for (int ch = 0; ch < 64; ++ch) {
                    if (ch < p.ko) {
                        float x = acc[ch];
                        if (p.bias)
                            x = __fadd_rn(x, p.bias[ch]);
                        if (p.act == CT_ACT_RELU)
                            x = __fmul_rn(x, x > 0.0f ? 1.0f : 0.0f);
                        pool_st[row * S::kPoolRowF + ch] = x;
                    }
                }
                if (!epi_sync())
                    break;
                const int pw = p.wo >> 1, ph = p.ho >> 1, prow0 = ty * (p.th >> 1);
                const int pcount = (p.th >> 1) * pw;
                if (lane < pcount) {
                    const int py = lane / pw, px = lane - py * pw;
                    if (prow0 + py < ph) {
                        const float *src = pool_st + ((2 * py) * p.wo + 2 * px) * S::kPoolRowF;
                        float *dst = p.out + (((int64_t)img * p.ko) * ph + prow0 + py) * pw + px;
                        for (int ch = warp - 2; ch < p.ko; ch += 4) {
                            float best = src[ch];
                            float v1 = src[S::kPoolRowF + ch], v2 = src[p.wo * S::kPoolRowF + ch];
                            float v3 = src[(p.wo + 1) * S::kPoolRowF + ch];
                            if (v1 > best)
                                best = v1;
                            if (v2 > best)
                                best = v2;
                            if (v3 > best)
                                best = v3;
                            dst[(int64_t)ch * ph * pw] = best;
                        }
                    }
                }
                if (!epi_sync()) // the block is rewritten by the next tile
                    break;
            } else if (row < p.rows && pix < p.pix) {
                float *dst = p.out + ((int64_t)img * p.ko) * p.pix + pix;
#pragma unroll
                for (int ch = 0; ch < 64; ++ch) {
                    if (ch < p.ko) {
                        float x = acc[ch];
                        if (p.bias)
                            x = __fadd_rn(x, p.bias[ch]);
                        if (p.act == CT_ACT_RELU)
                            x = __fmul_rn(x, x > 0.0f ? 1.0f : 0.0f);
                        dst[(int64_t)ch * p.pix] = x;
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, S::kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag)
        atomicExch(p.flags + FLAG_TIMEOUT, 1u + (uint32_t)blockIdx.x);
}

} // namespace

// ---- host side --------------------------------------------------------------------------

namespace {

typedef CUresult (*EncodeTiledFn)(
    CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
    const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is fetched through the runtime, so the library carries no link-time
// dependency on libcuda.
ct_status encode_fn(EncodeTiledFn *out) {
    static EncodeTiledFn fn = nullptr;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CT_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !sym)
            return fail(CT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    *out = fn;
    return CT_OK;
}

} // namespace

ct_status encode_tiled_map_f32(
    CUtensorMap *map, const void *base, int rank, const uint64_t *dims, const uint64_t *strides, const uint32_t *box,
    int swizzle_bytes) {
    EncodeTiledFn fn;
    CT_TRY(encode_fn(&fn));
    cuuint64_t d[5], s[4];
    cuuint32_t b[5], e[5];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        e[i] = 1;
        if (i + 1 < rank)
            s[i] = strides[i];
    }
    CUresult r = fn(
        map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void *>(base), d, s, b, e,
        CU_TENSOR_MAP_INTERLEAVE_NONE,
        swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                             : (swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(CT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return CT_OK;
}

namespace {

// Tensor map over a plane [rows][kp] (kp contiguous); box = one k-block x box_rows rows,
// 128-byte swizzle, out-of-range rows read as zero.
ct_status make_plane_map(
    CUtensorMap *map, const void *base, int elem_bytes, int64_t rows, int64_t kp, int box_rows,
    int batch /* 0: rank-2 map; >= 1: rank-3 map [batch][rows][kp] */, int row_bytes = ROW_B) {
    EncodeTiledFn fn;
    CT_TRY(encode_fn(&fn));
    cuuint64_t dims[3]    = {(cuuint64_t)kp, (cuuint64_t)rows, (cuuint64_t)(batch > 0 ? batch : 1)};
    cuuint64_t strides[2] = {(cuuint64_t)kp * (cuuint64_t)elem_bytes,
                             (cuuint64_t)kp * (cuuint64_t)elem_bytes * (cuuint64_t)rows};
    cuuint32_t box[3]     = {(cuuint32_t)(row_bytes / elem_bytes), (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3]    = {1, 1, 1};
    CUtensorMapDataType dt =
        elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    CUresult r = fn(
        map, dt, batch > 0 ? 3 : 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(CT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return CT_OK;
}

// Tensor map over NHWC input planes [batch][h][w][c_pad] (channels contiguous); box = 32 channels
// (one k-block) x wo columns x th rows of one image, 128-byte swizzle.  Written to shared memory
// the box is th*wo rows of 128 bytes: the K-major B tile of th*wo output pixels.
ct_status make_conv_map(
    CUtensorMap *map, const void *base, int elem_bytes, const ConvGeom &g, int batch, int row_bytes = ROW_B) {
    EncodeTiledFn fn;
    CT_TRY(encode_fn(&fn));
    cuuint64_t row        = (cuuint64_t)g.c_pad * (cuuint64_t)elem_bytes;
    cuuint64_t dims[4]    = {(cuuint64_t)g.c_pad, (cuuint64_t)g.w, (cuuint64_t)g.h, (cuuint64_t)batch};
    cuuint64_t strides[3] = {row, row * (cuuint64_t)g.w, row * (cuuint64_t)g.w * (cuuint64_t)g.h};
    cuuint32_t box[4]     = {(cuuint32_t)(row_bytes / elem_bytes), (cuuint32_t)g.wo, (cuuint32_t)g.th, 1};
    cuuint32_t estr[4]    = {1, 1, 1, 1};
    CUtensorMapDataType dt =
        elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    CUresult r = fn(
        map, dt, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(CT_ERR_CUDA, "cuTensorMapEncodeTiled (conv) failed with code %d", (int)r);
    return CT_OK;
}

// k-blocks of 128-byte rows per drain of the accumulator: 8 = 256 float32 values of k
constexpr int kChunkBlocks = 8;

template <int BN, int MODE, int RB = ROW_B>
ct_status launch_gemm(
    DeviceState *st, const void *a_hi, const void *a_lo, const void *b_hi, const void *b_lo,
    int64_t m, int64_t n, int64_t kp, const float *bias, int act, float *out, int batch,
    int64_t out_batch_stride, int bias_per_row, const ConvGeom *cg, int splits = 1) {
    using C = Cfg<BN, MODE, RB>;
    // split-K: `splits` slices of the k range, each writing m*n partial sums `out_batch_stride`
    // apart; the operand maps keep their own (single) batch entry
    const int grid_batch = splits > 1 ? splits : batch;
    CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo;
    CT_TRY(make_plane_map(&ma_hi, a_hi, C::kElem, m, kp, BM, 0, RB));
    if (cg)
        CT_TRY(make_conv_map(&mb_hi, b_hi, C::kElem, *cg, batch, RB));
    else
        CT_TRY(make_plane_map(&mb_hi, b_hi, C::kElem, n, kp, BN, batch, RB));
    if (MODE == MODE_3X) {
        CT_TRY(make_plane_map(&ma_lo, a_lo, C::kElem, m, kp, BM, 0, RB));
        if (cg)
            CT_TRY(make_conv_map(&mb_lo, b_lo, C::kElem, *cg, batch, RB));
        else
            CT_TRY(make_plane_map(&mb_lo, b_lo, C::kElem, n, kp, BN, batch, RB));
    } else {
        ma_lo = ma_hi;
        mb_lo = mb_hi;
    }
    GemmParams p;
    p.m            = m;
    p.n            = n;
    p.num_k_blocks = (int)(kp / C::kBlockK);
    p.chunk_blocks = kChunkBlocks * (ROW_B / RB); // same k extent per drain
    p.tiles_m      = (int)((m + BM - 1) / BM);
    p.tiles_n      = (int)((n + BN - 1) / BN);
    p.bias         = bias;
    p.act          = act;
    p.out          = out;
    p.ldc          = n;
    p.batch        = batch;
    p.out_batch_stride = out_batch_stride;
    p.bias_per_row = bias_per_row;
    p.flags        = st->flags_dev;
    p.tile_n       = BN;
    p.kb_per_split = splits > 1 ? (p.num_k_blocks + splits - 1) / splits : 0;
    p.conv         = 0;
    p.conv_cblocks = p.conv_kw = p.conv_pad = p.conv_th = 0;
    p.bands        = 0;
    p.band_done    = nullptr;
    if (g_band_plan.bands > 0 && !cg && splits == 1 && batch == 1) {
        p.bands     = g_band_plan.bands;
        p.band_done = g_band_plan.done;
        for (int b = 0; b <= p.bands; ++b)
            p.band_first[b] = g_band_plan.first[b];
        for (int b = 0; b < p.bands; ++b)
            p.band_out_off[b] = g_band_plan.out_off[b];
    }
    if (cg) {
        p.tile_n       = cg->th * cg->wo;
        p.tiles_n      = (cg->ho + cg->th - 1) / cg->th;
        p.conv         = 1;
        p.conv_cblocks = cg->c_pad / C::kBlockK;
        p.conv_kw      = cg->kw;
        p.conv_pad     = cg->pad;
        p.conv_th      = cg->th;
        if (p.tile_n > BN || (p.tile_n & 15) != 0)
            return fail(CT_ERR_INVALID, "conv2d: internal tile shape %d not usable", p.tile_n);
    }
    int64_t tiles  = (int64_t)p.tiles_m * p.tiles_n * grid_batch;
    if (tiles > 0x7fffffffll)
        return fail(CT_ERR_TOO_LARGE, "gemm: too many tiles");
    if constexpr (RB == 64) {
        // more tiles than SMs, each with a k range short enough for one accumulation (k <= 1024,
        // the error stays at the level of the chunked form): one CTA per SM walks the tiles
        if (splits == 1 && p.num_k_blocks <= 64 && tiles > st->sm_count && p.bands == 0) {
            using S = StreamCfg<BN, MODE>;
            static bool stream_attr_set_dev[16] = {}; // the attribute belongs to a device's context
            bool &stream_attr_set       = stream_attr_set_dev[st->device & 15];
            if (!stream_attr_set) {
                CT_CUDA(cudaFuncSetAttribute(
                    gemm_tc_stream_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes));
                stream_attr_set = true;
            }
            ProfScope prof("gemm_tc");
            gemm_tc_stream_kernel<BN, MODE><<<(unsigned)st->sm_count, C::kThreads, S::kSmemBytes, stream()>>>(
                ma_hi, ma_lo, mb_hi, mb_lo, p, (int)tiles);
            CT_LAUNCH_CHECK("gemm_tc_stream");
            return CT_OK;
        }
    }
    static bool attr_set_dev[16] = {}; // the attribute belongs to a device's context
    bool &attr_set = attr_set_dev[st->device & 15];
    if (!attr_set) {
        CT_CUDA(cudaFuncSetAttribute(
            gemm_tc_kernel<BN, MODE, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        attr_set = true;
    }
    ProfScope prof("gemm_tc");
    CT_CUDA(launch_dependent(
        gemm_tc_kernel<BN, MODE, RB>, dim3((unsigned)tiles), dim3(C::kThreads), (size_t)C::kSmemBytes, stream(), ma_hi,
        ma_lo, mb_hi, mb_lo, p));
    CT_LAUNCH_CHECK("gemm_tc");
    return CT_OK;
}

// conv2d with ko <= 64 output channels on the accumulator columns (conv_swap_stream_kernel).
// w_*: weight planes [ko][kp] (tap-major k), x_*: NHWC input planes [batch][h][w][c_pad].
template <int MODE>
ct_status launch_conv_swap(
    DeviceState *st, const void *w_hi, const void *w_lo, const void *x_hi, const void *x_lo, int ko, int64_t kp,
    const float *bias, int act, float *out, int batch, const ConvGeom &g) {
    using S = SwapCfg<MODE>;
    CUtensorMap mx_hi, mx_lo, mw_hi, mw_lo;
    CT_TRY(make_conv_map(&mx_hi, x_hi, S::kElem, g, batch, S::kRowB));
    CT_TRY(make_plane_map(&mw_hi, w_hi, S::kElem, ko, kp, S::kBN, 0, S::kRowB));
    if (MODE == MODE_3X) {
        CT_TRY(make_conv_map(&mx_lo, x_lo, S::kElem, g, batch, S::kRowB));
        CT_TRY(make_plane_map(&mw_lo, w_lo, S::kElem, ko, kp, S::kBN, 0, S::kRowB));
    } else {
        mx_lo = mx_hi;
        mw_lo = mw_hi;
    }
    ConvSwapParams p;
    p.ko           = ko;
    p.n_mma        = (ko + 15) / 16 * 16;
    p.num_k_blocks = (int)(kp / S::kBlockK);
    p.cblocks      = g.c_pad / S::kBlockK;
    p.kw           = g.kw;
    p.pad          = g.pad;
    p.th           = g.th;
    p.wo           = g.wo;
    p.rows         = g.th * g.wo;
    p.tiles_y      = (g.ho + g.th - 1) / g.th;
    p.pix          = (int64_t)g.ho * g.wo;
    p.bias         = bias;
    p.act          = act;
    p.out          = out;
    p.flags        = st->flags_dev;
    p.pool         = g.pool;
    p.ho           = g.ho;
    if (p.rows < 1 || p.rows > BM || p.num_k_blocks < 1)
        return fail(CT_ERR_INVALID, "conv2d: internal tile shape %d x %d not usable", g.th, g.wo);
    int64_t tiles = (int64_t)p.tiles_y * batch;
    if (tiles > 0x7fffffffll)
        return fail(CT_ERR_TOO_LARGE, "conv2d: too many tiles");
    static bool attr_set_dev[16] = {}; // the attribute belongs to a device's context
    bool &attr_set = attr_set_dev[st->device & 15];
    if (!attr_set) {
        CT_CUDA(cudaFuncSetAttribute(
            conv_swap_stream_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes));
        attr_set = true;
    }
    unsigned grid = (unsigned)(tiles < st->sm_count ? tiles : st->sm_count);
    ProfScope prof("gemm_tc");
    conv_swap_stream_kernel<MODE><<<grid, S::kThreads, S::kSmemBytes, stream()>>>(
        mx_hi, mx_lo, mw_hi, mw_lo, p, (int)tiles);
    CT_LAUNCH_CHECK("conv_swap_stream");
    return CT_OK;
}

} // namespace

namespace {
// out[i] = act(sum_z partial[z][i] + bias[i % n]), slices added in ascending order.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(
    const float *__restrict__ partial, int splits, int64_t total, int64_t n, const float *__restrict__ bias,
    int act, float *__restrict__ out, const uint32_t *__restrict__ flags) {
    // the slices were not computed if the launch before this one gave up (or never started because
    // an earlier failure is still on record): write nothing rather than sums of stale partials
    if (*reinterpret_cast<const volatile uint32_t *>(flags + FLAG_TIMEOUT) != 0)
        return;
    int64_t step = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
        float v = partial[i];
        for (int z = 1; z < splits; ++z)
            v = __fadd_rn(v, partial[(int64_t)z * total + i]);
        if (bias)
            v = __fadd_rn(v, bias[i % n]);
        if (act == CT_ACT_RELU)
            v = __fmul_rn(v, v > 0.0f ? 1.0f : 0.0f);
        out[i] = v;
    }
}
} // namespace

// Contraction over prepared operand planes: out[z][m][n] = act(A[m][kp] . B[z][n][kp]^T + bias).
// set (under the entry point's lock) while a product that must not touch the shared split-K workspace is enqueued
static bool g_no_splitk = false;

ct_status gemm_planes(
    DeviceState *st, int mode, const void *a_hi, const void *a_lo, const void *b_hi,
    const void *b_lo, int64_t m, int64_t n, int64_t kp, const float *bias, int act, float *out,
    int batch, int64_t out_batch_stride, int bias_per_row, const ConvGeom *conv) {
    // 128 x 256 tiles when they fill the machine, 128 x 128 otherwise
    int64_t tiles256 = ((m + BM - 1) / BM) * ((n + 255) / 256) * batch;
    bool wide        = n > 128 && tiles256 >= st->sm_count / 2;
    if (conv && m <= 64 && conv->wo <= 128 && kp <= 1024 * (mode == MODE_3X ? 1 : 2) && bias_per_row == (bias ? 1 : 0)) {
        // few output channels: pixels on the accumulator rows, channels on its columns; the whole k
        // range is one accumulation, so k stays within what keeps the error at float32 level
        ConvGeom g = *conv;
        g.th       = 128 / g.wo < g.ho ? 128 / g.wo : g.ho;
        if (g.pool)
            g.th &= ~1; // pooling windows must not straddle tiles
        if (mode == MODE_3X)
            return launch_conv_swap<MODE_3X>(st, a_hi, a_lo, b_hi, b_lo, (int)m, kp, bias, act, out, batch, g);
        return launch_conv_swap<MODE_BF>(st, a_hi, a_lo, b_hi, b_lo, (int)m, kp, bias, act, out, batch, g);
    }
    if (conv && conv->pool)
        return fail(CT_ERR_INVALID, "conv2d: the fused max-pool was requested for a shape its kernel does not take");
    if (conv)
        wide = conv->th * conv->wo > 128;
    // Few output tiles and a long reduction (e.g. a 12544 -> 128 layer): slice k across CTAs so
    // that the whole machine works, partial sums in a workspace, one pass to add them up.
    if (!conv && batch == 1 && !bias_per_row && !g_no_splitk) {
        const int kblock  = mode == MODE_3X ? 32 : 64;
        const int nkb     = (int)(kp / kblock);
        int64_t tiles     = ((m + BM - 1) / BM) * ((n + (wide ? 255 : 127)) / (wide ? 256 : 128));
        int splits        = (int)(st->sm_count / (tiles > 0 ? tiles : 1));
        if (splits > nkb / 8)
            splits = nkb / 8;
        if (splits > 32)
            splits = 32;
        if (tiles * 2 <= st->sm_count && splits >= 2) {
            int per = (nkb + splits - 1) / splits;
            splits  = (nkb + per - 1) / per; // no empty slice
            size_t bytes = (size_t)splits * m * n * sizeof(float);
            CT_TRY(ensure_ws(&st->splitk_ws, &st->splitk_ws_bytes, bytes));
            float *partial = static_cast<float *>(st->splitk_ws);
#define CT_SPLIT_ARGS st, a_hi, a_lo, b_hi, b_lo, m, n, kp, nullptr, CT_ACT_NONE, partial, 1, m * n, 0, nullptr, splits
            ct_status launched;
            if (mode == MODE_3X)
                launched = wide ? launch_gemm<256, MODE_3X>(CT_SPLIT_ARGS) : launch_gemm<128, MODE_3X>(CT_SPLIT_ARGS);
            else
                launched = wide ? launch_gemm<256, MODE_BF>(CT_SPLIT_ARGS) : launch_gemm<128, MODE_BF>(CT_SPLIT_ARGS);
#undef CT_SPLIT_ARGS
            CT_TRY(launched);
            int64_t total  = m * n;
            int64_t blocks = (total + 255) / 256;
            int64_t cap    = (int64_t)st->sm_count * 16;
            if (blocks > cap)
                blocks = cap;
            ProfScope prof("gemm_splitk_reduce");
            splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(partial, splits, total, n, bias, act, out, st->flags_dev);
            CT_LAUNCH_CHECK("splitk_reduce");
            return CT_OK;
        }
    }
#define CT_GEMM_ARGS st, a_hi, a_lo, b_hi, b_lo, m, n, kp, bias, act, out, batch, out_batch_stride, bias_per_row, conv
    if (mode == MODE_3X) {
        // 128 x 256 tiles of two float32 planes: 64-byte k-blocks give four 48 KB stages instead
        // of two 96 KB ones.  (A one-wave product, 128 such tiles on 148 SMs, is not served better
        // by 256 tiles of 128 x 128 walked by one CTA per SM: measured 56 instead of 42 us per layer
        // of a 4096 x 1024 x 1024 product - N = 128 MMAs cost 73 clocks against 138 for twice the
        // columns, and two tiles in a row per CTA outweigh the idle SMs.)
        if (wide)
            return launch_gemm<256, MODE_3X, 64>(CT_GEMM_ARGS);
        return launch_gemm<128, MODE_3X>(CT_GEMM_ARGS);
    }
    return wide ? launch_gemm<256, MODE_BF>(CT_GEMM_ARGS) : launch_gemm<128, MODE_BF>(CT_GEMM_ARGS);
#undef CT_GEMM_ARGS
}

ct_status nhwc_planes(
    DeviceState *st, int mode, const float *x, int64_t batch, int64_t c, int64_t hw, int64_t c_pad,
    void *hi, void *lo) {
    (void)st;
    if (batch == 0 || hw == 0)
        return CT_OK;
    if (batch > 65535 || c_pad / 32 > 65535)
        return fail(CT_ERR_TOO_LARGE, "conv2d: batch or channel count too large for the layout pre-pass");
    // per image: [c][hw] -> [hw][c_pad], i.e. the B-operand pre-pass of the GEMM with k = c, n = hw
    dim3 grid((unsigned)((hw + 31) / 32), (unsigned)(c_pad / 32), (unsigned)batch);
    if (mode == MODE_3X)
        split_transpose_kernel<MODE_3X><<<grid, 256, 0, stream()>>>(x, c, hw, c_pad, hi, lo, c * hw, hw * c_pad);
    else
        split_transpose_kernel<MODE_BF><<<grid, 256, 0, stream()>>>(x, c, hw, c_pad, hi, lo, c * hw, hw * c_pad);
    CT_LAUNCH_CHECK("nhwc_planes");
    return CT_OK;
}

ct_status split_rows_planes(
    DeviceState *st, int mode, const float *in, int64_t rows, int64_t k, int64_t kp, void *hi, void *lo) {
    int64_t total  = rows * kp;
    if (total == 0)
        return CT_OK;
    (void)st;
    const int64_t row_groups = (rows + kSplitRows - 1) / kSplitRows;
    dim3 grid((unsigned)((kp / 4 + 255) / 256), (unsigned)(row_groups < 65535 ? row_groups : 65535));
    int vec_ok = (k & 3) == 0 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0;
    if (mode == MODE_3X)
        CT_CUDA(launch_dependent(split_rows_vec_kernel<MODE_3X>, grid, dim3(256), 0, stream(), in, rows, k, kp, hi, lo, vec_ok));
    else
        CT_CUDA(launch_dependent(split_rows_vec_kernel<MODE_BF>, grid, dim3(256), 0, stream(), in, rows, k, kp, hi, lo, vec_ok));
    CT_LAUNCH_CHECK("split_rows");
    return CT_OK;
}

// Largest k for which the kernel's int32 TMA coordinates and k-block counter are safe.
constexpr int64_t kMaxDim = 1ll << 30;

ct_status gemm_f32_tc(
    DeviceState *st, const float *a, const float *b, const float *bias, int64_t m, int64_t k,
    int64_t n, int act, float *out, const PackedWeights *packed, bool a_is_km) {
    if (m == 0 || n == 0)
        return CT_OK;
    if (m > kMaxDim || n > kMaxDim || k > kMaxDim)
        return fail(CT_ERR_TOO_LARGE, "gemm: dimension too large");
    const int mode   = ct_get_precision() == CT_PREC_BF16 ? MODE_BF : MODE_3X;
    const int elem   = mode == MODE_3X ? 4 : 2;
    const int planes = mode == MODE_3X ? 2 : 1;
    const int kblock = ROW_B / elem;
    int64_t kp       = (k + kblock - 1) / kblock * kblock;
    if (kp == 0)
        kp = kblock; // k == 0: one all-zero k-block gives C = act(bias)
    // workspace: [A hi][A lo][B hi][B lo], each plane 1024-byte aligned
    auto align_up       = [](size_t v) { return (v + 1023) & ~(size_t)1023; };
    if (packed) {
        int dev = -1;
        CT_CUDA(cudaGetDevice(&dev));
        if (packed->magic != kPackedMagic || packed->mode != mode || packed->k != k || packed->n != n ||
            packed->kp != kp || packed->src != b || packed->device != dev)
            return fail(
                CT_ERR_INVALID,
                "dense: the packed weights were built from another matrix, shape, precision or device");
    }
    size_t a_plane      = align_up((size_t)m * kp * elem);
    size_t b_plane      = packed ? 0 : align_up((size_t)n * kp * elem);
    size_t total        = planes * (a_plane + b_plane);
    CT_TRY(ensure_ws(&st->gemm_ws, &st->gemm_ws_bytes, total));
    uint8_t *ws = static_cast<uint8_t *>(st->gemm_ws);
    void *a_hi = ws, *a_lo = ws + a_plane;
    void *b_hi = ws + planes * a_plane, *b_lo = ws + planes * a_plane + b_plane;
    if (packed) {
        b_hi = packed->hi;
        b_lo = packed->lo;
    }

    if (a_is_km) {
        // A is stored [k][m] (the product is A^T . B): its planes [m][kp] come out of the same
        // transposing pass that prepares B, so no transposed copy of A is ever written
        ProfScope prof("gemm_prepass");
        dim3 grid((unsigned)((m + 31) / 32), (unsigned)(kp / 32));
        if (grid.y > 65535)
            return fail(CT_ERR_TOO_LARGE, "gemm: k too large for the operand pre-pass");
        if (mode == MODE_3X)
            split_transpose_kernel<MODE_3X><<<grid, 256, 0, stream()>>>(a, k, m, kp, a_hi, a_lo);
        else
            split_transpose_kernel<MODE_BF><<<grid, 256, 0, stream()>>>(a, k, m, kp, a_hi, a_lo);
        CT_LAUNCH_CHECK("split_transpose");
    } else {
        ProfScope prof("gemm_prepass");
        CT_TRY(split_rows_planes(st, mode, a, m, k, kp, a_hi, a_lo));
    }
    if (!packed) {
        ProfScope prof("gemm_prepass");
        dim3 grid((unsigned)((n + 31) / 32), (unsigned)(kp / 32));
        if (grid.y > 65535)
            return fail(CT_ERR_TOO_LARGE, "gemm: k too large for the operand pre-pass");
        if (mode == MODE_3X)
            split_transpose_kernel<MODE_3X><<<grid, 256, 0, stream()>>>(b, k, n, kp, b_hi, b_lo);
        else
            split_transpose_kernel<MODE_BF><<<grid, 256, 0, stream()>>>(b, k, n, kp, b_hi, b_lo);
        CT_LAUNCH_CHECK("split_transpose");
    }

    return gemm_planes(st, mode, a_hi, a_lo, b_hi, b_lo, m, n, kp, bias, act, out, 1, 0, 0);
}

// ---- packed weights -----------------------------------------------------------------------

extern "C" ct_status ct_weights_pack(const float *w, int64_t k, int64_t n, void **packed_out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (!packed_out)
        return fail(CT_ERR_INVALID, "ct_weights_pack: packed_out is null");
    *packed_out = nullptr;
    if (k <= 0 || n <= 0 || !w)
        return fail(CT_ERR_INVALID, "ct_weights_pack: empty or null matrix");
    if (n > kMaxDim || k > kMaxDim)
        return fail(CT_ERR_TOO_LARGE, "ct_weights_pack: dimension too large");
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    CT_CUDA(cudaStreamIsCapturing(stream(), &cap));
    if (cap != cudaStreamCaptureStatusNone)
        return fail(CT_ERR_INVALID, "ct_weights_pack: cannot run while calls are being recorded");
    const int mode   = ct_get_precision() == CT_PREC_BF16 ? MODE_BF : MODE_3X;
    const int elem   = mode == MODE_3X ? 4 : 2;
    const int planes = mode == MODE_3X ? 2 : 1;
    const int kblock = ROW_B / elem;
    const int64_t kp = (k + kblock - 1) / kblock * kblock;
    const size_t plane = ((size_t)n * kp * elem + 1023) & ~(size_t)1023;
    dim3 grid((unsigned)((n + 31) / 32), (unsigned)(kp / 32));
    if (grid.y > 65535)
        return fail(CT_ERR_TOO_LARGE, "ct_weights_pack: k too large for the operand pre-pass");
    void *base = nullptr;
    CT_TRY(ct_alloc(&base, plane * planes));
    void *hi = base, *lo = static_cast<uint8_t *>(base) + plane;
    {
        ProfScope prof("weights_pack");
        if (mode == MODE_3X)
            split_transpose_kernel<MODE_3X><<<grid, 256, 0, stream()>>>(w, k, n, kp, hi, lo);
        else
            split_transpose_kernel<MODE_BF><<<grid, 256, 0, stream()>>>(w, k, n, kp, hi, lo);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            ct_free(base);
            return cuda_fail(e, "weights_pack");
        }
        count_launch(1);
    }
    // the handle may be used from any stream afterwards: finish the one-time pass here
    cudaError_t se = cudaStreamSynchronize(stream());
    if (se != cudaSuccess) {
        ct_free(base);
        return cuda_fail(se, "weights_pack");
    }
    int dev = -1;
    CT_CUDA(cudaGetDevice(&dev));
    PackedWeights *pw = new PackedWeights{kPackedMagic, mode, dev, k, n, kp, w, base, hi, lo};
    *packed_out       = pw;
    return CT_OK;
}

extern "C" ct_status ct_weights_free(void *packed) {
    if (!packed)
        return CT_OK;
    PackedWeights *pw = static_cast<PackedWeights *>(packed);
    if (pw->magic != kPackedMagic)
        return fail(CT_ERR_INVALID, "ct_weights_free: not a packed-weights handle");
    pw->magic    = 0;
    ct_status st = ct_free(pw->base);
    delete pw;
    return st;
}

// ---- packed left operand: split once, multiply row panels ------------------------------------
//
// A product whose rows are computed in several calls (the row panels of a sharded product, each
// all-gathered while the next is computed) should not pay one launch of the operand pre-pass per
// panel, and - since that pre-pass writes the library's one cached workspace - could not run two
// panels at the same time.  ct_rows_pack splits the whole left operand once into planes of its
// own; ct_matmul_packed_rows multiplies a row range of them with packed weights and touches no
// shared workspace, so panels enqueued on different streams fill each other's last, partly empty
// wave of tiles.
struct PackedRows {
    uint32_t magic;
    int mode;
    int device;
    int64_t m, k, kp;
    void *base;
    uint8_t *hi, *lo;
    size_t row_bytes; // bytes of one row of a plane
};
constexpr uint32_t kPackedRowsMagic = 0x43545052u; // "CTPR"

extern "C" ct_status ct_rows_pack(const float *a, int64_t m, int64_t k, void **packed_inout) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (!packed_inout)
        return fail(CT_ERR_INVALID, "ct_rows_pack: packed_inout is null");
    if (m <= 0 || k <= 0 || !a)
        return fail(CT_ERR_INVALID, "ct_rows_pack: empty or null matrix");
    if (m > kMaxDim || k > kMaxDim)
        return fail(CT_ERR_TOO_LARGE, "ct_rows_pack: dimension too large");
    const int mode   = ct_get_precision() == CT_PREC_BF16 ? MODE_BF : MODE_3X;
    const int elem   = mode == MODE_3X ? 4 : 2;
    const int planes = mode == MODE_3X ? 2 : 1;
    const int kblock = ROW_B / elem;
    const int64_t kp = (k + kblock - 1) / kblock * kblock;
    int dev = -1;
    CT_CUDA(cudaGetDevice(&dev));
    PackedRows *pr = static_cast<PackedRows *>(*packed_inout);
    if (pr && (pr->magic != kPackedRowsMagic || pr->mode != mode || pr->m != m || pr->k != k || pr->device != dev))
        return fail(CT_ERR_INVALID, "ct_rows_pack: the handle belongs to another shape, precision or device");
    if (!pr) {
        const size_t plane = ((size_t)m * kp * elem + 1023) & ~(size_t)1023;
        void *base         = nullptr;
        CT_TRY(ct_alloc(&base, plane * planes));
        uint8_t *hi = static_cast<uint8_t *>(base);
        pr          = new PackedRows{kPackedRowsMagic, mode, dev, m, k, kp, base, hi, hi + plane, (size_t)kp * elem};
        *packed_inout = pr;
    }
    ProfScope prof("gemm_prepass");
    return split_rows_planes(st, mode, a, m, k, kp, pr->hi, pr->lo);
}

extern "C" ct_status ct_rows_free(void *packed) {
    if (!packed)
        return CT_OK;
    PackedRows *pr = static_cast<PackedRows *>(packed);
    if (pr->magic != kPackedRowsMagic)
        return fail(CT_ERR_INVALID, "ct_rows_free: not a packed-rows handle");
    pr->magic    = 0;
    ct_status st = ct_free(pr->base);
    delete pr;
    return st;
}

extern "C" ct_status ct_matmul_packed_rows(
    const void *a_packed, int64_t row0, int64_t rows, const void *w_packed, float *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    const PackedRows *pr    = static_cast<const PackedRows *>(a_packed);
    const PackedWeights *pw = static_cast<const PackedWeights *>(w_packed);
    if (!pr || pr->magic != kPackedRowsMagic || !pw || pw->magic != kPackedMagic)
        return fail(CT_ERR_INVALID, "ct_matmul_packed_rows: not a packed operand");
    int dev = -1;
    CT_CUDA(cudaGetDevice(&dev));
    if (pr->mode != pw->mode || pr->k != pw->k || pr->kp != pw->kp || pr->device != dev || pw->device != dev)
        return fail(CT_ERR_INVALID, "ct_matmul_packed_rows: operands of different inner size, precision or device");
    if (row0 < 0 || rows < 0 || row0 + rows > pr->m)
        return fail(CT_ERR_INVALID, "ct_matmul_packed_rows: row range outside the packed matrix");
    if (rows == 0)
        return CT_OK;
    if (!out)
        return fail(CT_ERR_INVALID, "ct_matmul_packed_rows: null pointer");
    g_no_splitk   = true; // the split-K partial sums live in a shared workspace
    ct_status res = gemm_planes(
        st, pr->mode, pr->hi + (size_t)row0 * pr->row_bytes, pr->lo + (size_t)row0 * pr->row_bytes, pw->hi, pw->lo,
        rows, pw->n, pr->kp, nullptr, CT_ACT_NONE, out, 1, 0, 0);
    g_no_splitk = false;
    return res;
}

// A product in row bands with ONE launch.  Computing the bands of a sharded product as separate
// launches costs every band its own partly filled last wave of tiles (16384 columns are 64 tiles of
// 256: a band of 1024 rows is 512 tiles = 3.46 waves on 148 SMs); one launch over all bands has one
// last wave.  The tiles are dealt out band by band, every CTA counts itself into band_done[b] when its
// tile is stored, and a stream that has to move band b elsewhere waits for the count
// (ct_stream_wait_value) instead of for the whole launch.
extern "C" ct_status ct_matmul_packed_bands(
    const void *a_packed, const void *w_packed, int nbands, const int64_t *band_rows_host,
    float *const *band_out_host, uint32_t *band_done_dev, uint32_t *band_tiles_host) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    const PackedRows *pr    = static_cast<const PackedRows *>(a_packed);
    const PackedWeights *pw = static_cast<const PackedWeights *>(w_packed);
    if (!pr || pr->magic != kPackedRowsMagic || !pw || pw->magic != kPackedMagic)
        return fail(CT_ERR_INVALID, "ct_matmul_packed_bands: not a packed operand");
    int dev = -1;
    CT_CUDA(cudaGetDevice(&dev));
    if (pr->mode != pw->mode || pr->k != pw->k || pr->kp != pw->kp || pr->device != dev || pw->device != dev)
        return fail(CT_ERR_INVALID, "ct_matmul_packed_bands: operands of different inner size, precision or device");
    if (nbands < 1 || nbands > 8 || !band_rows_host || !band_out_host || !band_done_dev)
        return fail(CT_ERR_INVALID, "ct_matmul_packed_bands: 1 to 8 bands, with rows, outputs and counters");
    BandPlan plan;
    plan.bands   = nbands;
    plan.done    = band_done_dev;
    int64_t row  = 0;
    plan.first[0] = 0;
    const bool wide = pw->n > 128; // the tile width launch_gemm will pick is decided in gemm_planes; counts below use it
    for (int b = 0; b < nbands; ++b) {
        const int64_t rows = band_rows_host[b];
        if (rows <= 0 || !band_out_host[b] || (b + 1 < nbands && rows % BM != 0))
            return fail(CT_ERR_INVALID, "ct_matmul_packed_bands: bands are non-empty and all but the last a multiple of %d rows", BM);
        // tiles of band b write to band_out_host[b] + (row - first row of the band) * n
        plan.out_off[b] = (band_out_host[b] - band_out_host[0]) - row * pw->n;
        row += rows;
        plan.first[b + 1] = (int)((row + BM - 1) / BM);
    }
    if (row != pr->m)
        return fail(CT_ERR_INVALID, "ct_matmul_packed_bands: the bands hold %lld rows, the packed matrix %lld",
                    (long long)row, (long long)pr->m);
    // the tile width gemm_planes will choose (same rule)
    const int64_t tiles256 = ((pr->m + BM - 1) / BM) * ((pw->n + 255) / 256);
    const bool bn256       = wide && tiles256 >= st->sm_count / 2;
    const int64_t tiles_n  = (pw->n + (bn256 ? 255 : 127)) / (bn256 ? 256 : 128);
    for (int b = 0; b < nbands; ++b)
        if (band_tiles_host)
            band_tiles_host[b] = (uint32_t)((plan.first[b + 1] - plan.first[b]) * tiles_n);
    g_no_splitk   = true; // the split-K partial sums live in a shared workspace
    g_band_plan   = plan;
    ct_status res = gemm_planes(st, pr->mode, pr->hi, pr->lo, pw->hi, pw->lo, pr->m, pw->n, pr->kp, nullptr, CT_ACT_NONE,
                                band_out_host[0], 1, 0, 0);
    g_band_plan.bands = 0;
    g_no_splitk       = false;
    return res;
}

// The current stream waits (the host does not) until the 32-bit word at addr_dev is >= value.
extern "C" ct_status ct_stream_wait_value(const uint32_t *addr_dev, uint32_t value) {
    DeviceState *st;
    CT_TRY(current(&st));
    typedef CUresult (*WaitFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
    static WaitFn fn = nullptr;
    static std::mutex mu;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!fn) {
            void *sym = nullptr;
            cudaDriverEntryPointQueryResult qres;
            CT_CUDA(cudaGetDriverEntryPoint("cuStreamWaitValue32", &sym, cudaEnableDefault, &qres));
            if (qres != cudaDriverEntryPointSuccess || !sym)
                return fail(CT_ERR_CUDA, "cuStreamWaitValue32 is not available from this driver");
            fn = reinterpret_cast<WaitFn>(sym);
        }
    }
    if (!addr_dev)
        return fail(CT_ERR_INVALID, "ct_stream_wait_value: null address");
    CUresult r = fn(reinterpret_cast<CUstream>(stream()), reinterpret_cast<CUdeviceptr>(addr_dev), value,
                    CU_STREAM_WAIT_VALUE_GEQ);
    if (r != CUDA_SUCCESS)
        return fail(CT_ERR_CUDA, "cuStreamWaitValue32 failed with code %d", (int)r);
    return CT_OK;
}

// ---- matmul without any allocation --------------------------------------------------------
//
// Some hosts of this library may not allocate device memory when they call it: a plugin that is
// invoked while the embedding runtime holds a fixed memory budget, a call made from inside a
// region where cudaMalloc would synchronise the whole device (another thread's work in flight),
// or a real-time loop that has to stay free of allocator latency.  For them the operand planes
// of the 3xTF32 GEMM live in the fixed array below instead of in a growing workspace.  The array
// is part of the library image: every GPU on which the library is used holds these bytes from
// the first use until the process exits.

constexpr size_t kStaticScratchBytes = 16u << 20; // 16 MiB: e.g. m = n = k = 1024

static __device__ __align__(256) uint8_t g_static_scratch[kStaticScratchBytes];
static __device__ __align__(256) uint32_t g_static_flags[FLAG_COUNT];

namespace {

struct StaticState {
    bool ready       = false;
    uint8_t *scratch = nullptr; // device address of g_static_scratch on this device
    uint32_t *flags  = nullptr; // device address of g_static_flags on this device
    int sm_count     = 0;
};
StaticState g_static_state[16];
std::mutex g_static_mutex;

// In host code the names g_static_scratch / g_static_flags are only handles of the symbols;
// the addresses kernels can use come from cudaGetSymbolAddress, per device, with that device
// current.
ct_status static_state(StaticState **out) {
    int dev = -1;
    CT_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16)
        return fail(CT_ERR_INVALID, "device index %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticState *s = &g_static_state[dev];
    if (!s->ready) {
        int major = 0;
        CT_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10)
            return fail(CT_ERR_NO_DEVICE, "device %d is not sm_100: this library is built for sm_100a only", dev);
        CT_CUDA(cudaDeviceGetAttribute(&s->sm_count, cudaDevAttrMultiProcessorCount, dev));
        void *p = nullptr;
        CT_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        s->scratch = static_cast<uint8_t *>(p);
        CT_CUDA(cudaGetSymbolAddress(&p, g_static_flags));
        s->flags = static_cast<uint32_t *>(p);
        s->ready = true;
    }
    *out = s;
    return CT_OK;
}

template <int BN>
ct_status launch_static(
    StaticState *s, const void *a_hi, const void *a_lo, const void *b_hi, const void *b_lo,
    int64_t m, int64_t n, int64_t kp, float *out) {
    using C = Cfg<BN, MODE_3X>;
    CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo;
    CT_TRY(make_plane_map(&ma_hi, a_hi, C::kElem, m, kp, BM, 0));
    CT_TRY(make_plane_map(&ma_lo, a_lo, C::kElem, m, kp, BM, 0));
    CT_TRY(make_plane_map(&mb_hi, b_hi, C::kElem, n, kp, BN, 1));
    CT_TRY(make_plane_map(&mb_lo, b_lo, C::kElem, n, kp, BN, 1));
    GemmParams p;
    p.m                = m;
    p.n                = n;
    p.num_k_blocks     = (int)(kp / C::kBlockK);
    p.chunk_blocks     = 8;
    p.tiles_m          = (int)((m + BM - 1) / BM);
    p.tiles_n          = (int)((n + BN - 1) / BN);
    p.bias             = nullptr;
    p.act              = CT_ACT_NONE;
    p.out              = out;
    p.ldc              = n;
    p.batch            = 1;
    p.out_batch_stride = 0;
    p.bias_per_row     = 0;
    p.flags            = s->flags;
    p.tile_n           = BN;
    p.kb_per_split     = 0;
    p.conv             = 0;
    p.conv_cblocks = p.conv_kw = p.conv_pad = p.conv_th = 0;
    p.bands        = 0;
    p.band_done    = nullptr;
    CT_CUDA(cudaFuncSetAttribute(
        gemm_tc_kernel<BN, MODE_3X>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    gemm_tc_kernel<BN, MODE_3X><<<(unsigned)(p.tiles_m * p.tiles_n), C::kThreads, C::kSmemBytes, stream()>>>(
        ma_hi, ma_lo, mb_hi, mb_lo, p);
    CT_LAUNCH_CHECK("gemm_tc(static scratch)");
    return CT_OK;
}

} // namespace
} // namespace ct

extern "C" ct_status ct_matmul_f32_static(
    const float *a_dev, const float *b_dev, int64_t m, int64_t k, int64_t n, float *out_dev,
    uint32_t *status_dev) {
    using namespace ct;
    OpLock op_lock; // callers on several threads that share a stream are at least enqueued one after the other
    if (m < 0 || k < 0 || n < 0)
        return fail(CT_ERR_INVALID, "matmul: negative dimension");
    if (m == 0 || n == 0) {
        if (status_dev)
            CT_CUDA(cudaMemsetAsync(status_dev, 0, sizeof(uint32_t), stream()));
        return CT_OK;
    }
    if (!out_dev || (k > 0 && (!a_dev || !b_dev)))
        return fail(CT_ERR_INVALID, "matmul: null pointer");
    const int kblock = ROW_B / 4;
    int64_t kp       = (k + kblock - 1) / kblock * kblock;
    if (kp == 0)
        kp = kblock;
    auto align_up  = [](size_t v) { return (v + 1023) & ~(size_t)1023; };
    if (m > (1 << 20) || n > (1 << 20) || kp > (1 << 20))
        return fail(CT_ERR_TOO_LARGE, "ct_matmul_f32_static: dimension too large for the %zu-byte static scratch",
                    kStaticScratchBytes);
    size_t a_plane = align_up((size_t)m * kp * 4);
    size_t b_plane = align_up((size_t)n * kp * 4);
    if (2 * (a_plane + b_plane) > kStaticScratchBytes)
        return fail(
            CT_ERR_TOO_LARGE,
            "ct_matmul_f32_static: operand planes need %zu bytes (8*(m+n)*roundup(k,32)), the static scratch "
            "holds %zu; use ct_matmul for this size",
            2 * (a_plane + b_plane), kStaticScratchBytes);
    StaticState *s;
    CT_TRY(static_state(&s));
    // Every byte of the planes that the kernel reads is rewritten by the pre-pass below (padding
    // included), so nothing of an earlier call is reused; only the error words start from zero.
    CT_CUDA(cudaMemsetAsync(s->flags, 0, FLAG_COUNT * sizeof(uint32_t), stream()));
    uint8_t *ws = s->scratch;
    void *a_hi = ws, *a_lo = ws + a_plane, *b_hi = ws + 2 * a_plane, *b_lo = ws + 2 * a_plane + b_plane;
    {
        int64_t total  = m * kp;
        int64_t blocks = (total + 255) / 256;
        int64_t cap    = (int64_t)s->sm_count * 32;
        if (blocks > cap)
            blocks = cap;
        split_rows_kernel<MODE_3X><<<(unsigned)blocks, 256, 0, stream()>>>(a_dev, m, k, kp, a_hi, a_lo);
        CT_LAUNCH_CHECK("split_rows(static scratch)");
        dim3 grid((unsigned)((n + 31) / 32), (unsigned)(kp / 32));
        split_transpose_kernel<MODE_3X><<<grid, 256, 0, stream()>>>(b_dev, k, n, kp, b_hi, b_lo);
        CT_LAUNCH_CHECK("split_transpose(static scratch)");
    }
    int64_t tiles256 = ((m + BM - 1) / BM) * ((n + 255) / 256);
    if (n > 128 && tiles256 >= s->sm_count / 2)
        CT_TRY(launch_static<256>(s, a_hi, a_lo, b_hi, b_lo, m, n, kp, out_dev));
    else
        CT_TRY(launch_static<128>(s, a_hi, a_lo, b_hi, b_lo, m, n, kp, out_dev));
    if (status_dev) // stream-ordered copy of the kernel's error word into the caller's buffer
        CT_CUDA(cudaMemcpyAsync(
            status_dev, s->flags + FLAG_TIMEOUT, sizeof(uint32_t), cudaMemcpyDeviceToDevice, stream()));
    return CT_OK;
}

#ifdef CT_GEMM_TRACE
extern "C" int ct_debug_gemm_trace(unsigned long long *host, int count) {
    return (int)cudaMemcpyFromSymbol(host, ct::g_gemm_trace, sizeof(unsigned long long) * (size_t)count);
}
#endif
