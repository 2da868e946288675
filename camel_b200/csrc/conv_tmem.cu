// conv2d for layers with few channels on both sides (at most 32 in, at most 64 out, a small
// filter; the 32 -> 64 channel 3x3 layer of a small CNN): the filters live in tensor memory.
//
// Why another kernel.  With 64 output channels the tensor core cannot be given a wide tile:
// measured on B200 (ct_measure_mma_rate), tcgen05.mma kind::tf32 of 128 x N x 8 takes ~138 clocks
// at N = 256, ~73 at N = 128, ~54 at N = 64 and never less than ~49, and M = 64 takes as long as
// M = 128.  The pixels-on-rows kernel (conv_swap_stream_kernel) issues 128 x 64 x 8 MMAs and
// re-fetches, per filter tap, a shifted copy of the same pixels and the tap's filter rows; its
// operands cross shared memory twice (TMA in, MMA out), about 10 KB per MMA, and that traffic,
// not the tensor pipe, sets its pace (~80 clocks per MMA).  Here
//   * the filters are the A operand and stay in TENSOR MEMORY for the whole launch: rows 0..63
//     hold the tf32 "hi" part of the 64 filters, rows 64..127 the "lo" part, 8 columns per k-step
//     (tap, group of 8 input channels) - written once per CTA with tcgen05.st, never re-read from
//     shared memory;
//   * the pixels are the B operand, N = 128 per tile: th output rows of PW = w + 2 pad positions
//     (the two halo columns of every row are computed and dropped).  A tile's input - th + kh - 1
//     rows of PW positions, halo included, zeros outside the image - is fetched ONCE by one 4-D
//     TMA box per plane; because a position's row index in the box is y * PW + x, the pixels a
//     tap (r, s) needs are the same rows shifted by r * PW + s, i.e. the same shared memory
//     through a descriptor whose start address is moved by that many 128-byte rows;
//   * per k-step two MMAs, [W_hi; W_lo] x X_hi and [W_hi; W_lo] x X_lo, accumulate into one
//     128 x 128 accumulator: lane c holds W_hi . (X_hi + X_lo), lane 64 + c holds W_lo . (X_hi +
//     X_lo); the epilogue adds the two lanes (all four terms of the split product).
// Shared-memory traffic per k-step drops to ~9 KB for 146 clocks of tensor work, so the tensor
// pipe is the bound again: ~0.7 of the 3xTF32 ceiling for this shape instead of ~0.3.
//
// Roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer (and TMEM owner), warps 2-9
// epilogue: each drains a 32-lane x 64-column block of the accumulator into a shared-memory block
// [lane][position] (128-bit stores), which frees the accumulator for the next tile's MMAs; then
// warp e writes out channels e, e + 8, ...: hi lane + lo lane, bias, relu, optional 2x2 max-pool,
// its lanes over consecutive positions, so a store instruction covers consecutive pixels of one
// NCHW channel plane.  The epilogue of tile i runs while the MMAs of tile i + 1 are issued; it has
// to stay shorter than those (~2.7 us), which is why a position's pixel offset is computed once per
// kernel, not per value.  One CTA per SM walks the tiles.  Every wait is bounded.
#include "common.cuh"
#include "tc_ptx.cuh"
#include "split.cuh"
#include "tmap.cuh"

// Optional per-CTA clock accounting for tuning; compiled in only with -DCT_CONV_TRACE.
#ifdef CT_CONV_TRACE
__device__ unsigned long long g_conv_trace[256 * 16];
#define CV_CLOCK() clock64()
#define CV_ACCUM(slot, cycles)                                                          \
    do {                                                                                \
        if (blockIdx.x < 256)                                                           \
            g_conv_trace[blockIdx.x * 16 + (slot)] += (unsigned long long)(cycles);     \
    } while (0)
extern "C" int ct_debug_conv_trace(unsigned long long *host, int count, int clear) {
    int rc = (int)cudaMemcpyFromSymbol(host, g_conv_trace, sizeof(unsigned long long) * (size_t)count);
    if (clear) {
        static unsigned long long zeros[256 * 16];
        cudaMemcpyToSymbol(g_conv_trace, zeros, sizeof(zeros));
    }
    return rc;
}
#else
#define CV_CLOCK() 0ll
#define CV_ACCUM(slot, cycles) do { } while (0)
#endif

namespace ct {
namespace {

using namespace ptx;

constexpr int kTA_EpiWarps  = 8;
constexpr int kTA_Threads   = 64 + 32 * kTA_EpiWarps;
constexpr int kTA_CvtWarps  = 4;                  // raw mode: warps that turn float32 boxes into hi/lo planes
constexpr int kTA_ThreadsRaw = kTA_Threads + 32 * kTA_CvtWarps;
constexpr int kTA_RawStages = 2;
constexpr int kTA_MaxKSteps = 48;                 // 8 TMEM columns each: 384 of the 512 columns
constexpr int kTA_DCol      = kTA_MaxKSteps * 8;  // the accumulator's first column
constexpr int kTA_N         = 128;                // positions per tile (MMA N)
constexpr int kTA_StageRowF = kTA_N + 4;          // epilogue staging: [128 lanes][132] floats: rows 16-byte aligned,
                                                  // 128-bit stores of 8 consecutive lanes fall into distinct banks
constexpr int kTA_StagingBytes = 128 * kTA_StageRowF * 4;

struct ConvTmemParams {
    const float *w;   // filters [ko][c][kh][kw], float32
    const float *bias;
    float *out;       // [batch][ko][ho][wo], or [batch][ko][ho/2][wo/2] with pool
    uint32_t *flags;
    int ko, c, kh, kw, pad;
    int ho, wo, pw;   // pw = input width + 2 pad: positions per tile row
    int th;           // output rows per tile
    int tiles_y;      // ceil(ho / th)
    int ksteps;       // kh * kw * 4
    int box_bytes;    // bytes of one plane's TMA box
    int plane_bytes;  // shared-memory bytes reserved per plane (box plus the rows shifted reads run into)
    int stages;
    int act, pool;
    // raw mode (the input is read as it is, NCHW float32, and split into planes inside the kernel)
    int box_w;        // floats per row of the raw box (a multiple of four)
    int off_x;        // the tile's first position (x = -pad) sits this many floats into a raw row
    int box_rows;     // th + kh - 1
    int raw_bytes;    // bytes of one raw box: 32 channels x box_rows x box_w floats
    int raw_stride;   // shared-memory bytes reserved per raw stage
};

__device__ __forceinline__ void tmem_st_32x32_x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_tf32_a_tmem(
    uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// RAW = false: map_x_hi / map_x_lo cover NHWC hi / lo planes written by a pre-pass.
// RAW = true:  map_x_hi covers the input itself, [batch][c][h][w] float32 (map_x_lo is not used);
//              the producer fetches a tile's box of it - 32 channels x box_rows x box_w floats, zeros
//              outside the image and past the last channel - and four more warps rewrite it as the
//              two planes the MMAs read: position (y, x) becomes row y * pw + x, its 32 channels the
//              128 bytes of the row (swizzled as TMA would have), each value split into tf32 parts.
//              The pre-pass and its 12 bytes of traffic per input element are gone.
template <bool RAW>
__global__ void __launch_bounds__(kTA_ThreadsRaw, 1) conv_tmem_filters_kernel(
    const __grid_constant__ CUtensorMap map_x_hi, const __grid_constant__ CUtensorMap map_x_lo,
    const ConvTmemParams p, const int total_tiles) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[4];
    __shared__ uint64_t bar_empty[4];
    __shared__ uint64_t bar_raw_full[kTA_RawStages];
    __shared__ uint64_t bar_raw_empty[kTA_RawStages];
    __shared__ uint64_t bar_tmem_full;
    __shared__ uint64_t bar_tmem_empty;
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
    const uint32_t stage_bytes = 2u * (uint32_t)p.plane_bytes;
    // planes | raw boxes (raw mode) | epilogue staging
    const uint32_t raw_base = smem_base + (uint32_t)p.stages * stage_bytes;
    const uint32_t raw_all  = RAW ? (uint32_t)kTA_RawStages * (uint32_t)p.raw_stride : 0u;
    float *staging = reinterpret_cast<float *>(smem_raw + (raw_base - smem_u32(smem_raw)) + raw_all);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), RAW ? kTA_CvtWarps : 1); // raw mode: the converting warps fill a stage
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int s = 0; s < kTA_RawStages; ++s) {
            mbar_init(smem_u32(&bar_raw_full[s]), 1);
            mbar_init(smem_u32(&bar_raw_empty[s]), kTA_CvtWarps);
        }
        mbar_init(smem_u32(&bar_tmem_full), 1);
        mbar_init(smem_u32(&bar_tmem_empty), kTA_EpiWarps);
        mbar_init(smem_u32(&bar_done), 1);
        mbar_init(smem_u32(&bar_epi), kTA_EpiWarps);
        mbar_fence_init();
        prefetch_tensormap(&map_x_hi);
        prefetch_tensormap(&map_x_lo);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    // ---- the filters go to tensor memory, once: warps 2..5 own the four lane quarters ----------
    if (warp >= 2 && warp < 6) {
        const int quarter = warp & 3;
        const int m       = quarter * 32 + lane;      // TMEM lane = row of the A operand
        const int ch      = m & 63;                   // filter
        const bool lo_row = m >= 64;                  // rows 64..127: the low parts
        const int taps    = p.kh * p.kw;
        for (int ks = 0; ks < p.ksteps; ++ks) {
            const int tap = ks >> 2, c0 = (ks & 3) * 8;
            uint32_t v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float x = 0.0f;
                if (ch < p.ko && c0 + j < p.c)
                    x = p.w[((int64_t)ch * p.c + (c0 + j)) * taps + tap];
                float hi, lo;
                split_tf32(x, hi, lo);
                v[j] = __float_as_uint(lo_row ? lo : hi);
            }
            tmem_st_32x32_x8(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(ks * 8), v);
        }
        tmem_st_wait();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();

    if (warp == 0) {
        // ===== TMA producer: one halo box per plane and tile (raw mode: one box of the input) =====
        if (lane == 0) {
            int i = 0;
            bool ok = true;
            const int nstages = RAW ? kTA_RawStages : p.stages;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++i) {
                const int img = tile / p.tiles_y, ty = tile - img * p.tiles_y;
                const int s       = i % nstages;
                const uint32_t ph = (uint32_t)(i / nstages) & 1u;
                if (!mbar_wait_patient(smem_u32(RAW ? &bar_raw_empty[s] : &bar_empty[s]), ph ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                const int32_t h0 = ty * p.th - p.pad;
                if (RAW) {
                    const uint32_t full = smem_u32(&bar_raw_full[s]);
                    mbar_expect_tx(full, (uint32_t)p.raw_bytes);
                    // the box starts off_x floats left of x = -pad so that its first byte is 16-byte aligned
                    tma_load_4d(raw_base + (uint32_t)s * (uint32_t)p.raw_stride, &map_x_hi, full, -p.pad - p.off_x, h0, 0, img);
                } else {
                    const uint32_t full = smem_u32(&bar_full[s]);
                    const uint32_t dst  = smem_base + (uint32_t)s * stage_bytes;
                    mbar_expect_tx(full, 2u * (uint32_t)p.box_bytes);
                    const int32_t w0 = -p.pad;
                    tma_load_4d(dst, &map_x_hi, full, 0, w0, h0, img);
                    tma_load_4d(dst + (uint32_t)p.plane_bytes, &map_x_lo, full, 0, w0, h0, img);
                }
            }
            if (*abort_flag) {
                // unwind: let the copies still in flight land before the CTA goes away
                const int first = i - nstages < 0 ? 0 : i - nstages;
                for (int k2 = first; k2 < i; ++k2) {
                    const uint32_t bar = smem_u32(RAW ? &bar_raw_full[k2 % nstages] : &bar_full[k2 % nstages]);
                    const uint32_t ph  = (uint32_t)(k2 / nstages) & 1u;
                    const uint64_t t0  = globaltimer_ns();
                    while (!mbar_try_wait(bar, ph) && globaltimer_ns() - t0 < kWaitBudgetNs) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer =====
        if (lane == 0) {
            const uint32_t idesc  = make_idesc(2u, 128, (uint32_t)kTA_N);
            const uint32_t d_tmem = tmem_base + (uint32_t)kTA_DCol;
            int i = 0;
            bool ok = true;
            const long long t_start = CV_CLOCK();
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++i) {
                const int s       = i % p.stages;
                const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
                // the accumulator of the previous tile has been drained
                const long long t0 = CV_CLOCK();
                if (!mbar_wait(smem_u32(&bar_tmem_empty), ((uint32_t)i & 1u) ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                const long long t1 = CV_CLOCK();
                if (!mbar_wait(smem_u32(&bar_full[s]), ph, abort_flag)) {
                    ok = false;
                    break;
                }
                CV_ACCUM(0, t1 - t0);          // waiting for the accumulator
                CV_ACCUM(1, CV_CLOCK() - t1);  // waiting for the halo
                tc_fence_after_sync();
                const uint32_t x_hi = smem_base + (uint32_t)s * stage_bytes;
                const uint32_t x_lo = x_hi + (uint32_t)p.plane_bytes;
                int ks = 0;
                for (int r = 0; r < p.kh; ++r) {
                    for (int sx = 0; sx < p.kw; ++sx) {
                        // the tap's pixels: the same box, (r * pw + sx) rows of 128 bytes further on
                        const uint32_t shift = (uint32_t)(r * p.pw + sx) * 128u;
                        const uint64_t db_hi = smem_desc_k<128>(x_hi + shift), db_lo = smem_desc_k<128>(x_lo + shift);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk, ++ks) {
                            const uint64_t adv    = (uint64_t)(kk * 32 >> 4);
                            const uint32_t a_tmem = tmem_base + (uint32_t)(ks * 8);
                            mma_tf32_a_tmem(d_tmem, a_tmem, db_lo + adv, idesc, ks == 0 ? 0u : 1u);
                            mma_tf32_a_tmem(d_tmem, a_tmem, db_hi + adv, idesc, 1u);
                        }
                    }
                }
                tc_commit(smem_u32(&bar_empty[s]));   // the stage is free once these MMAs have retired
                tc_commit(smem_u32(&bar_tmem_full));  // and the accumulator is complete
            }
            CV_ACCUM(2, CV_CLOCK() - t_start); // the MMA thread's whole loop
            CV_ACCUM(3, i);
            if (!ok || *abort_flag) {
                tc_commit(smem_u32(&bar_done));
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(smem_u32(&bar_done), 0) && globaltimer_ns() - t0 < kWaitBudgetNs) {
                }
            }
        }
    } else if (RAW && warp < 2 + kTA_CvtWarps) {
        // ===== raw mode: float32 box -> hi / lo planes =====
        // A thread takes a position (y, x) of the box: its 32 channel values lie box_rows * box_w floats
        // apart in the raw box (consecutive lanes read consecutive x: no bank conflicts) and become the
        // 128-byte row y * pw + x of both planes, 16-byte chunk j at chunk j ^ (row & 7) - the 128-byte
        // swizzle the MMA's descriptors expect.
        // (these warps come before the epilogue warps: the schedulers favour older warps, and eight
        // epilogue warps polling their barrier kept younger converting warps from issuing - a tile's
        // conversion took 9900 clocks behind them)
        const int ct   = threadIdx.x - 64;
        const int npos = p.box_rows * p.pw;
        const int cstride = p.box_rows * p.box_w; // floats between two channels of one position
        int i = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++i) {
            const int rs       = i % kTA_RawStages;
            const uint32_t rph = (uint32_t)(i / kTA_RawStages) & 1u;
            const int s        = i % p.stages;
            const uint32_t ph  = (uint32_t)(i / p.stages) & 1u;
            const long long v0 = CV_CLOCK();
            bool got = mbar_wait_patient(smem_u32(&bar_raw_full[rs]), rph, abort_flag);
            const long long v1 = CV_CLOCK();
            got      = got && mbar_wait_patient(smem_u32(&bar_empty[s]), ph ^ 1u, abort_flag); // the planes' stage is free
            if (!__all_sync(0xffffffffu, got))
                break;
            const long long v2 = CV_CLOCK();
            const float *raw = reinterpret_cast<const float *>(smem_raw + (raw_base - smem_u32(smem_raw)) + (uint32_t)rs * (uint32_t)p.raw_stride);
            uint8_t *x_hi    = smem_raw + (smem_base - smem_u32(smem_raw)) + (uint32_t)s * stage_bytes;
            uint8_t *x_lo    = x_hi + p.plane_bytes;
            for (int pos = ct; pos < npos; pos += 32 * kTA_CvtWarps) {
                const int y = pos / p.pw, x = pos - y * p.pw;
                const float *src = raw + y * p.box_w + x + p.off_x;
                const uint32_t row_off = (uint32_t)pos * 128u;
                const uint32_t sw      = (uint32_t)pos & 7u;
                // sixteen channels at a time: all their loads first (a store to shared memory in between
                // would hold back the loads behind it), then the splits and the eight stores
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    float v[16];
#pragma unroll
                    for (int t = 0; t < 16; ++t)
                        v[t] = src[(16 * half + t) * cstride];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float hi[4], lo[4];
#pragma unroll
                        for (int t = 0; t < 4; ++t)
                            split_tf32_flat(v[4 * j + t], hi[t], lo[t]);
                        const uint32_t at = row_off + (((uint32_t)(4 * half + j) ^ sw) << 4);
                        *reinterpret_cast<float4 *>(x_hi + at) = make_float4(hi[0], hi[1], hi[2], hi[3]);
                        *reinterpret_cast<float4 *>(x_lo + at) = make_float4(lo[0], lo[1], lo[2], lo[3]);
                    }
                }
            }
            // the planes were written through the generic proxy and are read by the tensor core's
            // asynchronous proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&bar_full[s]));
                mbar_arrive(smem_u32(&bar_raw_empty[rs]));
            }
            if (ct == 0) {
                CV_ACCUM(9, v1 - v0);            // converter: waiting for the raw box
                CV_ACCUM(10, v2 - v1);           // waiting for a free plane stage
                CV_ACCUM(11, CV_CLOCK() - v2);   // converting
            }
        }
    } else {
        // ===== epilogue =====
        const int quarter = warp & 3;        // TMEM lanes this warp may read: 32 * quarter ..
        const int ew      = warp - (RAW ? 2 + kTA_CvtWarps : 2); // 0..7: which channels this warp writes out
        const int half    = ew >> 2;         // which 64 columns of the accumulator it drains
        uint32_t epi_phase = 0;
        auto epi_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&bar_epi));
            bool ok = mbar_wait_patient(smem_u32(&bar_epi), epi_phase, abort_flag);
            epi_phase ^= 1u;
            return __all_sync(0xffffffffu, ok);
        };
        // Where this lane's positions land, once for the whole kernel: position pos = lane + 32 g
        // of a tile is pixel (y, x) = (pos / pw, pos % pw) of the tile's rows; -1 for the halo columns
        // and past the tile.  With the pool: lane q = pooled pixel (py, px) of the tile.
        int off[4], yy[4];
        const int npos = p.th * p.pw;
        const int pw2 = p.wo >> 1, ph2 = p.ho >> 1;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const int pos = lane + 32 * g;
            off[g] = -1, yy[g] = 0;
            if (p.pool == 0) {
                const int y = pos / p.pw, x = pos - y * p.pw;
                if (pos < npos && x < p.wo)
                    off[g] = y * p.wo + x, yy[g] = y;
            } else {
                const int py = pos / pw2, px = pos - py * pw2;
                if (py < (p.th >> 1))
                    off[g] = (2 * py) * p.pw + 2 * px, yy[g] = py; // here: the window's first position
            }
        }
        // this warp's channels are the same for every tile: their bias values are read once (a load
        // per channel inside the tile loop costs a trip to L2 that the add then waits for)
        float bias_r[64 / kTA_EpiWarps];
#pragma unroll
        for (int j = 0; j < 64 / kTA_EpiWarps; ++j) {
            const int ch = ew + kTA_EpiWarps * j;
            bias_r[j]    = (p.bias && ch < p.ko) ? p.bias[ch] : 0.0f;
        }
        int i = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++i) {
            const int img = tile / p.tiles_y, ty = tile - img * p.tiles_y;
            const long long e0 = CV_CLOCK();
            bool got = mbar_wait_patient(smem_u32(&bar_tmem_full), (uint32_t)i & 1u, abort_flag);
            if (!__all_sync(0xffffffffu, got))
                break;
            const long long e1 = CV_CLOCK();
            const int y0 = ty * p.th;
            tc_fence_after_sync();
            // lane m of the accumulator -> row m of the staging block
            float4 *mine = reinterpret_cast<float4 *>(staging + (quarter * 32 + lane) * kTA_StageRowF + half * 64);
            const uint32_t taddr =
                tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(kTA_DCol + half * 64);
            // both halves of this warp's 64 columns are requested before the one wait, and the
            // accumulator is handed back as soon as the values are in registers: the next tile's
            // MMAs then start while these threads are still writing the staging block
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(taddr, r0);
            tmem_ld_32x32(taddr + 32, r1);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&bar_tmem_empty)); // the next tile's MMAs may start
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                mine[j]     = make_float4(__uint_as_float(r0[4 * j]), __uint_as_float(r0[4 * j + 1]),
                                          __uint_as_float(r0[4 * j + 2]), __uint_as_float(r0[4 * j + 3]));
                mine[8 + j] = make_float4(__uint_as_float(r1[4 * j]), __uint_as_float(r1[4 * j + 1]),
                                          __uint_as_float(r1[4 * j + 2]), __uint_as_float(r1[4 * j + 3]));
            }
            const long long e2 = CV_CLOCK();
            if (!epi_sync())
                break;
            const long long e3 = CV_CLOCK();
            // which of this lane's four positions are stored for this tile (rows past the image's
            // last row of a partial tile are not)
            unsigned okmask = 0;
#pragma unroll
            for (int g = 0; g < 4; ++g)
                if (off[g] >= 0 && (p.pool ? (y0 >> 1) + yy[g] < ph2 : y0 + yy[g] < p.ho))
                    okmask |= 1u << g;
            // Two channels at a time, every load of the pair before the first dependent instruction, no
            // branch inside: a channel past the last filter or a position that is not stored is masked
            // at the store (its loads read rows of the staging block that hold nothing of interest).
            if (p.pool == 0) {
#pragma unroll
                for (int jj = 0; jj < 64 / kTA_EpiWarps; jj += 2) {
                    float h[2][4], l[2][4];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int ch    = ew + kTA_EpiWarps * (jj + u);
                        const float *hi = staging + ch * kTA_StageRowF + lane, *lo = hi + 64 * kTA_StageRowF;
#pragma unroll
                        for (int g = 0; g < 4; ++g)
                            h[u][g] = hi[32 * g], l[u][g] = lo[32 * g];
                    }
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int ch = ew + kTA_EpiWarps * (jj + u);
                        const float b = bias_r[jj + u];
                        float *plane  = p.out + (((int64_t)img * p.ko + ch) * p.ho + y0) * p.wo;
                        const unsigned mask = ch < p.ko ? okmask : 0u;
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            float v = __fadd_rn(h[u][g], l[u][g]);
                            if (p.bias)
                                v = __fadd_rn(v, b);
                            if (p.act == CT_ACT_RELU)
                                v = __fmul_rn(v, v > 0.0f ? 1.0f : 0.0f);
                            if (mask & (1u << g))
                                plane[off[g]] = v;
                        }
                    }
                }
            } else {
                // 2x2 max-pool of the activated values; window order and strict '>' as in
                // maxpool2d (the first element seeds, a NaN never wins)
                const int pooled = (p.th >> 1) * pw2;           // pooled pixels of a tile
                const int groups = (pooled + 31) >> 5;          // the same for every lane: no divergence
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    if (g >= groups)
                        break;
                    const bool live = (okmask >> g) & 1u;
                    const int pos   = live ? off[g] : 0;
#pragma unroll
                    for (int jj = 0; jj < 64 / kTA_EpiWarps; jj += 2) {
                        float h[2][4], l[2][4];
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const int ch    = ew + kTA_EpiWarps * (jj + u);
                            const float *hi = staging + ch * kTA_StageRowF + pos, *lo = hi + 64 * kTA_StageRowF;
                            h[u][0] = hi[0], h[u][1] = hi[1], h[u][2] = hi[p.pw], h[u][3] = hi[p.pw + 1];
                            l[u][0] = lo[0], l[u][1] = lo[1], l[u][2] = lo[p.pw], l[u][3] = lo[p.pw + 1];
                        }
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const int ch  = ew + kTA_EpiWarps * (jj + u);
                            const float b = bias_r[jj + u];
                            float v[4];
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                v[t] = __fadd_rn(h[u][t], l[u][t]);
                                if (p.bias)
                                    v[t] = __fadd_rn(v[t], b);
                                if (p.act == CT_ACT_RELU)
                                    v[t] = __fmul_rn(v[t], v[t] > 0.0f ? 1.0f : 0.0f);
                            }
                            float best = v[0];
                            if (v[1] > best)
                                best = v[1];
                            if (v[2] > best)
                                best = v[2];
                            if (v[3] > best)
                                best = v[3];
                            if (live && ch < p.ko) {
                                float *plane = p.out + (((int64_t)img * p.ko + ch) * ph2 + (y0 >> 1)) * pw2;
                                plane[lane + 32 * g] = best; // pooled pixels of a tile are consecutive: py * pw2 + px
                            }
                        }
                    }
                }
            }
            const long long e4 = CV_CLOCK();
            if (!epi_sync()) // the staging block is rewritten by the next tile
                break;
            if (ew == 0 && lane == 0) {
                CV_ACCUM(4, e1 - e0);           // epilogue: waiting for the accumulator to be complete
                CV_ACCUM(5, e2 - e1);           // drain
                CV_ACCUM(6, e3 - e2);           // first meeting of the epilogue warps
                CV_ACCUM(7, e4 - e3);           // add, activate, store
                CV_ACCUM(8, CV_CLOCK() - e4);   // second meeting
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_flag)
        atomicExch(p.flags + FLAG_TIMEOUT, 1u + (uint32_t)blockIdx.x);
}

} // namespace

// Whether the filters-in-tensor-memory kernel takes this layer.  The answer does not depend on
// whether a max-pool is fused, so that conv2d and conv2d + pool of one layer run the same arithmetic;
// *pool_ok says whether the fused 2x2 pool is possible (even output extents, two rows per tile).
bool conv_tmem_applicable(int64_t c, int64_t h, int64_t w, int64_t ko, int64_t kh, int64_t kw, int64_t stride,
                          int64_t pad, bool *pool_ok) {
    if (pool_ok)
        *pool_ok = false;
    if (stride != 1 || c < 1 || c > 32 || ko < 1 || ko > 64 || kh * kw * 4 > kTA_MaxKSteps)
        return false;
    const int64_t pw = w + 2 * pad, wo = pw - kw + 1, ho = h + 2 * pad - kh + 1;
    if (wo < 1 || ho < 1 || pw > kTA_N || pw > 256)
        return false;
    int64_t th = kTA_N / pw;
    if (th > ho)
        th = ho;
    if (th < 1 || th + kh - 1 > 256)
        return false;
    // worth it only where the tile is reasonably full (else the pixels-on-rows kernel)
    if (!(th * pw >= 96 || th == ho))
        return false;
    if (pool_ok)
        *pool_ok = (wo & 1) == 0 && (ho & 1) == 0 && th >= 2;
    return true;
}

// Shared-memory plan of a launch: tile rows, bytes per plane and per raw box, pipeline stages.
static bool conv_tmem_plan(ConvTmemParams &p, int64_t h, int64_t wd, int64_t kh, int64_t kw, int64_t pad, int pool, bool raw) {
    p.pad = (int)pad, p.kh = (int)kh, p.kw = (int)kw;
    p.pw  = (int)(wd + 2 * pad);
    p.wo  = p.pw - (int)kw + 1;
    p.ho  = (int)(h + 2 * pad - kh + 1);
    p.th  = kTA_N / p.pw < p.ho ? kTA_N / p.pw : p.ho;
    if (pool)
        p.th &= ~1;
    if (p.th < 1)
        return false;
    p.tiles_y  = (p.ho + p.th - 1) / p.th;
    p.ksteps   = (int)(kh * kw * 4);
    p.box_rows = p.th + (int)kh - 1;
    p.box_bytes = p.box_rows * p.pw * 128;
    // a tap's shifted window of kTA_N rows may run past the box: reserve those rows too
    int rows_needed = ((int)kh - 1) * p.pw + ((int)kw - 1) + kTA_N;
    if (rows_needed < p.box_rows * p.pw)
        rows_needed = p.box_rows * p.pw;
    p.plane_bytes = (rows_needed * 128 + 1023) & ~1023;
    // raw mode: the box starts at the 16-byte boundary at or left of x = -pad and is a whole number
    // of 16-byte units wide
    const int pad_up = ((int)pad + 3) & ~3;
    p.off_x      = pad_up - (int)pad;
    p.box_w      = (p.off_x + p.pw + 3) & ~3;
    p.raw_bytes  = 32 * p.box_rows * p.box_w * 4;
    p.raw_stride = (p.raw_bytes + 127) & ~127;
    if (raw && (p.box_w > 256 || p.box_rows > 256))
        return false;
    const int budget = 226 * 1024 - 1024 - kTA_StagingBytes - (raw ? kTA_RawStages * p.raw_stride : 0);
    p.stages         = budget / (2 * p.plane_bytes);
    if (p.stages > 4)
        p.stages = 4;
    return p.stages >= 2;
}

// Whether the kernel can read this input as it is (NCHW float32) instead of pre-split NHWC planes:
// the tensor map over it needs row strides of whole 16-byte units and an aligned base, and the raw
// boxes have to fit into shared memory beside two stages of planes.
bool conv_tmem_reads_input_directly(const float *x, int64_t h, int64_t w, int64_t kh, int64_t kw, int64_t pad, int pool) {
    if ((w & 3) != 0 || (reinterpret_cast<uintptr_t>(x) & 15u) != 0)
        return false;
    ConvTmemParams p;
    return conv_tmem_plan(p, h, w, kh, kw, pad, pool, true);
}

// x_raw != nullptr: the input itself, [batch][c][h][w] float32 (see conv_tmem_reads_input_directly);
// else x_hi / x_lo: NHWC planes [batch][h][w][32] of the input (float32 hi / lo parts).
ct_status conv_tmem_filters(
    DeviceState *st, const float *x_raw, const void *x_hi, const void *x_lo, const float *w, const float *bias,
    int64_t batch, int64_t c, int64_t h, int64_t wd, int64_t ko, int64_t kh, int64_t kw, int64_t pad, int act, int pool,
    float *out) {
    const bool raw = x_raw != nullptr;
    ConvTmemParams p;
    p.w = w, p.bias = bias, p.out = out, p.flags = st->flags_dev;
    p.ko = (int)ko, p.c = (int)c;
    p.act = act, p.pool = pool;
    if (!conv_tmem_plan(p, h, wd, kh, kw, pad, pool, raw))
        return fail(CT_ERR_INVALID, "conv2d: internal tile shape %d x %d not usable", p.th, p.pw);
    const int box_rows = p.box_rows;
    const int64_t tiles = (int64_t)p.tiles_y * batch;
    if (tiles > 0x7fffffffll)
        return fail(CT_ERR_TOO_LARGE, "conv2d: too many tiles");
    CUtensorMap mx_hi, mx_lo;
    if (raw) {
        // the input [batch][c][h][w]; box = box_w floats x box_rows rows x 32 channels of one image, not
        // swizzled; outside the image and past the last channel it reads as zero: padding for free
        const uint64_t dims[4]    = {(uint64_t)wd, (uint64_t)h, (uint64_t)c, (uint64_t)batch};
        const uint64_t strides[3] = {4ull * (uint64_t)wd, 4ull * (uint64_t)wd * (uint64_t)h,
                                     4ull * (uint64_t)wd * (uint64_t)h * (uint64_t)c};
        const uint32_t box[4]     = {(uint32_t)p.box_w, (uint32_t)box_rows, 32, 1};
        CT_TRY(encode_tiled_map_f32(&mx_hi, x_raw, 4, dims, strides, box, /*swizzle_bytes=*/0));
        mx_lo = mx_hi;
    } else {
        // planes [batch][h][w][32 channels]; box = 32 channels x pw positions x (th + kh - 1) rows of one
        // image, 128-byte swizzle; positions outside the image read as zero: the padding
        const uint64_t dims[4]    = {32, (uint64_t)wd, (uint64_t)h, (uint64_t)batch};
        const uint64_t strides[3] = {128, 128ull * (uint64_t)wd, 128ull * (uint64_t)wd * (uint64_t)h};
        const uint32_t box[4]     = {32, (uint32_t)p.pw, (uint32_t)box_rows, 1};
        CT_TRY(encode_tiled_map_f32(&mx_hi, x_hi, 4, dims, strides, box, /*swizzle_bytes=*/128));
        CT_TRY(encode_tiled_map_f32(&mx_lo, x_lo, 4, dims, strides, box, 128));
    }
    const size_t smem = (size_t)p.stages * 2 * p.plane_bytes + (raw ? (size_t)kTA_RawStages * p.raw_stride : 0) +
                        kTA_StagingBytes + 1024;
    static bool attr_set_dev[16] = {}; // the attribute belongs to a device's context
    bool &attr_set = attr_set_dev[st->device & 15];
    if (!attr_set) {
        CT_CUDA(cudaFuncSetAttribute(conv_tmem_filters_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        CT_CUDA(cudaFuncSetAttribute(conv_tmem_filters_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        attr_set = true;
    }
    const unsigned grid = (unsigned)(tiles < st->sm_count ? tiles : st->sm_count);
    ProfScope prof("gemm_tc");
    if (raw)
        conv_tmem_filters_kernel<true><<<grid, kTA_ThreadsRaw, smem, stream()>>>(mx_hi, mx_lo, p, (int)tiles);
    else
        conv_tmem_filters_kernel<false><<<grid, kTA_Threads, smem, stream()>>>(mx_hi, mx_lo, p, (int)tiles);
    CT_LAUNCH_CHECK("conv_tmem_filters");
    return CT_OK;
}

} // namespace ct
