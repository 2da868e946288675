// Implicit-GEMM conv2d (stride 1) for layers with many output channels: the input halo of a tile is
// fetched once per channel block and serves all filter taps.
//
// The streaming implicit GEMM of gemm_tc.cu fetches, for every (tap, channel block), the tile's
// pixels again - the same values shifted by the tap.  Shared memory then carries, per k-block of 16
// channels, 28 KB of pixel planes and 16 KB of filter planes in (TMA) plus 66 KB out (six MMAs read
// their operands), and that traffic, not the tensor pipe, sets the kernel's pace (0.65 of the
// measured 3xTF32 ceiling on 64 -> 128 channels, 56 x 56).  Here a tile is th output rows of
// PW = w + 2 pad positions (the two halo columns of every row are computed and dropped), its
// input for one block of 16 channels - th + kh - 1 rows of PW positions, zeros outside the image -
// is ONE 4-D TMA box per plane, and tap (r, s) reads the same shared memory through a descriptor
// moved by r * PW + s rows of 64 bytes (a position's row in the box is y * PW + x).  Pixel planes
// enter shared memory once per nine taps; per k-block 19 KB in instead of 44.
//
// Structure as the streaming kernel: one CTA per SM walks the tiles, two TMEM accumulators, the
// epilogue of tile i (drain, bias, relu, store) runs under the MMAs of tile i + 1.  Two rings of
// stages: filter k-blocks (one per tap and channel block) and halos (one per channel block).
// Rows = 128 output channels, columns = positions.  Every wait is bounded.
#include "common.cuh"
#include "tc_ptx.cuh"
#include "tmap.cuh"

// Optional per-CTA clock accounting for tuning; compiled in only with -DCT_CONV_TRACE.
#ifdef CT_CONV_TRACE
__device__ unsigned long long g_halo_trace[256 * 16];
#define CH_CLOCK() clock64()
#define CH_ACCUM(slot, cycles)                                                          \
    do {                                                                                \
        if (blockIdx.x < 256)                                                           \
            g_halo_trace[blockIdx.x * 16 + (slot)] += (unsigned long long)(cycles);     \
    } while (0)
extern "C" int ct_debug_halo_trace(unsigned long long *host, int count, int clear) {
    int rc = (int)cudaMemcpyFromSymbol(host, g_halo_trace, sizeof(unsigned long long) * (size_t)count);
    if (clear) {
        static unsigned long long zeros[256 * 16];
        cudaMemcpyToSymbol(g_halo_trace, zeros, sizeof(zeros));
    }
    return rc;
}
#else
#define CH_CLOCK() 0ll
#define CH_ACCUM(slot, cycles) do { } while (0)
#endif

namespace ct {
namespace {

using namespace ptx;

constexpr int kH_RowB       = 64;                     // bytes of k per operand row and k-block: 16 float32
constexpr int kH_BlockK     = 16;
constexpr int kH_AStages    = 4;
constexpr int kH_HaloStages = 2;
constexpr int kH_ABytes     = 128 * kH_RowB;          // one filter plane of a k-block
constexpr int kH_AStageBytes = 2 * kH_ABytes;         // hi + lo
constexpr int kH_EpiWarps   = 8;
constexpr int kH_Threads    = 64 + 32 * kH_EpiWarps;
constexpr int kH_EpiRowBytes  = 64 * 4 + 16;          // 64 columns staged at a time, rows padded
constexpr int kH_EpiWarpBytes = 32 * kH_EpiRowBytes;
constexpr int kH_EpiBytes     = kH_EpiWarps * kH_EpiWarpBytes;
constexpr int kH_BiasSlots    = 256;                  // output channels whose bias is kept in shared memory

struct ConvHaloParams {
    const float *bias;
    float *out;       // [batch][ko][ho][wo]
    uint32_t *flags;
    int ko, tiles_m;
    int kh, kw, pad;
    int ho, wo, pw;   // pw = w + 2 pad
    int th, tiles_y;
    int cblocks;      // channel blocks of 16
    int c_pad;        // channels of the planes (k offset of a tap in the filter planes: tap * c_pad)
    int n_mma;        // th * pw rounded up to 16
    int box_bytes;    // one plane's halo box
    int halo_plane_bytes;
    int act;
};

__global__ void __launch_bounds__(kH_Threads, 1) conv_halo_stream_kernel(
    const __grid_constant__ CUtensorMap map_w_hi, const __grid_constant__ CUtensorMap map_w_lo,
    const __grid_constant__ CUtensorMap map_x_hi, const __grid_constant__ CUtensorMap map_x_lo,
    const ConvHaloParams p, const int total_tiles) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_a_full[kH_AStages], bar_a_empty[kH_AStages];
    __shared__ uint64_t bar_h_full[kH_HaloStages], bar_h_empty[kH_HaloStages];
    __shared__ uint64_t bar_tmem_full[2], bar_tmem_empty[2];
    __shared__ uint64_t bar_done;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag_s;
    // the layer's bias, read once: a load per stored row would put a trip to L2 in front of the add
    __shared__ float bias_s[kH_BiasSlots];
    volatile int *abort_flag = &abort_flag_s;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0)
        abort_flag_s = *reinterpret_cast<volatile uint32_t *>(p.flags + FLAG_TIMEOUT) != 0 ? 1 : 0;
    for (int c = threadIdx.x; c < kH_BiasSlots; c += kH_Threads)
        bias_s[c] = (p.bias && c < p.ko) ? p.bias[c] : 0.0f;
    __syncthreads();
    if (abort_flag_s)
        return;

    const uint32_t smem_base  = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t halo_base  = smem_base + kH_AStages * kH_AStageBytes;
    const uint32_t halo_stage = 2u * (uint32_t)p.halo_plane_bytes;
    uint8_t *epi_base = smem_raw + (smem_base - smem_u32(smem_raw)) + kH_AStages * kH_AStageBytes + kH_HaloStages * halo_stage;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kH_AStages; ++s) {
            mbar_init(smem_u32(&bar_a_full[s]), 1);
            mbar_init(smem_u32(&bar_a_empty[s]), 1);
        }
        for (int s = 0; s < kH_HaloStages; ++s) {
            mbar_init(smem_u32(&bar_h_full[s]), 1);
            mbar_init(smem_u32(&bar_h_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bar_tmem_full[b]), 1);
            mbar_init(smem_u32(&bar_tmem_empty[b]), kH_EpiWarps);
        }
        mbar_init(smem_u32(&bar_done), 1);
        mbar_fence_init();
        prefetch_tensormap(&map_w_hi);
        prefetch_tensormap(&map_w_lo);
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
    const int taps           = p.kh * p.kw;

    // tile -> (row tile of output channels, tile row, image): neighbouring CTAs take the row tiles
    // of one pixel tile, so they read the same halo out of L2
    auto coords = [&](int tile, int &tm, int &ty, int &img) {
        tm       = tile % p.tiles_m;
        int rest = tile / p.tiles_m;
        img      = rest / p.tiles_y;
        ty       = rest - img * p.tiles_y;
    };

    if (warp == 0) {
        // ===== TMA producer =====
        if (lane == 0) {
            int ka = 0, kh2 = 0; // filter k-blocks and halos issued so far
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                int tm, ty, img;
                coords(tile, tm, ty, img);
                for (int cb = 0; cb < p.cblocks && ok; ++cb, ++kh2) {
                    const int hs = kh2 % kH_HaloStages;
                    if (!mbar_wait(smem_u32(&bar_h_empty[hs]), ((uint32_t)(kh2 / kH_HaloStages) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t hfull = smem_u32(&bar_h_full[hs]);
                    const uint32_t hdst  = halo_base + (uint32_t)hs * halo_stage;
                    mbar_expect_tx(hfull, 2u * (uint32_t)p.box_bytes);
                    tma_load_4d(hdst, &map_x_hi, hfull, cb * kH_BlockK, -p.pad, ty * p.th - p.pad, img);
                    tma_load_4d(hdst + (uint32_t)p.halo_plane_bytes, &map_x_lo, hfull, cb * kH_BlockK, -p.pad,
                                ty * p.th - p.pad, img);
                    for (int tap = 0; tap < taps; ++tap, ++ka) {
                        const int s = ka % kH_AStages;
                        if (!mbar_wait(smem_u32(&bar_a_empty[s]), ((uint32_t)(ka / kH_AStages) & 1u) ^ 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        const uint32_t full = smem_u32(&bar_a_full[s]);
                        const uint32_t dst  = smem_base + (uint32_t)s * kH_AStageBytes;
                        mbar_expect_tx(full, (uint32_t)kH_AStageBytes);
                        const int32_t kc = tap * p.c_pad + cb * kH_BlockK;
                        tma_load_2d(dst, &map_w_hi, full, kc, tm * 128);
                        tma_load_2d(dst + kH_ABytes, &map_w_lo, full, kc, tm * 128);
                    }
                }
            }
            if (*abort_flag) {
                // unwind: let the copies still in flight land before the CTA goes away
                for (int k2 = ka - kH_AStages < 0 ? 0 : ka - kH_AStages; k2 < ka; ++k2) {
                    const uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(smem_u32(&bar_a_full[k2 % kH_AStages]), (uint32_t)(k2 / kH_AStages) & 1u) &&
                           globaltimer_ns() - t0 < kWaitBudgetNs) {
                    }
                }
                for (int k2 = kh2 - kH_HaloStages < 0 ? 0 : kh2 - kH_HaloStages; k2 < kh2; ++k2) {
                    const uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(smem_u32(&bar_h_full[k2 % kH_HaloStages]), (uint32_t)(k2 / kH_HaloStages) & 1u) &&
                           globaltimer_ns() - t0 < kWaitBudgetNs) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: accumulator buffer i & 1 for the CTA's i-th tile =====
        if (lane == 0) {
            const uint32_t idesc = make_idesc(2u, 128, (uint32_t)p.n_mma);
            int ka = 0, kh2 = 0, i = 0;
            bool ok = true;
            const long long t_start = CH_CLOCK();
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++i) {
                const int buf = i & 1;
                const long long t0 = CH_CLOCK();
                if (!mbar_wait(smem_u32(&bar_tmem_empty[buf]), (((uint32_t)i >> 1) & 1u) ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                CH_ACCUM(0, CH_CLOCK() - t0); // waiting for an accumulator
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)buf * 256u;
                bool first = true;
                for (int cb = 0; cb < p.cblocks && ok; ++cb, ++kh2) {
                    const int hs = kh2 % kH_HaloStages;
                    const long long t1 = CH_CLOCK();
                    if (!mbar_wait(smem_u32(&bar_h_full[hs]), (uint32_t)(kh2 / kH_HaloStages) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    CH_ACCUM(1, CH_CLOCK() - t1); // waiting for a halo
                    const uint32_t x_hi = halo_base + (uint32_t)hs * halo_stage;
                    const uint32_t x_lo = x_hi + (uint32_t)p.halo_plane_bytes;
                    int tap = 0;
                    for (int r = 0; r < p.kh && ok; ++r) {
                        for (int sx = 0; sx < p.kw; ++sx, ++tap, ++ka) {
                            const int s = ka % kH_AStages;
                            const long long t2 = CH_CLOCK();
                            if (!mbar_wait(smem_u32(&bar_a_full[s]), (uint32_t)(ka / kH_AStages) & 1u, abort_flag)) {
                                ok = false;
                                break;
                            }
                            CH_ACCUM(2, CH_CLOCK() - t2); // waiting for filter planes
                            tc_fence_after_sync();
                            const uint32_t a_hi = smem_base + (uint32_t)s * kH_AStageBytes, a_lo = a_hi + kH_ABytes;
                            // the tap's pixels: the halo, (r * pw + sx) rows of 64 bytes further on
                            const uint32_t shift = (uint32_t)(r * p.pw + sx) * (uint32_t)kH_RowB;
                            const uint64_t da_hi = smem_desc_k<kH_RowB>(a_hi), da_lo = smem_desc_k<kH_RowB>(a_lo);
                            const uint64_t db_hi = smem_desc_k<kH_RowB>(x_hi + shift), db_lo = smem_desc_k<kH_RowB>(x_lo + shift);
#pragma unroll
                            for (int kk = 0; kk < kH_RowB / 32; ++kk) {
                                const uint64_t adv = (uint64_t)(kk * 32 >> 4);
                                mma_tf32(d_tmem, da_lo + adv, db_hi + adv, idesc, first ? 0u : 1u);
                                mma_tf32(d_tmem, da_hi + adv, db_lo + adv, idesc, 1u);
                                mma_tf32(d_tmem, da_hi + adv, db_hi + adv, idesc, 1u);
                                first = false;
                            }
                            tc_commit(smem_u32(&bar_a_empty[s]));
                        }
                    }
                    if (ok)
                        tc_commit(smem_u32(&bar_h_empty[hs])); // the halo is free once its taps' MMAs have retired
                }
                if (ok)
                    tc_commit(smem_u32(&bar_tmem_full[buf]));
            }
            CH_ACCUM(3, CH_CLOCK() - t_start); // the MMA thread's whole loop
            CH_ACCUM(4, i);
            if (!ok || *abort_flag) {
                tc_commit(smem_u32(&bar_done));
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(smem_u32(&bar_done), 0) && globaltimer_ns() - t0 < kWaitBudgetNs) {
                }
            }
        }
    } else {
        // ===== epilogue: drain tile i to registers, release the accumulator, then store =====
        const int ew      = warp - 2;
        const int quarter = warp & 3;
        const int half    = ew >> 2;
        uint8_t *stg      = epi_base + (uint32_t)ew * kH_EpiWarpBytes;
        const int sub = lane & 15, rr = lane >> 4;
        // where this lane's columns land: column col = half * 128 + h2 * 64 + sub * 4 + q is position
        // (y, x) = (col / pw, col % pw); -1 for the halo columns and past the tile
        int off[2][4];
        const int npos = p.th * p.pw;
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int col = half * 128 + h2 * 64 + sub * 4 + q;
                const int y = col / p.pw, x = col - y * p.pw;
                off[h2][q] = (col < npos && x < p.wo) ? y * p.wo + x : -1;
            }
        const int col_base = half * 128 + sub * 4;
        int i = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++i) {
            int tm, ty, img;
            coords(tile, tm, ty, img);
            const int buf = i & 1;
            const long long e0 = CH_CLOCK();
            bool got = mbar_wait(smem_u32(&bar_tmem_full[buf]), ((uint32_t)i >> 1) & 1u, abort_flag);
            if (!__all_sync(0xffffffffu, got))
                break;
            const long long e1 = CH_CLOCK();
            tc_fence_after_sync();
            float acc[128];
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * 256 + half * 128);
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

            const int row0 = tm * 128 + quarter * 32; // first output channel of this warp's block
            const int y0   = ty * p.th;
            // positions of rows past the image's last row (a partial last tile) are dropped:
            // position col lies in row col / pw, so the valid ones are col < rows_left * pw
            const int col_limit = (p.ho - y0 < p.th ? p.ho - y0 : p.th) * p.pw;
            float *out_img = p.out + ((int64_t)img * p.ko) * p.ho * p.wo + (int64_t)y0 * p.wo;
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                if (half * 128 + h2 * 64 >= npos)
                    break;
                float4 *mine = reinterpret_cast<float4 *>(stg + lane * kH_EpiRowBytes);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    mine[j] = make_float4(acc[h2 * 64 + 4 * j], acc[h2 * 64 + 4 * j + 1], acc[h2 * 64 + 4 * j + 2],
                                          acc[h2 * 64 + 4 * j + 3]);
                __syncwarp();
#pragma unroll 4
                for (int it = 0; it < 16; ++it) {
                    const int r_in = it * 2 + rr; // channel within the warp's 32
                    const int ch   = row0 + r_in;
                    if (ch < p.ko) {
                        const float4 q4 = *reinterpret_cast<const float4 *>(stg + r_in * kH_EpiRowBytes + sub * 16);
                        const float v[4] = {q4.x, q4.y, q4.z, q4.w};
                        const float b    = ch < kH_BiasSlots ? bias_s[ch] : (p.bias ? p.bias[ch] : 0.0f);
                        float *plane     = out_img + (int64_t)ch * p.ho * p.wo;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (off[h2][q] >= 0 && col_base + h2 * 64 + q < col_limit) {
                                float x = v[q];
                                if (p.bias)
                                    x = __fadd_rn(x, b);
                                if (p.act == CT_ACT_RELU)
                                    x = __fmul_rn(x, x > 0.0f ? 1.0f : 0.0f);
                                plane[off[h2][q]] = x;
                            }
                        }
                    }
                }
                __syncwarp(); // the block is rewritten by the next half / tile
            }
            if (warp == 2 && lane == 0) {
                CH_ACCUM(5, e1 - e0);          // epilogue: waiting for a complete accumulator
                CH_ACCUM(6, CH_CLOCK() - e1);  // drain and store
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

struct HaloGeom {
    int pw, wo, ho, th, n_mma, box_rows, plane_bytes;
    size_t smem;
};

bool halo_geometry(int64_t h, int64_t w, int64_t kh, int64_t kw, int64_t pad, HaloGeom *g) {
    const int64_t pw = w + 2 * pad, wo = pw - kw + 1, ho = h + 2 * pad - kh + 1;
    if (wo < 1 || ho < 1 || pw > 256)
        return false;
    int64_t th = 256 / pw;
    if (th > ho)
        th = ho;
    if (th < 1 || th + kh - 1 > 256)
        return false;
    g->pw = (int)pw, g->wo = (int)wo, g->ho = (int)ho, g->th = (int)th;
    g->n_mma    = (int)((th * pw + 15) / 16 * 16);
    g->box_rows = (int)(th + kh - 1);
    // a tap's shifted window of n_mma rows may run past the box: reserve those rows too
    int64_t rows = (kh - 1) * pw + (kw - 1) + g->n_mma;
    if (rows < (int64_t)g->box_rows * pw)
        rows = (int64_t)g->box_rows * pw;
    g->plane_bytes = (int)((rows * kH_RowB + 1023) & ~1023ll);
    g->smem = (size_t)kH_AStages * kH_AStageBytes + (size_t)kH_HaloStages * 2 * g->plane_bytes + kH_EpiBytes + 1024;
    return g->smem <= 225 * 1024; // 227 KB per CTA less the kernel's static shared memory
}

} // namespace

// Whether the halo kernel takes this layer (3xTF32 only): stride 1, more than 64 filters (fewer go
// to the kernels that put pixels on the rows or filters in tensor memory), a k range short enough
// for one accumulation, and a tile that is reasonably full.
bool conv_halo_applicable(int64_t c_pad, int64_t h, int64_t w, int64_t ko, int64_t kh, int64_t kw, int64_t stride,
                          int64_t pad) {
    HaloGeom g;
    if (stride != 1 || ko <= 64 || kh * kw * c_pad > 1024 || (c_pad % kH_BlockK) != 0)
        return false;
    if (!halo_geometry(h, w, kh, kw, pad, &g))
        return false;
    return (int64_t)g.th * g.wo * 10 >= (int64_t)g.n_mma * 7; // at least 70 % of the columns carry an output
}

// w_hi / w_lo: filter planes [ko][taps * c_pad] (tap-major k); x_hi / x_lo: NHWC planes [batch][h][w][c_pad].
ct_status conv_halo_stream(
    DeviceState *st, const void *w_hi, const void *w_lo, const void *x_hi, const void *x_lo, int64_t batch,
    int64_t c_pad, int64_t h, int64_t wd, int64_t ko, int64_t kh, int64_t kw, int64_t pad, const float *bias, int act,
    float *out) {
    HaloGeom g;
    if (!halo_geometry(h, wd, kh, kw, pad, &g))
        return fail(CT_ERR_INVALID, "conv2d: internal tile shape not usable");
    ConvHaloParams p;
    p.bias = bias, p.out = out, p.flags = st->flags_dev;
    p.ko = (int)ko, p.tiles_m = (int)((ko + 127) / 128);
    p.kh = (int)kh, p.kw = (int)kw, p.pad = (int)pad;
    p.ho = g.ho, p.wo = g.wo, p.pw = g.pw, p.th = g.th;
    p.tiles_y = (g.ho + g.th - 1) / g.th;
    p.cblocks = (int)(c_pad / kH_BlockK);
    p.c_pad   = (int)c_pad;
    p.n_mma   = g.n_mma;
    p.box_bytes        = g.box_rows * g.pw * kH_RowB;
    p.halo_plane_bytes = g.plane_bytes;
    p.act = act;
    const int64_t tiles = (int64_t)p.tiles_m * p.tiles_y * batch;
    if (tiles > 0x7fffffffll)
        return fail(CT_ERR_TOO_LARGE, "conv2d: too many tiles");
    CUtensorMap mw_hi, mw_lo, mx_hi, mx_lo;
    const uint64_t kp = (uint64_t)(kh * kw * c_pad);
    const uint64_t wdims[2] = {kp, (uint64_t)ko}, wstr[1] = {kp * 4};
    const uint32_t wbox[2]  = {kH_BlockK, 128};
    CT_TRY(encode_tiled_map_f32(&mw_hi, w_hi, 2, wdims, wstr, wbox, kH_RowB));
    CT_TRY(encode_tiled_map_f32(&mw_lo, w_lo, 2, wdims, wstr, wbox, kH_RowB));
    const uint64_t row = (uint64_t)c_pad * 4;
    const uint64_t xdims[4] = {(uint64_t)c_pad, (uint64_t)wd, (uint64_t)h, (uint64_t)batch};
    const uint64_t xstr[3]  = {row, row * (uint64_t)wd, row * (uint64_t)wd * (uint64_t)h};
    const uint32_t xbox[4]  = {kH_BlockK, (uint32_t)g.pw, (uint32_t)g.box_rows, 1};
    CT_TRY(encode_tiled_map_f32(&mx_hi, x_hi, 4, xdims, xstr, xbox, kH_RowB));
    CT_TRY(encode_tiled_map_f32(&mx_lo, x_lo, 4, xdims, xstr, xbox, kH_RowB));
    // the kernel also has a little static shared memory (barriers, the bias): ask for exactly what
    // this geometry needs, remembering the largest request per device
    static size_t attr_bytes_dev[16] = {};
    size_t &attr_bytes = attr_bytes_dev[st->device & 15];
    if (g.smem > attr_bytes) {
        CT_CUDA(cudaFuncSetAttribute(conv_halo_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem));
        attr_bytes = g.smem;
    }
    const unsigned grid = (unsigned)(tiles < st->sm_count ? tiles : st->sm_count);
    ProfScope prof("gemm_tc");
    conv_halo_stream_kernel<<<grid, kH_Threads, g.smem, stream()>>>(mw_hi, mw_lo, mx_hi, mx_lo, p, (int)tiles);
    CT_LAUNCH_CHECK("conv_halo_stream");
    return CT_OK;
}

} // namespace ct
