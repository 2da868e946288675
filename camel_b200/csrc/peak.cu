// Measured ceiling of the tensor pipe for the roofline of the contraction kernels.
//
// One CTA per SM issues tcgen05.mma (128 x 256 x 32 bytes of k) back to back on operand tiles that
// already sit in shared memory - no TMA, no global memory, no epilogue in the loop - so the time of
// a launch is the time the tensor pipe needs for that many MMAs and nothing else.  The GEMM and
// conv kernels issue exactly this instruction shape; what they reach is reported against this
// number (divided by three for the 3xTF32 scheme, which spends three MMAs per product).
#include "common.cuh"
#include "tc_ptx.cuh"

namespace ct {
namespace {

using namespace ptx;

constexpr int kPeakBN      = 256;
constexpr int kPeakRowB    = 128;
constexpr int kPeakABytes  = 128 * kPeakRowB;
constexpr int kPeakBBytes  = kPeakBN * kPeakRowB;
constexpr int kPeakShiftMax = 16;                                   // B tiles may be read from up to 16 rows further on
constexpr int kPeakOperands = 2 * (kPeakABytes + kPeakBBytes) + kPeakShiftMax * kPeakRowB + 1024; // two operand sets, alternated
constexpr int kPeakSmem     = kPeakOperands > 120 * 1024 ? kPeakOperands : 120 * 1024; // more than half of an SM's shared
                                                                                        // memory: never two CTAs on one SM
constexpr int kPeakThreads = 128;

// SM cycles and nanoseconds that the MMA loop of the launch's first CTA took (the last launch wins):
// cycles / MMA is the pipe's rate in the clock domain it runs in, cycles / ns the SM clock the loop
// really ran at, whatever a sampled clock reading says.
__device__ unsigned long long g_peak_stamp[2];

// kind: 0 = kind::tf32, 1 = kind::f16 with bf16 operands
template <int KIND>
__global__ void __launch_bounds__(kPeakThreads, 1) mma_peak_kernel(
    int mma_groups, uint32_t *status, int mma_m, int mma_n, int b_row_shift, int a_in_tmem) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_done;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag_s;
    const int warp = threadIdx.x >> 5;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *base            = smem_raw + (smem_base - smem_u32(smem_raw));

    // Operand values: a fixed pattern of finite numbers in (-1, 1).  Their arrangement in the
    // swizzled tile is irrelevant here (no result is read), their being non-zero is not: an
    // all-zero operand draws less power and would flatter the sustained figure.
    for (int i = threadIdx.x; i < (2 * (kPeakABytes + kPeakBBytes) + kPeakShiftMax * kPeakRowB) / 4; i += kPeakThreads) {
        uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
        float v    = ((h >> 9) & 0xffff) * (1.0f / 32768.0f) - 1.0f;
        if (KIND == 0) {
            // tf32 values, as every kernel here feeds the pipe (the split rounds both parts to tf32):
            // the 13 low mantissa bits are zero
            reinterpret_cast<float *>(base)[i] = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
        } else {
            uint32_t b = __float_as_uint(v) >> 16; // the value truncated to bf16
            reinterpret_cast<uint32_t *>(base)[i] = b | (b << 16);
        }
    }
    if (threadIdx.x == 0) {
        abort_flag_s = 0;
        mbar_init(smem_u32(&bar_done), 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), 2 * kPeakBN);
        tmem_relinquish();
    }
    // make the generic-proxy writes of the operand tiles visible to the tensor core's async proxy
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 1 && (threadIdx.x & 31) == 0) {
        const uint32_t idesc = make_idesc(KIND == 0 ? 2u : 1u, (uint32_t)mma_m, (uint32_t)mma_n);
        const long long c0   = clock64();
        const uint64_t n0    = globaltimer_ns();
        for (int g = 0; g < mma_groups; ++g) {
            const uint32_t set = smem_base + (uint32_t)(g & 1) * (kPeakABytes + kPeakBBytes);
            const uint64_t da = smem_desc_k<kPeakRowB>(set);
            const uint64_t db = smem_desc_k<kPeakRowB>(set + kPeakABytes + (uint32_t)b_row_shift * kPeakRowB);
            // A from tensor memory: one accumulator (columns 0..255), the A tiles in columns 256..
            const uint32_t d  = tmem_base + (a_in_tmem ? 0u : (uint32_t)((g >> 1) & 1) * kPeakBN);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) { // four k-steps of 32 bytes per 128-byte operand row
                const uint64_t adv = (uint64_t)(kk * 32 >> 4);
                const uint32_t acc = g < 2 && kk == 0 ? 0u : 1u;
                if (KIND == 0 && a_in_tmem) {
                    asm volatile(
                        "{\n\t"
                        ".reg .pred p;\n\t"
                        "setp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t"
                        "}\n"
                        :
                        : "r"(d), "r"(tmem_base + 256u + (uint32_t)(((g & 7) * 4 + kk) * 8)), "l"(db + adv), "r"(idesc), "r"(acc)
                        : "memory");
                } else if (KIND == 0) {
                    mma_tf32(d, da + adv, db + adv, idesc, acc);
                } else {
                    mma_f16(d, da + adv, db + adv, idesc, acc);
                }
            }
        }
        tc_commit(smem_u32(&bar_done));
        if (!mbar_wait(smem_u32(&bar_done), 0, &abort_flag_s))
            atomicExch(status, 1u + blockIdx.x);
        if (blockIdx.x == 0) {
            g_peak_stamp[0] = (unsigned long long)(clock64() - c0);
            g_peak_stamp[1] = (unsigned long long)(globaltimer_ns() - n0);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 2 * kPeakBN);
    }
}

} // namespace
} // namespace ct

using namespace ct;

// Runs `launches` back-to-back launches of the MMA loop (mma_groups x 4 MMAs of 128 x 256 x 8
// (tf32) or 128 x 256 x 16 (bf16) per CTA, one CTA per SM), timed with CUDA events on the current
// stream.  *tflops_host = dense MMA rate over the whole timed region; *ms_host its duration.
// A launch also pays its set-up (operand fill, TMEM allocation, launch latency: some 15 us), so
// the pipe's own rate is the difference quotient of two launch sizes, (flop(g2) - flop(g1)) /
// (t(g2) - t(g1)); the caller forms it from two calls.
extern "C" ct_status ct_measure_mma_peak(
    ct_precision kind, int mma_groups, int launches, double *tflops_host, double *ms_host) {
    return ct_measure_mma_rate(kind, 128, kPeakBN, mma_groups, launches, tflops_host, ms_host);
}

// The same loop with another MMA shape (m = 64 or 128 rows, n = 16..256 columns in steps of 16):
// how the pipe's rate depends on the shape a kernel can give it.  A layer with 64 output channels
// cannot fill 256 columns; what its kernel reaches has to be read against the rate of its shape.
extern "C" ct_status ct_measure_mma_rate(
    ct_precision kind, int mma_m, int mma_n, int mma_groups, int launches, double *tflops_host, double *ms_host) {
    return ct_measure_mma_rate_shifted(kind, mma_m, mma_n, 0, mma_groups, launches, tflops_host, ms_host);
}

// ... and with the B tile read from b_row_shift rows (of 128 bytes) past a swizzle-aligned start:
// what an implicit-GEMM convolution does when it addresses a filter tap's pixels inside one halo
// box through a moved descriptor.
extern "C" ct_status ct_measure_mma_rate_shifted(
    ct_precision kind, int mma_m, int mma_n, int b_row_shift, int mma_groups, int launches, double *tflops_host,
    double *ms_host) {
    // b_row_shift + 256: the A operand comes from tensor memory instead of shared memory (tf32 only)
    const int a_in_tmem = b_row_shift >= 256 ? 1 : 0;
    b_row_shift -= 256 * a_in_tmem;
    if (a_in_tmem && kind != CT_PREC_3XTF32)
        return fail(CT_ERR_INVALID, "ct_measure_mma_rate_shifted: A from tensor memory is measured for tf32 only");
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (mma_groups < 2 || mma_groups > (1 << 20) || launches < 1 || launches > (1 << 20))
        return fail(CT_ERR_INVALID, "ct_measure_mma_peak: mma_groups in [2, 2^20], launches in [1, 2^20]");
    if (kind != CT_PREC_3XTF32 && kind != CT_PREC_BF16)
        return fail(CT_ERR_INVALID, "ct_measure_mma_peak: unknown kind");
    if (b_row_shift < 0 || b_row_shift > kPeakShiftMax)
        return fail(CT_ERR_INVALID, "ct_measure_mma_rate_shifted: shift of 0 to %d rows", kPeakShiftMax);
    if ((mma_m != 64 && mma_m != 128) || mma_n < 16 || mma_n > kPeakBN || (mma_n & 15) != 0)
        return fail(CT_ERR_INVALID, "ct_measure_mma_rate: m must be 64 or 128, n a multiple of 16 up to %d", kPeakBN);
    // the in-kernel wait for the last MMA is bounded by one second: keep a launch far below that
    if ((double)mma_groups * 4 * 70e-9 > 0.25)
        return fail(CT_ERR_TOO_LARGE, "ct_measure_mma_peak: a launch of %d MMA groups would run too long", mma_groups);
    auto kernel = kind == CT_PREC_3XTF32 ? mma_peak_kernel<0> : mma_peak_kernel<1>;
    CT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem));
    CT_CUDA(cudaMemsetAsync(st->flags_dev + 3, 0, sizeof(uint32_t), stream()));
    cudaEvent_t e0, e1;
    CT_CUDA(cudaEventCreate(&e0));
    CT_CUDA(cudaEventCreate(&e1));
    kernel<<<st->sm_count, kPeakThreads, kPeakSmem, stream()>>>(mma_groups, st->flags_dev + 3, mma_m, mma_n, b_row_shift, a_in_tmem); // warm-up
    CT_LAUNCH_CHECK("mma_peak");
    CT_CUDA(cudaEventRecord(e0, stream()));
    for (int i = 0; i < launches; ++i) {
        kernel<<<st->sm_count, kPeakThreads, kPeakSmem, stream()>>>(mma_groups, st->flags_dev + 3, mma_m, mma_n, b_row_shift, a_in_tmem);
        CT_LAUNCH_CHECK("mma_peak");
    }
    CT_CUDA(cudaEventRecord(e1, stream()));
    CT_CUDA(cudaEventSynchronize(e1));
    float ms = 0.0f;
    CT_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    uint32_t bad = 0;
    CT_CUDA(cudaMemcpy(&bad, st->flags_dev + 3, sizeof(bad), cudaMemcpyDeviceToHost));
    if (bad)
        return fail(CT_ERR_TIMEOUT, "ct_measure_mma_peak: the wait for the last MMA ran out (block %u)", bad - 1);
    const double k_per_mma = kind == CT_PREC_3XTF32 ? 8.0 : 16.0;
    const double flop = 2.0 * mma_m * mma_n * k_per_mma * 4.0 * mma_groups * (double)st->sm_count * launches;
    if (tflops_host)
        *tflops_host = ms > 0 ? flop / (ms * 1e-3) / 1e12 : 0.0;
    if (ms_host)
        *ms_host = ms;
    return CT_OK;
}

// The pipe's rate in its own clock domain: SM cycles per MMA of the given shape (difference
// quotient of two launch sizes, so that the loop's set-up and the final wait cancel) and the SM
// clock the loops really ran at (cycles / nanoseconds of the longer launch, both stamped inside
// the kernel).  flop per clock and SM = 2 * mma_m * mma_n * k / clocks_per_mma with k = 8 (tf32) or
// 16 (bf16); times the SM count and a clock it gives the ceiling at that clock, which is what a
// kernel timed under a power cap has to be read against.
extern "C" ct_status ct_measure_mma_clocks(
    ct_precision kind, int mma_m, int mma_n, double *clocks_per_mma_host, double *sm_mhz_host) {
    const int groups[2] = {200, 800};
    double cycles[2] = {0, 0}, ns[2] = {0, 0};
    for (int i = 0; i < 2; ++i) {
        double best = 0;
        for (int rep = 0; rep < 3; ++rep) {
            CT_TRY(ct_measure_mma_rate(kind, mma_m, mma_n, groups[i], 1, nullptr, nullptr));
            unsigned long long stamp[2];
            CT_CUDA(cudaMemcpyFromSymbol(stamp, g_peak_stamp, sizeof(stamp)));
            if (rep == 0 || (double)stamp[0] < best) {
                best      = (double)stamp[0];
                cycles[i] = (double)stamp[0];
                ns[i]     = (double)stamp[1];
            }
        }
    }
    if (clocks_per_mma_host)
        *clocks_per_mma_host = (cycles[1] - cycles[0]) / (4.0 * (groups[1] - groups[0]));
    if (sm_mhz_host)
        *sm_mhz_host = ns[1] > 0 ? cycles[1] / ns[1] * 1e3 : 0.0;
    return CT_OK;
}
