// Inline-PTX wrappers for the sm_100a features the contraction kernels use: mbarriers with
// BOUNDED waits, TMA tile loads (cp.async.bulk.tensor; every CTA fetches its own tiles), tensor memory (TMEM)
// allocation, tcgen05.mma / commit / ld, and the shared-memory matrix descriptors.
#pragma once

#include <cstdint>

namespace ct {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// The same with a time limit for the hardware's own suspension of the thread: a waiting thread
// sleeps until the phase completes (it is woken at once then) or the limit passes, instead of
// coming back after the much shorter system default and polling again.  For roles whose waits are
// long and whose polling would take issue slots from the warps that have work.
__device__ __forceinline__ bool mbar_try_wait_for(uint32_t bar, uint32_t parity, uint32_t limit_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(limit_ns)
        : "memory");
    return ok != 0;
}

// Wait budget of one barrier wait.  A healthy kernel waits microseconds; the budget only
// exists so that a protocol bug ends as an error status instead of a hung GPU.
constexpr uint64_t kWaitBudgetNs = 1000ull * 1000ull * 1000ull; // 1 s

// Bounded wait.  Returns false when the budget ran out or when another role has already
// given up (*abort_flag != 0); in the first case it raises *abort_flag itself.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity))
        return true;
    uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((it & 63u) == 0) {
            if (*abort_flag)
                return false;
            if (globaltimer_ns() - t0 > kWaitBudgetNs) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// Bounded wait for the patient roles (see mbar_try_wait_for): same contract as mbar_wait.
__device__ __forceinline__ bool mbar_wait_patient(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity))
        return true;
    uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait_for(bar, parity, 20000u))
            return true;
        if (*abort_flag)
            return false;
        if (globaltimer_ns() - t0 > kWaitBudgetNs) {
            *abort_flag = 1;
            return false;
        }
    }
}

// ---- TMA --------------------------------------------------------------------------------

__device__ __forceinline__ void prefetch_tensormap(const void *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tile load global -> shared of THIS CTA, completion counted on an mbarrier of this CTA.
// c0 is the innermost (contiguous) coordinate and must make a 16-byte aligned start.
__device__ __forceinline__ void tma_load_2d(
    uint32_t dst_smem, const void *map, uint32_t bar, int32_t c0, int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(
    uint32_t dst_smem, const void *map, uint32_t bar, int32_t c0, int32_t c1, int32_t c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        :
        : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// Only c0 carries the 16-byte alignment rule; c1..c3 may be negative or past the end (the
// out-of-range part of the box reads as zero), which is how a convolution's halo is fetched.
__device__ __forceinline__ void tma_load_4d(
    uint32_t dst_smem, const void *map, uint32_t bar, int32_t c0, int32_t c1, int32_t c2, int32_t c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        :
        : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2),
          "r"(c3)
        : "memory");
}

// ---- tensor memory ----------------------------------------------------------------------

// Whole-warp instructions (.sync.aligned): call from all 32 lanes of one warp.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Makes the mbarrier track completion of all MMAs this thread issued so far.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues.  accumulate == 0 overwrites D.
__device__ __forceinline__ void mma_tf32(
    uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_f16(
    uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- descriptors ------------------------------------------------------------------------

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with
// the 128-byte swizzle (what a TMA box of 128-byte rows with SWIZZLE_128B writes): 8-row groups
// 1024 bytes apart.  Fields (bit positions): start address >> 4 [0,14), leading byte offset
// >> 4 [16,30) (unused for swizzled K-major, 1), stride byte offset >> 4 [32,46) = 64,
// descriptor version 1 [46,48), layout type SWIZZLE_128B = 2 [61,64).
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Same for tiles whose rows are ROW_BYTES = 128 or 64 bytes wide, written by TMA with the
// matching swizzle (SWIZZLE_128B: layout type 2, SWIZZLE_64B: layout type 4); 8-row groups are
// 8 * ROW_BYTES apart.
template <int ROW_BYTES> __device__ __forceinline__ uint64_t smem_desc_k(uint32_t smem_addr) {
    static_assert(ROW_BYTES == 128 || ROW_BYTES == 64, "operand rows are 128 or 64 bytes");
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((8 * ROW_BYTES) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(ROW_BYTES == 128 ? 2 : 4) << 61;
    return d;
}

// Instruction descriptor, dense, float32 accumulator, both operands K-major.
// ab_format: 0 f16, 1 bf16, 2 tf32.  Fields: c format [4,6) = 1 (f32), a format [7,10),
// b format [10,13), n >> 3 [17,23), m >> 4 [24,29).
__host__ __device__ constexpr uint32_t make_idesc(uint32_t ab_format, uint32_t m, uint32_t n) {
    return (1u << 4) | (ab_format << 7) | (ab_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

} // namespace ptx
} // namespace ct
