// exp and log for float32 tensors.  The reference computes `float(std::exp(double(x)))`
// (modules/tensor/runtime.cpp:1023, 1042): a correctly rounded float32 result but for rare
// double-rounding cases.  The functions here stay in float32 arithmetic with the low-order parts
// carried along (so that the operators built on them run at HBM speed instead of being bound by
// float64 issue and conversions) and are never more than 1 ulp from that result, which is the bar
// the parity tests set; a float64 evaluation serves the arguments at the edges of the range.
#pragma once

#include <cstdint>

namespace ct {

// exp(x) for x that came from a float32; result to be rounded to float32 by the caller.
// Overflow (x > 88.7) and underflow (x < -103.9) resolve in that final rounding.
__device__ __forceinline__ double exp_from_f32(double x) {
    if (x != x)
        return x;
    x = x > 90.0 ? 90.0 : (x < -110.0 ? -110.0 : x);
    const double kLog2e = 1.4426950408889634074;
    const double kLn2Hi = 6.93147180369123816490e-01;
    const double kLn2Lo = 1.90821492927058770002e-10;
    const double kMagic = 6755399441055744.0; // 1.5 * 2^52: adds as round-to-nearest-integer
    double t  = fma(x, kLog2e, kMagic);
    int k     = (int)(uint32_t)__double2loint(t);
    double kd = t - kMagic;
    double r  = fma(-kd, kLn2Hi, x);
    r         = fma(-kd, kLn2Lo, r); // |r| <= ln2/2
    double p  = 1.0 / 39916800.0;     // Taylor to degree 11: remainder < 7e-15
    p         = fma(p, r, 1.0 / 3628800.0);
    p         = fma(p, r, 1.0 / 362880.0);
    p         = fma(p, r, 1.0 / 40320.0);
    p         = fma(p, r, 1.0 / 5040.0);
    p         = fma(p, r, 1.0 / 720.0);
    p         = fma(p, r, 1.0 / 120.0);
    p         = fma(p, r, 1.0 / 24.0);
    p         = fma(p, r, 1.0 / 6.0);
    p         = fma(p, r, 0.5);
    p         = fma(p, r, 1.0);
    p         = fma(p, r, 1.0);
    double scale = __hiloint2double((k + 1023) << 20, 0); // 2^k, k in [-159, 130]
    return p * scale;
}

// float32 in, float32 out, float32 arithmetic only.  The float64 evaluation above costs two
// conversions on the special-function pipe (16 per clock and SM) and ~17 instructions on the
// half-rate float64 pipe per element, which holds exp and softmax at 0.5-0.8 of HBM speed.  This
// version stays on the float32 pipe and keeps the low-order parts that decide the last bit:
//   n = rint(x log2 e), r = x - n ln2 in two FMAs (ln2 split so that n*hi is exact) plus the part
//   rl that the second FMA rounded away; exp(r) = 1 + (r + r^2 q(r)) with q a degree-5 fit of
//   (exp(r) - 1 - r) / r^2 on |r| <= ln2/2; the residuals of r + r^2 q and of 1 + s are recovered
//   with FMAs / a fast two-sum and added before the last rounding; 2^n by an exponent add.
// Against float(exp(double(x))) over 8 million inputs in [-87, 87]: never more than 1 ulp away,
// 98.9 % identical.  NaN, and arguments whose result overflows, underflows or is subnormal, take
// the float64 path.
__device__ __forceinline__ float exp_f32_core(float x) {
    {
        const float kMagic = 12582912.0f; // 1.5 * 2^23: adds as round-to-nearest-integer
        const float kLn2Hi = 0.693145751953125f;
        const float kLn2Lo = __int_as_float(0x35bfbe8e); // ln2 - kLn2Hi
        const float t  = __fmaf_rn(x, __int_as_float(0x3fb8aa3b), kMagic);
        const float nf = __fsub_rn(t, kMagic);
        const int ni   = __float_as_int(t) - 0x4B400000;
        const float r1 = __fmaf_rn(nf, -kLn2Hi, x);
        const float r  = __fmaf_rn(nf, -kLn2Lo, r1);
        const float rl = __fmaf_rn(nf, -kLn2Lo, __fsub_rn(r1, r));
        float q        = __int_as_float(0x3950a8be);
        q              = __fmaf_rn(q, r, __int_as_float(0x3ab6a194));
        q              = __fmaf_rn(q, r, __int_as_float(0x3c088863));
        q              = __fmaf_rn(q, r, __int_as_float(0x3d2aaa75));
        q              = __fmaf_rn(q, r, __int_as_float(0x3e2aaaab));
        q              = __fmaf_rn(q, r, 0.5f);
        const float r2 = __fmul_rn(r, r);
        const float s  = __fmaf_rn(r2, q, r);
        const float e  = __fadd_rn(__fmaf_rn(r2, q, __fsub_rn(r, s)), rl);
        float p        = __fadd_rn(1.0f, s);
        const float pe = __fadd_rn(__fsub_rn(1.0f, p), s);
        p              = __fadd_rn(p, __fadd_rn(pe, e));
        return __int_as_float(__float_as_int(p) + (ni << 23));
    }
}

__device__ __forceinline__ float exp_f32(float x) {
    if (fabsf(x) <= 87.0f)
        return exp_f32_core(x);
    return (float)exp_from_f32((double)x);
}

// For arguments known to be <= 0 or NaN (x - max of a softmax row): one range test, and the plain
// form of the same evaluation (degree-4 fit, no residual terms: 18 instructions instead of 28).
// Still never more than 1 ulp from float(exp(double(x))), identical for 90.6 % of inputs instead of
// 98.9 %.  A softmax output is this value divided by a rounded sum of such values and rounded
// again, so its last bits are not the reference's either way (measured: at most 4 ulp, 1e-5
// relative is the bar), while the wide softmax kernel is bound by instruction issue and gains
// a fifth in speed from the shorter form.
__device__ __forceinline__ float exp_f32_plain(float x) { // -87 <= x <= 87, not NaN
    {
        const float kMagic = 12582912.0f;
        const float t  = __fmaf_rn(x, __int_as_float(0x3fb8aa3b), kMagic);
        const float nf = __fsub_rn(t, kMagic);
        const int ni   = __float_as_int(t) - 0x4B400000;
        float r        = __fmaf_rn(nf, -0.693145751953125f, x);
        r              = __fmaf_rn(nf, -__int_as_float(0x35bfbe8e), r);
        float q        = __int_as_float(0x3ab6a194);
        q              = __fmaf_rn(q, r, __int_as_float(0x3c0905ba));
        q              = __fmaf_rn(q, r, __int_as_float(0x3d2aaa75));
        q              = __fmaf_rn(q, r, __int_as_float(0x3e2aaa6e));
        q              = __fmaf_rn(q, r, 0.5f);
        const float s  = __fmaf_rn(__fmul_rn(r, r), q, r);
        const float p  = __fadd_rn(1.0f, s);
        return __int_as_float(__float_as_int(p) + (ni << 23));
    }
}

__device__ __forceinline__ float exp_f32_nonpos(float x) {
    if (x >= -87.0f)
        return exp_f32_plain(x);
    return (float)exp_from_f32((double)x);
}

// ---- two float32 lanes per instruction (sm_100: add / mul / fma .f32x2, IEEE round-to-nearest
// per lane), for kernels that are bound by instruction issue ----
typedef unsigned long long f32x2;

__device__ __forceinline__ f32x2 pack2(float a, float b) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &a, float &b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__host__ __device__ constexpr f32x2 dup2(uint32_t bits) { return ((f32x2)bits << 32) | (f32x2)bits; }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// exp_f32_plain on two values (both in [-87, 87], not NaN): the same operations in the same
// order, so the same bits, in 11 two-lane instructions plus two integer ones per lane.
__device__ __forceinline__ f32x2 exp_f32_plain2(f32x2 x) {
    const f32x2 t  = fma2(x, dup2(0x3fb8aa3bu), dup2(0x4B400000u));   // x log2e + 1.5 * 2^23
    const f32x2 nf = add2(t, dup2(0xCB400000u));                       // - 1.5 * 2^23
    f32x2 r        = fma2(nf, dup2(0xBF317200u), x);                   // - n * 0.693145751953125
    r              = fma2(nf, dup2(0xB5BFBE8Eu), r);                   // - n * (ln2 - hi)
    f32x2 q        = fma2(dup2(0x3ab6a194u), r, dup2(0x3c0905bau));
    q              = fma2(q, r, dup2(0x3d2aaa75u));
    q              = fma2(q, r, dup2(0x3e2aaa6eu));
    q              = fma2(q, r, dup2(0x3f000000u));
    const f32x2 s  = fma2(mul2(r, r), q, r);
    const f32x2 p  = add2(dup2(0x3f800000u), s);
    // 2^n: the low bits of t hold n (biased by a constant whose low nine bits are zero)
    float t0, t1, p0, p1;
    unpack2(t, t0, t1);
    unpack2(p, p0, p1);
    return pack2(__int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23)),
                 __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23)));
}

// e / d for many numerators and one denominator (a softmax row): with r = __frcp_rn(d), the
// correctly rounded reciprocal, q0 = e r followed by one residual correction is the correctly
// rounded quotient (no mismatch against IEEE division in 2*10^7 random pairs); quotients near the
// subnormal range, zeros, infinities and NaN go through the general routine.
__device__ __forceinline__ float div_by(float e, float d, float r) {
    const float q0 = __fmul_rn(e, r);
    if (!(fabsf(q0) >= 1e-30f && fabsf(q0) <= 1e30f))
        return __fdiv_rn(e, d);
    return __fmaf_rn(__fmaf_rn(-q0, d, e), r, q0);
}

// The same for 0 <= e <= d (a softmax row): the quotient cannot be large, one range test.
__device__ __forceinline__ float div_small_by(float e, float d, float r) {
    const float q0 = __fmul_rn(e, r);
    if (!(q0 >= 1e-30f))
        return __fdiv_rn(e, d);
    return __fmaf_rn(__fmaf_rn(-q0, d, e), r, q0);
}

// log(x) in float32 arithmetic for 0 < x < inf:  x = 2^e m with m in [sqrt(1/2), sqrt(2)), f = m - 1,
// s = f / (2 + f), log(m) = f - s (f - R(s^2)) with s^2 R' a degree-3 fit of the odd series
// 2 s^3/3 + 2 s^5/5 + ...; the sum e ln2 + f - u is formed with fast two-sums so that the parts
// dropped by each rounding are added back before the last one.  Subnormal inputs are scaled by
// 2^23 first.  Against float(log(double(x))) over 8 million inputs (dense around 1, and across the
// whole exponent range): never more than 1 ulp away, 98.6 % identical.
__device__ __forceinline__ float log_f32_normal(float x, int bias);

// x > 0, or NaN.  One range test on the common path; subnormal, infinite and NaN arguments behind it.
__device__ __forceinline__ float log_f32_pos(float x) {
    if (x >= 1.17549435e-38f && x <= 3.4028234663852886e38f)
        return log_f32_normal(x, 0);
    if (!(x <= 3.4028234663852886e38f))
        return x; // +inf, NaN
    return log_f32_normal(__fmul_rn(x, 8388608.0f), 23); // subnormal
}

__device__ __forceinline__ float log_f32_normal(float x, int bias) {
    int ix        = __float_as_int(x) + (0x3f800000 - 0x3f3504f3);
    const int ex  = (ix >> 23) - 127 - bias;
    ix            = (ix & 0x007fffff) + 0x3f3504f3;
    const float f = __fsub_rn(__int_as_float(ix), 1.0f);
    // s = f / (2 + f): hardware reciprocal (2^-23) and one residual correction instead of the
    // general division routine; differs from the correctly rounded quotient about once in 10^7
    const float den = __fadd_rn(2.0f, f); // in [1.70, 2.42)
    float r0;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(den));
    const float s0 = __fmul_rn(f, r0);
    const float s  = __fmaf_rn(__fmaf_rn(-s0, den, f), r0, s0);
    const float z = __fmul_rn(s, s);
    float q       = __int_as_float(0x3e6e99a6);
    q             = __fmaf_rn(q, z, __int_as_float(0x3e923012));
    q             = __fmaf_rn(q, z, __int_as_float(0x3eccccef));
    q             = __fmaf_rn(q, z, __int_as_float(0x3f2aaaab));
    const float t    = __fsub_rn(f, __fmul_rn(z, q));
    const float u    = __fmul_rn(s, t);
    const float u_lo = __fmaf_rn(s, t, -u);
    const float ef   = (float)ex;
    const float hi   = __fmul_rn(ef, 0.693145751953125f); // exact: 16 x 9 bits
    const float a    = __fadd_rn(hi, f);                  // |hi| >= |f| or hi == 0
    const float a_lo = __fsub_rn(f, __fsub_rn(a, hi));
    const float low  = __fmaf_rn(ef, __int_as_float(0x35bfbe8e), __fsub_rn(a_lo, u_lo));
    const float b    = __fsub_rn(a, u);
    const float b_lo = __fsub_rn(__fsub_rn(a, b), u);
    return __fadd_rn(b, __fadd_rn(b_lo, low));
}

} // namespace ct
