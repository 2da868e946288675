// exp and log for float32 tensors, evaluated in float64 and rounded once - the reference's
// `float(std::exp(double(x)))` (modules/tensor/runtime.cpp:1023, 1042) - but with kernels cut to
// what a float32 result needs: ~2^-46 relative error instead of the full-double accuracy of the
// general-purpose device functions, which halves the float64 instruction count and lets the
// operators run at HBM speed.  Against the host libm the rounded float32 results are identical
// on every value tried (millions of inputs, dense around 1 for log); the parity tests allow
// 1 ulp.
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

// float32 in, float32 out.  The common range |x| <= 87 (result a normal float32) takes a path
// without clamps or special cases and scales by adding k to the exponent field; everything else
// (NaN, results that overflow, underflow or are subnormal) goes through exp_from_f32.  The
// operators built on this are bound by instruction issue, so every instruction counts.
__device__ __forceinline__ float exp_f32(float xf) {
    if (fabsf(xf) <= 87.0f) {
        const double kLog2e = 1.4426950408889634074;
        const double kLn2Hi = 6.93147180369123816490e-01;
        const double kLn2Lo = 1.90821492927058770002e-10;
        const double kMagic = 6755399441055744.0;
        double x  = (double)xf;
        double t  = fma(x, kLog2e, kMagic);
        int k     = __double2loint(t);
        double kd = t - kMagic;
        double r  = fma(-kd, kLn2Hi, x);
        r         = fma(-kd, kLn2Lo, r);
        double p  = 1.0 / 39916800.0;
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
        return (float)__hiloint2double(__double2hiint(p) + (k << 20), __double2loint(p));
    }
    return (float)exp_from_f32((double)xf);
}

// log tables: for m in [1, 2], j = round((m - 1) * 128), c_j = 1 + j/128:
// rc[j] = 1/c_j, lc[j] = log(c_j), with lc[128] the same double as ln 2 so that values just
// below a power of two cancel exactly.
constexpr int kLogTableSize = 129;

// log(x) for x > 0 that came from a float32 (so x is a normal double); table pointers are in
// shared memory.  log(x) = e*ln2 + log(c_j) + log1p(u), u = m/c_j - 1, |u| <= 2^-8.
__device__ __forceinline__ double log_from_f32(double x, const double *rc, const double *lc) {
    long long b = __double_as_longlong(x);
    if (b >= 0x7FF0000000000000LL)
        return x; // +inf, NaN
    int e       = (int)(b >> 52) - 1023;
    double m    = __longlong_as_double((b & 0xFFFFFFFFFFFFFLL) | 0x3FF0000000000000LL);
    int j       = ((int)((b >> 44) & 0xFF) + 1) >> 1;
    double u    = fma(m, rc[j], -1.0);
    double q    = 1.0 / 7.0;
    q           = fma(q, u, -1.0 / 6.0);
    q           = fma(q, u, 0.2);
    q           = fma(q, u, -0.25);
    q           = fma(q, u, 1.0 / 3.0);
    q           = fma(q, u, -0.5);
    double t    = fma(u * u, q, u);
    double base = fma((double)e, 0.693147180559945309417, lc[j]);
    return t + base;
}

} // namespace ct
