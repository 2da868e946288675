// Splitting float32 values into TF32 terms for the 3xTF32 contractions.
#pragma once

#include <cstdint>

namespace ct {

__device__ __forceinline__ float to_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

// v = hi + lo up to ~2^-22 |v|: hi is v rounded to TF32 (10 explicit mantissa bits), lo the
// TF32 rounding of the exact remainder.
__device__ __forceinline__ void split_tf32(float v, float &hi, float &lo) {
    hi = to_tf32(v);
    if (!isfinite(hi)) {
        if (!isfinite(v)) { // inf / NaN: carried by hi alone
            lo = 0.0f;
            return;
        }
        hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); // rounding overflowed: truncate
    }
    lo = to_tf32(v - hi); // v - hi is exact in float32
}

// The same split without a branch, for code that splits many values per thread and wants their
// dependency chains interleaved (a branch per value serialises them).  Rounding to TF32 (nearest,
// ties away from zero) is an integer operation on the bit pattern: add half a TF32 unit to the
// magnitude, clear the 13 low bits; the carry takes care of the exponent.  Same results as
// split_tf32 for every finite input; an infinity or NaN is carried by hi alone as there.
__device__ __forceinline__ void split_tf32_flat(float v, float &hi, float &lo) {
    const uint32_t u      = __float_as_uint(v);
    const bool v_special  = (u & 0x7f800000u) == 0x7f800000u;           // inf or NaN
    uint32_t h            = (u + 0x1000u) & 0xffffe000u;
    const bool h_overflow = (h & 0x7f800000u) == 0x7f800000u;           // rounding reached the top exponent
    h  = h_overflow ? (u & 0xffffe000u) : h;                            // finite v: truncate instead
    h  = v_special ? u : h;
    hi = __uint_as_float(h);
    const float d    = v - hi;                                          // exact for finite v
    const uint32_t l = (__float_as_uint(d) + 0x1000u) & 0xffffe000u;
    lo = __uint_as_float(v_special ? 0u : l);
}

} // namespace ct
