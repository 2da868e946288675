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


} // namespace ct
