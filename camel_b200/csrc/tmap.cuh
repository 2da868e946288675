// Tensor-map encoding shared by the contraction kernels (the driver entry point is fetched
// through the runtime, so the library carries no link-time dependency on libcuda).
#pragma once

#include "common.cuh"

#include <cuda.h>

namespace ct {

// A tiled float32 tensor map of `rank` dimensions (innermost first): extents `dims`, byte strides
// of dimensions 1.. in `strides` (rank - 1 entries), box extents `box`, the 128- or 64-byte
// swizzle (0: none), out-of-range elements read as zero.
ct_status encode_tiled_map_f32(
    CUtensorMap *map, const void *base, int rank, const uint64_t *dims, const uint64_t *strides, const uint32_t *box,
    int swizzle_bytes);

// conv2d with the filters in tensor memory (conv_tmem.cu).
bool conv_tmem_applicable(int64_t c, int64_t h, int64_t w, int64_t ko, int64_t kh, int64_t kw, int64_t stride,
                          int64_t pad, bool *pool_ok = nullptr);
bool conv_tmem_reads_input_directly(const float *x, int64_t h, int64_t w, int64_t kh, int64_t kw, int64_t pad, int pool);
ct_status conv_tmem_filters(
    DeviceState *st, const float *x_raw, const void *x_hi, const void *x_lo, const float *w, const float *bias,
    int64_t batch, int64_t c, int64_t h, int64_t wd, int64_t ko, int64_t kh, int64_t kw, int64_t pad, int act, int pool,
    float *out);

// conv2d with one input halo per tile and channel block serving every tap (conv_halo.cu).
bool conv_halo_applicable(int64_t c_pad, int64_t h, int64_t w, int64_t ko, int64_t kh, int64_t kw, int64_t stride,
                          int64_t pad);
ct_status conv_halo_stream(
    DeviceState *st, const void *w_hi, const void *w_lo, const void *x_hi, const void *x_lo, int64_t batch,
    int64_t c_pad, int64_t h, int64_t wd, int64_t ko, int64_t kh, int64_t kw, int64_t pad, const float *bias, int act,
    float *out);

} // namespace ct
