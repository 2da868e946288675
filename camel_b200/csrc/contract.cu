// Entry points of the contractions (matmul, dense, conv2d) and maxpool2d: argument checks,
// dispatch between the tensor-core kernel and the CUDA-core kernels, and the conv2d lowering.
#include "common.cuh"
#include "tmap.cuh"
#include "split.cuh"

#include <cuda_bf16.h>

#include <cstdlib>
#include <type_traits>

namespace ct {
namespace {

// Problems below this many multiply-adds stay on the CUDA-core kernel: the tensor-core path
// costs three launches and a tile of 128 rows.
constexpr int64_t kTinyMacs = 64ll * 64 * 64;

// ---- conv2d lowering ----------------------------------------------------------------------
//
// out[img][ko][pix] = sum_{c,r,s} w[ko][c][r][s] * x[img][c][y*stride-pad+r][x*stride-pad+s]
// is the GEMM  W[ko][kdim] . P[img][pix][kdim]^T  with kdim = c*kh*kw in (c,r,s) order, which is
// exactly the OIHW weight layout.  The patch matrix P is written once, already split into the
// operand planes the tensor-core kernel reads (zero for padded taps and for kdim..kp), and the
// kernel's output rows are output channels, so the result lands in NCHW without a transpose.
template <int MODE>
__global__ void __launch_bounds__(256) im2col_planes_kernel(
    const float *__restrict__ x, int64_t c, int64_t h, int64_t w, int64_t kh, int64_t kw,
    int64_t stride, int64_t pad, int64_t ho, int64_t wo, int64_t kdim, int64_t kp, int64_t total,
    void *__restrict__ p_hi, void *__restrict__ p_lo) {
    int64_t step = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
        int64_t kk  = i % kp;
        int64_t row = i / kp; // img * ho*wo + pix
        float v     = 0.0f;
        if (kk < kdim) {
            int64_t pix = row % (ho * wo), img = row / (ho * wo);
            int64_t oy = pix / wo, ox = pix - oy * wo;
            int64_t s = kk % kw, r = (kk / kw) % kh, ic = kk / (kw * kh);
            int64_t iy = oy * stride - pad + r, ix = ox * stride - pad + s;
            if (iy >= 0 && iy < h && ix >= 0 && ix < w)
                v = __ldg(x + ((img * c + ic) * h + iy) * w + ix);
        }
        if (MODE == 0) {
            float hi, lo;
            split_tf32(v, hi, lo);
            static_cast<float *>(p_hi)[i] = hi;
            static_cast<float *>(p_lo)[i] = lo;
        } else {
            static_cast<__nv_bfloat16 *>(p_hi)[i] = __float2bfloat16_rn(v);
        }
    }
}

// Weights [ko][c][kh][kw] -> A-operand planes [ko][taps * c_pad] with k = (r*kw + s) * c_pad + ic:
// tap-major, so that one k-block is 32 channels of one filter tap (what the implicit-GEMM
// producer fetches from the NHWC input with one shifted TMA box).
template <int MODE>
__global__ void __launch_bounds__(256) conv_weight_planes_kernel(
    const float *__restrict__ w, int64_t ko, int64_t c, int64_t taps, int64_t c_pad,
    void *__restrict__ p_hi, void *__restrict__ p_lo) {
    int64_t kp    = taps * c_pad;
    int64_t total = ko * kp;
    int64_t step  = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
        int64_t o = i / kp, kk = i - o * kp;
        int64_t rs = kk / c_pad, ic = kk - rs * c_pad;
        float v = ic < c ? w[(o * c + ic) * taps + rs] : 0.0f;
        if (MODE == 0) {
            float hi, lo;
            split_tf32(v, hi, lo);
            static_cast<float *>(p_hi)[i] = hi;
            static_cast<float *>(p_lo)[i] = lo;
        } else {
            static_cast<__nv_bfloat16 *>(p_hi)[i] = __float2bfloat16_rn(v);
        }
    }
}

// Output rows per implicit-GEMM tile: the largest th <= ho with th*wo <= 256 and th*wo a
// multiple of 16 (the MMA's N granularity); 0 when there is none.
int conv_tile_rows(int64_t ho, int64_t wo) {
    for (int64_t th = ho < 256 ? ho : 256; th >= 1; --th)
        if (th * wo <= 256 && (th * wo) % 16 == 0)
            return (int)th;
    return 0;
}

// Small problems: one thread per output, float64 accumulation in (c,r,s) order.
__global__ void __launch_bounds__(256) conv2d_direct_kernel(
    const float *__restrict__ x, const float *__restrict__ wt, const float *__restrict__ bias,
    int64_t n, int64_t c, int64_t h, int64_t w, int64_t ko, int64_t kh, int64_t kw, int64_t stride,
    int64_t pad, int64_t ho, int64_t wo, int act, float *__restrict__ out) {
    int64_t total = n * ko * ho * wo;
    int64_t step  = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
        int64_t ox = i % wo, oy = (i / wo) % ho, o = (i / (wo * ho)) % ko, img = i / (wo * ho * ko);
        double acc = 0.0;
        for (int64_t ic = 0; ic < c; ++ic)
            for (int64_t r = 0; r < kh; ++r) {
                int64_t iy = oy * stride - pad + r;
                if (iy < 0 || iy >= h)
                    continue;
                for (int64_t s = 0; s < kw; ++s) {
                    int64_t ix = ox * stride - pad + s;
                    if (ix < 0 || ix >= w)
                        continue;
                    acc += (double)x[((img * c + ic) * h + iy) * w + ix] *
                           (double)wt[((o * c + ic) * kh + r) * kw + s];
                }
            }
        if (bias)
            acc += (double)bias[o];
        float v = (float)acc;
        if (act == CT_ACT_RELU)
            v = __fmul_rn(v, v > 0.0f ? 1.0f : 0.0f);
        out[i] = v;
    }
}

// Few input channels (c*kh*kw <= 64, e.g. the first layer of a CNN on grey images): the
// contraction is too short for tensor-core tiles and the layer is bound by writing its output.
// One thread per output pixel keeps the patch in registers and walks the filters from shared
// memory; float64 accumulation in (c,r,s) order, bias last, as the reference style prescribes.
// Stores are coalesced: consecutive threads own consecutive pixels of one output plane.
constexpr int kSmallPatch = 64;
template <int KD> // register capacity of the patch: the smallest of 9 / 16 / 32 / 64 that holds kdim
__global__ void __launch_bounds__(256) conv2d_small_c_kernel(
    const float *__restrict__ x, const float *__restrict__ wt, const float *__restrict__ bias,
    int64_t n, int c, int64_t h, int64_t w, int ko, int kh, int kw, int64_t stride, int64_t pad,
    int64_t ho, int64_t wo, int act, float *__restrict__ out) {
    // [ko][kdim], widened to float64 once per block: float32 -> float64 conversions are the slow
    // instruction here, so none is left in the multiply-add loop when the patch is short
    extern __shared__ double w_s[];
    using patch_t  = typename std::conditional<(KD <= 16), double, float>::type;
    const int kdim = c * kh * kw;
    for (int i = threadIdx.x; i < ko * kdim; i += 256)
        w_s[i] = (double)wt[i];
    __syncthreads();
    const int64_t pix   = ho * wo;
    const int64_t total = n * pix;
    const int64_t step  = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
        int64_t img = i / pix, p = i - img * pix;
        int64_t oy = p / wo, ox = p - oy * wo;
        patch_t patch[KD];
#pragma unroll
        for (int t = 0; t < KD; ++t)
            patch[t] = 0;
        int t = 0;
        for (int ic = 0; ic < c; ++ic)
            for (int r = 0; r < kh; ++r)
                for (int s = 0; s < kw; ++s, ++t) {
                    int64_t iy = oy * stride - pad + r, ix = ox * stride - pad + s;
                    float v = 0.0f;
                    if (iy >= 0 && iy < h && ix >= 0 && ix < w)
                        v = __ldg(x + ((img * c + ic) * h + iy) * w + ix);
#pragma unroll
                    for (int u = 0; u < KD; ++u)
                        if (u == t)
                            patch[u] = (patch_t)v;
                }
        float *dst = out + img * ko * pix + p;
        for (int o = 0; o < ko; ++o) {
            const double *wr = w_s + o * kdim;
            double acc       = 0.0;
#pragma unroll
            for (int u = 0; u < KD; ++u)
                if (u < kdim)
                    acc = __fma_rn((double)patch[u], wr[u], acc); // exact product: same bits as mul, add
            if (bias)
                acc += (double)bias[o];
            float v = (float)acc;
            if (act == CT_ACT_RELU)
                v = __fmul_rn(v, v > 0.0f ? 1.0f : 0.0f);
            dst[(int64_t)o * pix] = v;
        }
    }
}

// One input channel, 3x3, stride 1 (the first layer of a CNN on grey images).  A thread owns four
// horizontally adjacent outputs: their patches overlap in a 3 x 6 window, which is loaded once and
// widened to float64 once, and every filter value read from shared memory then feeds four
// multiply-adds.  With one output per thread (the kernel above) each multiply-add needs its own
// 8-byte broadcast read and the layer is bound by the return bandwidth of shared memory (128 B per
// clock and SM), four times above what writing the result costs.  Same arithmetic: float64
// accumulation in (r, s) order, bias last, one rounding.
__global__ void __launch_bounds__(256) conv2d_c1_3x3_kernel(
    const float *__restrict__ x, const float *__restrict__ wt, const float *__restrict__ bias,
    int64_t n, int64_t h, int64_t w, int ko, int64_t pad, int64_t ho, int64_t wo, int act,
    float *__restrict__ out) {
    extern __shared__ double w_s[]; // [ko][9]
    for (int i = threadIdx.x; i < ko * 9; i += 256)
        w_s[i] = (double)wt[i];
    __syncthreads();
    const int64_t quads = wo >> 2; // wo is a multiple of 4
    const int64_t pix   = ho * wo;
    const int64_t total = n * ho * quads;
    const int64_t step  = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
        const int64_t qx = i % quads, oy = (i / quads) % ho, img = i / (quads * ho);
        const int64_t ox = qx * 4;
        double patch[3][6];
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const int64_t iy  = oy - pad + r;
            const bool row_ok = iy >= 0 && iy < h;
            const float *src  = x + (img * h + (row_ok ? iy : 0)) * w;
#pragma unroll
            for (int s = 0; s < 6; ++s) {
                const int64_t ix = ox - pad + s;
                patch[r][s]      = (row_ok && ix >= 0 && ix < w) ? (double)__ldg(src + ix) : 0.0;
            }
        }
        float *dst = out + img * ko * pix + oy * wo + ox;
        for (int o = 0; o < ko; ++o) {
            const double *wr = w_s + o * 9;
            double acc[4]    = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
            for (int r = 0; r < 3; ++r)
#pragma unroll
                for (int s = 0; s < 3; ++s) {
                    const double wv = wr[r * 3 + s];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        acc[j] = __fma_rn(patch[r][s + j], wv, acc[j]); // exact product: same bits as mul, add
                }
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                double a = acc[j];
                if (bias)
                    a += (double)bias[o];
                v[j] = (float)a;
                if (act == CT_ACT_RELU)
                    v[j] = __fmul_rn(v[j], v[j] > 0.0f ? 1.0f : 0.0f);
            }
            *reinterpret_cast<float4 *>(dst + (int64_t)o * pix) = make_float4(v[0], v[1], v[2], v[3]);
        }
    }
}

// maxpool, window == stride: one thread per output, strict '>' from the window's first element.
__global__ void __launch_bounds__(256) maxpool2d_kernel(
    const float *__restrict__ x, int64_t planes, int64_t h, int64_t w, int64_t win, int64_t ho,
    int64_t wo, float *__restrict__ out) {
    int64_t total = planes * ho * wo;
    int64_t step  = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
        int64_t ox = i % wo, oy = (i / wo) % ho, p = i / (wo * ho);
        const float *src = x + (p * h + oy * win) * w + ox * win;
        float best       = src[0];
        for (int64_t r = 0; r < win; ++r)
            for (int64_t s = 0; s < win; ++s) {
                float v = src[r * w + s];
                if (v > best)
                    best = v;
            }
        out[i] = best;
    }
}

// 2x2 windows on even widths: each thread reads two float2 and writes one value, so a warp
// reads 2 x 256 contiguous bytes.
__global__ void __launch_bounds__(256) maxpool2x2_kernel(
    const float *__restrict__ x, int64_t planes, int64_t h, int64_t w, int64_t ho, int64_t wo,
    float *__restrict__ out) {
    int64_t total = planes * ho * wo;
    int64_t step  = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
        int64_t ox = i % wo, oy = (i / wo) % ho, p = i / (wo * ho);
        const float *src = x + (p * h + oy * 2) * w + ox * 2;
        float2 a         = __ldcs(reinterpret_cast<const float2 *>(src));
        float2 b         = __ldcs(reinterpret_cast<const float2 *>(src + w));
        float best       = a.x;
        if (a.y > best)
            best = a.y;
        if (b.x > best)
            best = b.x;
        if (b.y > best)
            best = b.y;
        out[i] = best;
    }
}

// The same on widths that are a multiple of 4: two 128-bit loads and one 64-bit store per thread.
// IDX: the type the flat index is divided in (32-bit divisions where the element count allows:
// two 64-bit divisions per thread cost more than the loads they address).
template <typename IDX>
__global__ void __launch_bounds__(256) maxpool2x2_wide_kernel(
    const float *__restrict__ x, int64_t planes, int64_t h, int64_t w, int64_t ho, int64_t wo,
    float *__restrict__ out) {
    const IDX pairs = (IDX)(wo >> 1), rows = (IDX)ho;
    const IDX total = (IDX)(planes * ho) * pairs;
    const IDX step  = (IDX)gridDim.x * 256;
    for (IDX i = (IDX)blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
        const IDX row = i / pairs, px = i - row * pairs; // row = plane * ho + oy
        const IDX p64 = row / rows, oy = row - p64 * rows;
        const int64_t p  = (int64_t)p64;
        const float *src = x + (p * h + (int64_t)oy * 2) * w + (int64_t)px * 4;
        float4 a         = __ldcs(reinterpret_cast<const float4 *>(src));
        float4 b         = __ldcs(reinterpret_cast<const float4 *>(src + w));
        float m0 = a.x, m1 = a.z; // the window's first element seeds, later ones win on strict '>'
        if (a.y > m0)
            m0 = a.y;
        if (b.x > m0)
            m0 = b.x;
        if (b.y > m0)
            m0 = b.y;
        if (a.w > m1)
            m1 = a.w;
        if (b.z > m1)
            m1 = b.z;
        if (b.w > m1)
            m1 = b.w;
        __stcs(reinterpret_cast<float2 *>(out + (p * ho + (int64_t)oy) * wo + (int64_t)px * 2), make_float2(m0, m1));
    }
}

unsigned capped_blocks(DeviceState *st, int64_t total, int per_sm) {
    int64_t blocks = (total + 255) / 256;
    int64_t cap    = (int64_t)st->sm_count * per_sm;
    if (blocks > cap)
        blocks = cap;
    return (unsigned)(blocks < 1 ? 1 : blocks);
}

} // namespace
} // namespace ct

using namespace ct;

namespace ct {

// matmul with k == 1 is an outer product: out[i][j] = float(0.0 + double(a[i]) * double(b[j])), one
// exact product rounded once.  The reference's programs broadcast a column this way
// (`v[n, 1] @ ones([1, k])`, test/run/nn/mnist.cml:18), so it has to return v exactly, which a
// split-precision tensor-core product does not.  Bound by the write of the result.
template <bool VEC>
__global__ void __launch_bounds__(256) outer_product_kernel(
    const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out, int64_t n, int64_t total) {
    int64_t step = (int64_t)gridDim.x * 256;
    auto one     = [](float x, float y) { return (float)(0.0 + (double)x * (double)y); };
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
        if (VEC) { // n % 4 == 0: four neighbours of one row
            int64_t r = (i * 4) / n, c = i * 4 - r * n;
            float x   = a[r];
            float4 y  = *reinterpret_cast<const float4 *>(b + c);
            float4 o  = make_float4(one(x, y.x), one(x, y.y), one(x, y.z), one(x, y.w));
            *reinterpret_cast<float4 *>(out + i * 4) = o;
        } else {
            int64_t r = i / n, c = i - r * n;
            out[i]    = one(a[r], b[c]);
        }
    }
}

static ct_status outer_product(DeviceState *st, const float *a, const float *b, int64_t m, int64_t n, float *out) {
    bool vec      = (n & 3) == 0 && ((reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    int64_t total = vec ? m * n / 4 : m * n;
    int64_t want  = (total + 255) / 256, cap = (int64_t)st->sm_count * 16;
    unsigned grid = (unsigned)(want < cap ? want : cap);
    if (vec)
        outer_product_kernel<true><<<grid, 256, 0, stream()>>>(a, b, out, n, total);
    else
        outer_product_kernel<false><<<grid, 256, 0, stream()>>>(a, b, out, n, total);
    CT_LAUNCH_CHECK("outer_product");
    return CT_OK;
}

} // namespace ct

extern "C" {

ct_status ct_matmul(
    ct_dtype adt, const void *a, ct_dtype bdt, const void *b, int64_t m, int64_t k, int64_t n,
    void *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (!valid_dtype(adt) || !valid_dtype(bdt))
        return fail(CT_ERR_INVALID, "matmul: bad dtype");
    if (m < 0 || k < 0 || n < 0)
        return fail(CT_ERR_INVALID, "matmul: negative dimension");
    if (m == 0 || n == 0)
        return CT_OK;
    if (!out || (k > 0 && (!a || !b)))
        return fail(CT_ERR_INVALID, "matmul: null pointer");
    if (adt == CT_F32 && bdt == CT_F32) {
        const float *af = static_cast<const float *>(a), *bf = static_cast<const float *>(b);
        float *of = static_cast<float *>(out);
        if (n <= 32)
            return gemm_f32_skinny(st, af, bf, nullptr, m, k, n, CT_ACT_NONE, of, nullptr);
        if (k == 1)
            return outer_product(st, af, bf, m, n, of);
        if (m * n * (k > 0 ? k : 1) < kTinyMacs)
            return matmul_generic(adt, a, bdt, b, m, k, n, out);
        return gemm_f32_tc(st, af, bf, nullptr, m, k, n, CT_ACT_NONE, of);
    }
    return matmul_generic(adt, a, bdt, b, m, k, n, out);
}

ct_status ct_matmul_tn(const float *a_km, const float *b, int64_t m, int64_t k, int64_t n, float *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (m < 0 || k < 0 || n < 0)
        return fail(CT_ERR_INVALID, "matmul: negative dimension");
    if (m == 0 || n == 0)
        return CT_OK;
    if (!out || (k > 0 && (!a_km || !b)))
        return fail(CT_ERR_INVALID, "matmul: null pointer");
    if (n <= 32)
        return gemm_f32_tn_skinny(st, a_km, b, m, k, n, out);
    if (m * n * (k > 0 ? k : 1) < kTinyMacs) {
        // too small for the tensor-core kernel: materialise the transpose, then as ct_matmul
        void *at = nullptr;
        CT_TRY(ct_alloc(&at, (size_t)(m * k > 0 ? m * k : 1) * sizeof(float)));
        ct_status s = k > 0 ? ct_transpose(CT_F32, a_km, k, m, at) : CT_OK;
        if (s == CT_OK)
            s = ct_matmul(CT_F32, at, CT_F32, b, m, k, n, out);
        ct_status f = ct_free(at);
        return s != CT_OK ? s : f;
    }
    return gemm_f32_tc(st, a_km, b, nullptr, m, k, n, CT_ACT_NONE, out, nullptr, /*a_is_km=*/true);
}

ct_status ct_dense(
    const float *x, const float *w, const float *bias, int64_t m, int64_t k, int64_t n,
    ct_activation act, float *out, int64_t *argmax) {
    return ct_dense_packed(x, w, nullptr, bias, m, k, n, act, out, argmax);
}

ct_status ct_dense_packed(
    const float *x, const float *w, const void *packed, const float *bias, int64_t m, int64_t k,
    int64_t n, ct_activation act, float *out, int64_t *argmax) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (m < 0 || k < 0 || n < 0)
        return fail(CT_ERR_INVALID, "dense: negative dimension");
    if (act != CT_ACT_NONE && act != CT_ACT_RELU && act != CT_ACT_SOFTMAX)
        return fail(CT_ERR_INVALID, "dense: unknown activation");
    if (m == 0 || n == 0)
        return CT_OK;
    if (!out || (k > 0 && (!x || !w)))
        return fail(CT_ERR_INVALID, "dense: null pointer");
    if (n <= 32)
        return gemm_f32_skinny(st, x, w, bias, m, k, n, act, out, argmax);
    int gemm_act = act == CT_ACT_RELU ? CT_ACT_RELU : CT_ACT_NONE;
    CT_TRY(gemm_f32_tc(st, x, w, bias, m, k, n, gemm_act, out, static_cast<const PackedWeights *>(packed)));
    if (act == CT_ACT_SOFTMAX) {
        // wide classifier: logits are complete rows in `out`; finish in place
        if (argmax)
            CT_TRY(ct_argmax_axis(CT_F32, out, m, n, 1, argmax));
        CT_TRY(ct_softmax_rows(out, m, n, out));
    }
    return CT_OK;
}

ct_status ct_matmul_host(
    const float *a, const float *b, int64_t m, int64_t k, int64_t n, float *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (m < 0 || k < 0 || n < 0)
        return fail(CT_ERR_INVALID, "matmul: negative dimension");
    if (m == 0 || n == 0)
        return CT_OK;
    size_t ab = (size_t)m * k * 4, bb = (size_t)k * n * 4, ob = (size_t)m * n * 4;
    CT_TRY(ensure_ws(&st->stage_ws[0], &st->stage_ws_bytes[0], ab ? ab : 4));
    CT_TRY(ensure_ws(&st->stage_ws[1], &st->stage_ws_bytes[1], bb ? bb : 4));
    CT_TRY(ensure_ws(&st->stage_ws[2], &st->stage_ws_bytes[2], ob));
    if (ab)
        CT_CUDA(cudaMemcpyAsync(st->stage_ws[0], a, ab, cudaMemcpyHostToDevice, stream()));
    if (bb)
        CT_CUDA(cudaMemcpyAsync(st->stage_ws[1], b, bb, cudaMemcpyHostToDevice, stream()));
    CT_TRY(ct_matmul(CT_F32, st->stage_ws[0], CT_F32, st->stage_ws[1], m, k, n, st->stage_ws[2]));
    CT_CUDA(cudaMemcpyAsync(out, st->stage_ws[2], ob, cudaMemcpyDeviceToHost, stream()));
    CT_TRY(fetch_flags(st));
    return report_timeout(st, "matmul");
}

// Largest even number of output rows whose pixels fit the 128 accumulator rows; the fused
// conv + 2x2 max-pool needs at least two, even output height and width, at most 64 filters and a
// k range of one accumulation (the conditions of the pixels-on-rows kernel).
static int pooled_tile_rows(int64_t ho, int64_t wo) {
    int64_t th = wo > 0 ? 128 / wo : 0;
    if (th > ho)
        th = ho;
    return (int)(th & ~(int64_t)1);
}

static ct_status conv2d_run(
    const float *x, const float *w, const float *bias, int64_t n, int64_t c, int64_t h,
    int64_t wd, int64_t ko, int64_t kh, int64_t kw, int64_t stride, int64_t pad,
    ct_activation act, float *out, int pool);

ct_status ct_conv2d(
    const float *x, const float *w, const float *bias, int64_t n, int64_t c, int64_t h,
    int64_t wd, int64_t ko, int64_t kh, int64_t kw, int64_t stride, int64_t pad,
    ct_activation act, float *out) {
    return conv2d_run(x, w, bias, n, c, h, wd, ko, kh, kw, stride, pad, act, out, 0);
}

ct_status ct_conv2d_maxpool2(
    const float *x, const float *w, const float *bias, int64_t n, int64_t c, int64_t h,
    int64_t wd, int64_t ko, int64_t kh, int64_t kw, int64_t stride, int64_t pad,
    ct_activation act, float *out) {
    if (n < 0 || c < 0 || h < 0 || wd < 0 || ko < 0 || kh <= 0 || kw <= 0 || stride <= 0 || pad < 0)
        return fail(CT_ERR_INVALID, "conv2d: bad dimension");
    if (h + 2 * pad < kh || wd + 2 * pad < kw)
        return fail(CT_ERR_INVALID, "conv2d: kernel larger than padded input");
    const int64_t ho = (h + 2 * pad - kh) / stride + 1, wo = (wd + 2 * pad - kw) / stride + 1;
    const int kblock   = ct_get_precision() == CT_PREC_BF16 ? 64 : 32;
    const int64_t kp_i = kh * kw * ((c + kblock - 1) / kblock * kblock);
    // only where ct_conv2d itself takes the tensor-core path (same kernel, so the same bits): not
    // the short-patch, tiny or few-filter shapes that it serves with float64 CUDA-core kernels
    const int64_t kdim = c * kh * kw, pix = ho * wo;
    const bool tensor_core = kdim > kSmallPatch && !(kdim * ko * pix * n < kTinyMacs * 8 || ko < 16 || pix < 64);
    const bool swap_kernel = ko <= 64 && ko > 0 && wo <= 128 && kp_i <= 1024 * (kblock / 32) && pooled_tile_rows(ho, wo) >= 2;
    // the layer's kernel is chosen without regard to the pool (conv2d_run), so that the fused and the
    // two-step form run the same arithmetic; the pool is fused where that kernel can do it
    bool tmem_pool         = false;
    const bool tmem_kernel = kblock == 32 && conv_tmem_applicable(c, h, wd, ko, kh, kw, stride, pad, &tmem_pool);
    const bool fused = tensor_core && stride == 1 && c >= 16 && (wo & 1) == 0 && (ho & 1) == 0 && conv_tile_rows(ho, wo) > 0 &&
                       n > 0 && (tmem_kernel ? tmem_pool : swap_kernel);
    if (fused)
        return conv2d_run(x, w, bias, n, c, h, wd, ko, kh, kw, stride, pad, act, out, 2);
    // not a shape of the fused kernel: the convolution into a temporary, then maxpool2d
    void *tmp      = nullptr;
    size_t bytes   = (size_t)(n * ko * ho * wo > 0 ? n * ko * ho * wo : 1) * sizeof(float);
    CT_TRY(ct_alloc(&tmp, bytes));
    ct_status s = conv2d_run(x, w, bias, n, c, h, wd, ko, kh, kw, stride, pad, act, static_cast<float *>(tmp), 0);
    if (s == CT_OK)
        s = ct_maxpool2d(static_cast<const float *>(tmp), n, ko, ho, wo, 2, out);
    ct_status f = ct_free(tmp);
    return s != CT_OK ? s : f;
}

static ct_status conv2d_run(
    const float *x, const float *w, const float *bias, int64_t n, int64_t c, int64_t h,
    int64_t wd, int64_t ko, int64_t kh, int64_t kw, int64_t stride, int64_t pad,
    ct_activation act, float *out, int pool) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (n < 0 || c < 0 || h < 0 || wd < 0 || ko < 0 || kh <= 0 || kw <= 0 || stride <= 0 || pad < 0)
        return fail(CT_ERR_INVALID, "conv2d: bad dimension");
    if (act != CT_ACT_NONE && act != CT_ACT_RELU)
        return fail(CT_ERR_INVALID, "conv2d: activation must be none or relu");
    if (h + 2 * pad < kh || wd + 2 * pad < kw)
        return fail(CT_ERR_INVALID, "conv2d: kernel larger than padded input");
    int64_t ho = (h + 2 * pad - kh) / stride + 1, wo = (wd + 2 * pad - kw) / stride + 1;
    int64_t total_out = n * ko * ho * wo;
    if (total_out == 0)
        return CT_OK;
    if (!x || !w || !out)
        return fail(CT_ERR_INVALID, "conv2d: null pointer");
    int64_t kdim = c * kh * kw;
    int64_t pix  = ho * wo;
    if (pool == 0 && c == 1 && kh == 3 && kw == 3 && stride == 1 && (wo & 3) == 0 && (pix & 3) == 0 && ko * 72 <= 48 * 1024 &&
        (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
        ProfScope prof("conv_small_c");
        conv2d_c1_3x3_kernel<<<capped_blocks(st, n * ho * (wo >> 2), 16), 256, (size_t)ko * 72, stream()>>>(
            x, w, bias, n, h, wd, (int)ko, pad, ho, wo, act, out);
        CT_LAUNCH_CHECK("conv2d_c1_3x3");
        return CT_OK;
    }
    if (pool == 0 && kdim <= kSmallPatch && ko * kdim * 8 <= 48 * 1024 && ko <= 0x7fffffff) {
        ProfScope prof("conv_small_c");
        unsigned blocks = capped_blocks(st, n * pix, 16);
        size_t smem     = (size_t)(ko * kdim * 8);
#define CT_SMALL_C_ARGS x, w, bias, n, (int)c, h, wd, (int)ko, (int)kh, (int)kw, stride, pad, ho, wo, act, out
        if (kdim <= 9)
            conv2d_small_c_kernel<9><<<blocks, 256, smem, stream()>>>(CT_SMALL_C_ARGS);
        else if (kdim <= 16)
            conv2d_small_c_kernel<16><<<blocks, 256, smem, stream()>>>(CT_SMALL_C_ARGS);
        else if (kdim <= 32)
            conv2d_small_c_kernel<32><<<blocks, 256, smem, stream()>>>(CT_SMALL_C_ARGS);
        else
            conv2d_small_c_kernel<64><<<blocks, 256, smem, stream()>>>(CT_SMALL_C_ARGS);
#undef CT_SMALL_C_ARGS
        CT_LAUNCH_CHECK("conv2d_small_c");
        return CT_OK;
    }
    if (pool == 0 && (kdim * ko * pix * n < kTinyMacs * 8 || ko < 16 || pix < 64 || n > 0x7fffffff)) {
        conv2d_direct_kernel<<<capped_blocks(st, total_out, 16), 256, 0, stream()>>>(
            x, w, bias, n, c, h, wd, ko, kh, kw, stride, pad, ho, wo, act, out);
        CT_LAUNCH_CHECK("conv2d_direct");
        return CT_OK;
    }
    const int mode   = ct_get_precision() == CT_PREC_BF16 ? 1 : 0;
    const int elem   = mode == 0 ? 4 : 2;
    const int planes = mode == 0 ? 2 : 1;
    const int kblock = 128 / elem;
    auto align_up    = [](size_t v) { return (v + 1023) & ~(size_t)1023; };

    // Implicit GEMM: stride 1, enough channels to fill k-blocks, and a row tile that the MMA
    // accepts.  The input is rewritten once as NHWC hi/lo planes (12 B per input element); the
    // patch matrix is never materialised - each k-block is one shifted 4-D TMA box.
    const int th = (stride == 1 && c >= 16 && wo <= 256 && wd <= 0x7fffffff && h <= 0x7fffffff)
                       ? conv_tile_rows(ho, wo) : 0;
    if (th > 0 && mode == 0 && conv_tmem_applicable(c, h, wd, ko, kh, kw, stride, pad)) {
        // few channels on both sides: the filters stay in tensor memory, a tile's input is fetched
        // once (conv_tmem.cu) - as it is where its rows allow a tensor map over it (the kernel then
        // splits it itself: no pre-pass, no workspace), else from NHWC hi/lo planes
        if (conv_tmem_reads_input_directly(x, h, wd, kh, kw, pad, pool))
            return conv_tmem_filters(st, x, nullptr, nullptr, w, bias, n, c, h, wd, ko, kh, kw, pad, act, pool, out);
        size_t x_plane = align_up((size_t)n * h * wd * 32 * 4);
        CT_TRY(ensure_ws(&st->gemm_ws, &st->gemm_ws_bytes, 2 * x_plane));
        uint8_t *ws = static_cast<uint8_t *>(st->gemm_ws);
        {
            ProfScope prof("conv_prepass");
            CT_TRY(nhwc_planes(st, mode, x, n, c, h * wd, 32, ws, ws + x_plane));
        }
        return conv_tmem_filters(st, nullptr, ws, ws + x_plane, w, bias, n, c, h, wd, ko, kh, kw, pad, act, pool, out);
    }
    if (th > 0) {
        int64_t c_pad  = (c + kblock - 1) / kblock * kblock;
        int64_t taps   = kh * kw;
        int64_t kp_i   = taps * c_pad;
        size_t w_plane = align_up((size_t)ko * kp_i * elem);
        size_t x_plane = align_up((size_t)n * h * wd * c_pad * elem);
        CT_TRY(ensure_ws(&st->gemm_ws, &st->gemm_ws_bytes, planes * (w_plane + x_plane)));
        uint8_t *ws = static_cast<uint8_t *>(st->gemm_ws);
        void *w_hi = ws, *w_lo = ws + w_plane;
        void *x_hi = ws + planes * w_plane, *x_lo = ws + planes * w_plane + x_plane;
        {
            ProfScope prof("conv_prepass");
            int64_t wtotal = ko * kp_i;
            if (mode == 0)
                conv_weight_planes_kernel<0><<<capped_blocks(st, wtotal, 8), 256, 0, stream()>>>(
                    w, ko, c, taps, c_pad, w_hi, w_lo);
            else
                conv_weight_planes_kernel<1><<<capped_blocks(st, wtotal, 8), 256, 0, stream()>>>(
                    w, ko, c, taps, c_pad, w_hi, w_lo);
            CT_LAUNCH_CHECK("conv_weight_planes");
            CT_TRY(nhwc_planes(st, mode, x, n, c, h * wd, c_pad, x_hi, x_lo));
        }
        if (mode == 0 && pool == 0 && conv_halo_applicable(c_pad, h, wd, ko, kh, kw, stride, pad))
            // many filters: one input halo per tile and channel block serves every tap (conv_halo.cu)
            return conv_halo_stream(st, w_hi, w_lo, x_hi, x_lo, n, c_pad, h, wd, ko, kh, kw, pad, bias, act, out);
        ConvGeom g;
        g.c_pad = (int)c_pad;
        g.h = (int)h, g.w = (int)wd, g.ho = (int)ho, g.wo = (int)wo;
        g.kh = (int)kh, g.kw = (int)kw, g.pad = (int)pad, g.th = th;
        g.pool = pool; // only set for shapes ct_conv2d_maxpool2 has checked against the fused kernel
        return gemm_planes(
            st, mode, w_hi, w_lo, x_hi, x_lo, ko, pix, kp_i, bias, act, out, (int)n, ko * pix,
            bias ? 1 : 0, &g);
    }

    int64_t kp       = (kdim + kblock - 1) / kblock * kblock;
    size_t w_plane   = align_up((size_t)ko * kp * elem);
    size_t p_plane   = align_up((size_t)n * pix * kp * elem);
    CT_TRY(ensure_ws(&st->gemm_ws, &st->gemm_ws_bytes, planes * (w_plane + p_plane)));
    uint8_t *ws = static_cast<uint8_t *>(st->gemm_ws);
    void *w_hi = ws, *w_lo = ws + w_plane;
    void *p_hi = ws + planes * w_plane, *p_lo = ws + planes * w_plane + p_plane;
    CT_TRY(split_rows_planes(st, mode, w, ko, kdim, kp, w_hi, w_lo));
    int64_t total = n * pix * kp;
    {
        ProfScope prof("im2col");
        if (mode == 0)
        im2col_planes_kernel<0><<<capped_blocks(st, total, 32), 256, 0, stream()>>>(
            x, c, h, wd, kh, kw, stride, pad, ho, wo, kdim, kp, total, p_hi, p_lo);
    else
        im2col_planes_kernel<1><<<capped_blocks(st, total, 32), 256, 0, stream()>>>(
            x, c, h, wd, kh, kw, stride, pad, ho, wo, kdim, kp, total, p_hi, p_lo);
    }
    CT_LAUNCH_CHECK("im2col_planes");
    return gemm_planes(
        st, mode, w_hi, w_lo, p_hi, p_lo, ko, pix, kp, bias, act, out, (int)n, ko * pix,
        bias ? 1 : 0);
}

ct_status ct_maxpool2d(
    const float *x, int64_t n, int64_t c, int64_t h, int64_t w, int64_t window, float *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (n < 0 || c < 0 || h < 0 || w < 0 || window <= 0)
        return fail(CT_ERR_INVALID, "maxpool2d: bad dimension");
    int64_t ho = h / window, wo = w / window;
    int64_t total = n * c * ho * wo;
    if (total == 0)
        return CT_OK;
    if (!x || !out)
        return fail(CT_ERR_INVALID, "maxpool2d: null pointer");
    ProfScope prof("maxpool");
    if (window == 2 && (w & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 7u) == 0)
        if (total / 2 + (int64_t)st->sm_count * 32 * 256 < 0x7fffffffll)
            maxpool2x2_wide_kernel<uint32_t><<<capped_blocks(st, total / 2, 32), 256, 0, stream()>>>(x, n * c, h, w, ho, wo, out);
        else
            maxpool2x2_wide_kernel<uint64_t><<<capped_blocks(st, total / 2, 32), 256, 0, stream()>>>(x, n * c, h, w, ho, wo, out);
    else if (window == 2 && (w & 1) == 0 && (reinterpret_cast<uintptr_t>(x) & 7u) == 0)
        maxpool2x2_kernel<<<capped_blocks(st, total, 32), 256, 0, stream()>>>(x, n * c, h, w, ho, wo, out);
    else
        maxpool2d_kernel<<<capped_blocks(st, total, 32), 256, 0, stream()>>>(x, n * c, h, w, window, ho, wo, out);
    CT_LAUNCH_CHECK("maxpool2d");
    return CT_OK;
}

} // extern "C"
