// Elementwise operators: binary / scalar-broadcast arithmetic, comparisons, exp, log, relu,
// constructors.  All are HBM-bound: every thread moves 4-element vectors (128-bit for float32)
// with coalesced, streaming accesses and no reuse.
//
// Arithmetic follows the reference: read as double, compute in double, round once into the
// output dtype (modules/tensor/runtime.cpp:298-355).  For float32 (+,-,*,/) the double detour
// is provably the IEEE float32 result (53 >= 2*24+2), so the fast path uses the correctly
// rounded single-precision instructions directly, with no fused multiply-add.
#include "common.cuh"
#include "fastmath.cuh"

#include <cmath>
#include <mutex>

namespace ct {
namespace {

constexpr int kThreads = 256;
constexpr int kVec     = 4; // elements per thread per step
constexpr int kUnroll  = 4; // steps per thread

template <typename T> struct alignas(sizeof(T) * kVec > 16 ? 16 : sizeof(T) * kVec) VecT {
    T v[kVec];
};

template <typename T> __device__ __forceinline__ VecT<T> load_vec(const T *p, uint64_t i) {
    return __ldcs(reinterpret_cast<const VecT<T> *>(p) + i);
}
template <> __device__ __forceinline__ VecT<float> load_vec<float>(const float *p, uint64_t i) {
    float4 q = __ldcs(reinterpret_cast<const float4 *>(p) + i);
    VecT<float> r;
    r.v[0] = q.x, r.v[1] = q.y, r.v[2] = q.z, r.v[3] = q.w;
    return r;
}
template <>
__device__ __forceinline__ VecT<int64_t> load_vec<int64_t>(const int64_t *p, uint64_t i) {
    longlong2 a = __ldcs(reinterpret_cast<const longlong2 *>(p) + 2 * i);
    longlong2 b = __ldcs(reinterpret_cast<const longlong2 *>(p) + 2 * i + 1);
    VecT<int64_t> r;
    r.v[0] = a.x, r.v[1] = a.y, r.v[2] = b.x, r.v[3] = b.y;
    return r;
}
template <>
__device__ __forceinline__ VecT<uint8_t> load_vec<uint8_t>(const uint8_t *p, uint64_t i) {
    uchar4 q = __ldcs(reinterpret_cast<const uchar4 *>(p) + i);
    VecT<uint8_t> r;
    r.v[0] = q.x, r.v[1] = q.y, r.v[2] = q.z, r.v[3] = q.w;
    return r;
}

__device__ __forceinline__ void store_vec(float *p, uint64_t i, const VecT<float> &r) {
    __stcs(reinterpret_cast<float4 *>(p) + i, make_float4(r.v[0], r.v[1], r.v[2], r.v[3]));
}
__device__ __forceinline__ void store_vec(int64_t *p, uint64_t i, const VecT<int64_t> &r) {
    __stcs(reinterpret_cast<longlong2 *>(p) + 2 * i, make_longlong2(r.v[0], r.v[1]));
    __stcs(reinterpret_cast<longlong2 *>(p) + 2 * i + 1, make_longlong2(r.v[2], r.v[3]));
}
__device__ __forceinline__ void store_vec(uint8_t *p, uint64_t i, const VecT<uint8_t> &r) {
    __stcs(reinterpret_cast<uchar4 *>(p) + i, make_uchar4(r.v[0], r.v[1], r.v[2], r.v[3]));
}

// TensorObject::getAsDouble / setFromDouble (runtime.cpp:298-310, 340-355).
__device__ __forceinline__ double as_double(float v) { return (double)v; }
__device__ __forceinline__ double as_double(int64_t v) { return (double)v; }
__device__ __forceinline__ double as_double(uint8_t v) { return v != 0 ? 1.0 : 0.0; }
template <typename T> __device__ __forceinline__ T from_double(double v);
template <> __device__ __forceinline__ float from_double<float>(double v) { return (float)v; }
template <> __device__ __forceinline__ int64_t from_double<int64_t>(double v) {
    return (int64_t)v;
}
template <> __device__ __forceinline__ uint8_t from_double<uint8_t>(double v) {
    return v != 0.0 ? 1 : 0;
}

// applyBinary in double (runtime.cpp:113-130); a zero divisor raises the device flag.
__device__ __forceinline__ double apply_binary_d(int op, double a, double b, uint32_t *flags) {
    switch (op) {
    case CT_ADD:
        return a + b;
    case CT_SUB:
        return a - b;
    case CT_MUL:
        return a * b;
    case CT_DIV:
        if (b == 0.0) {
            flags[FLAG_DIV_ZERO] = 1;
            return 0.0;
        }
        return a / b;
    default:
        return pow(a, b);
    }
}

// Same, float32 operands and result.
template <int OP>
__device__ __forceinline__ float apply_binary_f(float a, float b, uint32_t *flags) {
    if (OP == CT_ADD)
        return __fadd_rn(a, b);
    if (OP == CT_SUB)
        return __fsub_rn(a, b);
    if (OP == CT_MUL)
        return __fmul_rn(a, b);
    if (OP == CT_DIV) {
        if (b == 0.0f) {
            flags[FLAG_DIV_ZERO] = 1;
            return 0.0f;
        }
        return __fdiv_rn(a, b);
    }
    return (float)pow((double)a, (double)b);
}

// applyCompare in double (runtime.cpp:132-146).
__device__ __forceinline__ uint8_t apply_compare_d(int op, double a, double b) {
    switch (op) {
    case CT_LT:
        return a < b;
    case CT_LE:
        return a <= b;
    case CT_GT:
        return a > b;
    case CT_GE:
        return a >= b;
    default:
        return a == b;
    }
}

// Generic driver: out[i] = f(i-th elements).  VEC=true: all pointers are vector-aligned and
// the body covers numel/4 vectors; the tail (and the unaligned case) runs with VEC=false.
template <bool VEC, typename F> __global__ void __launch_bounds__(kThreads) map_kernel(uint64_t count, F f) {
    uint64_t base = (uint64_t)blockIdx.x * (kThreads * kUnroll) + threadIdx.x;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        uint64_t i = base + (uint64_t)u * kThreads;
        if (i < count)
            f(i);
    }
}

template <typename F> ct_status launch_map(uint64_t count, F f, const char *name) {
    if (count == 0)
        return CT_OK;
    uint64_t per_block = (uint64_t)kThreads * kUnroll;
    uint64_t blocks    = (count + per_block - 1) / per_block;
    if (blocks > 0x7fffffffull)
        return fail(CT_ERR_TOO_LARGE, "%s: too many elements", name);
    ProfScope prof("elementwise");
    map_kernel<true, F><<<(unsigned)blocks, kThreads, 0, stream()>>>(count, f);
    CT_LAUNCH_CHECK(name);
    return CT_OK;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
template <typename T> inline bool vec_aligned(const void *p) {
    size_t a = sizeof(T) * kVec > 16 ? 16 : sizeof(T) * kVec;
    return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

// ---- binary, tensor (x) tensor --------------------------------------------------------

template <typename LT, typename RT, typename OT> struct BinaryGenericVec {
    const LT *l;
    const RT *r;
    OT *o;
    int op;
    uint32_t *flags;
    __device__ void operator()(uint64_t i) const {
        VecT<LT> a = load_vec<LT>(l, i);
        VecT<RT> b = load_vec<RT>(r, i);
        VecT<OT> c;
#pragma unroll
        for (int k = 0; k < kVec; ++k)
            c.v[k] = from_double<OT>(apply_binary_d(op, as_double(a.v[k]), as_double(b.v[k]), flags));
        store_vec(o, i, c);
    }
};
template <typename LT, typename RT, typename OT> struct BinaryGenericScalar {
    const LT *l;
    const RT *r;
    OT *o;
    int op;
    uint32_t *flags;
    uint64_t offset;
    __device__ void operator()(uint64_t i) const {
        uint64_t j = i + offset;
        o[j]       = from_double<OT>(apply_binary_d(op, as_double(l[j]), as_double(r[j]), flags));
    }
};
template <int OP> struct BinaryF32Vec {
    const float *l;
    const float *r;
    float *o;
    uint32_t *flags;
    __device__ void operator()(uint64_t i) const {
        VecT<float> a = load_vec<float>(l, i);
        VecT<float> b = load_vec<float>(r, i);
        VecT<float> c;
#pragma unroll
        for (int k = 0; k < kVec; ++k)
            c.v[k] = apply_binary_f<OP>(a.v[k], b.v[k], flags);
        store_vec(o, i, c);
    }
};

template <typename LT, typename RT, typename OT>
ct_status binary_typed(int op, const void *l, const void *r, uint64_t n, void *o, uint32_t *flags) {
    const LT *lp = static_cast<const LT *>(l);
    const RT *rp = static_cast<const RT *>(r);
    OT *op_      = static_cast<OT *>(o);
    uint64_t nv  = 0;
    if (vec_aligned<LT>(l) && vec_aligned<RT>(r) && vec_aligned<OT>(o)) {
        nv = n / kVec;
        CT_TRY(launch_map(nv, BinaryGenericVec<LT, RT, OT>{lp, rp, op_, op, flags}, "binary"));
    }
    uint64_t done = nv * kVec;
    return launch_map(
        n - done, BinaryGenericScalar<LT, RT, OT>{lp, rp, op_, op, flags, done}, "binary(tail)");
}

template <int OP>
ct_status binary_f32(const float *l, const float *r, uint64_t n, float *o, uint32_t *flags) {
    uint64_t nv = 0;
    if (aligned16(l) && aligned16(r) && aligned16(o)) {
        nv = n / kVec;
        CT_TRY(launch_map(nv, BinaryF32Vec<OP>{l, r, o, flags}, "binary_f32"));
    }
    uint64_t done = nv * kVec;
    return launch_map(
        n - done, BinaryGenericScalar<float, float, float>{l, r, o, OP, flags, done},
        "binary_f32(tail)");
}

template <typename LT, typename RT>
ct_status binary_out(int op, int odt, const void *l, const void *r, uint64_t n, void *o, uint32_t *f) {
    switch (odt) {
    case CT_F32:
        return binary_typed<LT, RT, float>(op, l, r, n, o, f);
    case CT_I64:
        return binary_typed<LT, RT, int64_t>(op, l, r, n, o, f);
    default:
        return binary_typed<LT, RT, uint8_t>(op, l, r, n, o, f);
    }
}

template <typename LT>
ct_status binary_rhs(int op, int rdt, int odt, const void *l, const void *r, uint64_t n, void *o, uint32_t *f) {
    switch (rdt) {
    case CT_F32:
        return binary_out<LT, float>(op, odt, l, r, n, o, f);
    case CT_I64:
        return binary_out<LT, int64_t>(op, odt, l, r, n, o, f);
    default:
        return binary_out<LT, uint8_t>(op, odt, l, r, n, o, f);
    }
}

// ---- binary, tensor (x) scalar --------------------------------------------------------

template <typename TT, typename OT, bool VEC> struct ScalarBinary {
    const TT *t;
    OT *o;
    double s;
    int op;
    int left;
    uint32_t *flags;
    uint64_t offset;
    __device__ __forceinline__ OT one(TT v) const {
        double d = as_double(v);
        return from_double<OT>(left ? apply_binary_d(op, s, d, flags) : apply_binary_d(op, d, s, flags));
    }
    __device__ void operator()(uint64_t i) const {
        if (VEC) {
            VecT<TT> a = load_vec<TT>(t, i);
            VecT<OT> c;
#pragma unroll
            for (int k = 0; k < kVec; ++k)
                c.v[k] = one(a.v[k]);
            store_vec(o, i, c);
        } else {
            o[i + offset] = one(t[i + offset]);
        }
    }
};

// float32 tensor with a scalar that is exactly a float32: single-precision fast path.
template <int OP, bool VEC> struct ScalarBinaryF32 {
    const float *t;
    float *o;
    float s;
    int left;
    uint32_t *flags;
    uint64_t offset;
    __device__ __forceinline__ float one(float v) const {
        return left ? apply_binary_f<OP>(s, v, flags) : apply_binary_f<OP>(v, s, flags);
    }
    __device__ void operator()(uint64_t i) const {
        if (VEC) {
            VecT<float> a = load_vec<float>(t, i);
            VecT<float> c;
#pragma unroll
            for (int k = 0; k < kVec; ++k)
                c.v[k] = one(a.v[k]);
            store_vec(o, i, c);
        } else {
            o[i + offset] = one(t[i + offset]);
        }
    }
};

template <typename TT, typename OT>
ct_status scalar_typed(int op, const void *t, double s, int left, uint64_t n, void *o, uint32_t *f) {
    const TT *tp = static_cast<const TT *>(t);
    OT *op_      = static_cast<OT *>(o);
    uint64_t nv  = 0;
    if (vec_aligned<TT>(t) && vec_aligned<OT>(o)) {
        nv = n / kVec;
        CT_TRY(launch_map(nv, ScalarBinary<TT, OT, true>{tp, op_, s, op, left, f, 0}, "binary_scalar"));
    }
    uint64_t done = nv * kVec;
    return launch_map(
        n - done, ScalarBinary<TT, OT, false>{tp, op_, s, op, left, f, done}, "binary_scalar(tail)");
}

template <int OP>
ct_status scalar_f32(const float *t, float s, int left, uint64_t n, float *o, uint32_t *f) {
    uint64_t nv = 0;
    if (aligned16(t) && aligned16(o)) {
        nv = n / kVec;
        CT_TRY(launch_map(nv, ScalarBinaryF32<OP, true>{t, o, s, left, f, 0}, "binary_scalar_f32"));
    }
    uint64_t done = nv * kVec;
    return launch_map(
        n - done, ScalarBinaryF32<OP, false>{t, o, s, left, f, done}, "binary_scalar_f32(tail)");
}

template <typename TT>
ct_status scalar_out(int op, int odt, const void *t, double s, int left, uint64_t n, void *o, uint32_t *f) {
    switch (odt) {
    case CT_F32:
        return scalar_typed<TT, float>(op, t, s, left, n, o, f);
    case CT_I64:
        return scalar_typed<TT, int64_t>(op, t, s, left, n, o, f);
    default:
        return scalar_typed<TT, uint8_t>(op, t, s, left, n, o, f);
    }
}

// ---- comparisons ----------------------------------------------------------------------

template <typename LT, typename RT, bool VEC> struct CompareTT {
    const LT *l;
    const RT *r;
    uint8_t *o;
    int op;
    uint64_t offset;
    __device__ void operator()(uint64_t i) const {
        if (VEC) {
            VecT<LT> a = load_vec<LT>(l, i);
            VecT<RT> b = load_vec<RT>(r, i);
            VecT<uint8_t> c;
#pragma unroll
            for (int k = 0; k < kVec; ++k)
                c.v[k] = apply_compare_d(op, as_double(a.v[k]), as_double(b.v[k]));
            store_vec(o, i, c);
        } else {
            uint64_t j = i + offset;
            o[j]       = apply_compare_d(op, as_double(l[j]), as_double(r[j]));
        }
    }
};

template <typename TT, bool VEC> struct CompareTS {
    const TT *t;
    uint8_t *o;
    double s;
    int op;
    int left;
    uint64_t offset;
    __device__ __forceinline__ uint8_t one(TT v) const {
        double d = as_double(v);
        return left ? apply_compare_d(op, s, d) : apply_compare_d(op, d, s);
    }
    __device__ void operator()(uint64_t i) const {
        if (VEC) {
            VecT<TT> a = load_vec<TT>(t, i);
            VecT<uint8_t> c;
#pragma unroll
            for (int k = 0; k < kVec; ++k)
                c.v[k] = one(a.v[k]);
            store_vec(o, i, c);
        } else {
            o[i + offset] = one(t[i + offset]);
        }
    }
};

template <typename LT, typename RT>
ct_status compare_typed(int op, const void *l, const void *r, uint64_t n, uint8_t *o) {
    const LT *lp = static_cast<const LT *>(l);
    const RT *rp = static_cast<const RT *>(r);
    uint64_t nv  = 0;
    if (vec_aligned<LT>(l) && vec_aligned<RT>(r) && vec_aligned<uint8_t>(o)) {
        nv = n / kVec;
        CT_TRY(launch_map(nv, CompareTT<LT, RT, true>{lp, rp, o, op, 0}, "compare"));
    }
    uint64_t done = nv * kVec;
    return launch_map(n - done, CompareTT<LT, RT, false>{lp, rp, o, op, done}, "compare(tail)");
}

template <typename LT> ct_status compare_rhs(int op, int rdt, const void *l, const void *r, uint64_t n, uint8_t *o) {
    switch (rdt) {
    case CT_F32:
        return compare_typed<LT, float>(op, l, r, n, o);
    case CT_I64:
        return compare_typed<LT, int64_t>(op, l, r, n, o);
    default:
        return compare_typed<LT, uint8_t>(op, l, r, n, o);
    }
}

template <typename TT>
ct_status compare_scalar_typed(int op, const void *t, double s, int left, uint64_t n, uint8_t *o) {
    const TT *tp = static_cast<const TT *>(t);
    uint64_t nv  = 0;
    if (vec_aligned<TT>(t) && vec_aligned<uint8_t>(o)) {
        nv = n / kVec;
        CT_TRY(launch_map(nv, CompareTS<TT, true>{tp, o, s, op, left, 0}, "compare_scalar"));
    }
    uint64_t done = nv * kVec;
    return launch_map(n - done, CompareTS<TT, false>{tp, o, s, op, left, done}, "compare_scalar(tail)");
}

// ---- unary ----------------------------------------------------------------------------

enum { UN_EXP = 0, UN_LOG = 1, UN_RELU = 2 };

template <int OP> __device__ __forceinline__ float apply_unary(float x, uint32_t *flags) {
    if (OP == UN_EXP)
        return exp_f32(x); // tensorExp, runtime.cpp:1023
    if (OP == UN_LOG) {
        if (x <= 0.0f) { // v <= 0 throws; NaN does not (runtime.cpp:1038-1042)
            flags[FLAG_LOG_DOMAIN] = 1;
            return 0.0f;
        }
        return (float)log((double)x);
    }
    // relu := x * (x > 0), both factors as the reference's operators would produce them
    return __fmul_rn(x, x > 0.0f ? 1.0f : 0.0f);
}

template <int OP, bool VEC> struct Unary {
    const float *t;
    float *o;
    uint32_t *flags;
    uint64_t offset;
    __device__ void operator()(uint64_t i) const {
        if (VEC) {
            VecT<float> a = load_vec<float>(t, i);
            VecT<float> c;
#pragma unroll
            for (int k = 0; k < kVec; ++k)
                c.v[k] = apply_unary<OP>(a.v[k], flags);
            store_vec(o, i, c);
        } else {
            o[i + offset] = apply_unary<OP>(t[i + offset], flags);
        }
    }
};

template <int OP> ct_status unary(const float *t, uint64_t n, float *o, uint32_t *flags, const char *name) {
    uint64_t nv = 0;
    if (aligned16(t) && aligned16(o)) {
        nv = n / kVec;
        CT_TRY(launch_map(nv, Unary<OP, true>{t, o, flags, 0}, name));
    }
    uint64_t done = nv * kVec;
    return launch_map(n - done, Unary<OP, false>{t, o, flags, done}, name);
}

// ---- w - g * lr in one pass (the parameter update of the reference's training loops) ------

// Same roundings as the two operators it replaces: t = float(double(g) * lr) (tensor * scalar,
// runtime.cpp:795-812), then float(double(w) - double(t)) = the IEEE float32 difference.
template <bool VEC> struct ScaledSub {
    const float *w;
    const float *g;
    float *o;
    double lr;
    uint64_t offset;
    __device__ float one(float wv, float gv) const { return __fsub_rn(wv, (float)((double)gv * lr)); }
    __device__ void operator()(uint64_t i) const {
        if (VEC) {
            VecT<float> a = load_vec<float>(w, i);
            VecT<float> b = load_vec<float>(g, i);
            VecT<float> c;
#pragma unroll
            for (int k = 0; k < kVec; ++k)
                c.v[k] = one(a.v[k], b.v[k]);
            store_vec(o, i, c);
        } else {
            o[i + offset] = one(w[i + offset], g[i + offset]);
        }
    }
};

// ---- log ------------------------------------------------------------------------------

// tensorLog (runtime.cpp:1029-1045): any x <= 0 raises the flag (the reference throws there).
__global__ void __launch_bounds__(kThreads) log_kernel(
    const float *__restrict__ in, float *__restrict__ out, uint64_t n, int vec, uint32_t *flags) {
    auto one = [&](float x) -> float {
        if (x >= 1.17549435e-38f && x <= 3.4028234663852886e38f)
            return log_f32_normal(x, 0); // the common case behind one range test
        if (x <= 0.0f) {
            flags[FLAG_LOG_DOMAIN] = 1;
            return 0.0f;
        }
        return log_f32_pos(x);
    };
    if (vec) {
        uint64_t nv   = n / kVec;
        uint64_t base = (uint64_t)blockIdx.x * (kThreads * kUnroll) + threadIdx.x;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            uint64_t i = base + (uint64_t)u * kThreads;
            if (i < nv) {
                VecT<float> a = load_vec<float>(in, i);
                VecT<float> c;
#pragma unroll
                for (int k = 0; k < kVec; ++k)
                    c.v[k] = one(a.v[k]);
                store_vec(out, i, c);
            }
        }
        // the last block also finishes the < 4 element tail
        if (blockIdx.x == gridDim.x - 1)
            for (uint64_t i = nv * kVec + threadIdx.x; i < n; i += kThreads)
                out[i] = one(in[i]);
    } else {
        uint64_t base = (uint64_t)blockIdx.x * (kThreads * kUnroll * kVec) + threadIdx.x;
        for (int u = 0; u < kUnroll * kVec; ++u) {
            uint64_t i = base + (uint64_t)u * kThreads;
            if (i < n)
                out[i] = one(in[i]);
        }
    }
}

// ---- constructors ---------------------------------------------------------------------

template <typename T> struct Fill {
    T *o;
    T value;
    __device__ void operator()(uint64_t i) const { o[i] = value; }
};
template <typename T> struct FillVec {
    T *o;
    T value;
    __device__ void operator()(uint64_t i) const {
        VecT<T> c;
#pragma unroll
        for (int k = 0; k < kVec; ++k)
            c.v[k] = value;
        store_vec(o, i, c);
    }
};
template <typename T> struct FillTail {
    T *o;
    T value;
    uint64_t offset;
    __device__ void operator()(uint64_t i) const { o[i + offset] = value; }
};

template <typename T> ct_status fill_typed(T value, uint64_t n, void *out) {
    T *o        = static_cast<T *>(out);
    uint64_t nv = 0;
    if (vec_aligned<T>(out)) {
        nv = n / kVec;
        CT_TRY(launch_map(nv, FillVec<T>{o, value}, "fill"));
    }
    uint64_t done = nv * kVec;
    return launch_map(n - done, FillTail<T>{o, value, done}, "fill(tail)");
}

struct Eye {
    float *o;
    int64_t size;
    __device__ void operator()(uint64_t i) const {
        uint64_t r = i / (uint64_t)size, c = i % (uint64_t)size;
        o[i] = r == c ? 1.0f : 0.0f;
    }
};

struct Arange {
    int64_t *o;
    int64_t start, step;
    __device__ void operator()(uint64_t i) const { o[i] = start + (int64_t)i * step; }
};

bool is_float_scalar_exact(double s) { return (double)(float)s == s || s != s; }

} // namespace
} // namespace ct

using namespace ct;

extern "C" {

ct_status ct_binary(
    ct_binary_op op, ct_dtype ldt, const void *l, ct_dtype rdt, const void *r, uint64_t n,
    void *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (op < CT_ADD || op > CT_POW || !valid_dtype(ldt) || !valid_dtype(rdt))
        return fail(CT_ERR_INVALID, "ct_binary: bad operator or dtype");
    if (n == 0)
        return CT_OK;
    if (!l || !r || !out)
        return fail(CT_ERR_INVALID, "ct_binary: null pointer");
    bool checks = op == CT_DIV;
    if (checks)
        CT_TRY(clear_data_flags(st));
    ct_status rc;
    if (ldt == CT_F32 && rdt == CT_F32) {
        const float *lf = static_cast<const float *>(l), *rf = static_cast<const float *>(r);
        float *of = static_cast<float *>(out);
        switch (op) {
        case CT_ADD:
            rc = binary_f32<CT_ADD>(lf, rf, n, of, st->flags_dev);
            break;
        case CT_SUB:
            rc = binary_f32<CT_SUB>(lf, rf, n, of, st->flags_dev);
            break;
        case CT_MUL:
            rc = binary_f32<CT_MUL>(lf, rf, n, of, st->flags_dev);
            break;
        case CT_DIV:
            rc = binary_f32<CT_DIV>(lf, rf, n, of, st->flags_dev);
            break;
        default:
            rc = binary_f32<CT_POW>(lf, rf, n, of, st->flags_dev);
            break;
        }
    } else {
        int odt = ct_result_dtype(op, ldt, rdt);
        switch (ldt) {
        case CT_F32:
            rc = binary_rhs<float>(op, rdt, odt, l, r, n, out, st->flags_dev);
            break;
        case CT_I64:
            rc = binary_rhs<int64_t>(op, rdt, odt, l, r, n, out, st->flags_dev);
            break;
        default:
            rc = binary_rhs<uint8_t>(op, rdt, odt, l, r, n, out, st->flags_dev);
            break;
        }
    }
    CT_TRY(rc);
    if (checks) {
        CT_TRY(fetch_flags(st));
        if (st->flags_host[FLAG_DIV_ZERO])
            return fail(CT_ERR_DIV_ZERO, "Division by zero");
    }
    return CT_OK;
}

ct_status ct_binary_scalar(
    ct_binary_op op, ct_dtype tdt, const void *t, double scalar, ct_dtype sdt, int left,
    uint64_t n, void *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (op < CT_ADD || op > CT_POW || !valid_dtype(tdt) || !valid_dtype(sdt))
        return fail(CT_ERR_INVALID, "ct_binary_scalar: bad operator or dtype");
    // The reference evaluates the scalar divisor per element and throws on the first one,
    // so an empty tensor never throws (runtime.cpp:806-808).
    if (n == 0)
        return CT_OK;
    if (!t || !out)
        return fail(CT_ERR_INVALID, "ct_binary_scalar: null pointer");
    if (op == CT_DIV && !left && scalar == 0.0)
        return fail(CT_ERR_DIV_ZERO, "Division by zero");
    bool checks = op == CT_DIV && left;
    if (checks)
        CT_TRY(clear_data_flags(st));
    int odt = left ? ct_result_dtype(op, sdt, tdt) : ct_result_dtype(op, tdt, sdt);
    ct_status rc;
    if (tdt == CT_F32 && op != CT_POW && is_float_scalar_exact(scalar)) {
        const float *tf = static_cast<const float *>(t);
        float *of       = static_cast<float *>(out);
        float s         = (float)scalar;
        switch (op) {
        case CT_ADD:
            rc = scalar_f32<CT_ADD>(tf, s, left, n, of, st->flags_dev);
            break;
        case CT_SUB:
            rc = scalar_f32<CT_SUB>(tf, s, left, n, of, st->flags_dev);
            break;
        case CT_MUL:
            rc = scalar_f32<CT_MUL>(tf, s, left, n, of, st->flags_dev);
            break;
        default:
            rc = scalar_f32<CT_DIV>(tf, s, left, n, of, st->flags_dev);
            break;
        }
    } else {
        switch (tdt) {
        case CT_F32:
            rc = scalar_out<float>(op, odt, t, scalar, left, n, out, st->flags_dev);
            break;
        case CT_I64:
            rc = scalar_out<int64_t>(op, odt, t, scalar, left, n, out, st->flags_dev);
            break;
        default:
            rc = scalar_out<uint8_t>(op, odt, t, scalar, left, n, out, st->flags_dev);
            break;
        }
    }
    CT_TRY(rc);
    if (checks) {
        CT_TRY(fetch_flags(st));
        if (st->flags_host[FLAG_DIV_ZERO])
            return fail(CT_ERR_DIV_ZERO, "Division by zero");
    }
    return CT_OK;
}

ct_status ct_compare(
    ct_compare_op op, ct_dtype ldt, const void *l, ct_dtype rdt, const void *r, uint64_t n,
    uint8_t *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (op < CT_LT || op > CT_EQ || !valid_dtype(ldt) || !valid_dtype(rdt))
        return fail(CT_ERR_INVALID, "ct_compare: bad operator or dtype");
    if (n == 0)
        return CT_OK;
    if (!l || !r || !out)
        return fail(CT_ERR_INVALID, "ct_compare: null pointer");
    switch (ldt) {
    case CT_F32:
        return compare_rhs<float>(op, rdt, l, r, n, out);
    case CT_I64:
        return compare_rhs<int64_t>(op, rdt, l, r, n, out);
    default:
        return compare_rhs<uint8_t>(op, rdt, l, r, n, out);
    }
}

ct_status ct_compare_scalar(
    ct_compare_op op, ct_dtype tdt, const void *t, double scalar, int left, uint64_t n,
    uint8_t *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (op < CT_LT || op > CT_EQ || !valid_dtype(tdt))
        return fail(CT_ERR_INVALID, "ct_compare_scalar: bad operator or dtype");
    if (n == 0)
        return CT_OK;
    if (!t || !out)
        return fail(CT_ERR_INVALID, "ct_compare_scalar: null pointer");
    switch (tdt) {
    case CT_F32:
        return compare_scalar_typed<float>(op, t, scalar, left, n, out);
    case CT_I64:
        return compare_scalar_typed<int64_t>(op, t, scalar, left, n, out);
    default:
        return compare_scalar_typed<uint8_t>(op, t, scalar, left, n, out);
    }
}

ct_status ct_exp(const float *in, uint64_t n, float *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (n == 0)
        return CT_OK;
    if (!in || !out)
        return fail(CT_ERR_INVALID, "ct_exp: null pointer");
    return unary<UN_EXP>(in, n, out, st->flags_dev, "exp");
}

ct_status ct_log(const float *in, uint64_t n, float *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (n == 0)
        return CT_OK;
    if (!in || !out)
        return fail(CT_ERR_INVALID, "ct_log: null pointer");
    CT_TRY(clear_data_flags(st));
    {
        uint64_t per_block = (uint64_t)kThreads * kUnroll * kVec;
        uint64_t blocks    = (n + per_block - 1) / per_block;
        if (blocks > 0x7fffffffull)
            return fail(CT_ERR_TOO_LARGE, "log: too many elements");
        int vec = aligned16(in) && aligned16(out);
        ProfScope prof("elementwise");
        log_kernel<<<(unsigned)blocks, kThreads, 0, stream()>>>(in, out, n, vec, st->flags_dev);
        CT_LAUNCH_CHECK("log");
    }
    CT_TRY(fetch_flags(st));
    if (st->flags_host[FLAG_LOG_DOMAIN])
        return fail(CT_ERR_LOG_DOMAIN, "log: input must be positive");
    return CT_OK;
}

ct_status ct_scaled_sub(const float *w, const float *g, double lr, uint64_t n, float *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (n == 0)
        return CT_OK;
    if (!w || !g || !out)
        return fail(CT_ERR_INVALID, "ct_scaled_sub: null pointer");
    uint64_t nv = 0;
    if (aligned16(w) && aligned16(g) && aligned16(out)) {
        nv = n / kVec;
        CT_TRY(launch_map(nv, ScaledSub<true>{w, g, out, lr, 0}, "scaled_sub"));
    }
    uint64_t done = nv * kVec;
    return launch_map(n - done, ScaledSub<false>{w, g, out, lr, done}, "scaled_sub");
}

ct_status ct_relu(const float *in, uint64_t n, float *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (n == 0)
        return CT_OK;
    if (!in || !out)
        return fail(CT_ERR_INVALID, "ct_relu: null pointer");
    return unary<UN_RELU>(in, n, out, st->flags_dev, "relu");
}

ct_status ct_fill(ct_dtype dt, double value, uint64_t n, void *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (!valid_dtype(dt))
        return fail(CT_ERR_INVALID, "ct_fill: bad dtype");
    if (n == 0)
        return CT_OK;
    if (!out)
        return fail(CT_ERR_INVALID, "ct_fill: null pointer");
    switch (dt) {
    case CT_F32:
        return fill_typed<float>((float)value, n, out);
    case CT_I64:
        return fill_typed<int64_t>((int64_t)value, n, out);
    default:
        return fill_typed<uint8_t>(value != 0.0 ? 1 : 0, n, out);
    }
}

ct_status ct_eye(int64_t size, float *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (size < 0)
        return fail(CT_ERR_INVALID, "eye size cannot be negative");
    if (size == 0)
        return CT_OK;
    return launch_map((uint64_t)size * (uint64_t)size, Eye{out, size}, "eye");
}

ct_status ct_arange(int64_t start, int64_t step, int64_t count, int64_t *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (step == 0)
        return fail(CT_ERR_INVALID, "range step cannot be zero");
    if (count <= 0)
        return CT_OK;
    return launch_map((uint64_t)count, Arange{out, start, step}, "arange");
}

ct_status ct_binary_host(
    ct_binary_op op, const float *lhs, const float *rhs, uint64_t n, float *out) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (n == 0)
        return CT_OK;
    size_t bytes = n * sizeof(float);
    for (int i = 0; i < 3; ++i)
        CT_TRY(ensure_ws(&st->stage_ws[i], &st->stage_ws_bytes[i], bytes));
    CT_CUDA(cudaMemcpyAsync(st->stage_ws[0], lhs, bytes, cudaMemcpyHostToDevice, stream()));
    CT_CUDA(cudaMemcpyAsync(st->stage_ws[1], rhs, bytes, cudaMemcpyHostToDevice, stream()));
    CT_TRY(ct_binary(op, CT_F32, st->stage_ws[0], CT_F32, st->stage_ws[1], n, st->stage_ws[2]));
    CT_CUDA(cudaMemcpyAsync(out, st->stage_ws[2], bytes, cudaMemcpyDeviceToHost, stream()));
    CT_CUDA(cudaStreamSynchronize(stream()));
    return CT_OK;
}

} // extern "C"
