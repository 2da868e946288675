// Operator bodies and registration tables of the B200 `tensor` plugin.
//
// Same entry points, group names, URIs and signature strings as the reference module
// (modules/tensor/operators.h:31-63, operators.cpp:160-583), so programs resolve and dispatch
// exactly as before; each body unpacks its ArgsView the way the reference body does and then
// calls one function of the C ABI (include/camel_tensor_b200.h) instead of looping on the host.
// Operators added on top: relu, softmax, dense*, conv2d*, conv2d_relu_maxpool2, maxpool2d, flatten,
// matmul_tn, scaled_sub.
#include "tensor_ops.h"

#include "camel/core/error/runtime.h"
#include "camel/core/mm.h"
#include "camel/core/rtdata/array.h"
#include "camel/core/type/composite/array.h"
#include "device_tensor.h"
#include "type.h"

#include <iostream>
#include <mutex>
#include <random>
#include <optional>
#include <stdexcept>
#include <vector>

namespace mm = camel::core::mm;
using namespace camel::core::error;
using namespace camel::core::type;
using namespace camel::core::rtdata;
using camel::tensor::TensorObject;
using camel::tensor::TensorType;
namespace ctn = camel::tensor;

namespace {

// ---- argument helpers --------------------------------------------------------------------

Type *tensorType(Type *dtype = nullptr) { return TensorType::Dynamic(dtype ? dtype : Type::Float32()); }

bool isTensor(Type *t) { return t && t->code() == TensorType::typeCode(); }
bool isArray(Type *t) { return t && t->code() == TypeCode::Array; }

double scalarValue(ArgsView &args, size_t i) {
    switch (args.type(i)->code()) {
    case TypeCode::Int32:
        return static_cast<double>(args.get<Int32>(i));
    case TypeCode::Int64:
        return static_cast<double>(args.get<Int64>(i));
    case TypeCode::Float32:
        return static_cast<double>(args.get<Float32>(i));
    case TypeCode::Float64:
        return args.get<Float64>(i);
    case TypeCode::Bool:
        return args.get<Bool>(i) ? 1.0 : 0.0;
    default:
        throw std::invalid_argument("Unsupported scalar type for Tensor operation");
    }
}

int64_t intValue(ArgsView &args, size_t i) {
    return args.type(i)->code() == TypeCode::Int32 ? static_cast<int64_t>(args.get<Int32>(i)) : args.get<Int64>(i);
}

TensorObject *tensorArg(ArgsView &args, size_t i) {
    if (!isTensor(args.type(i)))
        throwRuntimeFault(RuntimeDiag::RuntimeError, "Expected Tensor argument");
    TensorObject *t = args.get<TensorObject *>(i);
    if (!t)
        throwRuntimeFault(RuntimeDiag::RuntimeError, "Tensor argument cannot be null");
    return t;
}

// Nested Camel array -> tensor (the reference's tensorFromArray, runtime.cpp:153-219,
// 1067-1077): dtype from the leaf element type, rectangular shape required.
struct ArrayShape {
    TypeCode dtype;
    std::vector<int64_t> dims;
};

ArrayShape inferArray(slot_t slot, Type *valueType) {
    auto *arrayType = static_cast<ArrayType *>(valueType);
    auto *array     = fromSlot<::Array *>(slot);
    Type *elem      = arrayType->elemType();
    int64_t size    = array ? static_cast<int64_t>(array->size()) : 0;
    ArrayShape out{TypeCode::Float32, {size}};
    if (elem->code() != TypeCode::Array) {
        if (!ctn::isSupportedTensorScalar(elem->code()))
            throw std::invalid_argument("Only numeric arrays can be converted to Tensor");
        out.dtype = ctn::normalizeTensorDType(elem->code());
        return out;
    }
    if (size == 0)
        return out;
    ArrayShape first = inferArray(array->data()[0], elem);
    for (int64_t i = 1; i < size; ++i) {
        ArrayShape other = inferArray(array->data()[i], elem);
        if (other.dims != first.dims || other.dtype != first.dtype)
            throw std::invalid_argument("Nested array shape or dtype mismatch");
    }
    out.dtype = first.dtype;
    out.dims.insert(out.dims.end(), first.dims.begin(), first.dims.end());
    return out;
}

template <typename T> void flattenInto(const ::Array *array, Type *valueType, std::vector<T> &out) {
    Type *elem = static_cast<ArrayType *>(valueType)->elemType();
    for (size_t i = 0; i < array->size(); ++i) {
        slot_t v = array->data()[i];
        if (elem->code() == TypeCode::Array) {
            flattenInto<T>(fromSlot<::Array *>(v), elem, out);
            continue;
        }
        double d;
        switch (elem->code()) {
        case TypeCode::Int32:
            d = static_cast<double>(fromSlot<Int32>(v));
            break;
        case TypeCode::Int64:
            d = static_cast<double>(fromSlot<Int64>(v));
            break;
        case TypeCode::Float32:
            d = static_cast<double>(fromSlot<Float32>(v));
            break;
        case TypeCode::Float64:
            d = fromSlot<Float64>(v);
            break;
        default:
            d = fromSlot<Bool>(v) ? 1.0 : 0.0;
            break;
        }
        if constexpr (std::is_same_v<T, uint8_t>)
            out.push_back(d != 0.0 ? 1 : 0);
        else
            out.push_back(static_cast<T>(d));
    }
}

TensorObject *tensorFromArray(slot_t slot, Type *valueType) {
    ArrayShape info = inferArray(slot, valueType);
    auto *array     = fromSlot<::Array *>(slot);
    auto build      = [&](auto tag) {
        using T = decltype(tag);
        std::vector<T> flat;
        if (array)
            flattenInto<T>(array, valueType, flat);
        return TensorObject::fromHost(info.dtype, info.dims, flat.data(), mm::autoSpace());
    };
    if (info.dtype == TypeCode::Float32)
        return build(float{});
    if (info.dtype == TypeCode::Int64)
        return build(int64_t{});
    return build(uint8_t{});
}

TensorObject *tensorOrArrayArg(ArgsView &args, size_t i) {
    if (isTensor(args.type(i)))
        return tensorArg(args, i);
    if (isArray(args.type(i)))
        return tensorFromArray(args.slot(i), args.type(i));
    throwRuntimeFault(RuntimeDiag::RuntimeError, "Expected Tensor or numeric array");
}

// parseShapeArray, runtime.cpp:582-604
std::vector<int64_t> shapeArg(ArgsView &args, size_t i) {
    Type *t = args.type(i);
    auto *a = args.get<::Array *>(i);
    if (!a || !isArray(t))
        throw std::invalid_argument("Shape must be an integer array");
    TypeCode ec = static_cast<ArrayType *>(t)->elemTypeCode();
    if (ec != TypeCode::Int32 && ec != TypeCode::Int64)
        throw std::invalid_argument("Shape array must contain integers");
    std::vector<int64_t> shape;
    for (size_t k = 0; k < a->size(); ++k) {
        int64_t v = ec == TypeCode::Int32 ? static_cast<int64_t>(a->get<Int32>(k)) : a->get<Int64>(k);
        if (v < 0)
            throw std::invalid_argument("Shape cannot contain negative values");
        shape.push_back(v);
    }
    return shape;
}

slot_t wrap(TensorObject *t) { return toSlot(static_cast<Object *>(t)); }

TensorObject *newTensor(TypeCode dtype, std::span<const int64_t> shape) {
    return TensorObject::create(dtype, shape, mm::autoSpace(), false);
}

std::span<const int64_t> shapeOf(const TensorObject *t) { return {t->shape(), t->rank()}; }

// Every std::exception raised in a body becomes a RuntimeFault, like withTensorErrors
// (operators.cpp:103-109); ct_* failures arrive here through ctCheck.
template <typename Fn> slot_t guarded(Fn &&fn) {
    try {
        return fn();
    } catch (const RuntimeFault &) {
        throw;
    } catch (const std::exception &e) {
        throwRuntimeFault(RuntimeDiag::RuntimeError, e.what());
    }
}

// ---- closing an idiom: operators that look at how their operands came about -----------------

using ctn::Expr;
using ctn::ExprKind;

bool isF32(const Expr *e) { return e->dtype == CT_F32; }
bool stillPending(const Expr *e) { return e->pending.load(std::memory_order_relaxed); }
const float *f32(Expr *e) { return static_cast<const float *>(ctn::bufferOf(e)); }

// mask == (h > 0)
bool isPositiveMaskOf(const Expr *mask, const Expr *h) {
    return mask->kind == ExprKind::CompareScalar && mask->a == h && mask->op == CT_GT && mask->tensorOnLeft &&
           mask->scalar == 0.0 && isF32(h);
}

// h * (h > 0), either order (test/run/nn/svm.cml:31): one relu pass; on top of a matmul that has
// not run, the GEMM with relu in its epilogue.  Returns nullptr if the operands are not that.
TensorObject *tryRelu(TensorObject *a, TensorObject *b) {
    Expr *ea = a->expr(), *eb = b->expr();
    Expr *h  = isPositiveMaskOf(eb, ea) ? ea : (isPositiveMaskOf(ea, eb) ? eb : nullptr);
    if (!h)
        return nullptr;
    Expr *mask        = h == ea ? eb : ea;
    TensorObject *out = newTensor(TypeCode::Float32, shapeOf(a));
    if (h->numel == 0)
        return out;
    bool transposedLhs = h->kind == ExprKind::MatMul && h->a->kind == ExprKind::Transpose && stillPending(h->a);
    if (h->kind == ExprKind::MatMul && stillPending(h) && !transposedLhs) {
        ctn::evaluate(h->a);
        ctn::evaluate(h->b);
        ctn::ctCheck(ct_dense(f32(h->a), f32(h->b), nullptr, h->rows, h->a->cols, h->cols, CT_ACT_RELU,
                              static_cast<float *>(out->deviceData()), nullptr));
        // The product of the matmul was never written.  If the mask is read later it is taken from
        // the result: (h > 0) == (h * (h > 0) > 0) for every h (-0.0, NaN and infinities included).
        if (stillPending(mask))
            ctn::rebindOperand(mask, 0, out->expr());
    } else {
        ctn::evaluate(h);
        ctn::ctCheck(ct_relu(f32(h), h->numel, static_cast<float *>(out->deviceData())));
    }
    return out;
}

// w - (s * g) or w - (g * s) with the product not yet computed (mnist.cml:40): one pass.
TensorObject *tryScaledSub(TensorObject *a, TensorObject *b) {
    Expr *w = a->expr(), *sg = b->expr();
    if (!(isF32(w) && sg->kind == ExprKind::ScaleByScalar && stillPending(sg) && isF32(sg->a)))
        return nullptr;
    TensorObject *out = newTensor(TypeCode::Float32, shapeOf(a));
    ctn::evaluate(w);
    ctn::evaluate(sg->a);
    ctn::ctCheck(ct_scaled_sub(f32(w), f32(sg->a), sg->scalar, w->numel, static_cast<float *>(out->deviceData())));
    return out;
}

// The softmax of test/run/nn/mnist.cml:13-25, recognised at its last operator:
//   exp(L - spread(max(L, 1))) / spread(sum(exp(...), 1)),  spread(v) = reshape(v, [n, 1]) @ ones([1, k]).
// One ct_softmax_rows pass over L; where L is a matmul that has not run, the classifier GEMM with
// softmax fused (ct_dense).  The row sums are >= 1 (the row maximum contributes exp(0)) or NaN, so
// the division-by-zero check of divide can never fire on this pattern.
TensorObject *trySoftmax(TensorObject *a, TensorObject *b) {
    Expr *num = a->expr(), *den = b->expr();
    auto spreadOf = [](const Expr *e, ExprKind reduction) -> const Expr * {
        if (e->kind != ExprKind::Spread || e->a->kind != ExprKind::Column || e->a->a->kind != reduction)
            return nullptr;
        return e->a->a->a;
    };
    if (num->kind != ExprKind::Exp || num->a->kind != ExprKind::Subtract)
        return nullptr;
    Expr *logits = num->a->a;
    if (spreadOf(num->a->b, ExprKind::MaxAxis1) != logits || spreadOf(den, ExprKind::SumAxis1) != num)
        return nullptr;
    if (!isF32(logits) || logits->rank != 2 || logits->numel == 0)
        return nullptr;
    if (logits->dead.load(std::memory_order_acquire))
        return nullptr; // matched through records that have already run: the logits themselves are gone
    TensorObject *out = newTensor(TypeCode::Float32, shapeOf(a));
    auto *dst         = static_cast<float *>(out->deviceData());
    bool transposedLhs =
        logits->kind == ExprKind::MatMul && logits->a->kind == ExprKind::Transpose && stillPending(logits->a);
    if (logits->kind == ExprKind::MatMul && stillPending(logits) && !transposedLhs) {
        ctn::evaluate(logits->a);
        ctn::evaluate(logits->b);
        ctn::ctCheck(ct_dense(f32(logits->a), f32(logits->b), nullptr, logits->rows, logits->a->cols, logits->cols,
                              CT_ACT_SOFTMAX, dst, nullptr));
    } else {
        ctn::evaluate(logits);
        ctn::ctCheck(ct_softmax_rows(f32(logits), logits->rows, logits->cols, dst));
    }
    return out;
}

// ---- generic bodies ----------------------------------------------------------------------

slot_t binaryBody(ArgsView &norm, ct_binary_op op, bool lhsMustBeTensor) {
    return guarded([&]() -> slot_t {
        bool lt = isTensor(norm.type(0)), rt = isTensor(norm.type(1));
        if (lhsMustBeTensor)
            lt = (tensorArg(norm, 0), true);
        if (lt && rt) {
            TensorObject *a = tensorArg(norm, 0), *b = tensorArg(norm, 1);
            if (!a->sameShape(b))
                throw std::invalid_argument("Tensor binary operation requires matching shapes");
            if (op == CT_MUL || op == CT_SUB || op == CT_DIV) {
                std::lock_guard<std::recursive_mutex> lock(ctn::exprMutex());
                TensorObject *fused = op == CT_MUL ? tryRelu(a, b) : (op == CT_SUB ? tryScaledSub(a, b) : trySoftmax(a, b));
                if (fused)
                    return wrap(fused);
            }
            ct_dtype odt      = ct_result_dtype(op, a->ctDType(), b->ctDType());
            TensorObject *out = newTensor(ctn::fromCtDType(odt), shapeOf(a));
            if (op == CT_SUB && a->dtype() == TypeCode::Float32 && b->dtype() == TypeCode::Float32) {
                ctn::defer(out, ExprKind::Subtract, a, b); // `logits - row_max_broadcast` of the softmax idiom
                return wrap(out);
            }
            ctn::ctCheck(ct_binary(op, a->ctDType(), a->deviceData(), b->ctDType(), b->deviceData(), a->numel(),
                                   out->deviceData()));
            return wrap(out);
        }
        size_t ti = lt ? 0 : 1, si = lt ? 1 : 0;
        TensorObject *t   = tensorArg(norm, ti);
        ct_dtype sdt      = ctn::toCtDType(norm.type(si)->code());
        double s          = scalarValue(norm, si);
        ct_dtype odt      = lt ? ct_result_dtype(op, t->ctDType(), sdt) : ct_result_dtype(op, sdt, t->ctDType());
        TensorObject *out = newTensor(ctn::fromCtDType(odt), shapeOf(t));
        if (op == CT_MUL && t->dtype() == TypeCode::Float32) {
            ctn::defer(out, ExprKind::ScaleByScalar, t, nullptr, 0, s, sdt, lt ? 1 : 0); // `lr * g` of the update
            return wrap(out);
        }
        ctn::ctCheck(
            ct_binary_scalar(op, t->ctDType(), t->deviceData(), s, sdt, lt ? 0 : 1, t->numel(), out->deviceData()));
        return wrap(out);
    });
}

slot_t compareBody(ArgsView &norm, ct_compare_op op, bool arraysAllowed) {
    return guarded([&]() -> slot_t {
        auto tensorLike = [&](size_t i) {
            return isTensor(norm.type(i)) || (arraysAllowed && isArray(norm.type(i)));
        };
        auto fetch = [&](size_t i) { return arraysAllowed ? tensorOrArrayArg(norm, i) : tensorArg(norm, i); };
        bool lt = tensorLike(0), rt = tensorLike(1);
        if (lt && rt) {
            TensorObject *a = fetch(0), *b = fetch(1);
            if (!a->sameShape(b))
                throw std::invalid_argument("Tensor comparison requires matching shapes");
            TensorObject *out = newTensor(TypeCode::Bool, shapeOf(a));
            ctn::ctCheck(ct_compare(op, a->ctDType(), a->deviceData(), b->ctDType(), b->deviceData(), a->numel(),
                                    static_cast<uint8_t *>(out->deviceData())));
            return wrap(out);
        }
        size_t ti = lt ? 0 : 1, si = lt ? 1 : 0;
        TensorObject *t   = fetch(ti);
        double s          = scalarValue(norm, si);
        TensorObject *out = newTensor(TypeCode::Bool, shapeOf(t));
        ctn::defer(out, ExprKind::CompareScalar, t, nullptr, op, s, CT_F32, lt ? 1 : 0); // `h > 0` of the relu idiom
        return wrap(out);
    });
}

enum class AxisKind { Sum, Max, Argmax };

slot_t axisBody(ArgsView &norm, AxisKind kind, const char *name) {
    return guarded([&]() -> slot_t {
        TensorObject *t = tensorArg(norm, 0);
        int64_t axis    = intValue(norm, 1);
        if (t->rank() != 2)
            throw std::invalid_argument(std::string(name) + "(axis) currently only supports rank-2 tensors");
        int64_t a = axis < 0 ? axis + 2 : axis;
        if (a != 0 && a != 1)
            throw std::invalid_argument(std::string(name) + "(axis): axis must be 0 or 1 for rank-2 tensors");
        int64_t rows = t->dim(0), cols = t->dim(1);
        int64_t outShape[1] = {a == 0 ? cols : rows};
        TensorObject *out   = newTensor(kind == AxisKind::Argmax ? TypeCode::Int64 : TypeCode::Float32, outShape);
        if (a == 1 && kind != AxisKind::Argmax && t->dtype() == TypeCode::Float32) {
            ctn::defer(out, kind == AxisKind::Sum ? ExprKind::SumAxis1 : ExprKind::MaxAxis1, t); // softmax idiom
            return wrap(out);
        }
        ct_status s;
        if (kind == AxisKind::Sum)
            s = ct_sum_axis(t->ctDType(), t->deviceData(), rows, cols, a, static_cast<float *>(out->deviceData()));
        else if (kind == AxisKind::Max)
            s = ct_max_axis(t->ctDType(), t->deviceData(), rows, cols, a, static_cast<float *>(out->deviceData()));
        else
            s = ct_argmax_axis(t->ctDType(), t->deviceData(), rows, cols, a, static_cast<int64_t *>(out->deviceData()));
        ctn::ctCheck(s);
        return wrap(out);
    });
}

slot_t fillBody(ArgsView &norm, TypeCode dtype, double value, bool ones = false) {
    return guarded([&]() -> slot_t {
        auto shape        = shapeArg(norm, 0);
        TensorObject *out = newTensor(dtype, shape);
        if (ones) {
            ctn::defer(out, ExprKind::Ones, nullptr); // `v @ ones([1, k])` is how the programs broadcast
            return wrap(out);
        }
        ctn::ctCheck(ct_fill(out->ctDType(), value, out->numel(), out->deviceData()));
        return wrap(out);
    });
}

TensorObject *requireFloat(TensorObject *t, const char *name) {
    if (!ctn::isFloatingTensorType(t->dtype()))
        throw std::invalid_argument(std::string(name) + " requires floating-point tensor");
    return t;
}

slot_t unaryBody(ArgsView &norm, const char *name, ct_status (*fn)(const float *, uint64_t, float *)) {
    return guarded([&]() -> slot_t {
        TensorObject *t   = requireFloat(tensorArg(norm, 0), name);
        TensorObject *out = newTensor(TypeCode::Float32, shapeOf(t));
        if (fn == ct_exp) {
            ctn::defer(out, ExprKind::Exp, t); // softmax idiom; exp raises no error
            return wrap(out);
        }
        ctn::ctCheck(fn(static_cast<const float *>(t->deviceData()), t->numel(), static_cast<float *>(out->deviceData())));
        return wrap(out);
    });
}

slot_t denseBody(ArgsView &with, ArgsView &norm, ct_activation act) {
    return guarded([&]() -> slot_t {
        TensorObject *x = requireFloat(tensorArg(norm, 0), "dense");
        TensorObject *w = requireFloat(tensorArg(with, 0), "dense");
        TensorObject *b = with.size() > 1 ? requireFloat(tensorArg(with, 1), "dense") : nullptr;
        if (x->rank() != 2 || w->rank() != 2)
            throw std::invalid_argument("matmul currently only supports rank-2 tensors");
        if (x->dim(1) != w->dim(0))
            throw std::invalid_argument("matmul dimension mismatch");
        int64_t m = x->dim(0), k = x->dim(1), n = w->dim(1);
        if (b && static_cast<int64_t>(b->numel()) != n)
            throw std::invalid_argument("dense: bias must have one value per output column");
        int64_t outShape[2] = {m, n};
        TensorObject *out   = newTensor(TypeCode::Float32, outShape);
        ctn::ctCheck(ct_dense_packed(
            static_cast<const float *>(x->deviceData()), static_cast<const float *>(w->deviceData()),
            ctn::packedWeightsFor(w, k, n), b ? static_cast<const float *>(b->deviceData()) : nullptr, m, k, n, act,
            static_cast<float *>(out->deviceData()), nullptr));
        return wrap(out);
    });
}

slot_t convBody(ArgsView &with, ArgsView &norm, ct_activation act, bool pool2 = false) {
    return guarded([&]() -> slot_t {
        TensorObject *x = requireFloat(tensorArg(norm, 0), "conv2d");
        TensorObject *w = requireFloat(tensorArg(with, 0), "conv2d");
        TensorObject *b = requireFloat(tensorArg(with, 1), "conv2d");
        int64_t stride = intValue(with, 2), pad = intValue(with, 3);
        if (x->rank() != 4 || w->rank() != 4)
            throw std::invalid_argument("conv2d requires rank-4 input [n,c,h,w] and weights [k,c,kh,kw]");
        if (x->dim(1) != w->dim(1))
            throw std::invalid_argument("conv2d channel mismatch");
        if (static_cast<int64_t>(b->numel()) != w->dim(0))
            throw std::invalid_argument("conv2d: bias must have one value per output channel");
        int64_t n = x->dim(0), c = x->dim(1), h = x->dim(2), wd = x->dim(3);
        int64_t ko = w->dim(0), kh = w->dim(2), kw = w->dim(3);
        if (stride <= 0 || pad < 0 || h + 2 * pad < kh || wd + 2 * pad < kw)
            throw std::invalid_argument("conv2d: kernel larger than padded input");
        int64_t outShape[4] = {n, ko, (h + 2 * pad - kh) / stride + 1, (wd + 2 * pad - kw) / stride + 1};
        if (pool2) {
            outShape[2] /= 2;
            outShape[3] /= 2;
        }
        TensorObject *out = newTensor(TypeCode::Float32, outShape);
        ctn::ctCheck((pool2 ? ct_conv2d_maxpool2 : ct_conv2d)(
            static_cast<const float *>(x->deviceData()), static_cast<const float *>(w->deviceData()),
            static_cast<const float *>(b->deviceData()), n, c, h, wd, ko, kh, kw, stride, pad, act,
            static_cast<float *>(out->deviceData())));
        return wrap(out);
    });
}

} // namespace

// ---- the reference's 31 entry points (modules/tensor/operators.h:31-61) -------------------

#define CT_OP(name) slot_t name(ArgsView &with, ArgsView &norm, ctx::Context &ctx)
#define CT_UNUSED (void)with, (void)ctx

CT_OP(__tensor_add__) { CT_UNUSED; return binaryBody(norm, CT_ADD, false); }
CT_OP(__tensor_subtract__) { CT_UNUSED; return binaryBody(norm, CT_SUB, false); }
CT_OP(__tensor_multiply__) { CT_UNUSED; return binaryBody(norm, CT_MUL, false); }
CT_OP(__tensor_divide__) { CT_UNUSED; return binaryBody(norm, CT_DIV, false); }
CT_OP(__tensor_pow__) { CT_UNUSED; return binaryBody(norm, CT_POW, true); }
CT_OP(__tensor_lt__) { CT_UNUSED; return compareBody(norm, CT_LT, false); }
CT_OP(__tensor_le__) { CT_UNUSED; return compareBody(norm, CT_LE, false); }
CT_OP(__tensor_gt__) { CT_UNUSED; return compareBody(norm, CT_GT, false); }
CT_OP(__tensor_ge__) { CT_UNUSED; return compareBody(norm, CT_GE, false); }
CT_OP(__tensor_eq__) { CT_UNUSED; return compareBody(norm, CT_EQ, true); }
CT_OP(__tensor_sum_axis__) { CT_UNUSED; return axisBody(norm, AxisKind::Sum, "sum"); }
CT_OP(__tensor_max_axis__) { CT_UNUSED; return axisBody(norm, AxisKind::Max, "max"); }
CT_OP(__tensor_argmax_axis__) { CT_UNUSED; return axisBody(norm, AxisKind::Argmax, "argmax"); }
CT_OP(__tensor_exp__) { CT_UNUSED; return unaryBody(norm, "exp", ct_exp); }
CT_OP(__tensor_log__) { CT_UNUSED; return unaryBody(norm, "log", ct_log); }
CT_OP(__tensor_empty__) { CT_UNUSED; return fillBody(norm, TypeCode::Float32, 0.0); }
CT_OP(__tensor_zeros__) { CT_UNUSED; return fillBody(norm, TypeCode::Float32, 0.0); }
CT_OP(__tensor_ones__) { CT_UNUSED; return fillBody(norm, TypeCode::Float32, 1.0, true); }

CT_OP(__tensor_full__) {
    CT_UNUSED;
    // dtype follows the value's type (operators.cpp:1003-1014)
    return guarded([&]() -> slot_t {
        return fillBody(norm, ctn::normalizeTensorDType(norm.type(1)->code()), scalarValue(norm, 1));
    });
}

CT_OP(__tensor_random__) {
    CT_UNUSED;
    // Unseedable in the reference (std::random_device, runtime.cpp:648); values are drawn on the
    // host the same way and uploaded - not part of parity and not a measured path.
    return guarded([&]() -> slot_t {
        auto shape  = shapeArg(norm, 0);
        double low  = scalarValue(norm, 1), high = scalarValue(norm, 2);
        if (low > high)
            std::swap(low, high);
        uint64_t n = 1;
        for (int64_t d : shape)
            n *= static_cast<uint64_t>(d);
        std::vector<float> host(n);
        std::mt19937 rng(std::random_device{}());
        std::uniform_real_distribution<float> dist(static_cast<float>(low), static_cast<float>(high));
        for (auto &v : host)
            v = dist(rng);
        return wrap(TensorObject::fromHost(TypeCode::Float32, shape, host.data(), mm::autoSpace()));
    });
}

CT_OP(__tensor_range__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        int64_t start = 0, stop = 0, step = 1;
        if (norm.size() == 1) {
            stop = intValue(norm, 0);
        } else {
            start = intValue(norm, 0);
            stop  = intValue(norm, 1);
            if (norm.size() == 3)
                step = intValue(norm, 2);
        }
        if (step == 0)
            throw std::invalid_argument("range step cannot be zero");
        int64_t count = 0; // tensorArange, runtime.cpp:652-673
        if (step > 0 && stop > start)
            count = (stop - start + step - 1) / step;
        else if (step < 0 && stop < start)
            count = (start - stop + (-step) - 1) / (-step);
        int64_t shape[1]  = {count};
        TensorObject *out = newTensor(TypeCode::Int64, shape);
        ctn::ctCheck(ct_arange(start, step, count, static_cast<int64_t *>(out->deviceData())));
        return wrap(out);
    });
}

CT_OP(__tensor_eye__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        int64_t size = intValue(norm, 0);
        if (size < 0)
            throw std::invalid_argument("eye size cannot be negative");
        int64_t shape[2]  = {size, size};
        TensorObject *out = newTensor(TypeCode::Float32, shape);
        ctn::ctCheck(ct_eye(size, static_cast<float *>(out->deviceData())));
        return wrap(out);
    });
}

CT_OP(__tensor_shape__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *t = tensorArg(norm, 0);
        ::Array *shape  = ::Array::create(mm::autoSpace(), t->rank());
        for (size_t i = 0; i < t->rank(); ++i)
            shape->set(i, static_cast<Int64>(t->dim(i)));
        return toSlot(shape);
    });
}

CT_OP(__tensor_sum__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *t = tensorArg(norm, 0);
        double total    = 0.0;
        ctn::ctCheck(ct_sum(t->ctDType(), t->deviceData(), t->numel(), &total));
        return toSlot(total);
    });
}

CT_OP(__tensor_idx__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *t = tensorArg(norm, 0);
        int64_t i       = norm.get<Int64>(1);
        if (t->rank() != 1)
            throw std::invalid_argument("Single-index tensor access requires rank-1 tensor");
        if (i < 0 || i >= t->dim(0))
            throw std::invalid_argument("Tensor index out of bounds");
        return toSlot(t->getAsDouble(static_cast<uint64_t>(i)));
    });
}

CT_OP(__tensor_idx2d__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *t = tensorArg(norm, 0);
        int64_t r = norm.get<Int64>(1), c = norm.get<Int64>(2);
        if (t->rank() != 2)
            throw std::invalid_argument("Two-index tensor access requires rank-2 tensor");
        if (r < 0 || r >= t->dim(0) || c < 0 || c >= t->dim(1))
            throw std::invalid_argument("Tensor index out of bounds");
        return toSlot(t->getAsDouble(static_cast<uint64_t>(r * t->dim(1) + c)));
    });
}

CT_OP(__tensor_matmul__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *a = tensorArg(norm, 0), *b = tensorArg(norm, 1);
        if (a->rank() != 2 || b->rank() != 2)
            throw std::invalid_argument("matmul currently only supports rank-2 tensors");
        if (a->dim(1) != b->dim(0))
            throw std::invalid_argument("matmul dimension mismatch");
        int64_t shape[2]  = {a->dim(0), b->dim(1)};
        TensorObject *out = newTensor(ctn::promoteTensorTypes(a->dtype(), b->dtype()), shape);
        if (a->dtype() == TypeCode::Float32 && b->dtype() == TypeCode::Float32) {
            // Deferred: multiply, divide and the readers decide whether it runs alone, with an
            // activation in its epilogue, or without the transposed copy of its left operand.
            bool spread = a->dim(1) == 1 && b->expr()->kind == ExprKind::Ones;
            ctn::defer(out, spread ? ExprKind::Spread : ExprKind::MatMul, a, b);
            return wrap(out);
        }
        ctn::ctCheck(ct_matmul(a->ctDType(), a->deviceData(), b->ctDType(), b->deviceData(), a->dim(0), a->dim(1),
                               b->dim(1), out->deviceData()));
        return wrap(out);
    });
}

CT_OP(__tensor_transpose__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *t = tensorArg(norm, 0);
        if (t->rank() != 2)
            throw std::invalid_argument("transpose currently only supports rank-2 tensors");
        int64_t shape[2]  = {t->dim(1), t->dim(0)};
        TensorObject *out = newTensor(t->dtype(), shape);
        ctn::defer(out, ExprKind::Transpose, t); // `transpose(X) @ G`: matmul reads X in place
        return wrap(out);
    });
}

CT_OP(__tensor_concat__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *a = tensorOrArrayArg(norm, 0), *b = tensorOrArrayArg(norm, 1);
        int64_t axis    = norm.get<Int64>(2);
        if (a->rank() != b->rank())
            throw std::invalid_argument("concat requires tensors with the same rank");
        if (axis < 0 || axis >= static_cast<int64_t>(a->rank()))
            throw std::invalid_argument("concat axis out of range");
        if (a->dtype() != b->dtype())
            throw std::invalid_argument("concat currently requires matching dtypes");
        std::vector<int64_t> shape(a->shape(), a->shape() + a->rank());
        uint64_t outer = 1, inner = 1;
        for (size_t i = 0; i < a->rank(); ++i) {
            if (static_cast<int64_t>(i) == axis)
                continue;
            if (a->dim(i) != b->dim(i))
                throw std::invalid_argument("concat requires equal non-axis dimensions");
            (static_cast<int64_t>(i) < axis ? outer : inner) *= static_cast<uint64_t>(a->dim(i));
        }
        shape[static_cast<size_t>(axis)] += b->dim(static_cast<size_t>(axis));
        TensorObject *out = newTensor(a->dtype(), shape);
        ctn::ctCheck(ct_concat(a->ctDType(), a->deviceData(), b->deviceData(), outer,
                               static_cast<uint64_t>(a->dim(static_cast<size_t>(axis))),
                               static_cast<uint64_t>(b->dim(static_cast<size_t>(axis))), inner, out->deviceData()));
        return wrap(out);
    });
}

CT_OP(__tensor_reshape__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *t = tensorOrArrayArg(norm, 0);
        auto shape      = shapeArg(norm, 1);
        uint64_t n      = 1;
        for (int64_t d : shape)
            n *= static_cast<uint64_t>(d);
        if (n != t->numel())
            throw std::invalid_argument("reshape changes tensor element count");
        TensorObject *out = newTensor(t->dtype(), shape);
        if (t->rank() == 1 && shape.size() == 2 && shape[1] == 1 && t->dtype() == TypeCode::Float32) {
            ctn::defer(out, ExprKind::Column, t); // `reshape(row_max, [n, 1])` of the softmax idiom
            return wrap(out);
        }
        // the reference copies (runtime.cpp:692-702); tensors are immutable values, so a second shape
        // over the same device buffer is the same value without the pass over HBM.  An array
        // argument was just uploaded into a tensor of its own: that tensor is the source.
        ctn::makeAlias(out, t);
        return wrap(out);
    });
}

CT_OP(__tensor_show__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *t = tensorOrArrayArg(norm, 0);
        t->print(std::cout, isTensor(norm.type(0)) ? norm.type(0) : tensorType());
        std::cout << std::endl;
        return NullSlot;
    });
}

// ---- operators added by this plugin ---------------------------------------------------------

CT_OP(__tensor_relu__) { CT_UNUSED; return unaryBody(norm, "relu", ct_relu); }

CT_OP(__tensor_softmax__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *t = requireFloat(tensorArg(norm, 0), "softmax");
        if (t->rank() != 2)
            throw std::invalid_argument("softmax currently only supports rank-2 tensors");
        TensorObject *out = newTensor(TypeCode::Float32, shapeOf(t));
        ctn::ctCheck(ct_softmax_rows(static_cast<const float *>(t->deviceData()), t->dim(0), t->dim(1),
                                     static_cast<float *>(out->deviceData())));
        return wrap(out);
    });
}

CT_OP(__tensor_dense__) { (void)ctx; return denseBody(with, norm, CT_ACT_NONE); }
CT_OP(__tensor_dense_relu__) { (void)ctx; return denseBody(with, norm, CT_ACT_RELU); }
CT_OP(__tensor_dense_softmax__) { (void)ctx; return denseBody(with, norm, CT_ACT_SOFTMAX); }
CT_OP(__tensor_conv2d__) { (void)ctx; return convBody(with, norm, CT_ACT_NONE); }
CT_OP(__tensor_conv2d_relu__) { (void)ctx; return convBody(with, norm, CT_ACT_RELU); }
CT_OP(__tensor_conv2d_relu_maxpool2__) { (void)ctx; return convBody(with, norm, CT_ACT_RELU, true); }

CT_OP(__tensor_maxpool2d__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *x = requireFloat(tensorArg(norm, 0), "maxpool2d");
        int64_t win     = intValue(norm, 1);
        if (x->rank() != 4 || win <= 0)
            throw std::invalid_argument("maxpool2d requires a rank-4 input [n,c,h,w] and a positive window");
        int64_t shape[4]  = {x->dim(0), x->dim(1), x->dim(2) / win, x->dim(3) / win};
        TensorObject *out = newTensor(TypeCode::Float32, shape);
        ctn::ctCheck(ct_maxpool2d(static_cast<const float *>(x->deviceData()), x->dim(0), x->dim(1), x->dim(2),
                                  x->dim(3), win, static_cast<float *>(out->deviceData())));
        return wrap(out);
    });
}

CT_OP(__tensor_flatten__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *x = tensorArg(norm, 0);
        if (x->rank() < 1)
            throw std::invalid_argument("flatten requires rank >= 1");
        int64_t rows      = x->dim(0);
        int64_t shape[2]  = {rows, rows ? static_cast<int64_t>(x->numel()) / rows : 0};
        TensorObject *out = newTensor(x->dtype(), shape);
        ctn::makeAlias(out, x); // reshape(x, [n, rest]): the same buffer under another shape
        return wrap(out);
    });
}

// transpose(a) @ b in one call (test/run/nn/mnist.cml:39), float tensors.
CT_OP(__tensor_matmul_tn__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *a = requireFloat(tensorArg(norm, 0), "matmul_tn");
        TensorObject *b = requireFloat(tensorArg(norm, 1), "matmul_tn");
        if (a->rank() != 2 || b->rank() != 2)
            throw std::invalid_argument("matmul currently only supports rank-2 tensors");
        if (a->dim(0) != b->dim(0))
            throw std::invalid_argument("matmul dimension mismatch");
        int64_t shape[2]  = {a->dim(1), b->dim(1)};
        TensorObject *out = newTensor(TypeCode::Float32, shape);
        ctn::ctCheck(ct_matmul_tn(
            static_cast<const float *>(a->deviceData()), static_cast<const float *>(b->deviceData()), a->dim(1),
            a->dim(0), b->dim(1), static_cast<float *>(out->deviceData())));
        return wrap(out);
    });
}

// w - lr * g in one pass (test/run/nn/mnist.cml:40), float tensors of one shape.
CT_OP(__tensor_scaled_sub__) {
    CT_UNUSED;
    return guarded([&]() -> slot_t {
        TensorObject *w = requireFloat(tensorArg(norm, 0), "scaled_sub");
        TensorObject *g = requireFloat(tensorArg(norm, 1), "scaled_sub");
        if (!w->sameShape(g))
            throw std::invalid_argument("Tensor binary operation requires matching shapes");
        double lr         = scalarValue(norm, 2);
        TensorObject *out = newTensor(TypeCode::Float32, std::span<const int64_t>(w->shape(), w->rank()));
        ctn::ctCheck(ct_scaled_sub(
            static_cast<const float *>(w->deviceData()), static_cast<const float *>(g->deviceData()), lr, w->numel(),
            static_cast<float *>(out->deviceData())));
        return wrap(out);
    });
}

#undef CT_OP
#undef CT_UNUSED
