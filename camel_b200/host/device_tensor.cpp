#include "device_tensor.h"

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <ostream>
#include <stdexcept>
#include <map>
#include <unordered_set>
#include <utility>
#include <vector>

namespace camel::tensor {

using type::TypeCode;

namespace {
std::mutex g_registryMutex;
std::unordered_set<void *> g_deviceBuffers;
// (device buffer, precision) -> packed form of a weight tensor.  A device buffer is written once,
// when its tensor is created, and lives until releaseAllDeviceBuffers, so the address identifies
// the contents.
std::map<std::pair<void *, int>, void *> g_packedWeights;
// The expression records of all tensors, released with the device buffers.
std::vector<Expr *> g_exprs;
std::atomic<int> g_lazy{-1}; // -1: not read from the environment yet

void *allocDevice(size_t bytes) {
    void *p = nullptr;
    ctCheck(ct_alloc(&p, bytes));
    std::lock_guard<std::mutex> lock(g_registryMutex);
    g_deviceBuffers.insert(p);
    return p;
}

uint64_t product(std::span<const int64_t> shape) {
    uint64_t n = 1;
    for (int64_t d : shape) {
        if (d < 0)
            throw std::invalid_argument("Tensor shape cannot contain negative dimensions");
        n *= static_cast<uint64_t>(d);
    }
    return n;
}
} // namespace

void ctCheck(ct_status status) {
    if (status != CT_OK)
        throw std::runtime_error(ct_last_error());
}

void releaseAllDeviceBuffers() {
    std::lock_guard<std::mutex> lock(g_registryMutex);
    for (auto &entry : g_packedWeights)
        ct_weights_free(entry.second);
    g_packedWeights.clear();
    for (void *p : g_deviceBuffers)
        ct_free(p);
    g_deviceBuffers.clear();
    for (Expr *e : g_exprs)
        delete e;
    g_exprs.clear();
}

const void *packedWeightsFor(const TensorObject *w, int64_t k, int64_t n) {
    if (n <= 32 || k <= 0 || w->dtype() != TypeCode::Float32)
        return nullptr; // narrow outputs read the matrix itself
    const auto key = std::make_pair(const_cast<void *>(w->deviceData()), static_cast<int>(ct_get_precision()));
    std::lock_guard<std::mutex> lock(g_registryMutex);
    auto it = g_packedWeights.find(key);
    if (it != g_packedWeights.end())
        return it->second;
    void *handle = nullptr;
    ctCheck(ct_weights_pack(static_cast<const float *>(w->deviceData()), k, n, &handle));
    g_packedWeights.emplace(key, handle);
    return handle;
}

size_t liveDeviceBuffers() {
    std::lock_guard<std::mutex> lock(g_registryMutex);
    return g_deviceBuffers.size();
}

size_t elementSize(TypeCode dtype) {
    switch (dtype) {
    case TypeCode::Float32:
        return 4;
    case TypeCode::Int64:
        return 8;
    case TypeCode::Bool:
        return 1;
    default:
        throw std::invalid_argument("Unsupported Tensor dtype");
    }
}

bool isSupportedTensorScalar(TypeCode code) {
    return code == TypeCode::Int32 || code == TypeCode::Int64 || code == TypeCode::Float32 ||
           code == TypeCode::Float64 || code == TypeCode::Bool;
}

bool isFloatingTensorType(TypeCode code) { return code == TypeCode::Float32 || code == TypeCode::Float64; }

TypeCode normalizeTensorDType(TypeCode code) {
    if (code == TypeCode::Float32 || code == TypeCode::Float64)
        return TypeCode::Float32;
    if (code == TypeCode::Int32 || code == TypeCode::Int64)
        return TypeCode::Int64;
    if (code == TypeCode::Bool)
        return TypeCode::Bool;
    throw std::invalid_argument("Unsupported Tensor dtype");
}

TypeCode promoteTensorTypes(TypeCode lhs, TypeCode rhs) {
    return fromCtDType(ct_result_dtype(CT_ADD, toCtDType(normalizeTensorDType(lhs)), toCtDType(normalizeTensorDType(rhs))));
}

ct_dtype toCtDType(TypeCode code) {
    switch (normalizeTensorDType(code)) {
    case TypeCode::Float32:
        return CT_F32;
    case TypeCode::Int64:
        return CT_I64;
    default:
        return CT_BOOL;
    }
}

TypeCode fromCtDType(ct_dtype dt) {
    return dt == CT_F32 ? TypeCode::Float32 : (dt == CT_I64 ? TypeCode::Int64 : TypeCode::Bool);
}

TensorObject::TensorObject(TypeCode dtype, uint32_t rank, uint64_t numel, uint64_t byteSize)
    : dtype_(dtype), rank_(rank), numel_(numel), byteSize_(byteSize), expr_(nullptr),
      host_(nullptr), shape_(nullptr) {}

TensorObject *
TensorObject::create(TypeCode dtype, std::span<const int64_t> shape, mm::IAllocator &allocator, bool zeroInit) {
    dtype          = normalizeTensorDType(dtype);
    uint64_t numel = product(shape);
    uint64_t bytes = numel * elementSize(dtype);
    size_t total   = sizeof(TensorObject) + shape.size() * sizeof(int64_t);
    void *memory   = allocator.alloc(total, alignof(TensorObject));
    if (!memory)
        throw std::bad_alloc();
    auto *t   = new (memory) TensorObject(dtype, static_cast<uint32_t>(shape.size()), numel, bytes);
    t->shape_ = t->dims_;
    if (!shape.empty())
        std::memcpy(t->dims_, shape.data(), shape.size() * sizeof(int64_t));
    auto *e  = new Expr;
    e->bytes = bytes;
    e->dtype = toCtDType(dtype);
    e->rank  = static_cast<uint32_t>(shape.size());
    e->numel = numel;
    e->rows  = shape.empty() ? 1 : shape[0];
    e->cols  = shape.size() == 2 ? shape[1] : (e->rows ? static_cast<int64_t>(numel) / e->rows : 0);
    t->expr_ = e;
    {
        std::lock_guard<std::mutex> lock(g_registryMutex);
        g_exprs.push_back(e);
    }
    if (zeroInit && numel > 0)
        ctCheck(ct_fill(toCtDType(dtype), 0.0, numel, t->deviceData()));
    return t;
}

TensorObject *TensorObject::fromHost(
    TypeCode dtype, std::span<const int64_t> shape, const void *hostData, mm::IAllocator &allocator) {
    TensorObject *t = create(dtype, shape, allocator, false);
    if (t->byteSize_ > 0)
        ctCheck(ct_h2d(t->deviceData(), hostData, static_cast<size_t>(t->byteSize_)));
    return t;
}

ct_dtype TensorObject::ctDType() const { return toCtDType(dtype_); }

// ---- deferred device expressions ---------------------------------------------------------

std::recursive_mutex &exprMutex() {
    static std::recursive_mutex m;
    return m;
}

bool lazyEvaluation() {
    int v = g_lazy.load(std::memory_order_relaxed);
    if (v < 0) {
        const char *env = std::getenv("CAMEL_TENSOR_EAGER");
        v               = (env && env[0] && env[0] != '0') ? 0 : 1;
        g_lazy.store(v, std::memory_order_relaxed);
    }
    return v != 0;
}

void setLazyEvaluation(bool on) { g_lazy.store(on ? 1 : 0, std::memory_order_relaxed); }

void *bufferOf(Expr *e) {
    static std::mutex once;
    std::lock_guard<std::mutex> lock(once);
    void *p = e->out.load(std::memory_order_relaxed);
    if (!p) {
        p = allocDevice(static_cast<size_t>(e->bytes));
        e->out.store(p, std::memory_order_release);
    }
    return p;
}

void defer(TensorObject *out, ExprKind kind, const TensorObject *a, const TensorObject *b, int op, double scalar,
           ct_dtype scalarDType, int tensorOnLeft) {
    Expr *e         = out->expr();
    e->kind         = kind;
    e->a            = a ? a->expr() : nullptr;
    e->b            = b ? b->expr() : nullptr;
    e->op           = op;
    e->scalar       = scalar;
    e->scalarDType  = scalarDType;
    e->tensorOnLeft = tensorOnLeft;
    e->pending.store(true, std::memory_order_release);
    if (!lazyEvaluation()) {
        evaluate(e);
        e->kind = ExprKind::Value; // no record: nothing downstream is fused
        e->a = e->b = nullptr;
    }
}

void evaluate(Expr *e) {
    if (!e || !e->pending.load(std::memory_order_acquire))
        return;
    std::lock_guard<std::recursive_mutex> lock(exprMutex());
    if (!e->pending.load(std::memory_order_relaxed))
        return;
    Expr *a = e->a, *b = e->b;
    auto buf = [](Expr *x) { return bufferOf(x); };
    auto f32 = [](Expr *x) { return static_cast<const float *>(bufferOf(x)); };
    ct_status status = CT_OK;
    if (e->numel == 0) {
        e->pending.store(false, std::memory_order_release);
        return;
    }
    switch (e->kind) {
    case ExprKind::Value:
        break;
    case ExprKind::CompareScalar:
        evaluate(a);
        status = ct_compare_scalar(static_cast<ct_compare_op>(e->op), a->dtype, buf(a), e->scalar,
                                   e->tensorOnLeft ? 0 : 1, e->numel, static_cast<uint8_t *>(buf(e)));
        break;
    case ExprKind::ScaleByScalar:
        evaluate(a);
        status = ct_binary_scalar(CT_MUL, a->dtype, buf(a), e->scalar, e->scalarDType, e->tensorOnLeft ? 0 : 1,
                                  e->numel, buf(e));
        break;
    case ExprKind::Transpose:
        evaluate(a);
        status = ct_transpose(a->dtype, buf(a), a->rows, a->cols, buf(e));
        break;
    case ExprKind::MatMul:
        if (a->kind == ExprKind::Transpose && a->pending.load(std::memory_order_relaxed) && a->a->dtype == CT_F32 &&
            b->dtype == CT_F32) {
            // transpose(X) @ G with the transposed copy never made (mnist.cml:39)
            evaluate(a->a);
            evaluate(b);
            status = ct_matmul_tn(f32(a->a), f32(b), e->rows, a->cols, e->cols, static_cast<float *>(buf(e)));
        } else {
            evaluate(a);
            evaluate(b);
            status = ct_matmul(a->dtype, buf(a), b->dtype, buf(b), a->rows, a->cols, b->cols, buf(e));
        }
        break;
    case ExprKind::Ones:
        status = ct_fill(e->dtype, 1.0, e->numel, buf(e));
        break;
    case ExprKind::MaxAxis1:
        evaluate(a);
        status = ct_max_axis(a->dtype, buf(a), a->rows, a->cols, 1, static_cast<float *>(buf(e)));
        break;
    case ExprKind::SumAxis1:
        evaluate(a);
        status = ct_sum_axis(a->dtype, buf(a), a->rows, a->cols, 1, static_cast<float *>(buf(e)));
        break;
    case ExprKind::Column:
        evaluate(a);
        status = ct_d2d(buf(e), buf(a), static_cast<size_t>(e->numel) * 4);
        break;
    case ExprKind::Spread:
        evaluate(a);
        evaluate(b);
        status = ct_matmul(CT_F32, buf(a), CT_F32, buf(b), a->rows, 1, b->cols, buf(e));
        break;
    case ExprKind::Subtract:
        evaluate(a);
        evaluate(b);
        status = ct_binary(CT_SUB, a->dtype, buf(a), b->dtype, buf(b), e->numel, buf(e));
        break;
    case ExprKind::Exp:
        evaluate(a);
        status = ct_exp(f32(a), e->numel, static_cast<float *>(buf(e)));
        break;
    }
    ctCheck(status); // a failed launch leaves the record pending: the next reader sees the error too
    e->pending.store(false, std::memory_order_release);
}

bool TensorObject::sameShape(const TensorObject *other) const {
    if (!other || rank_ != other->rank_)
        return false;
    for (size_t i = 0; i < rank_; ++i)
        if (shape_[i] != other->shape_[i])
            return false;
    return true;
}

const std::byte *TensorObject::rawData() const {
    // several operators may read the same tensor on the host at once (idx on one tensor from two
    // scheduler threads): the mirror is made once, under a lock
    std::byte *mirror = host_.load(std::memory_order_acquire);
    if (mirror)
        return mirror;
    static std::mutex once;
    std::lock_guard<std::mutex> lock(once);
    mirror = host_.load(std::memory_order_relaxed);
    if (!mirror) {
        mirror = static_cast<std::byte *>(std::malloc(byteSize_ ? static_cast<size_t>(byteSize_) : 1));
        if (!mirror)
            throw std::bad_alloc();
        if (byteSize_ > 0) {
            ct_status status = ct_d2h(mirror, deviceData(), static_cast<size_t>(byteSize_));
            if (status != CT_OK) {
                std::free(mirror);
                ctCheck(status);
            }
        }
        host_.store(mirror, std::memory_order_release);
    }
    return mirror;
}

void TensorObject::invalidateHost() const { std::free(host_.exchange(nullptr, std::memory_order_acq_rel)); }

double TensorObject::getAsDouble(uint64_t i) const {
    const std::byte *p = rawData();
    switch (dtype_) {
    case TypeCode::Float32:
        return static_cast<double>(reinterpret_cast<const float *>(p)[i]);
    case TypeCode::Int64:
        return static_cast<double>(reinterpret_cast<const int64_t *>(p)[i]);
    case TypeCode::Bool:
        return reinterpret_cast<const uint8_t *>(p)[i] != 0 ? 1.0 : 0.0;
    default:
        throw std::invalid_argument("Unsupported Tensor dtype");
    }
}

bool TensorObject::equals(const rtdata::Object *other, const type::Type *, bool) const {
    if (this == other)
        return true;
    auto *rhs = dynamic_cast<const TensorObject *>(other);
    if (!rhs || rhs->dtype_ != dtype_ || !sameShape(rhs))
        return false;
    return byteSize_ == 0 || std::memcmp(rawData(), rhs->rawData(), static_cast<size_t>(byteSize_)) == 0;
}

rtdata::Object *TensorObject::clone(mm::IAllocator &allocator, const type::Type *, bool) const {
    TensorObject *copy = create(dtype_, std::span<const int64_t>(shape_, rank_), allocator, false);
    if (byteSize_ > 0)
        ctCheck(ct_d2d(copy->deviceData(), deviceData(), static_cast<size_t>(byteSize_)));
    return copy;
}

void TensorObject::printLevel(std::ostream &os, size_t level, uint64_t &flat) const {
    if (rank_ == 0) {
        os << getAsDouble(0);
        return;
    }
    os << "[";
    for (int64_t i = 0; i < shape_[level]; ++i) {
        if (i > 0)
            os << ", ";
        if (level + 1 == rank_) {
            if (dtype_ == TypeCode::Bool)
                os << (getAsDouble(flat) != 0.0 ? "true" : "false");
            else
                os << getAsDouble(flat);
            ++flat;
        } else {
            printLevel(os, level + 1, flat);
        }
    }
    os << "]";
}

void TensorObject::print(std::ostream &os, const type::Type *) const {
    os << "tensor(";
    uint64_t flat = 0;
    printLevel(os, 0, flat);
    os << ", dtype=" << (dtype_ == TypeCode::Float32 ? "float32" : dtype_ == TypeCode::Int64 ? "int64" : "bool") << ")";
}

void TensorObject::onMoved() { shape_ = dims_; }

void TensorObject::updateRefs(const std::function<rtdata::Object *(rtdata::Object *)> &, const type::Type *) {}

} // namespace camel::tensor
