#include "device_tensor.h"

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <ostream>
#include <stdexcept>
#include <map>
#include <unordered_set>
#include <utility>

namespace camel::tensor {

using type::TypeCode;

namespace {
std::mutex g_registryMutex;
std::unordered_set<void *> g_deviceBuffers;
// (device buffer, precision) -> packed form of a weight tensor.  A device buffer is written once,
// when its tensor is created, and lives until releaseAllDeviceBuffers, so the address identifies
// the contents.
std::map<std::pair<void *, int>, void *> g_packedWeights;

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
    : dtype_(dtype), rank_(rank), numel_(numel), byteSize_(byteSize), dev_(nullptr), host_(nullptr),
      shape_(nullptr) {}

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
    t->dev_ = allocDevice(static_cast<size_t>(bytes));
    if (zeroInit && numel > 0)
        ctCheck(ct_fill(toCtDType(dtype), 0.0, numel, t->dev_));
    return t;
}

TensorObject *TensorObject::fromHost(
    TypeCode dtype, std::span<const int64_t> shape, const void *hostData, mm::IAllocator &allocator) {
    TensorObject *t = create(dtype, shape, allocator, false);
    if (t->byteSize_ > 0)
        ctCheck(ct_h2d(t->dev_, hostData, static_cast<size_t>(t->byteSize_)));
    return t;
}

ct_dtype TensorObject::ctDType() const { return toCtDType(dtype_); }

void TensorObject::deferCompare(const TensorObject *src, ct_compare_op op, double scalar, bool tensorOnLeft) {
    deferred_.src          = src->deviceData(); // a finished buffer: a deferred source is evaluated here
    deferred_.srcDType     = src->ctDType();
    deferred_.op           = op;
    deferred_.scalar       = scalar;
    deferred_.tensorOnLeft = tensorOnLeft ? 1 : 0;
    pending_.store(true, std::memory_order_release);
}

void TensorObject::materialise() const {
    if (!pending_.load(std::memory_order_acquire))
        return;
    static std::mutex once;
    std::lock_guard<std::mutex> lock(once);
    if (!pending_.load(std::memory_order_relaxed))
        return;
    const DeferredCompare &d = deferred_;
    ctCheck(ct_compare_scalar(
        d.op, d.srcDType, d.src, d.scalar, d.tensorOnLeft ? 0 : 1, numel_, static_cast<uint8_t *>(dev_)));
    pending_.store(false, std::memory_order_release);
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
    if (!host_) {
        host_ = static_cast<std::byte *>(std::malloc(byteSize_ ? static_cast<size_t>(byteSize_) : 1));
        if (!host_)
            throw std::bad_alloc();
        if (byteSize_ > 0)
            ctCheck(ct_d2h(host_, deviceData(), static_cast<size_t>(byteSize_)));
    }
    return host_;
}

void TensorObject::invalidateHost() const {
    std::free(host_);
    host_ = nullptr;
}

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
        ctCheck(ct_d2d(copy->dev_, deviceData(), static_cast<size_t>(byteSize_)));
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
