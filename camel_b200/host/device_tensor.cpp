#include "device_tensor.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <ostream>
#include <stdexcept>
#include <map>
#include <unordered_map>
#include <utility>
#include <vector>

namespace camel::tensor {

using type::TypeCode;

namespace {
std::mutex g_registryMutex;
// device buffer -> its size; the sum is g_liveBytes
std::unordered_map<void *, uint64_t> g_deviceBuffers;
uint64_t g_liveBytes = 0;
// (device buffer, precision) -> packed form of a weight tensor and its size.  A device buffer is
// written once, when its tensor is created, and the entry goes when the buffer goes, so the
// address identifies the contents.
struct PackedEntry {
    void *handle;
    uint64_t bytes;
};
std::map<std::pair<void *, int>, PackedEntry> g_packedWeights;
// Every record ever made (freed at unload), and the creation log the scopes work on: the records
// whose object header still holds its claim, in creation order.
std::vector<Expr *> g_exprs;
std::vector<Expr *> g_created;
std::atomic<uint64_t> g_hostReads{0};
std::atomic<int> g_lazy{-1}; // -1: not read from the environment yet

void *allocDevice(size_t bytes) {
    void *p = nullptr;
    ctCheck(ct_alloc(&p, bytes));
    std::lock_guard<std::mutex> lock(g_registryMutex);
    g_deviceBuffers.emplace(p, bytes);
    g_liveBytes += bytes;
    return p;
}

void freeDevice(void *p) {
    std::lock_guard<std::mutex> lock(g_registryMutex);
    for (int prec = 0; prec < 2; ++prec) {
        auto it = g_packedWeights.find(std::make_pair(p, prec));
        if (it != g_packedWeights.end()) {
            ct_weights_free(it->second.handle);
            g_liveBytes -= it->second.bytes;
            g_packedWeights.erase(it);
        }
    }
    auto it = g_deviceBuffers.find(p);
    if (it != g_deviceBuffers.end()) {
        g_liveBytes -= it->second;
        g_deviceBuffers.erase(it);
        ct_free(p); // stream-ordered: kernels already enqueued on the stream still see the data
    }
}

// One user of the record's buffer is gone (the object header at the end of its scope, or a
// deferred computation that has run or will never run).  Call under exprMutex().
void dropUser(Expr *e) {
    if (!e || e->users.fetch_sub(1, std::memory_order_acq_rel) != 1)
        return;
    e->dead.store(true, std::memory_order_release);
    if (e->aliasOf) {
        e->out.store(nullptr, std::memory_order_release); // the buffer belongs to the record it is a view of
        dropUser(e->aliasOf);
    } else if (void *buf = e->out.exchange(nullptr, std::memory_order_acq_rel)) {
        freeDevice(buf);
    }
    std::free(e->host.exchange(nullptr, std::memory_order_acq_rel));
    if (e->pending.exchange(false, std::memory_order_acq_rel)) { // it will never run: its operands are free of it
        dropUser(e->a);
        dropUser(e->b);
    }
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
    std::lock_guard<std::recursive_mutex> exprLock(exprMutex());
    std::lock_guard<std::mutex> lock(g_registryMutex);
    for (auto &entry : g_packedWeights)
        ct_weights_free(entry.second.handle);
    g_packedWeights.clear();
    for (auto &entry : g_deviceBuffers)
        ct_free(entry.first);
    g_deviceBuffers.clear();
    g_liveBytes = 0;
    for (Expr *e : g_exprs) {
        std::free(e->host.load(std::memory_order_relaxed));
        delete e;
    }
    g_exprs.clear();
    g_created.clear();
}

uint64_t beginScope() {
    std::lock_guard<std::mutex> lock(g_registryMutex);
    return g_created.size();
}

void endScope(uint64_t token, std::span<TensorObject *const> keep) {
    std::lock_guard<std::recursive_mutex> exprLock(exprMutex());
    std::vector<Expr *> ended;
    {
        std::lock_guard<std::mutex> lock(g_registryMutex);
        if (token > g_created.size())
            throw std::invalid_argument("endScope: the scope has already been ended by an enclosing one");
        ended.assign(g_created.begin() + static_cast<std::ptrdiff_t>(token), g_created.end());
        g_created.resize(static_cast<size_t>(token));
        for (Expr *e : ended)
            for (TensorObject *k : keep)
                if (k && k->expr() == e) {
                    g_created.push_back(e); // passes to the enclosing scope
                    break;
                }
    }
    for (Expr *e : ended) {
        bool kept = false;
        for (TensorObject *k : keep)
            kept = kept || (k && k->expr() == e);
        if (!kept)
            dropUser(e); // the object header's claim
    }
}

void releaseTensor(TensorObject *t) {
    if (!t)
        return;
    std::lock_guard<std::recursive_mutex> exprLock(exprMutex());
    Expr *e = t->expr();
    {
        std::lock_guard<std::mutex> lock(g_registryMutex);
        auto it = std::find(g_created.rbegin(), g_created.rend(), e); // recent values are near the end
        if (it == g_created.rend())
            return; // its header's claim has been dropped before
        g_created.erase(std::next(it).base());
    }
    dropUser(e);
}

uint64_t liveDeviceBytes() {
    std::lock_guard<std::mutex> lock(g_registryMutex);
    return g_liveBytes;
}

uint64_t hostReadCopies() { return g_hostReads.load(std::memory_order_relaxed); }

const void *packedWeightsFor(const TensorObject *w, int64_t k, int64_t n) {
    if (n <= 32 || k <= 0 || w->dtype() != TypeCode::Float32)
        return nullptr; // narrow outputs read the matrix itself
    const int prec = static_cast<int>(ct_get_precision());
    const auto key = std::make_pair(const_cast<void *>(w->deviceData()), prec);
    std::lock_guard<std::mutex> lock(g_registryMutex);
    auto it = g_packedWeights.find(key);
    if (it != g_packedWeights.end())
        return it->second.handle;
    void *handle = nullptr;
    ctCheck(ct_weights_pack(static_cast<const float *>(w->deviceData()), k, n, &handle));
    // size of the packed planes, for the books: [n][k rounded up to the k-block], two float32
    // planes (3xTF32) or one bf16 plane, each rounded up to 1 KiB
    const int64_t kblock = prec == CT_PREC_BF16 ? 64 : 32, elem = prec == CT_PREC_BF16 ? 2 : 4;
    const uint64_t plane = (static_cast<uint64_t>(n) * ((k + kblock - 1) / kblock * kblock) * elem + 1023) & ~1023ull;
    const uint64_t bytes = plane * (prec == CT_PREC_BF16 ? 1 : 2);
    g_packedWeights.emplace(key, PackedEntry{handle, bytes});
    g_liveBytes += bytes;
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
    : dtype_(dtype), rank_(rank), numel_(numel), byteSize_(byteSize), expr_(nullptr), shape_(nullptr) {}

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
        g_created.push_back(e);
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

void makeAlias(TensorObject *out, const TensorObject *src) {
    Expr *root = src->expr();
    while (root->aliasOf)
        root = root->aliasOf;
    root->users.fetch_add(1, std::memory_order_acq_rel);
    out->expr()->aliasOf = root;
}

void *bufferOf(Expr *e) {
    if (e->aliasOf) {
        if (e->dead.load(std::memory_order_acquire))
            throw std::runtime_error("Tensor used after the scope that created it has ended");
        evaluate(e->aliasOf);
        void *p = bufferOf(e->aliasOf);
        e->out.store(p, std::memory_order_release); // later reads take the fast path
        return p;
    }
    static std::mutex once;
    std::lock_guard<std::mutex> lock(once);
    void *p = e->out.load(std::memory_order_relaxed);
    if (!p) {
        if (e->dead.load(std::memory_order_acquire))
            throw std::runtime_error("Tensor used after the scope that created it has ended");
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
    // until it has run, the record is a user of its operands' buffers
    if (e->a)
        e->a->users.fetch_add(1, std::memory_order_acq_rel);
    if (e->b)
        e->b->users.fetch_add(1, std::memory_order_acq_rel);
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
        dropUser(a);
        dropUser(b);
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
    dropUser(a); // it has run: its operands are free of it (the pointers stay, as facts)
    dropUser(b);
}

void rebindOperand(Expr *e, int which, Expr *to) {
    std::lock_guard<std::recursive_mutex> lock(exprMutex());
    Expr *&slot = which == 0 ? e->a : e->b;
    if (slot == to)
        return;
    if (e->pending.load(std::memory_order_acquire)) {
        if (to)
            to->users.fetch_add(1, std::memory_order_acq_rel);
        Expr *old = slot;
        slot      = to;
        dropUser(old);
    } else {
        slot = to;
    }
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
    std::byte *mirror = expr_->host.load(std::memory_order_acquire);
    if (mirror)
        return mirror;
    static std::mutex once;
    std::lock_guard<std::mutex> lock(once);
    mirror = expr_->host.load(std::memory_order_relaxed);
    if (!mirror) {
        mirror = static_cast<std::byte *>(std::malloc(byteSize_ ? static_cast<size_t>(byteSize_) : 1));
        if (!mirror)
            throw std::bad_alloc();
        if (byteSize_ > 0) {
            // the graph boundary: one device-to-host copy, then the device's error record - a
            // contraction whose bounded wait ran out must not hand its undefined output to the host
            // (one call, one synchronisation: two separate round trips cost a 4096-sample MLP step
            // 20 of its 440 microseconds)
            ct_status status = ct_d2h_checked(mirror, deviceData(), static_cast<size_t>(byteSize_));
            if (status != CT_OK) {
                std::free(mirror);
                ctCheck(status);
            }
            g_hostReads.fetch_add(1, std::memory_order_relaxed);
        }
        expr_->host.store(mirror, std::memory_order_release);
    }
    return mirror;
}

void TensorObject::invalidateHost() const { std::free(expr_->host.exchange(nullptr, std::memory_order_acq_rel)); }

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

// Text form of one element, as the reference prints it (modules/tensor/runtime.cpp:417-448):
// float32 as "% 7.0f." when integral and below 1e10 in magnitude, else "% 7.4g"; int64 right
// aligned in 7 columns; bool as "  true" / " false".
static std::string elementText(const TensorObject &t, uint64_t flat) {
    char text[48];
    switch (t.dtype()) {
    case TypeCode::Float32: {
        const double v = t.getAsDouble(flat);
        const bool whole = v == std::floor(v) && std::abs(v) < 1e10;
        std::snprintf(text, sizeof(text), whole ? "% 7.0f." : "% 7.4g", v);
        return text;
    }
    case TypeCode::Int64:
        std::snprintf(text, sizeof(text), "%7lld", static_cast<long long>(reinterpret_cast<const int64_t *>(t.rawData())[flat]));
        return text;
    case TypeCode::Bool:
        return t.getAsDouble(flat) != 0.0 ? "  true" : " false";
    default:
        return "?";
    }
}

// Layout of modules/tensor/runtime.cpp:484-528: the innermost dimension on one line, wrapped
// (", newline, indent") before an element that would pass column 100; every outer dimension puts
// its slices on lines of their own, indented by 8 columns per level.
void TensorObject::printLevel(std::ostream &os, size_t level, uint64_t &flat) const {
    constexpr size_t kIndentStep = 8, kMaxWidth = 100;
    if (rank_ == 0) {
        os << elementText(*this, 0);
        return;
    }
    const std::string inner((level + 1) * kIndentStep, ' ');
    os << "[";
    if (level + 1 == rank_) {
        size_t width = inner.size();
        for (int64_t i = 0; i < shape_[level]; ++i) {
            const std::string text = elementText(*this, flat++);
            if (i > 0) {
                if (width + 2 + text.size() > kMaxWidth) {
                    os << ",\n" << inner;
                    width = inner.size();
                } else {
                    os << ", ";
                    width += 2;
                }
            }
            os << text;
            width += text.size();
        }
    } else {
        for (int64_t i = 0; i < shape_[level]; ++i) {
            if (i > 0)
                os << ",\n" << inner;
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
