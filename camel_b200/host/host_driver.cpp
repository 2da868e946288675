// Plain-C test harness around the plugin's operator table: builds ArgsViews from raw buffers,
// calls an operator body exactly as Camel's executors do - op(withView, normView, ctx)
// (src/passes/sched/nodevm/nodevm.cpp:588) - and hands the result back as raw buffers.  The
// argument and result structs have the layout of the oracle's reference driver, so one Python
// front end drives both the reference module and this plugin.
#include "dlpack.h"
#include "camel/core/error/runtime.h"
#include "camel/core/mm.h"
#include "camel/core/operator.h"
#include "camel/core/rtdata/array.h"
#include "camel/core/type/composite/array.h"
#include "device_tensor.h"
#include "tensor_ops.h"
#include "type.h"

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

using camel::tensor::TensorObject;
using camel::tensor::TensorType;
namespace mm = camel::core::mm;
using camel::core::type::ArrayType;
using camel::core::type::Type;
using camel::core::type::TypeCode;

namespace {

struct VecArgsView final : ArgsView {
    std::vector<slot_t> slots;
    std::vector<Type *> types;
    size_t size() const override { return slots.size(); }
    slot_t slot(size_t i) const override { return slots[i]; }
    void setSlot(size_t i, slot_t v) override { slots[i] = v; }
    TypeCode code(size_t i) const override { return types[i]->code(); }
    Type *type(size_t i) const override { return types[i]; }
};

// Object headers of the arguments live in malloc blocks that are released after the call.
class ScratchAllocator final : public mm::IAllocator {
  public:
    void *alloc(size_t size, size_t) override {
        auto *base = static_cast<std::byte *>(std::calloc(1, size + 64));
        if (!base)
            return nullptr;
        blocks_.push_back(base);
        return base + 64;
    }
    void free(void *) override {}
    void releaseAll() {
        for (auto *b : blocks_)
            std::free(b);
        blocks_.clear();
    }

  private:
    std::vector<std::byte *> blocks_;
};

ScratchAllocator g_scratch;
void *g_lastOut = nullptr;

TypeCode dtypeCode(int d) { return d == 0 ? TypeCode::Float32 : (d == 1 ? TypeCode::Int64 : TypeCode::Bool); }
Type *dtypeType(int d) { return d == 0 ? Type::Float32() : (d == 1 ? Type::Int64() : Type::Bool()); }

Type *tensorTypeFor(int dtype) {
    static Type *cache[3] = {nullptr, nullptr, nullptr};
    int k                 = dtype < 0 || dtype > 2 ? 2 : dtype;
    if (!cache[k])
        cache[k] = TensorType::Dynamic(dtypeType(k));
    return cache[k];
}

} // namespace

extern "C" {

// kind (low byte): 0 tensor, 1 int64, 2 float64, 3 float32, 4 int32, 5 bool, 6 int64 array;
// kind | 0x100 places the argument in the `with` list instead of the `norm` list.
struct camel_host_arg {
    int32_t kind, dtype, rank, pad_;
    const int64_t *shape;
    const void *data;
    double f64;
    int64_t i64;
};

struct camel_host_out {
    int32_t kind, dtype, rank, pad_; // kind: 0 tensor, 1 float64, 2 int64 array, 3 null
    int64_t shape[8];
    uint64_t numel;
    const void *data; // owned by the harness until the next call
    double f64;
    double seconds;
};

int camel_ref_call(const char *op, int nargs, const camel_host_arg *args, camel_host_out *out, char *err, int errlen) {
    auto fail = [&](int rc, const std::string &msg) {
        if (err && errlen > 0) {
            std::strncpy(err, msg.c_str(), static_cast<size_t>(errlen) - 1);
            err[errlen - 1] = '\0';
        }
        return rc;
    };
    try {
        // everything the previous call created is garbage now
        g_scratch.releaseAll();
        camel::tensor::releaseAllDeviceBuffers();
        std::free(g_lastOut);
        g_lastOut = nullptr;

        static const auto ops = getTensorOpsMap();
        auto it               = ops.find(op);
        if (it == ops.end())
            return fail(2, std::string("unknown operator: ") + op);

        VecArgsView with, norm;
        for (int i = 0; i < nargs; ++i) {
            const camel_host_arg &a = args[i];
            VecArgsView &dst        = (a.kind & 0x100) ? with : norm;
            switch (a.kind & 0xff) {
            case 0: {
                std::span<const int64_t> shape(a.shape, static_cast<size_t>(a.rank));
                TensorObject *t = TensorObject::fromHost(dtypeCode(a.dtype), shape, a.data, g_scratch);
                dst.slots.push_back(camel::core::rtdata::toSlot(static_cast<camel::core::rtdata::Object *>(t)));
                dst.types.push_back(tensorTypeFor(a.dtype));
                break;
            }
            case 1:
                dst.slots.push_back(camel::core::rtdata::toSlot<int64_t>(a.i64));
                dst.types.push_back(Type::Int64());
                break;
            case 2:
                dst.slots.push_back(camel::core::rtdata::toSlot<double>(a.f64));
                dst.types.push_back(Type::Float64());
                break;
            case 3:
                dst.slots.push_back(camel::core::rtdata::toSlot<float>(static_cast<float>(a.f64)));
                dst.types.push_back(Type::Float32());
                break;
            case 4:
                dst.slots.push_back(camel::core::rtdata::toSlot<int32_t>(static_cast<int32_t>(a.i64)));
                dst.types.push_back(Type::Int32());
                break;
            case 5:
                dst.slots.push_back(camel::core::rtdata::toSlot<bool>(a.i64 != 0));
                dst.types.push_back(Type::Bool());
                break;
            case 6: {
                ::Array *arr = ::Array::create(g_scratch, static_cast<size_t>(a.rank));
                for (int k = 0; k < a.rank; ++k)
                    arr->set<int64_t>(static_cast<size_t>(k), a.shape[k]);
                dst.slots.push_back(camel::core::rtdata::toSlot(static_cast<camel::core::rtdata::Object *>(arr)));
                static Type *intArray = ArrayType::create(Type::Int64());
                dst.types.push_back(intArray);
                break;
            }
            default:
                return fail(2, "bad argument kind");
            }
        }

        camel::core::context::Context *nullCtx = nullptr; // no operator body touches the context
        auto t0       = std::chrono::steady_clock::now();
        slot_t result = it->second(with, norm, *nullCtx);
        ct_sync();
        auto t1 = std::chrono::steady_clock::now();

        std::memset(out, 0, sizeof(*out));
        out->seconds  = std::chrono::duration<double>(t1 - t0).count();
        std::string n = op;
        if (n == "sum" || n == "idx" || n == "idx2d") {
            out->kind = 1;
            out->f64  = camel::core::rtdata::fromSlot<double>(result);
        } else if (n == "shape") {
            auto *arr = camel::core::rtdata::fromSlot<::Array *>(result);
            out->kind = 2;
            out->rank = static_cast<int32_t>(arr->size());
            for (size_t k = 0; k < arr->size() && k < 8; ++k)
                out->shape[k] = arr->get<int64_t>(k);
        } else if (n == "show") {
            out->kind = 3;
        } else {
            auto *t    = camel::core::rtdata::fromSlot<TensorObject *>(result);
            out->kind  = 0;
            out->dtype = static_cast<int32_t>(t->ctDType());
            out->rank  = static_cast<int32_t>(t->rank());
            for (size_t k = 0; k < t->rank() && k < 8; ++k)
                out->shape[k] = t->dim(k);
            out->numel = t->numel();
            if (t->byteSize() > 0) {
                g_lastOut = std::malloc(t->byteSize());
                std::memcpy(g_lastOut, t->rawData(), t->byteSize());
            }
            out->data = g_lastOut;
            t->invalidateHost();
        }
        ct_status async = ct_check();
        if (async != CT_OK)
            return fail(1, ct_last_error());
        return 0;
    } catch (const camel::core::error::RuntimeFault &f) {
        std::string msg;
        for (const auto &s : f.formatArgs())
            msg += s;
        if (msg.empty())
            msg = f.what();
        return fail(1, msg);
    } catch (const std::exception &e) {
        return fail(1, e.what());
    }
}

int camel_ref_list_ops(char *buf, int buflen) {
    std::string s;
    for (const auto &kv : getTensorOpsMap())
        s += kv.first + "\n";
    if (static_cast<int>(s.size()) + 1 > buflen)
        return -static_cast<int>(s.size()) - 1;
    std::memcpy(buf, s.c_str(), s.size() + 1);
    return static_cast<int>(s.size());
}

// DLPack round trip of a float32 matrix, for the tests: host -> tensor -> device export (must be
// the tensor's own buffer, kDLCUDA) -> import (device copy) -> host export -> import -> host.
// Returns 0, or a negative step number; out_host receives the matrix after both round trips.
int camel_host_dlpack_roundtrip(const float *host, int64_t rows, int64_t cols, float *out_host, char *err, int errlen) {
    try {
        int64_t shape[2] = {rows, cols};
        TensorObject *t  = TensorObject::fromHost(TypeCode::Float32, shape, host, g_scratch);
        camel::tensor::DLManagedTensor *dev = camel::tensor::tensorToDLPackDevice(t);
        if (dev->dl_tensor.device.device_type != camel::tensor::kDLCUDA || dev->dl_tensor.data != t->deviceData() ||
            dev->dl_tensor.ndim != 2 || dev->dl_tensor.shape[0] != rows || dev->dl_tensor.shape[1] != cols)
            return -1;
        TensorObject *u = camel::tensor::tensorFromDLPackCopy(dev, g_scratch);
        dev->deleter(dev);
        if (u->deviceData() == t->deviceData())
            return -2;
        camel::tensor::DLManagedTensor *cpu = camel::tensor::tensorToDLPackCopy(u);
        if (cpu->dl_tensor.device.device_type != camel::tensor::kDLCPU)
            return -3;
        TensorObject *v = camel::tensor::tensorFromDLPackCopy(cpu, g_scratch);
        cpu->deleter(cpu);
        std::memcpy(out_host, v->rawData(), v->byteSize());
        return 0;
    } catch (const std::exception &e) {
        if (err && errlen > 0) {
            std::strncpy(err, e.what(), static_cast<size_t>(errlen) - 1);
            err[errlen - 1] = '\0';
        }
        return -9;
    }
}

// The relu idiom of the reference's programs, `h * (h > threshold)`, as one operator chain on one
// tensor, for the tests.  out_product receives the product, out_mask the comparison (read after the
// product).  Returns 1 if the comparison was still unevaluated after the multiply (so the multiply
// did not read it), 0 if the multiply evaluated it, negative on error.
int camel_host_relu_idiom(const float *host, int64_t n, double threshold, int mask_first, float *out_product,
                          uint8_t *out_mask, char *err, int errlen) {
    try {
        static const auto ops = getTensorOpsMap();
        int64_t shape[1]      = {n};
        TensorObject *h       = TensorObject::fromHost(TypeCode::Float32, shape, host, g_scratch);
        camel::core::context::Context *nullCtx = nullptr;
        Type *f32Tensor                        = tensorTypeFor(0);

        VecArgsView with, cmp;
        cmp.slots.push_back(camel::core::rtdata::toSlot(static_cast<camel::core::rtdata::Object *>(h)));
        cmp.types.push_back(f32Tensor);
        cmp.slots.push_back(camel::core::rtdata::toSlot<double>(threshold));
        cmp.types.push_back(Type::Float64());
        slot_t maskSlot = ops.at("gt")(with, cmp, *nullCtx);
        auto *mask      = camel::core::rtdata::fromSlot<TensorObject *>(maskSlot);

        VecArgsView mul;
        auto push = [&](TensorObject *t, int dtype) {
            mul.slots.push_back(camel::core::rtdata::toSlot(static_cast<camel::core::rtdata::Object *>(t)));
            mul.types.push_back(tensorTypeFor(dtype));
        };
        if (mask_first) {
            push(mask, 2);
            push(h, 0);
        } else {
            push(h, 0);
            push(mask, 2);
        }
        auto *prod   = camel::core::rtdata::fromSlot<TensorObject *>(ops.at("multiply")(with, mul, *nullCtx));
        int deferred = mask->deferred() != nullptr ? 1 : 0;
        if (prod->dtype() != TypeCode::Float32 || prod->numel() != static_cast<uint64_t>(n))
            return -1;
        std::memcpy(out_product, prod->rawData(), prod->byteSize());
        std::memcpy(out_mask, mask->rawData(), mask->byteSize());
        if (mask->deferred() != nullptr)
            return -2;
        return deferred;
    } catch (const std::exception &e) {
        if (err && errlen > 0) {
            std::strncpy(err, e.what(), static_cast<size_t>(errlen) - 1);
            err[errlen - 1] = '\0';
        }
        return -9;
    }
}

int camel_ref_list_groups(char *buf, int buflen) {
    std::string s;
    for (const auto &g : getTensorOperatorGroups())
        for (const auto &[uri, resolver] : g->resolvers())
            s += g->name() + "\t" + uri + "\t" + resolver->signature() + "\n";
    if (static_cast<int>(s.size()) + 1 > buflen)
        return -static_cast<int>(s.size()) - 1;
    std::memcpy(buf, s.c_str(), s.size() + 1);
    return static_cast<int>(s.size());
}

} // extern "C"
