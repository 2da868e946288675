// TEST INFRASTRUCTURE, not product code.
//
// Plain-C driver around the UNMODIFIED reference tensor module (OpenCML/Camel,
// modules/tensor/{runtime,operators,type}.cpp plus the src/core closure), which the
// Makefile next to this file compiles from the reference checkout into
// oracle/_ref/libcamel_tensor_ref.so.  Operators are fetched from the reference's own
// getTensorOpsMap() (modules/tensor/operators.cpp:160-194) and called exactly as the graph
// executors call them: op(withView, normView, ctx) (src/passes/sched/nodevm/nodevm.cpp:588).
// Only tests, the smoke check and the bench's CPU-baseline leg may load the result.
//
// Nothing here restates reference arithmetic; it only marshals arguments.

#include "camel/core/error/runtime.h"
#include "camel/core/mm.h"
#include "camel/core/operator.h"
#include "camel/core/rtdata/array.h"
#include "camel/core/type/composite/array.h"
#include "operators.h"
#include "runtime.h"
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

// Vector-backed ArgsView (abstract interface: include/camel/core/operator.h:51-63).
struct VecArgsView final : ArgsView {
    std::vector<slot_t> slots;
    std::vector<Type *> types;
    size_t size() const override { return slots.size(); }
    slot_t slot(size_t i) const override { return slots[i]; }
    void setSlot(size_t i, slot_t v) override { slots[i] = v; }
    TypeCode code(size_t i) const override { return types[i]->code(); }
    Type *type(size_t i) const override { return types[i]; }
};

// Input tensors are built in plain malloc blocks (TensorObject::create takes any allocator,
// modules/tensor/runtime.cpp:256-279) so that they can be released after the call; only the
// operator's own result comes from the reference's collector-owned space.
class InputAllocator final : public mm::IAllocator {
  public:
    void *alloc(size_t size, size_t align) override {
        (void)align;
        constexpr size_t kHeader = 64; // room for an object header in front, zeroed
        auto *base               = static_cast<std::byte *>(std::calloc(1, size + kHeader));
        if (!base)
            return nullptr;
        blocks_.push_back(base);
        return base + kHeader;
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

InputAllocator g_inputs;
size_t g_nurseryBytes = 0;

// A nested Camel array (the value of a literal such as [[1.0, 2.0], [3.0, 4.0]]) and its type.
Type *leafType(int dtype) {
    switch (dtype) {
    case 0:
        return Type::Float32();
    case 1:
        return Type::Int64();
    case 2:
        return Type::Bool();
    case 3:
        return Type::Float64();
    default:
        return Type::Int32();
    }
}

Type *nestedArrayType(int dtype, int rank) {
    Type *t = leafType(dtype);
    for (int level = 0; level < rank; ++level)
        t = ArrayType::create(t);
    return t;
}

::Array *nestedArray(int dtype, int rank, const int64_t *shape, const double *&leaves, mm::IAllocator &alloc) {
    ::Array *arr = ::Array::create(alloc, static_cast<size_t>(shape[0]));
    for (int64_t i = 0; i < shape[0]; ++i) {
        if (rank > 1) {
            arr->set<camel::core::rtdata::Object *>(
                static_cast<size_t>(i),
                static_cast<camel::core::rtdata::Object *>(nestedArray(dtype, rank - 1, shape + 1, leaves, alloc)));
            continue;
        }
        double v = *leaves++;
        switch (dtype) {
        case 0:
            arr->set<float>(static_cast<size_t>(i), static_cast<float>(v));
            break;
        case 1:
            arr->set<int64_t>(static_cast<size_t>(i), static_cast<int64_t>(v));
            break;
        case 2:
            arr->set<bool>(static_cast<size_t>(i), v != 0.0);
            break;
        case 3:
            arr->set<double>(static_cast<size_t>(i), v);
            break;
        default:
            arr->set<int32_t>(static_cast<size_t>(i), static_cast<int32_t>(v));
            break;
        }
    }
    return arr;
}
void *g_lastOut       = nullptr;

TypeCode dtypeCode(int dtype) {
    switch (dtype) {
    case 0:
        return TypeCode::Float32;
    case 1:
        return TypeCode::Int64;
    default:
        return TypeCode::Bool;
    }
}

int dtypeId(TypeCode code) {
    if (code == TypeCode::Float32)
        return 0;
    if (code == TypeCode::Int64)
        return 1;
    return 2;
}

Type *dtypeType(int dtype) {
    switch (dtype) {
    case 0:
        return Type::Float32();
    case 1:
        return Type::Int64();
    default:
        return Type::Bool();
    }
}

// Types are bump-allocated and never freed (src/core/type/base.cpp:438), so make each once.
Type *tensorTypeFor(int dtype) {
    static Type *cache[3] = {nullptr, nullptr, nullptr};
    int k                 = dtype < 0 || dtype > 2 ? 2 : dtype;
    if (!cache[k])
        cache[k] = TensorType::Dynamic(dtypeType(k));
    return cache[k];
}

} // namespace

extern "C" {

// kind: 0 tensor, 1 int64 scalar, 2 float64 scalar, 3 float32 scalar, 4 int32 scalar,
//       5 bool scalar, 6 int64 array (e.g. a shape), 8 nested array literal: `rank` levels of
//       extents `shape`, leaves read from `data` (doubles, row-major) as the type `dtype` names
// dtype (tensors): 0 float32, 1 int64, 2 bool(u8); (array leaves): also 3 float64, 4 int32
struct camel_ref_arg {
    int32_t kind;
    int32_t dtype;
    int32_t rank;
    int32_t pad_;
    const int64_t *shape; // tensor shape, or the int64 array's items (rank = length)
    const void *data;
    double f64;
    int64_t i64;
};

// kind: 0 tensor, 1 float64 scalar, 2 int64 array, 3 null
struct camel_ref_out {
    int32_t kind;
    int32_t dtype;
    int32_t rank;
    int32_t pad_;
    int64_t shape[8];
    uint64_t numel;
    const void *data; // owned by the driver until the next call
    double f64;
    double seconds; // steady_clock time of the operator_t call alone
};

// Returns 0 on success, 1 when the operator raised (message in err), 2 on a driver error.
int camel_ref_call(
    const char *op, int nargs, const camel_ref_arg *args, camel_ref_out *out, char *err,
    int errlen) {
    auto fail = [&](int rc, const std::string &msg) {
        if (err && errlen > 0) {
            std::strncpy(err, msg.c_str(), static_cast<size_t>(errlen) - 1);
            err[errlen - 1] = '\0';
        }
        return rc;
    };
    try {
        auto &space = mm::autoSpace();
        g_inputs.releaseAll();
        // Operator results of <= 4 KB come from a 32 MB bump-allocated nursery
        // (include/camel/core/mm/gen.h:256-288).  When it fills the reference collects it,
        // and with no root set installed by any host (setObjectRootSet has no caller in the
        // reference) that collection is not survivable.  Stop short of it with a clear error.
        if (g_nurseryBytes > 24u * 1024u * 1024u)
            return fail(2, "reference nursery nearly full: start a fresh process");
        std::free(g_lastOut);
        g_lastOut = nullptr;

        static const auto ops = getTensorOpsMap();
        auto it               = ops.find(op);
        if (it == ops.end())
            return fail(2, std::string("unknown operator: ") + op);

        VecArgsView with, norm;
        for (int i = 0; i < nargs; ++i) {
            const camel_ref_arg &a = args[i];
            switch (a.kind) {
            case 0: {
                std::span<const int64_t> shape(a.shape, static_cast<size_t>(a.rank));
                TensorObject *t = TensorObject::create(dtypeCode(a.dtype), shape, g_inputs, false);
                if (t->byteSize() > 0)
                    std::memcpy(t->rawData(), a.data, t->byteSize());
                norm.slots.push_back(
                    camel::core::rtdata::toSlot(static_cast<camel::core::rtdata::Object *>(t)));
                norm.types.push_back(tensorTypeFor(a.dtype));
                break;
            }
            case 1:
                norm.slots.push_back(camel::core::rtdata::toSlot<int64_t>(a.i64));
                norm.types.push_back(Type::Int64());
                break;
            case 2:
                norm.slots.push_back(camel::core::rtdata::toSlot<double>(a.f64));
                norm.types.push_back(Type::Float64());
                break;
            case 3:
                norm.slots.push_back(camel::core::rtdata::toSlot<float>(static_cast<float>(a.f64)));
                norm.types.push_back(Type::Float32());
                break;
            case 4:
                norm.slots.push_back(
                    camel::core::rtdata::toSlot<int32_t>(static_cast<int32_t>(a.i64)));
                norm.types.push_back(Type::Int32());
                break;
            case 5:
                norm.slots.push_back(camel::core::rtdata::toSlot<bool>(a.i64 != 0));
                norm.types.push_back(Type::Bool());
                break;
            case 6: {
                ::Array *arr = ::Array::create(g_inputs, static_cast<size_t>(a.rank));
                for (int k = 0; k < a.rank; ++k)
                    arr->set<int64_t>(static_cast<size_t>(k), a.shape[k]);
                norm.slots.push_back(
                    camel::core::rtdata::toSlot(static_cast<camel::core::rtdata::Object *>(arr)));
                static Type *intArray = ArrayType::create(Type::Int64());
                norm.types.push_back(intArray);
                break;
            }
            case 8: {
                const double *leaves = static_cast<const double *>(a.data);
                ::Array *arr         = nestedArray(a.dtype, a.rank, a.shape, leaves, g_inputs);
                norm.slots.push_back(
                    camel::core::rtdata::toSlot(static_cast<camel::core::rtdata::Object *>(arr)));
                norm.types.push_back(nestedArrayType(a.dtype, a.rank));
                break;
            }
            default:
                return fail(2, "bad argument kind");
            }
        }

        // No tensor operator dereferences the context (each body starts `(void)ctx;`,
        // modules/tensor/operators.cpp:585-587), so a null reference stands in for it.
        camel::core::context::Context *nullCtx = nullptr;
        auto t0                                = std::chrono::steady_clock::now();
        slot_t result                          = it->second(with, norm, *nullCtx);
        auto t1                                = std::chrono::steady_clock::now();

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
            out->dtype = dtypeId(t->dtype());
            out->rank  = static_cast<int32_t>(t->rank());
            for (size_t k = 0; k < t->rank() && k < 8; ++k)
                out->shape[k] = t->dim(k);
            out->numel = t->numel();
            if (t->byteSize() + sizeof(TensorObject) + 8 * t->rank() <= 4096 + 64)
                g_nurseryBytes += t->byteSize() + sizeof(TensorObject) + 8 * t->rank() + 64;
            if (t->byteSize() > 0) {
                g_lastOut = std::malloc(t->byteSize());
                std::memcpy(g_lastOut, t->rawData(), t->byteSize());
            }
            out->data = g_lastOut;
        }
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

// Operator URI suffixes the reference registers (keys of getTensorOpsMap()), '\n'-joined.
int camel_ref_list_ops(char *buf, int buflen) {
    std::string s;
    for (const auto &kv : getTensorOpsMap())
        s += kv.first + "\n";
    if (static_cast<int>(s.size()) + 1 > buflen)
        return -static_cast<int>(s.size()) - 1;
    std::memcpy(buf, s.c_str(), s.size() + 1);
    return static_cast<int>(s.size());
}

// "group\turi\tsignature" lines from getTensorOperatorGroups()
// (modules/tensor/operators.cpp:196-583); static resolvers print "<static>".
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
