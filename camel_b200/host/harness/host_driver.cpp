// NOT part of tensor.cmo: a plain-C harness around the plugin's operator table, linked only into
// libcamel_tensor_host_test.so (tests and the bench's plugin leg).  It stands in for the `camel`
// executable, which cannot be built without Clang/Conan/ANTLR: it builds ArgsViews from raw
// buffers, calls an operator body exactly as Camel's executors do - op(withView, normView, ctx)
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
#include <thread>
#include <utility>
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
ScratchAllocator g_persist; // values that outlive the steps of a loop (weights); released when the loop starts
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

// A nested Camel array (the value of a literal such as [[1.0, 2.0], [3.0, 4.0]]) and its type;
// leaf codes: 0 float32, 1 int64, 2 bool, 3 float64, 4 int32.
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

::Array *nestedArray(int dtype, int rank, const int64_t *shape, const double *&leaves) {
    using camel::core::rtdata::Object;
    ::Array *arr = ::Array::create(g_scratch, static_cast<size_t>(shape[0]));
    for (int64_t i = 0; i < shape[0]; ++i) {
        const size_t at = static_cast<size_t>(i);
        if (rank > 1) {
            arr->set<Object *>(at, static_cast<Object *>(nestedArray(dtype, rank - 1, shape + 1, leaves)));
            continue;
        }
        const double v = *leaves++;
        if (dtype == 0)
            arr->set<float>(at, static_cast<float>(v));
        else if (dtype == 1)
            arr->set<int64_t>(at, static_cast<int64_t>(v));
        else if (dtype == 2)
            arr->set<bool>(at, v != 0.0);
        else if (dtype == 3)
            arr->set<double>(at, v);
        else
            arr->set<int32_t>(at, static_cast<int32_t>(v));
    }
    return arr;
}

} // namespace

extern "C" {

// kind (low byte): 0 tensor, 1 int64, 2 float64, 3 float32, 4 int32, 5 bool, 6 int64 array,
// 7 session handle, 8 nested array literal (`rank` levels of extents `shape`, leaves from `data`
// as doubles, leaf type `dtype`); kind | 0x100 places the argument in the `with` list instead of
// the `norm` list.
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

// Values kept between the calls of a session (below): what an operator returned, with its type.
struct SessionValue {
    slot_t slot;
    Type *type;
    int kind; // as camel_host_out.kind
};
static std::vector<SessionValue> g_session;

static Type *intArrayType() {
    static Type *t = ArrayType::create(Type::Int64());
    return t;
}

// Appends the arguments to the `with` and `norm` views; returns an empty string or the complaint.
static std::string buildArgs(int nargs, const camel_host_arg *args, VecArgsView &with, VecArgsView &norm) {
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
            dst.types.push_back(intArrayType());
            break;
        }
        case 7: { // the value an earlier call of the session returned
            if (a.i64 < 0 || a.i64 >= static_cast<int64_t>(g_session.size()))
                return "bad session handle";
            dst.slots.push_back(g_session[static_cast<size_t>(a.i64)].slot);
            dst.types.push_back(g_session[static_cast<size_t>(a.i64)].type);
            break;
        }
        case 8: {
            const double *leaves = static_cast<const double *>(a.data);
            ::Array *arr         = nestedArray(a.dtype, a.rank, a.shape, leaves);
            dst.slots.push_back(camel::core::rtdata::toSlot(static_cast<camel::core::rtdata::Object *>(arr)));
            dst.types.push_back(nestedArrayType(a.dtype, a.rank));
            break;
        }
        default:
            return "bad argument kind";
        }
    }
    return "";
}

static int resultKind(const std::string &op) {
    if (op == "sum" || op == "idx" || op == "idx2d")
        return 1;
    if (op == "shape")
        return 2;
    return op == "show" ? 3 : 0;
}

// Copies a result out (a tensor through its host view: the device-to-host read of a graph boundary).
static void exportResult(int kind, slot_t result, camel_host_out *out) {
    out->kind = kind;
    if (kind == 1) {
        out->f64 = camel::core::rtdata::fromSlot<double>(result);
    } else if (kind == 2) {
        auto *arr = camel::core::rtdata::fromSlot<::Array *>(result);
        out->rank = static_cast<int32_t>(arr->size());
        for (size_t k = 0; k < arr->size() && k < 8; ++k)
            out->shape[k] = arr->get<int64_t>(k);
    } else if (kind == 0) {
        auto *t    = camel::core::rtdata::fromSlot<TensorObject *>(result);
        out->dtype = static_cast<int32_t>(t->ctDType());
        out->rank  = static_cast<int32_t>(t->rank());
        for (size_t k = 0; k < t->rank() && k < 8; ++k)
            out->shape[k] = t->dim(k);
        out->numel = t->numel();
        std::free(g_lastOut);
        g_lastOut = nullptr;
        if (t->byteSize() > 0) {
            g_lastOut = std::malloc(t->byteSize());
            std::memcpy(g_lastOut, t->rawData(), t->byteSize());
        }
        out->data = g_lastOut;
        t->invalidateHost();
    }
}

static int failWith(char *err, int errlen, int rc, const std::string &msg) {
    if (err && errlen > 0) {
        std::strncpy(err, msg.c_str(), static_cast<size_t>(errlen) - 1);
        err[errlen - 1] = '\0';
    }
    return rc;
}

static std::string faultText(const camel::core::error::RuntimeFault &f) {
    std::string msg;
    for (const auto &s : f.formatArgs())
        msg += s;
    return msg.empty() ? std::string(f.what()) : msg;
}

int camel_ref_call(const char *op, int nargs, const camel_host_arg *args, camel_host_out *out, char *err, int errlen) {
    try {
        // everything the previous call created is garbage now
        g_session.clear();
        g_scratch.releaseAll();
        camel::tensor::releaseAllDeviceBuffers();
        std::free(g_lastOut);
        g_lastOut = nullptr;

        static const auto ops = getTensorOpsMap();
        auto it               = ops.find(op);
        if (it == ops.end())
            return failWith(err, errlen, 2, std::string("unknown operator: ") + op);

        VecArgsView with, norm;
        std::string complaint = buildArgs(nargs, args, with, norm);
        if (!complaint.empty())
            return failWith(err, errlen, 2, complaint);

        camel::core::context::Context *nullCtx = nullptr; // no operator body touches the context
        int kind      = resultKind(op);
        auto t0       = std::chrono::steady_clock::now();
        slot_t result = it->second(with, norm, *nullCtx);
        if (kind == 0) // an operator may only have recorded its work: have it run inside the timed region
            camel::core::rtdata::fromSlot<TensorObject *>(result)->deviceData();
        ct_sync();
        auto t1 = std::chrono::steady_clock::now();

        std::memset(out, 0, sizeof(*out));
        out->seconds = std::chrono::duration<double>(t1 - t0).count();
        exportResult(kind, result, out);
        ct_status async = ct_check();
        if (async != CT_OK)
            return failWith(err, errlen, 1, ct_last_error());
        return 0;
    } catch (const camel::core::error::RuntimeFault &f) {
        return failWith(err, errlen, 1, faultText(f));
    } catch (const std::exception &e) {
        return failWith(err, errlen, 1, e.what());
    }
}

// ---- sessions: a chain of operator calls whose values stay on the device -------------------
//
// camel_ref_call uploads its arguments and reads its result back, like a program of one operator.
// A session runs a program of many: every call's value is kept (handle = its index) and can be
// an argument of later calls (argument kind 7), so tensors pass from operator to operator exactly
// as they do between the nodes of a Camel graph - on the device and, where the plugin defers work,
// unevaluated.  begin releases everything earlier calls created.

int camel_host_session_begin(int lazy) {
    g_session.clear();
    g_scratch.releaseAll();
    camel::tensor::releaseAllDeviceBuffers();
    if (lazy >= 0)
        camel::tensor::setLazyEvaluation(lazy != 0);
    return 0;
}

// Keeps a host tensor (or scalar) as a session value without calling an operator.
int camel_host_session_put(const camel_host_arg *arg, int64_t *handle, char *err, int errlen) {
    try {
        VecArgsView with, norm;
        std::string complaint = buildArgs(1, arg, with, norm);
        if (!complaint.empty())
            return failWith(err, errlen, 2, complaint);
        VecArgsView &v = norm.slots.empty() ? with : norm;
        g_session.push_back({v.slots[0], v.types[0], (arg->kind & 0xff) == 0 ? 0 : -1});
        *handle = static_cast<int64_t>(g_session.size()) - 1;
        return 0;
    } catch (const std::exception &e) {
        return failWith(err, errlen, 1, e.what());
    }
}

int camel_host_session_call(
    const char *op, int nargs, const camel_host_arg *args, int64_t *handle, char *err, int errlen) {
    try {
        static const auto ops = getTensorOpsMap();
        auto it               = ops.find(op);
        if (it == ops.end())
            return failWith(err, errlen, 2, std::string("unknown operator: ") + op);
        VecArgsView with, norm;
        std::string complaint = buildArgs(nargs, args, with, norm);
        if (!complaint.empty())
            return failWith(err, errlen, 2, complaint);
        camel::core::context::Context *nullCtx = nullptr;
        slot_t result = it->second(with, norm, *nullCtx);
        int kind      = resultKind(op);
        Type *type    = nullptr;
        if (kind == 0)
            type = tensorTypeFor(static_cast<int>(camel::core::rtdata::fromSlot<TensorObject *>(result)->ctDType()));
        else if (kind == 1)
            type = Type::Float64();
        else if (kind == 2)
            type = intArrayType();
        g_session.push_back({result, type, kind});
        *handle = static_cast<int64_t>(g_session.size()) - 1;
        return 0;
    } catch (const camel::core::error::RuntimeFault &f) {
        return failWith(err, errlen, 1, faultText(f));
    } catch (const std::exception &e) {
        return failWith(err, errlen, 1, e.what());
    }
}

// Reads a session value back (evaluating it if need be).
int camel_host_session_fetch(int64_t handle, camel_host_out *out, char *err, int errlen) {
    try {
        if (handle < 0 || handle >= static_cast<int64_t>(g_session.size()) || g_session[handle].kind < 0)
            return failWith(err, errlen, 2, "bad session handle");
        std::memset(out, 0, sizeof(*out));
        exportResult(g_session[handle].kind, g_session[handle].slot, out);
        ct_status async = ct_check();
        if (async != CT_OK)
            return failWith(err, errlen, 1, ct_last_error());
        return 0;
    } catch (const camel::core::error::RuntimeFault &f) {
        return failWith(err, errlen, 1, faultText(f));
    } catch (const std::exception &e) {
        return failWith(err, errlen, 1, e.what());
    }
}

// Makes sure a tensor value has been computed (without reading it back) and waits for the device;
// returns the number of kernels the library has launched so far, or -1.
int64_t camel_host_session_finish(int64_t handle, char *err, int errlen) {
    try {
        if (handle >= 0 && handle < static_cast<int64_t>(g_session.size()) && g_session[handle].kind == 0)
            camel::core::rtdata::fromSlot<TensorObject *>(g_session[handle].slot)->deviceData();
        if (ct_sync() != CT_OK)
            return failWith(err, errlen, -1, ct_last_error());
        return static_cast<int64_t>(ct_launch_count());
    } catch (const camel::core::error::RuntimeFault &f) {
        return failWith(err, errlen, -1, faultText(f));
    } catch (const std::exception &e) {
        return failWith(err, errlen, -1, e.what());
    }
}

// 1 if the tensor value still waits to be computed, 0 if it has been, -1 if it is no tensor.
int camel_host_session_pending(int64_t handle) {
    if (handle < 0 || handle >= static_cast<int64_t>(g_session.size()) || g_session[handle].kind != 0)
        return -1;
    return camel::core::rtdata::fromSlot<TensorObject *>(g_session[handle].slot)->expr()->pending.load() ? 1 : 0;
}

// The idioms of the reference's programs from many threads at once, the way the Taskflow scheduler
// calls operators (src/passes/sched/taskflow/taskflow.cpp:157-196, up to 32 workers).  All threads
// share one input tensor h[rows, cols] and one mask `h > 0` - whose deferred evaluation, buffer
// allocation and host mirror they therefore race for - and each computes h * mask and the softmax
// chain of mnist.cml:13-25 over h.  out_prod / out_probs receive every thread's results
// ([threads][rows*cols]), out_mask the mask read at the end.  Returns 0 or the number of threads
// that raised (the first message in err).
int camel_host_threads_idioms(const float *host, int64_t rows, int64_t cols, int threads, float *out_prod,
                              float *out_probs, uint8_t *out_mask, char *err, int errlen) {
    try {
        g_session.clear();
        g_scratch.releaseAll();
        camel::tensor::releaseAllDeviceBuffers();
        camel::tensor::setLazyEvaluation(true);
        static const auto ops = getTensorOpsMap();
        camel::core::context::Context *nullCtx = nullptr;
        using camel::core::rtdata::fromSlot;
        using camel::core::rtdata::toSlot;
        auto objSlot = [](TensorObject *t) { return toSlot(static_cast<camel::core::rtdata::Object *>(t)); };
        int64_t shape[2] = {rows, cols};
        TensorObject *h  = TensorObject::fromHost(TypeCode::Float32, shape, host, g_scratch);
        Type *f32T = tensorTypeFor(0), *boolT = tensorTypeFor(2);
        auto call = [&](const char *op, std::initializer_list<std::pair<slot_t, Type *>> args) {
            VecArgsView with, norm;
            for (const auto &a : args) {
                norm.slots.push_back(a.first);
                norm.types.push_back(a.second);
            }
            return ops.at(op)(with, norm, *nullCtx);
        };
        auto shapeSlot = [&](int64_t a, int64_t b) { // int[] argument; the allocator behind it is mutex-guarded
            ::Array *arr = ::Array::create(mm::autoSpace(), 2);
            arr->set<int64_t>(0, a);
            arr->set<int64_t>(1, b);
            return toSlot(static_cast<camel::core::rtdata::Object *>(arr));
        };
        slot_t hs   = objSlot(h);
        slot_t mask = call("gt", {{hs, f32T}, {toSlot<double>(0.0), Type::Float64()}});
        const size_t count = static_cast<size_t>(rows * cols);
        std::vector<std::string> failures(static_cast<size_t>(threads));
        std::vector<std::thread> pool;
        for (int t = 0; t < threads; ++t) {
            pool.emplace_back([&, t]() {
                try {
                    slot_t prod = (t & 1) ? call("multiply", {{mask, boolT}, {hs, f32T}})
                                          : call("multiply", {{hs, f32T}, {mask, boolT}});
                    Type *ia    = intArrayType();
                    slot_t i1   = toSlot<int64_t>(1);
                    slot_t rmax = call("max_axis", {{hs, f32T}, {i1, Type::Int64()}});
                    slot_t rm2  = call("reshape", {{rmax, f32T}, {shapeSlot(rows, 1), ia}});
                    slot_t one1 = call("ones", {{shapeSlot(1, cols), ia}});
                    slot_t rmb  = call("matmul", {{rm2, f32T}, {one1, f32T}});
                    slot_t stab = call("subtract", {{hs, f32T}, {rmb, f32T}});
                    slot_t ex   = call("exp", {{stab, f32T}});
                    slot_t rsum = call("sum_axis", {{ex, f32T}, {i1, Type::Int64()}});
                    slot_t rs2  = call("reshape", {{rsum, f32T}, {shapeSlot(rows, 1), ia}});
                    slot_t one2 = call("ones", {{shapeSlot(1, cols), ia}});
                    slot_t rsb  = call("matmul", {{rs2, f32T}, {one2, f32T}});
                    slot_t prob = call("divide", {{ex, f32T}, {rsb, f32T}});
                    if (t % 3 == 2) // some threads read the shared mask while others still multiply by it
                        (void)fromSlot<TensorObject *>(mask)->rawData();
                    std::memcpy(out_prod + t * count, fromSlot<TensorObject *>(prod)->rawData(), count * 4);
                    std::memcpy(out_probs + t * count, fromSlot<TensorObject *>(prob)->rawData(), count * 4);
                } catch (const camel::core::error::RuntimeFault &f) {
                    failures[static_cast<size_t>(t)] = faultText(f);
                } catch (const std::exception &e) {
                    failures[static_cast<size_t>(t)] = e.what();
                }
            });
        }
        for (auto &th : pool)
            th.join();
        std::memcpy(out_mask, fromSlot<TensorObject *>(mask)->rawData(), count);
        int failed = 0;
        for (const auto &f : failures)
            if (!f.empty() && failed++ == 0)
                failWith(err, errlen, 1, f);
        if (ct_check() != CT_OK && failed++ == 0)
            failWith(err, errlen, 1, ct_last_error());
        return failed;
    } catch (const std::exception &e) {
        return failWith(err, errlen, -1, e.what());
    }
}

// ---- what the module keeps on the device, and the scopes that end it -------------------------

uint64_t camel_host_live_device_bytes(void) { return camel::tensor::liveDeviceBytes(); }
uint64_t camel_host_live_device_buffers(void) { return camel::tensor::liveDeviceBuffers(); }
uint64_t camel_host_read_copies(void) { return camel::tensor::hostReadCopies(); }

// A scope over session values: everything created after `begin` except the handles in `keep` is
// released at `end` (the values stay in the session table but must not be used again).
uint64_t camel_host_scope_begin(void) { return camel::tensor::beginScope(); }

int camel_host_scope_end(uint64_t token, int nkeep, const int64_t *keep, char *err, int errlen) {
    try {
        std::vector<TensorObject *> kept;
        for (int i = 0; i < nkeep; ++i) {
            if (keep[i] < 0 || keep[i] >= static_cast<int64_t>(g_session.size()) || g_session[keep[i]].kind != 0)
                return failWith(err, errlen, 2, "bad session handle in the keep list");
            kept.push_back(camel::core::rtdata::fromSlot<TensorObject *>(g_session[keep[i]].slot));
        }
        camel::tensor::endScope(token, kept);
        return 0;
    } catch (const std::exception &e) {
        return failWith(err, errlen, 1, e.what());
    }
}

// The training loop of test/run/nn/mnist.cml:27-41 (`update`, applied `steps` times), operator by
// operator through the plugin's bodies, each step inside a scope whose only surviving value is the
// new W - what a scheduler does that ends a frame when `update` returns.  x [n, d] (bias column
// included), y one-hot [n, classes], w [d, classes] in, w out.  live_bytes_out (may be null)
// receives the module's device bytes after every step; seconds_out the wall time of the loop
// including the final read-back.  use_scopes == 0 runs the same loop without scopes.
int camel_host_sgd_loop(
    const float *x, const float *y, float *w, int64_t n, int64_t d, int64_t classes, double lr, int steps,
    int use_scopes, uint64_t *live_bytes_out, double *seconds_out, char *err, int errlen) {
    try {
        g_session.clear();
        g_scratch.releaseAll();
        camel::tensor::releaseAllDeviceBuffers();
        static const auto ops = getTensorOpsMap();
        camel::core::context::Context *nullCtx = nullptr;
        using camel::core::rtdata::fromSlot;
        using camel::core::rtdata::toSlot;
        using Arg = std::pair<slot_t, Type *>;
        auto call = [&](const char *op, std::initializer_list<Arg> args) {
            VecArgsView with, norm;
            for (const auto &a : args) {
                norm.slots.push_back(a.first);
                norm.types.push_back(a.second);
            }
            return ops.at(op)(with, norm, *nullCtx);
        };
        auto objSlot = [](TensorObject *t) { return toSlot(static_cast<camel::core::rtdata::Object *>(t)); };
        auto shapeArg = [&](int64_t a, int64_t b) -> Arg {
            ::Array *arr = ::Array::create(g_scratch, 2);
            arr->set<int64_t>(0, a);
            arr->set<int64_t>(1, b);
            return {toSlot(static_cast<camel::core::rtdata::Object *>(arr)), intArrayType()};
        };
        Type *f32T = tensorTypeFor(0);
        int64_t xs[2] = {n, d}, ys[2] = {n, classes}, ws[2] = {d, classes};
        Arg X{objSlot(TensorObject::fromHost(TypeCode::Float32, xs, x, g_scratch)), f32T};
        Arg Y{objSlot(TensorObject::fromHost(TypeCode::Float32, ys, y, g_scratch)), f32T};
        Arg W{objSlot(TensorObject::fromHost(TypeCode::Float32, ws, w, g_scratch)), f32T};
        Arg one{toSlot<int64_t>(1), Type::Int64()};
        ct_sync();
        auto t0 = std::chrono::steady_clock::now();
        for (int step = 0; step < steps; ++step) {
            uint64_t scope = use_scopes ? camel::tensor::beginScope() : 0;
            // let logits = X @ W;  let probs = softmax(logits)            (mnist.cml:13-25, 29-30)
            Arg logits{call("matmul", {X, W}), f32T};
            Arg rowMax{call("max_axis", {logits, one}), f32T};
            Arg rowMax2{call("reshape", {rowMax, shapeArg(n, 1)}), f32T};
            Arg ones1{call("ones", {shapeArg(1, classes)}), f32T};
            Arg spreadMax{call("matmul", {rowMax2, ones1}), f32T};
            Arg stable{call("subtract", {logits, spreadMax}), f32T};
            Arg expLogits{call("exp", {stable}), f32T};
            Arg rowSum{call("sum_axis", {expLogits, one}), f32T};
            Arg rowSum2{call("reshape", {rowSum, shapeArg(n, 1)}), f32T};
            Arg ones2{call("ones", {shapeArg(1, classes)}), f32T};
            Arg spreadSum{call("matmul", {rowSum2, ones2}), f32T};
            Arg probs{call("divide", {expLogits, spreadSum}), f32T};
            // let grad = transpose(X) @ (probs - y_onehot);  W - lr * (1.0 / m) * grad   (mnist.cml:32-33)
            Arg diff{call("subtract", {probs, Y}), f32T};
            Arg xt{call("transpose", {X}), f32T};
            Arg grad{call("matmul", {xt, diff}), f32T};
            Arg scale{toSlot<double>(lr * (1.0 / static_cast<double>(n))), Type::Float64()};
            Arg scaled{call("multiply", {scale, grad}), f32T};
            Arg next{call("subtract", {W, scaled}), f32T};
            if (use_scopes) {
                TensorObject *keep[1] = {fromSlot<TensorObject *>(next.first)};
                keep[0]->deviceData(); // the frame's result is computed before the frame ends
                camel::tensor::endScope(scope, keep);
            }
            if (use_scopes) // the loop variable has been replaced: the old weights have had their last use
                camel::tensor::releaseTensor(fromSlot<TensorObject *>(W.first));
            W = next;
            if (live_bytes_out)
                live_bytes_out[step] = camel::tensor::liveDeviceBytes();
        }
        TensorObject *wt = fromSlot<TensorObject *>(W.first);
        std::memcpy(w, wt->rawData(), wt->byteSize());
        auto t1 = std::chrono::steady_clock::now();
        if (seconds_out)
            *seconds_out = std::chrono::duration<double>(t1 - t0).count();
        if (ct_check() != CT_OK)
            return failWith(err, errlen, 1, ct_last_error());
        return 0;
    } catch (const camel::core::error::RuntimeFault &f) {
        return failWith(err, errlen, 1, faultText(f));
    } catch (const std::exception &e) {
        return failWith(err, errlen, 1, e.what());
    }
}

// The MLP forward of a Camel program, per step, the way a scheduler runs it: the batch arrives in
// host memory (a tensor is made from it: one host-to-device copy), three operator calls through
// operator_t, then the host reads the probabilities and the arg-max back (two device-to-host
// copies through the tensor's host view); the step's values die with its frame (a scope).
// Weights are tensors that live across steps.  mode 0: the fused operators dense_relu<w,b>,
// dense_relu<w,b>, dense_softmax<w,b>, argmax.  mode 1: the module's small operators only, as the
// reference's programs spell them - `x @ w`, `h * (h > 0)`, the softmax function of
// mnist.cml:13-25 (no bias terms) - which run through the deferred-expression recognisers.
// x: [steps_distinct][batch][d0] host batches used round-robin.  probs/argmax receive the last
// step's results; step_seconds[steps] the wall time of every step.
int camel_host_mlp_forward(
    int mode, const float *x, int steps_distinct, int64_t batch, int64_t d0, int64_t d1, int64_t d2, int64_t d3,
    const float *w1, const float *b1, const float *w2, const float *b2, const float *w3, const float *b3, int steps,
    float *probs, int64_t *argmax, double *step_seconds, uint64_t *launches_out, char *err, int errlen) {
    try {
        g_session.clear();
        g_scratch.releaseAll();
        g_persist.releaseAll();
        camel::tensor::releaseAllDeviceBuffers();
        camel::tensor::setLazyEvaluation(true);
        static const auto ops = getTensorOpsMap();
        camel::core::context::Context *nullCtx = nullptr;
        using camel::core::rtdata::fromSlot;
        using camel::core::rtdata::toSlot;
        using Arg = std::pair<slot_t, Type *>;
        auto call = [&](const char *op, std::initializer_list<Arg> with_args, std::initializer_list<Arg> args) {
            VecArgsView with, norm;
            for (const auto &a : with_args) {
                with.slots.push_back(a.first);
                with.types.push_back(a.second);
            }
            for (const auto &a : args) {
                norm.slots.push_back(a.first);
                norm.types.push_back(a.second);
            }
            return ops.at(op)(with, norm, *nullCtx);
        };
        auto objSlot = [](TensorObject *t) { return toSlot(static_cast<camel::core::rtdata::Object *>(t)); };
        auto shapeArg = [&](int64_t a, int64_t b) -> Arg {
            ::Array *arr = ::Array::create(g_scratch, 2);
            arr->set<int64_t>(0, a);
            arr->set<int64_t>(1, b);
            return {toSlot(static_cast<camel::core::rtdata::Object *>(arr)), intArrayType()};
        };
        Type *f32T = tensorTypeFor(0), *i64T = tensorTypeFor(1);
        auto weight = [&](const float *host, int64_t r, int64_t c) -> Arg {
            int64_t shape[2] = {r, c};
            return {objSlot(TensorObject::fromHost(TypeCode::Float32, std::span<const int64_t>(shape, c ? 2 : 1), host, g_persist)), f32T};
        };
        Arg W1 = weight(w1, d0, d1), W2 = weight(w2, d1, d2), W3 = weight(w3, d2, d3);
        Arg B1 = weight(b1, d1, 0), B2 = weight(b2, d2, 0), B3 = weight(b3, d3, 0);
        Arg one{toSlot<int64_t>(1), Type::Int64()};
        auto softmaxIdiom = [&](Arg logits, int64_t n, int64_t k) -> Arg {
            Arg rowMax2{call("reshape", {}, {Arg{call("max_axis", {}, {logits, one}), f32T}, shapeArg(n, 1)}), f32T};
            Arg spreadMax{call("matmul", {}, {rowMax2, Arg{call("ones", {}, {shapeArg(1, k)}), f32T}}), f32T};
            Arg expLogits{call("exp", {}, {Arg{call("subtract", {}, {logits, spreadMax}), f32T}}), f32T};
            Arg rowSum2{call("reshape", {}, {Arg{call("sum_axis", {}, {expLogits, one}), f32T}, shapeArg(n, 1)}), f32T};
            Arg spreadSum{call("matmul", {}, {rowSum2, Arg{call("ones", {}, {shapeArg(1, k)}), f32T}}), f32T};
            return {call("divide", {}, {expLogits, spreadSum}), f32T};
        };
        auto reluIdiom = [&](Arg h) -> Arg {
            Arg zero{toSlot<double>(0.0), Type::Float64()};
            Arg mask{call("gt", {}, {h, zero}), tensorTypeFor(2)};
            return {call("multiply", {}, {h, mask}), f32T};
        };
        const uint64_t launches0 = ct_launch_count();
        for (int step = 0; step < steps; ++step) {
            const float *batch_host = x + static_cast<size_t>(step % steps_distinct) * batch * d0;
            auto t0           = std::chrono::steady_clock::now();
            uint64_t scope    = camel::tensor::beginScope();
            int64_t xshape[2] = {batch, d0};
            Arg X{objSlot(TensorObject::fromHost(TypeCode::Float32, xshape, batch_host, g_scratch)), f32T};
            Arg P{0, f32T};
            if (mode == 0) {
                Arg h1{call("dense_relu", {W1, B1}, {X}), f32T};
                Arg h2{call("dense_relu", {W2, B2}, {h1}), f32T};
                P = Arg{call("dense_softmax", {W3, B3}, {h2}), f32T};
            } else {
                Arg h1 = reluIdiom(Arg{call("matmul", {}, {X, W1}), f32T});
                Arg h2 = reluIdiom(Arg{call("matmul", {}, {h1, W2}), f32T});
                P      = softmaxIdiom(Arg{call("matmul", {}, {h2, W3}), f32T}, batch, d3);
            }
            Arg A{call("argmax_axis", {}, {P, one}), i64T};
            TensorObject *pt = fromSlot<TensorObject *>(P.first), *at = fromSlot<TensorObject *>(A.first);
            std::memcpy(probs, pt->rawData(), pt->byteSize());
            std::memcpy(argmax, at->rawData(), at->byteSize());
            camel::tensor::endScope(scope, {});
            if ((step & 15) == 15)
                g_scratch.releaseAll(); // headers of finished steps (the weights' come from g_persist)
            step_seconds[step] = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        }
        if (launches_out)
            *launches_out = ct_launch_count() - launches0;
        if (ct_check() != CT_OK)
            return failWith(err, errlen, 1, ct_last_error());
        return 0;
    } catch (const camel::core::error::RuntimeFault &f) {
        return failWith(err, errlen, 1, faultText(f));
    } catch (const std::exception &e) {
        return failWith(err, errlen, 1, e.what());
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
