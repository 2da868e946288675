// Device-resident tensor object of the `tensor` plugin.
//
// Takes the place of the reference's TensorObject (modules/tensor/runtime.h:55-109) behind the
// same accessors the operator bodies and the Camel runtime use (rank, numel, dtype, shape, dim,
// rawData, getAsDouble, equals / clone / print / onMoved / updateRefs).  The payload lives in
// device memory owned through the C ABI (ct_alloc / ct_free); a host mirror is created only when
// the runtime reads elements (print, equals, indexing, array conversion) - those reads are the
// graph boundaries where a device-to-host copy is due.
//
// The collector that owns these objects has no finalisers and its root set is never installed
// (include/camel/core/mm/gen.h:224-227), so nothing ever tells the module that a tensor is dead.
// The module therefore keeps its own books: every tensor has a record (Expr) on the C++ heap that
// owns the device buffer and the host mirror and counts who still needs the buffer - the object
// header, and every deferred computation that has it as an operand.  A host that knows where values
// die brackets that region with beginScope() / endScope(): endScope releases what was created
// inside, except the values it is told to keep (and whatever those still need).  A program of
// the reference's training loops (test/run/nn/mnist.cml:33-41) then holds device memory flat.
// Without scopes everything lives until releaseAllDeviceBuffers() at module unload.  A tensor whose
// scope has ended must not be used again; using it raises instead of reading freed memory.
#pragma once

#include "camel/core/mm/alloc/allocator.h"
#include "camel/core/rtdata/base.h"
#include "camel/core/type/base.h"
#include "camel_tensor_b200.h"

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <mutex>
#include <span>
#include <vector>
#include <string>

namespace camel::tensor {

namespace mm     = camel::core::mm;
namespace rtdata = camel::core::rtdata;
namespace type   = camel::core::type;

// Same enumerators as ct_binary_op / ct_compare_op, which follow modules/tensor/runtime.h:39-53.
using BinaryOp  = ct_binary_op;
using CompareOp = ct_compare_op;

// ---- deferred device expressions ---------------------------------------------------------
//
// The reference's programs spell their networks with the module's small operators: relu is
// `h * (h > 0)` (test/run/nn/svm.cml:31), softmax is ten operators with two matmul-by-ones
// broadcasts (test/run/nn/mnist.cml:13-25), the gradient is `transpose(X) @ (probs - y)` and the
// update `W - lr * g` (mnist.cml:39-40).  Run one by one, each of those is a pass over HBM.  So
// the cheap, error-free operators of these idioms do not launch when they are called: they
// allocate their result and record how to compute it (an Expr).  The record is evaluated the
// first time anything reads the tensor's data, and an operator that closes an idiom (multiply,
// subtract, divide, matmul) looks at the records of its operands and calls the fused entry point
// instead (ct_relu, ct_dense with an activation, ct_softmax_rows, ct_matmul_tn, ct_scaled_sub);
// the intermediate tensors are then never written.  Tensors are immutable values
// (src/builtin/operators/ops.cpp:210) and a pending record keeps its operands' buffers alive
// (it counts as a user of each), so it can be evaluated at any later time with the same result.
//
// Operators that can raise a data-dependent error (divide, log, pow) are never deferred, so every
// error is still raised by the operator that the reference raises it from.
enum class ExprKind : uint8_t {
    Value,         // computed when it was created (or uploaded); nothing recorded
    CompareScalar, // a <op> scalar, Bool
    ScaleByScalar, // a * scalar, float32
    Transpose,     // rank-2 transpose of a
    MatMul,        // a @ b, float32
    Ones,          // ones(shape), float32
    MaxAxis1,      // max(a, 1)
    SumAxis1,      // sum(a, 1)
    Column,        // reshape of the vector a[n] to [n, 1]
    Spread,        // a[n, 1] @ ones[1, k]: every row's value k times (b is the ones tensor)
    Subtract,      // a - b, float32
    Exp,           // exp(a)
};

// One record per tensor, on the C++ heap: operands refer to each other through these, because the
// collector moves small object headers (include/camel/core/mm/gen.h:460-520).  `kind` and the
// operand pointers stay after evaluation - they are facts about an immutable value, and the idiom
// recognisers compare them by identity - and only `pending`, `users` and `dead` change.  Fields
// other than those are written before the tensor is handed out, or under exprMutex().
//
// Lifetime.  `users` counts who needs the device buffer: the object header (one, from creation
// until the tensor's scope ends) and every record that is still pending and has this one as an
// operand.  When it drops to zero the buffer, the packed form of a weight tensor and the host
// mirror are freed and the record is marked dead.  The record itself stays allocated until the
// module is unloaded (about a hundred bytes), so operand pointers never dangle and a use after the
// end of a scope is caught instead of reading freed memory.
struct Expr {
    ExprKind kind = ExprKind::Value;
    std::atomic<bool> pending{false};
    std::atomic<bool> dead{false};
    std::atomic<int> users{1};
    Expr *aliasOf = nullptr; // this tensor is another shape over that record's buffer (reshape, flatten)
    Expr *a = nullptr, *b = nullptr;
    std::atomic<void *> out{nullptr}; // the tensor's device buffer, allocated at first use (bufferOf)
    std::atomic<std::byte *> host{nullptr}; // malloc'd host mirror, nullptr while there is none
    uint64_t bytes = 0;
    ct_dtype dtype = CT_F32;
    uint32_t rank  = 0;
    uint64_t numel = 0;
    int64_t rows = 0, cols = 0; // of a rank-2 tensor; [n] counts as n rows of one
    int op             = 0;     // ct_compare_op of CompareScalar
    double scalar      = 0.0;
    ct_dtype scalarDType = CT_F32;
    int tensorOnLeft   = 1;
};

class TensorObject;

// Serialises evaluation and every look at operand records (operators run on up to 32 threads).
std::recursive_mutex &exprMutex();
// Runs the kernels of a pending record (operands first); no-op when it has run.
void evaluate(Expr *e);
// The record's device buffer, allocated on the first call.
void *bufferOf(Expr *e);
// Records how `out` (freshly created, not yet visible to anyone) is computed.  With deferral
// switched off it is computed at once and keeps no record.
void defer(TensorObject *out, ExprKind kind, const TensorObject *a, const TensorObject *b = nullptr, int op = 0,
           double scalar = 0.0, ct_dtype scalarDType = CT_F32, int tensorOnLeft = 1);
// Deferral is on unless CAMEL_TENSOR_EAGER=1 is set when the module is loaded.
bool lazyEvaluation();
void setLazyEvaluation(bool on);
// Replaces operand `which` (0: a, 1: b) of a pending record, moving its claim on the buffer.
void rebindOperand(Expr *e, int which, Expr *to);
// Makes `out` (freshly created, same dtype and element count) a second shape over `src`'s device
// buffer instead of a copy: tensors are immutable values, so no reader can tell the difference.
// `out` keeps `src`'s buffer alive for as long as it lives itself.
void makeAlias(TensorObject *out, const TensorObject *src);

// ---- scopes ------------------------------------------------------------------------------
// beginScope() returns a token; endScope(token, keep) ends the life of every tensor created since
// that token (on any thread) except those in `keep`, which pass to the enclosing scope.  What a kept
// tensor still needs (operands of a computation it has deferred) survives with it.  Scopes nest;
// tokens must be ended innermost first.  A scheduler calls these around a region whose only
// surviving values it knows - a `sync` block or a function frame: its result slot is the keep list.
uint64_t beginScope();
void endScope(uint64_t token, std::span<TensorObject *const> keep);
// Ends the life of one tensor, whichever scope it belongs to: for a host that knows a value's last
// use (a loop variable that has just been replaced).  No effect on a tensor already released.
void releaseTensor(TensorObject *t);
// Bytes of device memory the module's tensors own right now (packed weight layouts included).
uint64_t liveDeviceBytes();
// Device-to-host copies made for host reads (print, equals, indexing) since the module was loaded.
uint64_t hostReadCopies();

class TensorObject : public rtdata::Object {
  public:
    TensorObject(const TensorObject &)            = delete;
    TensorObject &operator=(const TensorObject &) = delete;

    // Header (and shape) come from `allocator`; the payload is a device buffer.  With zeroInit
    // the buffer is cleared on the device.
    static TensorObject *
    create(type::TypeCode dtype, std::span<const int64_t> shape, mm::IAllocator &allocator, bool zeroInit = false);
    // Same, filled from host memory (one host-to-device copy).
    static TensorObject *fromHost(
        type::TypeCode dtype, std::span<const int64_t> shape, const void *hostData, mm::IAllocator &allocator);

    size_t rank() const { return rank_; }
    uint64_t numel() const { return numel_; }
    type::TypeCode dtype() const { return dtype_; }
    ct_dtype ctDType() const;
    size_t byteSize() const { return byteSize_; }
    const int64_t *shape() const { return shape_; }
    int64_t dim(size_t index) const { return shape_[index]; }
    bool sameShape(const TensorObject *other) const;

    // Device payload.  The buffer is allocated when it is first asked for, so a tensor whose
    // expression (below) is never evaluated never owns device memory; an expression that has not
    // run yet is evaluated first, so every reader sees finished data.
    void *deviceData() { return const_cast<void *>(static_cast<const TensorObject *>(this)->deviceData()); }
    const void *deviceData() const {
        if (expr_->pending.load(std::memory_order_acquire))
            evaluate(expr_);
        void *p = expr_->out.load(std::memory_order_acquire);
        return p ? p : bufferOf(expr_); // bufferOf raises for a tensor whose scope has ended
    }
    // How this tensor came about (see Expr); never null, stable while the object moves.
    Expr *expr() const { return expr_; }

    // Host view of the payload: copies device -> host on first use after a device write.
    const std::byte *rawData() const;
    double getAsDouble(uint64_t flatIndex) const;

    bool equals(const rtdata::Object *other, const type::Type *type, bool deep = false) const override;
    rtdata::Object *clone(mm::IAllocator &allocator, const type::Type *type, bool deep = false) const override;
    void print(std::ostream &os, const type::Type *type) const override;
    void onMoved() override;
    void updateRefs(
        const std::function<rtdata::Object *(rtdata::Object *)> &relocate, const type::Type *type) override;

    // Drops the host mirror (after the device payload was rewritten in place).
    void invalidateHost() const;

  private:
    TensorObject(type::TypeCode dtype, uint32_t rank, uint64_t numel, uint64_t byteSize);
    void printLevel(std::ostream &os, size_t level, uint64_t &flat) const;

    type::TypeCode dtype_;
    uint32_t rank_;
    uint64_t numel_;
    uint64_t byteSize_;
    Expr *expr_;
    int64_t *shape_;
    int64_t dims_[]; // rank_ entries, in the same allocation as the header
};

// Storage dtype rules of the reference (modules/tensor/runtime.cpp:530-580).
size_t elementSize(type::TypeCode dtype);
bool isSupportedTensorScalar(type::TypeCode code);
bool isFloatingTensorType(type::TypeCode code);
type::TypeCode normalizeTensorDType(type::TypeCode code);
type::TypeCode promoteTensorTypes(type::TypeCode lhs, type::TypeCode rhs);
ct_dtype toCtDType(type::TypeCode code);
type::TypeCode fromCtDType(ct_dtype dt);

// Throws std::runtime_error carrying ct_last_error() when a C-ABI call fails; the operator
// wrapper turns it into a RuntimeFault exactly like the reference's withTensorErrors
// (modules/tensor/operators.cpp:103-109).
void ctCheck(ct_status status);

// Tensor-core layout of a weight tensor (ct_weights_pack), built at its first use as the `with`
// argument of dense and kept until the device buffers are released; nullptr where dense does not
// take one.  Tensors are immutable values, so the layout never goes stale.
const void *packedWeightsFor(const TensorObject *w, int64_t k, int64_t n);

// Releases every device buffer and record created so far (module unload).
void releaseAllDeviceBuffers();
size_t liveDeviceBuffers();

} // namespace camel::tensor
