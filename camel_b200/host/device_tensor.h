// Device-resident tensor object of the `tensor` plugin.
//
// Takes the place of the reference's TensorObject (modules/tensor/runtime.h:55-109) behind the
// same accessors the operator bodies and the Camel runtime use (rank, numel, dtype, shape, dim,
// rawData, getAsDouble, equals / clone / print / onMoved / updateRefs).  The payload lives in
// device memory owned through the C ABI (ct_alloc / ct_free); a host mirror is created only when
// the runtime reads elements (print, equals, indexing, array conversion) - those reads are the
// graph boundaries where a device-to-host copy is due.
//
// The collector that owns these objects has no finalisers (include/camel/core/mm/gen.h:224-227),
// so device buffers are tracked in a registry and released by releaseAllDeviceBuffers() when the
// module is unloaded or a host asks for it; objects released that way must not be used again.
#pragma once

#include "camel/core/mm/alloc/allocator.h"
#include "camel/core/rtdata/base.h"
#include "camel/core/type/base.h"
#include "camel_tensor_b200.h"

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <span>
#include <string>

namespace camel::tensor {

namespace mm     = camel::core::mm;
namespace rtdata = camel::core::rtdata;
namespace type   = camel::core::type;

// Same enumerators as ct_binary_op / ct_compare_op, which follow modules/tensor/runtime.h:39-53.
using BinaryOp  = ct_binary_op;
using CompareOp = ct_compare_op;

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

    // Device payload (never null for numel > 0).  A deferred comparison (below) is evaluated
    // first, so every reader sees the finished mask.
    void *deviceData() {
        materialise();
        return dev_;
    }
    const void *deviceData() const {
        materialise();
        return dev_;
    }

    // `t > s`, `t < s`, ... against a scalar may stay unevaluated until somebody reads the mask.
    // The reference's programs write relu as `h * (h > 0)` (test/run/nn/svm.cml:31): multiply sees
    // the deferred `h > 0` and runs one relu kernel (8 bytes per element instead of 14 for the two
    // operators), and the mask is never written unless something else asks for it.  The source is
    // remembered by its device buffer, which neither moves nor dies before the module is unloaded.
    struct DeferredCompare {
        const void *src = nullptr; // device buffer of the compared tensor; set once, by deferCompare
        ct_dtype srcDType = CT_F32;
        ct_compare_op op  = CT_GT;
        double scalar     = 0.0;
        int tensorOnLeft  = 1;
    };
    void deferCompare(const TensorObject *src, ct_compare_op op, double scalar, bool tensorOnLeft);
    // The record of a comparison that has not run yet, or nullptr.  Operators run on many threads:
    // the flag is the only field written after deferCompare, and materialise() is serialised.
    const DeferredCompare *deferred() const { return pending_.load(std::memory_order_acquire) ? &deferred_ : nullptr; }
    void materialise() const;

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
    void *dev_;
    DeferredCompare deferred_;
    mutable std::atomic<bool> pending_{false};
    mutable std::byte *host_; // malloc'd mirror, nullptr while stale
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

// Releases every device buffer created so far (module unload / explicit scope end).
void releaseAllDeviceBuffers();
size_t liveDeviceBuffers();

} // namespace camel::tensor
