// DLPack import / export for the device-resident TensorObject (see dlpack.h).
#include "dlpack.h"

#include <cstring>
#include <stdexcept>
#include <vector>

namespace camel::tensor {

using type::TypeCode;

namespace {

constexpr uint8_t kInt = 0, kUInt = 1, kFloat = 2, kBool = 6; // DLDataTypeCode

DLDataType toDLPackType(TypeCode dtype) {
    switch (dtype) {
    case TypeCode::Float32:
        return {kFloat, 32, 1};
    case TypeCode::Int64:
        return {kInt, 64, 1};
    case TypeCode::Bool:
        return {kBool, 8, 1};
    default:
        throw std::invalid_argument("Unsupported Tensor dtype");
    }
}

TypeCode fromDLPackType(DLDataType t) {
    if (t.lanes == 1 && t.code == kFloat && t.bits == 32)
        return TypeCode::Float32;
    if (t.lanes == 1 && t.code == kInt && t.bits == 64)
        return TypeCode::Int64;
    if (t.lanes == 1 && (t.code == kBool || t.code == kUInt) && t.bits == 8)
        return TypeCode::Bool;
    throw std::invalid_argument("Unsupported DLPack dtype");
}

struct Descriptor {
    int64_t *shape = nullptr;
    void *host     = nullptr; // owned copy of the payload (kDLCPU export), else null
};

DLManagedTensor *describe(const TensorObject *tensor, void *data, DLDevice device, void *ownedHost) {
    auto *managed        = new DLManagedTensor{};
    auto *ctx            = new Descriptor{};
    ctx->shape           = new int64_t[tensor->rank() ? tensor->rank() : 1];
    ctx->host            = ownedHost;
    managed->manager_ctx = ctx;
    managed->deleter     = [](DLManagedTensor *self) {
        if (!self)
            return;
        auto *inner = static_cast<Descriptor *>(self->manager_ctx);
        delete[] inner->shape;
        ::operator delete(inner->host);
        delete inner;
        delete self;
    };
    std::memcpy(ctx->shape, tensor->shape(), tensor->rank() * sizeof(int64_t));
    managed->dl_tensor.data        = data;
    managed->dl_tensor.device      = device;
    managed->dl_tensor.ndim        = static_cast<int32_t>(tensor->rank());
    managed->dl_tensor.dtype       = toDLPackType(tensor->dtype());
    managed->dl_tensor.shape       = ctx->shape;
    managed->dl_tensor.strides     = nullptr;
    managed->dl_tensor.byte_offset = 0;
    return managed;
}

} // namespace

DLManagedTensor *tensorToDLPackCopy(const TensorObject *tensor) {
    void *copy = ::operator new(tensor->byteSize() ? tensor->byteSize() : 1);
    std::memcpy(copy, tensor->rawData(), tensor->byteSize());
    return describe(tensor, copy, DLDevice{kDLCPU, 0}, copy);
}

DLManagedTensor *tensorToDLPackDevice(const TensorObject *tensor) {
    int device = 0;
    ctCheck(ct_get_device(&device));
    ctCheck(ct_sync()); // the consumer may read on any stream
    return describe(tensor, const_cast<void *>(tensor->deviceData()), DLDevice{kDLCUDA, device}, nullptr);
}

TensorObject *tensorFromDLPackCopy(const DLManagedTensor *managed, mm::IAllocator &allocator) {
    if (!managed)
        throw std::invalid_argument("Null DLPack tensor");
    const DLTensor &dl = managed->dl_tensor;
    if (dl.device.device_type != kDLCPU && dl.device.device_type != kDLCUDA)
        throw std::invalid_argument("Only CPU and CUDA DLPack tensors are supported");
    if (dl.strides != nullptr || dl.byte_offset != 0)
        throw std::invalid_argument("Only contiguous DLPack tensors are supported");
    TypeCode dtype = fromDLPackType(dl.dtype);
    std::vector<int64_t> shape(dl.shape, dl.shape + dl.ndim);
    if (dl.device.device_type == kDLCPU)
        return TensorObject::fromHost(dtype, shape, dl.data, allocator);
    int device = 0;
    ctCheck(ct_get_device(&device));
    if (dl.device.device_id != device)
        throw std::invalid_argument("The DLPack tensor lives on another CUDA device");
    TensorObject *tensor = TensorObject::create(dtype, shape, allocator, false);
    if (tensor->byteSize() > 0)
        ctCheck(ct_d2d(tensor->deviceData(), dl.data, tensor->byteSize()));
    return tensor;
}

} // namespace camel::tensor
