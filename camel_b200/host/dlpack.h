// DLPack exchange of device-resident tensors.
//
// The reference's modules/tensor/dlpack.h declares the DLPack structures with the CPU device only
// and its runtime copies through host memory (modules/tensor/runtime.cpp:1079-1124).  The layout
// of the structures is the DLPack ABI, so it is the same here; what is added is the CUDA device
// type and an export that hands out the tensor's own device buffer.
#pragma once

#include "device_tensor.h"

#include <cstdint>

namespace camel::tensor {

enum DLDeviceType : int32_t {
    kDLCPU  = 1,
    kDLCUDA = 2,
};

struct DLDevice {
    int32_t device_type;
    int32_t device_id;
};

struct DLDataType {
    uint8_t code;
    uint8_t bits;
    uint16_t lanes;
};

struct DLTensor {
    void *data;
    DLDevice device;
    int32_t ndim;
    DLDataType dtype;
    int64_t *shape;
    int64_t *strides;
    uint64_t byte_offset;
};

struct DLManagedTensor {
    DLTensor dl_tensor;
    void *manager_ctx;
    void (*deleter)(DLManagedTensor *self);
};

// Same contract as the reference: a host copy (kDLCPU) that the deleter frees.
DLManagedTensor *tensorToDLPackCopy(const TensorObject *tensor);
// The device buffer itself (kDLCUDA, no copy).  The buffer belongs to the module and lives until
// the device buffers are released; the deleter frees only the descriptor.
DLManagedTensor *tensorToDLPackDevice(const TensorObject *tensor);
// Accepts kDLCPU (one host-to-device copy) and kDLCUDA on the current device (one device copy);
// dense row-major only, like the reference.
TensorObject *tensorFromDLPackCopy(const DLManagedTensor *managed, mm::IAllocator &allocator);

} // namespace camel::tensor
