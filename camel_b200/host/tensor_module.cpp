// Plugin entry of the B200 `tensor` module: the same two C symbols and the same registration
// steps as the reference plugin (modules/camel_module_abi.cpp:22, modules/tensor/module.cpp:30-54,
// modules/tensor/executor.cpp:36-61), wired to the operator tables of tensor_registry.cpp.
#include "camel/compile/gir.h"
#include "camel/core/context/context.h"
#include "camel/core/context/frame.h"
#include "camel/core/error/diagnostics.h"
#include "camel/core/error/runtime.h"
#include "camel/core/module/builtin.h"
#include "camel/core/module/dynamic.h"
#include "camel/execute/executor.h"
#include "device_tensor.h"
#include "tensor_ops.h"
#include "type.h"

using namespace camel::core::context;
using namespace camel::core::error;
using namespace camel::core::module;

namespace {

// Dispatches `tensor:<uri>` nodes: collects the node's with/norm input slots into frame views
// and calls the operator body, storing its result slot on the node.
class B200TensorExecutor : public Executor {
  public:
    explicit B200TensorExecutor(context_ptr_t ctx) : Executor(std::move(ctx), getTensorOpsMap()) {}

    void eval(std::string uri, GIR::Node *self, Frame &frame) override {
        auto found = opsMap_.find(uri);
        if (found == opsMap_.end())
            throw DiagnosticBuilder::of(RuntimeDiag::UnrecognizedOperatorURI).commit(uri);
        std::vector<GIR::data_idx_t> withIdx, normIdx;
        for (const auto &in : self->withInputs())
            withIdx.push_back(in->index());
        for (const auto &in : self->normInputs())
            normIdx.push_back(in->index());
        FrameArgsView withView(frame, data_arr_t{withIdx.data(), static_cast<GIR::arr_size_t>(withIdx.size())});
        FrameArgsView normView(frame, data_arr_t{normIdx.data(), static_cast<GIR::arr_size_t>(normIdx.size())});
        frame.set(self->index(), found->second(withView, normView, *context_));
    }
};

class B200TensorModule : public BuiltinModule {
  public:
    explicit B200TensorModule(context_ptr_t ctx) : BuiltinModule("tensor", ctx) {
        exportType(Reference("Tensor"), camel::tensor::TensorType::Default());
        for (const auto &g : getTensorOperatorGroups()) {
            exportEntity(g->name(), g);
            if (g->name().starts_with("__")) // infix operators resolve without an explicit import
                exportDefaultImportRef(g->name());
        }
    }
    ~B200TensorModule() override { camel::tensor::releaseAllDeviceBuffers(); }

    bool load() override {
        if (!loaded_) {
            context_->registerExecutorFactory(
                "tensor", [ctx = context_]() { return std::make_shared<B200TensorExecutor>(ctx); });
            loaded_ = true;
        }
        return true;
    }
};

} // namespace

extern "C" {
int camel_module_abi_version(void) { return CAMEL_MODULE_ABI_VERSION; }
Module *camel_module_create(Context *ctx) { return new B200TensorModule(ctx->shared_from_this()); }

// Optional hooks for a host that knows where values die (it finds them with dlsym on the loaded
// module; a host that does not look for them loses nothing but device memory).  The collector has
// no finalisers (include/camel/core/mm/gen.h:224-227), so without these the module keeps every
// device buffer until it is unloaded.  A scheduler calls begin when it enters a function frame or a
// `sync` block and end when it leaves, passing the Tensor objects among the values that leave the
// region (its result slot; for a tail call, the arguments of the next iteration): everything else
// the region created on the device is released, and what a kept value still needs survives with it.
uint64_t camel_tensor_scope_begin(void) { return camel::tensor::beginScope(); }

void camel_tensor_scope_end(uint64_t token, void *const *kept_tensor_objects, size_t count) {
    std::vector<camel::tensor::TensorObject *> keep;
    for (size_t i = 0; i < count; ++i)
        keep.push_back(static_cast<camel::tensor::TensorObject *>(
            static_cast<camel::core::rtdata::Object *>(kept_tensor_objects[i])));
    camel::tensor::endScope(token, keep);
}

// One value's last use (a loop variable that has just been replaced).
void camel_tensor_release(void *tensor_object) {
    camel::tensor::releaseTensor(static_cast<camel::tensor::TensorObject *>(
        static_cast<camel::core::rtdata::Object *>(tensor_object)));
}

uint64_t camel_tensor_live_device_bytes(void) { return camel::tensor::liveDeviceBytes(); }
}
