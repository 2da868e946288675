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
}
