// CUDA-graph capture of a sequence of library calls: a launch-bound chain of small operators
// (an MLP forward is seven launches of 5-50 us each) is recorded once and replayed with one
// cudaGraphLaunch, which removes the per-call host cost (argument checks, tensor-map encoding,
// allocator calls, launch latency) from the steady state.
#include "common.cuh"

namespace ct {
namespace {
struct GraphHandle {
    cudaGraphExec_t exec;
    uint64_t launches; // kernels recorded in the graph, for ct_launch_count
};
cudaStream_t g_capture_stream = nullptr;
cudaStream_t g_saved_stream   = nullptr;
bool g_capturing              = false;
uint64_t g_launches_at_begin  = 0;
} // namespace
} // namespace ct

using namespace ct;

extern "C" {

ct_status ct_graph_begin(void) {
    OpLock op_lock;
    DeviceState *st;
    CT_TRY(current(&st));
    if (g_capturing)
        return fail(CT_ERR_INVALID, "ct_graph_begin: a capture is already in progress");
    if (!g_capture_stream)
        CT_CUDA(cudaStreamCreateWithFlags(&g_capture_stream, cudaStreamNonBlocking));
    // everything enqueued so far must be complete before the captured work may run
    CT_CUDA(cudaStreamSynchronize(stream()));
    g_saved_stream = stream();
    ct_set_stream(g_capture_stream);
    cudaError_t e = cudaStreamBeginCapture(g_capture_stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) {
        ct_set_stream(g_saved_stream);
        return cuda_fail(e, "cudaStreamBeginCapture");
    }
    g_capturing         = true;
    g_launches_at_begin = ct_launch_count();
    return CT_OK;
}

ct_status ct_graph_end(void **graph_out) {
    if (!g_capturing)
        return fail(CT_ERR_INVALID, "ct_graph_end: no capture in progress");
    if (!graph_out)
        return fail(CT_ERR_INVALID, "ct_graph_end: null output");
    g_capturing       = false;
    cudaGraph_t graph = nullptr;
    cudaError_t e     = cudaStreamEndCapture(g_capture_stream, &graph);
    ct_set_stream(g_saved_stream);
    if (e != cudaSuccess || !graph) {
        cudaGetLastError();
        return fail(
            CT_ERR_CUDA,
            "graph capture failed (%s): calls that synchronise or grow a workspace cannot be "
            "captured - run the sequence once before capturing it",
            cudaGetErrorString(e));
    }
    cudaGraphExec_t exec = nullptr;
    // tensors created inside the capture that are still alive at the next launch are released
    // by that launch and created again at the same place in the sequence
    e = cudaGraphInstantiateWithFlags(&exec, graph, cudaGraphInstantiateFlagAutoFreeOnLaunch);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess)
        return cuda_fail(e, "cudaGraphInstantiateWithFlags");
    GraphHandle *h = new GraphHandle{exec, ct_launch_count() - g_launches_at_begin};
    *graph_out     = h;
    return CT_OK;
}

ct_status ct_graph_launch(void *graph) {
    if (!graph)
        return fail(CT_ERR_INVALID, "ct_graph_launch: null graph");
    GraphHandle *h = static_cast<GraphHandle *>(graph);
    CT_CUDA(cudaGraphLaunch(h->exec, stream()));
    count_launch((unsigned)h->launches);
    return CT_OK;
}

ct_status ct_graph_destroy(void *graph) {
    if (!graph)
        return CT_OK;
    GraphHandle *h = static_cast<GraphHandle *>(graph);
    cudaError_t e  = cudaGraphExecDestroy(h->exec);
    delete h;
    if (e != cudaSuccess)
        return cuda_fail(e, "cudaGraphExecDestroy");
    return CT_OK;
}

} // extern "C"
