// C ABI: contexts, kernel timing, stream capture and graph replay.
#include "api_internal.hpp"

using namespace psi;

extern "C" {

int32_t psi_last_error(char* buf, size_t n) { return copy_message(g_thread_error, buf, n); }

static int32_t ctx_create(int32_t device, void* stream, bool own, psi_ctx** out) {
    return guarded(nullptr, [&] {
        require(out != nullptr, "out must not be null");
        *out = nullptr;
        int count = 0;
        cudaError_t err = cudaGetDeviceCount(&count);
        if (err != cudaSuccess || count == 0) {
            (void)cudaGetLastError();
            throw CudaError("no CUDA device is available; this library has no CPU fallback");
        }
        require(device >= 0 && device < count, "device index out of range");
        auto ctx = std::make_unique<psi_ctx>();
        ctx->device = device;
        ctx->bind();
        cuda_check(cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device),
                   "cudaDeviceGetAttribute");
        if (own) {
            cuda_check(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
            ctx->owns_stream = true;
        } else {
            ctx->stream = static_cast<cudaStream_t>(stream);
        }
        *out = ctx.release();
    });
}

int32_t psi_ctx_create(int32_t device, psi_ctx** out) { return ctx_create(device, nullptr, true, out); }

int32_t psi_ctx_create_on_stream(int32_t device, void* cuda_stream, psi_ctx** out) {
    return ctx_create(device, cuda_stream, false, out);
}

int32_t psi_ctx_destroy(psi_ctx* ctx) {
    if (ctx == nullptr) return PSI_OK;
    int32_t status = guarded(nullptr, [&] {
        ctx->bind();
        (void)cudaStreamSynchronize(ctx->stream);
        ctx->clear_timing();
        if (ctx->owns_stream) (void)cudaStreamDestroy(ctx->stream);
    });
    delete ctx;
    return status;
}

int32_t psi_ctx_sync(psi_ctx* ctx) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        ctx->bind();
        cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
    });
}

int32_t psi_ctx_read_bandwidth(psi_ctx* ctx, uint64_t bytes, uint32_t iterations, double* out_gbs) {
    if (ctx == nullptr || out_gbs == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        require(bytes >= 16 && iterations > 0, "the probe needs at least 16 bytes and one iteration");
        require(!ctx->capturing, "the bandwidth probe synchronises and stays outside captured graphs");
        ctx->bind();
        bytes &= ~uint64_t(15);
        DeviceBuffer scratch, sink;
        struct Release {
            DeviceBuffer& a;
            DeviceBuffer& b;
            ~Release() {
                a.release();
                b.release();
            }
        } release{scratch, sink};
        scratch.ensure(ctx, bytes, true);
        sink.ensure(ctx, sizeof(uint32_t), true);
        cudaEvent_t begin = nullptr, end = nullptr;
        cuda_check(cudaEventCreate(&begin), "cudaEventCreate");
        cuda_check(cudaEventCreate(&end), "cudaEventCreate");
        const uint32_t num_ctas = static_cast<uint32_t>(ctx->sm_count) * 8;
        float best_ms = 0.0f;
        cudaError_t err = cudaSuccess;
        for (uint32_t it = 0; it <= iterations && err == cudaSuccess; ++it) {  // pass 0 warms up
            err = cudaEventRecord(begin, ctx->stream);
            if (err == cudaSuccess) err = launch_read_stream(scratch.ptr, bytes, static_cast<uint32_t*>(sink.ptr), num_ctas, ctx->stream);
            if (err == cudaSuccess) err = cudaEventRecord(end, ctx->stream);
            if (err == cudaSuccess) err = cudaEventSynchronize(end);
            float ms = 0.0f;
            if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, begin, end);
            if (err == cudaSuccess && it > 0 && (best_ms == 0.0f || ms < best_ms)) best_ms = ms;
        }
        (void)cudaEventDestroy(begin);
        (void)cudaEventDestroy(end);
        cuda_check(err, "read bandwidth probe");
        *out_gbs = best_ms > 0.0f ? static_cast<double>(bytes) / (static_cast<double>(best_ms) * 1e6) : 0.0;
    });
}

int32_t psi_ctx_stream(psi_ctx* ctx, void** out) {
    if (ctx == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    *out = ctx->stream;
    return PSI_OK;
}

int32_t psi_ctx_sm_count(psi_ctx* ctx, int32_t* out) {
    if (ctx == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    *out = ctx->sm_count;
    return PSI_OK;
}

int32_t psi_ctx_last_error(psi_ctx* ctx, char* buf, size_t n) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return copy_message(ctx->last_error, buf, n);
}

int32_t psi_ctx_enable_kernel_timing(psi_ctx* ctx, int32_t enable) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        ctx->bind();
        cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
        ctx->clear_timing();
        ctx->timing = enable != 0;
    });
}

int32_t psi_ctx_kernel_timing(psi_ctx* ctx, uint32_t kernel_class, float* out_total_ms, uint64_t* out_launches) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        require(kernel_class < kKernelClasses, "unknown kernel class");
        require(out_total_ms != nullptr && out_launches != nullptr, "outputs must not be null");
        ctx->bind();
        cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
        float total = 0.0f;
        for (const auto& pair : ctx->timed[kernel_class]) {
            float ms = 0.0f;
            cuda_check(cudaEventElapsedTime(&ms, pair.first, pair.second), "cudaEventElapsedTime");
            total += ms;
        }
        *out_total_ms = total;
        *out_launches = ctx->timed[kernel_class].size();
    });
}

int32_t psi_ctx_capture_begin(psi_ctx* ctx) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        require(!ctx->capturing, "a stream capture is already open on this context");
        require(!ctx->timing, "switch kernel timing off before capturing");
        require(ctx->stream != nullptr && ctx->stream != cudaStreamLegacy,
                "the legacy default stream cannot be captured: create the context on a stream of its own");
        ctx->bind();
        cuda_check(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
        ctx->capturing = true;
    });
}

int32_t psi_ctx_capture_end(psi_ctx* ctx, psi_graph** out) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        require(out != nullptr, "out must not be null");
        *out = nullptr;
        require(ctx->capturing, "no stream capture is open on this context");
        ctx->capturing = false;
        cudaGraph_t graph = nullptr;
        cuda_check(cudaStreamEndCapture(ctx->stream, &graph), "cudaStreamEndCapture");
        auto holder = std::make_unique<psi_graph>();
        holder->ctx = ctx;
        holder->graph = graph;
        size_t nodes = 0;
        cuda_check(cudaGraphGetNodes(graph, nullptr, &nodes), "cudaGraphGetNodes");
        std::vector<cudaGraphNode_t> list(nodes);
        if (nodes > 0) cuda_check(cudaGraphGetNodes(graph, list.data(), &nodes), "cudaGraphGetNodes");
        for (cudaGraphNode_t node : list) {
            cudaGraphNodeType type;
            cuda_check(cudaGraphNodeGetType(node, &type), "cudaGraphNodeGetType");
            if (type == cudaGraphNodeTypeKernel) holder->kernel_nodes += 1;
        }
        cudaError_t err = cudaGraphInstantiate(&holder->exec, graph, 0);
        if (err != cudaSuccess) {
            (void)cudaGraphDestroy(graph);
            cuda_check(err, "cudaGraphInstantiate");
        }
        *out = holder.release();
    });
}

int32_t psi_graph_launch(psi_graph* graph) {
    if (graph == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(graph->ctx, [&] {
        require(!graph->ctx->capturing, "a graph cannot be launched into an open capture of its own context");
        graph->ctx->bind();
        cuda_check(cudaGraphLaunch(graph->exec, graph->ctx->stream), "cudaGraphLaunch");
        graph->ctx->launches += graph->kernel_nodes;
    });
}

int32_t psi_graph_kernel_count(psi_graph* graph, uint64_t* out) {
    if (graph == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    *out = graph->kernel_nodes;
    return PSI_OK;
}

int32_t psi_graph_destroy(psi_graph* graph) {
    return guarded(nullptr, [&] {
        if (graph == nullptr) return;
        if (graph->exec != nullptr) (void)cudaGraphExecDestroy(graph->exec);
        if (graph->graph != nullptr) (void)cudaGraphDestroy(graph->graph);
        delete graph;
    });
}

int32_t psi_ctx_launch_count(psi_ctx* ctx, uint64_t* out) {
    if (ctx == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    *out = ctx->launches;
    return PSI_OK;
}

}  // extern "C"
