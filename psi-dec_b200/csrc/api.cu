// C ABI of the library: opaque objects, host-side validation, metadata upload and kernel launches.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <new>
#include <string>
#include <vector>

#include "host_logic.hpp"
#include "kernels.cuh"
#include "psi_cuda.h"
#include "snapshot.hpp"

using namespace psi;

namespace {

struct CudaError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

thread_local std::string g_thread_error;

void cuda_check(cudaError_t err, const char* what) {
    if (err != cudaSuccess) {
        throw CudaError(std::string(what) + ": " + cudaGetErrorName(err) + " (" + cudaGetErrorString(err) + ")");
    }
}

constexpr uint32_t kWordAlign = 8;  // sections of the device metadata block start on 32-byte boundaries
uint64_t pad_words(uint64_t n) { return (n + kWordAlign - 1) / kWordAlign * kWordAlign; }

}  // namespace

constexpr uint32_t kKernelClasses = 7;

struct psi_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 0;
    uint64_t launches = 0;
    std::string last_error;
    bool timing = false;
    bool capturing = false;  // between psi_ctx_capture_begin and psi_ctx_capture_end
    // (begin, end) event pairs per kernel class, recorded while timing is on
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> timed[kKernelClasses];
    void bind() const { cuda_check(cudaSetDevice(device), "cudaSetDevice"); }
    void clear_timing() {
        for (auto& list : timed) {
            for (auto& pair : list) {
                (void)cudaEventDestroy(pair.first);
                (void)cudaEventDestroy(pair.second);
            }
            list.clear();
        }
    }
};

namespace {

// Counts one launch and, while timing is on, brackets it with events on the context's stream.
struct LaunchScope {
    psi_ctx* ctx;
    cudaEvent_t end = nullptr;
    LaunchScope(psi_ctx* c, uint32_t kernel_class) : ctx(c) {
        ctx->launches += 1;
        if (!ctx->timing || ctx->capturing) return;
        cudaEvent_t begin = nullptr;
        cuda_check(cudaEventCreate(&begin), "cudaEventCreate");
        cuda_check(cudaEventCreate(&end), "cudaEventCreate");
        ctx->timed[kernel_class].emplace_back(begin, end);
        cuda_check(cudaEventRecord(begin, ctx->stream), "cudaEventRecord");
    }
    ~LaunchScope() {
        if (end != nullptr) (void)cudaEventRecord(end, ctx->stream);
    }
};

}  // namespace

namespace {

// Grow-only device allocation owned by a context.
struct DeviceBuffer {
    void* ptr = nullptr;
    uint64_t bytes = 0;
    void ensure(psi_ctx* ctx, uint64_t wanted, bool zero) {
        if (wanted <= bytes) return;
        require(!ctx->capturing, "a device buffer would have to grow during stream capture: reserve replay capacity first");
        if (ptr != nullptr) {
            cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
            cuda_check(cudaFree(ptr), "cudaFree");
            ptr = nullptr;
            bytes = 0;
        }
        cudaError_t err = cudaMalloc(&ptr, wanted);
        if (err == cudaErrorMemoryAllocation) {
            (void)cudaGetLastError();
            throw ExhaustedError("out of device memory");
        }
        cuda_check(err, "cudaMalloc");
        bytes = wanted;
        if (zero) cuda_check(cudaMemsetAsync(ptr, 0, wanted, ctx->stream), "cudaMemsetAsync");
    }
    void release() {
        if (ptr != nullptr) (void)cudaFree(ptr);
        ptr = nullptr;
        bytes = 0;
    }
};

}  // namespace

struct psi_pages {
    psi_ctx* ctx = nullptr;
    void* ptr = nullptr;
    bool owned = false;
    uint64_t num_pages = 0;
    uint32_t page_bytes = 0;
};

struct psi_table {
    psi_ctx* ctx = nullptr;
    psi_page_table_layout layout{};
    uint32_t* dev = nullptr;
    std::vector<uint32_t> host;
    uint64_t row_words() const { return uint64_t(layout.num_blocks) * layout.num_page_ids_per_block; }
    uint64_t start_index(uint32_t slot, uint32_t layer, uint32_t block) const {
        return ((uint64_t(slot) * layout.num_gqa_layers + layer) * layout.num_blocks + block) *
               layout.num_page_ids_per_block;
    }
};

struct psi_graph {
    psi_ctx* ctx = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t kernel_nodes = 0;
};

struct psi_snapshot_writer {
    SnapshotWriter impl;
    psi_snapshot_writer(const std::string& d, const std::vector<uint32_t>& f, const SnapshotPlan& p) : impl(d, f, p) {}
};

struct psi_snapshot_reader {
    SnapshotReader impl;
    psi_snapshot_reader(const std::string& d, const std::vector<uint32_t>& f, const SnapshotPlan& p) : impl(d, f, p) {}
};

struct psi_id_allocator {
    IdAllocator impl;
    explicit psi_id_allocator(uint64_t capacity) : impl(capacity) {}
};

struct psi_gqa {
    psi_ctx* ctx = nullptr;
    psi_gqa_config cfg{};
    uint32_t tokens_per_page = 0;
    uint32_t kernel = PSI_KERNEL_GENERIC;  // resolved kernel
    uint32_t grid_cap = 1;
    uint32_t item_start_cost = 0;  // KV tiles one item switch is worth when shares are balanced
    PlanGeometry geo{};
    std::unique_ptr<SplitKvSelector> selector;  // null when the profile is outside the reference selector's domain
    std::unique_ptr<ReferenceMetadata> md;
    std::vector<uint32_t> boundaries;
    psi_replay_shape shape{};
    psi_split_kv_variant variant{};
    WorkPlan plan;
    ChunkPlan chunk;            // long query runs (balanced plan + mma kernel only)
    bool chunk_supported = false;
    bool prepared = false;

    DeviceBuffer block;       // device metadata block
    uint32_t* staging = nullptr;  // pinned mirror of the block
    uint64_t staging_words = 0;
    cudaEvent_t upload_done = nullptr;
    // section offsets (in words) of the block uploaded by the last prepare
    uint64_t off_req_slots = 0, off_token_indices = 0, off_cta = 0, off_reduces = 0, off_items = 0;
    uint64_t off_chunk_cta = 0, off_chunk_items = 0;
    uint64_t off_first_items = 0;  // copies of every CTA's first item (mma kernel)
    // Replay reservation: every array of the device block at a fixed offset sized for max_tokens, every scratch buffer
    // at its largest, every launch at its capacity grid, so that a captured graph stays valid from step to step.
    bool replay_reserved = false;
    uint64_t cap_items = 0, cap_chunk_items = 0, cap_reduces = 0;

    DeviceBuffer partial_o, partial_ml;  // [slots][16][D] and [2][slots][16]
    DeviceBuffer unit_counters;          // [slots] u32, zero between launches
    uint64_t partial_slots_cap = 0;
    DeviceBuffer step_k, step_v, step_q, step_out;  // psi_gqa_decode_step_host staging
    DeviceBuffer combine_ptrs;
    DeviceBuffer status_word;  // u32 written by bounded device-side waits
    bool chunk_umma = false;   // long query runs on the tcgen05 kernel (else the mma.sync chunk kernel)
    uint32_t chunk_launches[2] = {0, 0};  // tcgen05, mma.sync
    DeviceBuffer norm_rope;    // q weight bf16[D] | k weight bf16[D] | inverse frequencies f32[rope_dim/2]
    psi_norm_rope_config norm_rope_cfg{};
    float norm_rope_attention_factor = 1.0f;
    bool has_norm_rope = false;
};

namespace {

template <typename F>
int32_t guarded(psi_ctx* ctx, F&& body) {
    int32_t status = PSI_OK;
    std::string message;
    try {
        body();
    } catch (const ContractError& e) {
        status = PSI_ERR_INVALID_ARGUMENT;
        message = e.what();
    } catch (const ExhaustedError& e) {
        status = PSI_ERR_RESOURCE_EXHAUSTED;
        message = e.what();
    } catch (const CudaError& e) {
        status = PSI_ERR_CUDA;
        message = e.what();
    } catch (const std::bad_alloc&) {
        status = PSI_ERR_RESOURCE_EXHAUSTED;
        message = "out of host memory";
    } catch (const std::exception& e) {
        status = PSI_ERR_INTERNAL;
        message = e.what();
    } catch (...) {
        status = PSI_ERR_INTERNAL;
        message = "unknown error";
    }
    if (status != PSI_OK) {
        g_thread_error = message;
        if (ctx != nullptr) ctx->last_error = message;
    }
    return status;
}

int32_t copy_message(const std::string& message, char* buf, size_t n) {
    if (buf == nullptr || n == 0) return PSI_ERR_INVALID_ARGUMENT;
    size_t len = std::min(message.size(), n - 1);
    std::memcpy(buf, message.data(), len);
    buf[len] = '\0';
    return PSI_OK;
}

void validate_layout(const psi_page_table_layout& l) {
    require(l.num_req_slots > 0 && l.num_blocks > 0 && l.num_gqa_layers > 0 && l.num_page_ids_per_block > 0,
            "GQA page-table layout dimensions must be positive");
    const uint64_t per_req = uint64_t(l.num_blocks) * l.num_page_ids_per_block;
    require(per_req <= kU32Max, "GQA per-request physical page count must fit u32");
    const long double total = (long double)l.num_req_slots * l.num_gqa_layers * (long double)per_req;
    require(total < 4.0e18L, "GQA page-table element count must fit usize");
}

PageGeometry page_geometry(const psi_gqa* g, const psi_pages* pages, const psi_table* table, uint32_t layer) {
    require(pages != nullptr && table != nullptr, "pages and table must not be null");
    require(pages->ctx == g->ctx && table->ctx == g->ctx, "pages, table and GQA component must share one context");
    require(pages->ptr != nullptr, "page arena state must be loaded before execution");
    require(pages->page_bytes == g->cfg.page_bytes, "page arena page_bytes differs from the GQA configuration");
    const auto& a = table->layout;
    const auto& b = g->cfg.layout;
    require(a.num_req_slots == b.num_req_slots && a.num_gqa_layers == b.num_gqa_layers &&
                a.num_blocks == b.num_blocks && a.num_page_ids_per_block == b.num_page_ids_per_block,
            "page table layout differs from the GQA configuration");
    require(layer < b.num_gqa_layers, "GQA page-table index exceeds layer count");
    PageGeometry geo{};
    geo.pages = pages->ptr;
    geo.page_ids = table->dev;
    geo.elem_bytes = dtype_bytes(g->cfg.dtype);
    geo.page_elems = g->cfg.page_bytes / geo.elem_bytes;
    geo.num_pages = pages->num_pages;
    geo.layer = layer;
    geo.num_layers = b.num_gqa_layers;
    geo.pages_per_req = static_cast<uint32_t>(table->row_words());
    geo.tokens_per_page = g->tokens_per_page;
    geo.num_kv_heads = g->cfg.num_kv_heads;
    geo.head_dim = g->cfg.head_dim;
    return geo;
}

const uint32_t* block_words(const psi_gqa* g, uint64_t offset) {
    return static_cast<const uint32_t*>(g->block.ptr) + offset;
}

// Requests whose query run spans at least this many query tiles go to the chunk kernels.
constexpr uint32_t kChunkMinTiles = 5;
// psi_gqa_step_host: from this many bytes of q + k + v the attention launch reads pinned host buffers in place.
constexpr uint64_t kDirectHostBytes = 1ull << 20;

AttendParams attend_params(psi_gqa* g, const psi_pages* pages, const psi_table* table, uint32_t layer, const void* q) {
    require(g->prepared, "GQA batch metadata must be updated before recording");
    require(q != nullptr, "q must not be null");
    AttendParams p{};
    p.geo = page_geometry(g, pages, table, layer);
    p.q = q;
    p.items = reinterpret_cast<const DeviceItem*>(block_words(g, g->off_items));
    p.cta_item_begin = block_words(g, g->off_cta);
    if (g->kernel == PSI_KERNEL_MMA) p.cta_first_items = reinterpret_cast<const DeviceItem*>(block_words(g, g->off_first_items));
    p.reduces = reinterpret_cast<const ReduceUnit*>(block_words(g, g->off_reduces));
    p.partial_o = static_cast<float*>(g->partial_o.ptr);
    p.partial_m = static_cast<float*>(g->partial_ml.ptr);
    p.partial_l = p.partial_m == nullptr ? nullptr : p.partial_m + g->partial_slots_cap * kMaxRows;
    p.unit_counters = static_cast<uint32_t*>(g->unit_counters.ptr);
    p.scalars = block_words(g, 0);
    p.num_q_heads = g->cfg.num_q_heads;
    p.tokens_per_tile = g->geo.tokens_per_tile;
    p.dtype = g->cfg.dtype;
    p.scale_log2 = g->cfg.scale * 1.4426950408889634f;
    return p;
}

void run_attend(psi_gqa* g, const AttendParams& params) {
    psi_ctx* ctx = g->ctx;
    AttendParams p = params;
    // Under a replay reservation a captured launch sequence has to be right for every later plan: always the same
    // launches (append, map, chunk, reduce where the kernel needs one), each at its capacity grid, each reading its
    // active counts from the device block.
    const bool fixed = g->replay_reserved;
    if (p.new_k != nullptr && (fixed || g->chunk.num_ctas() > 0)) {
        // A fused step that carries long query runs: their K/V tiles are fetched page-wise by TMA, so the step's rows
        // go to their pages first (one more launch, against milliseconds of attention) and both kernels read pages only.
        AppendParams a{};
        a.geo = p.geo;
        a.flat_k = p.new_k;
        a.flat_v = p.new_v;
        a.req_slots = block_words(g, g->off_req_slots);
        a.flat_token_indices = block_words(g, g->off_token_indices);
        a.scalars = block_words(g, 0);
        a.num_total_tokens = g->shape.num_total_tokens;
        {
            LaunchScope scope(ctx, PSI_KERNEL_CLASS_APPEND);
            cuda_check(launch_kv_append(a, ctx->stream), "kv append launch");
        }
        p.new_k = nullptr;
        p.new_v = nullptr;
    }
    const uint32_t num_ctas = fixed ? g->grid_cap : g->plan.num_ctas();
    if (num_ctas > 0) {
        LaunchScope scope(ctx, PSI_KERNEL_CLASS_ATTEND_MAP);
        if (g->kernel == PSI_KERNEL_MMA) {
            cuda_check(launch_attend_mma(p, num_ctas, ctx->stream), "attend (mma) launch");
        } else {
            cuda_check(launch_attend_generic(p, num_ctas, ctx->stream), "attend (generic) launch");
        }
    }
    const uint32_t chunk_ctas = fixed ? (g->chunk_supported ? g->grid_cap : 0u) : g->chunk.num_ctas();
    if (chunk_ctas > 0) {
        AttendParams c = p;
        c.items = reinterpret_cast<const DeviceItem*>(block_words(g, g->off_chunk_items));
        c.cta_item_begin = block_words(g, g->off_chunk_cta);
        LaunchScope scope(ctx, PSI_KERNEL_CLASS_ATTEND_CHUNK);
        cudaError_t launched = cudaErrorNotSupported;
        if (g->chunk_umma) {
            c.status = static_cast<uint32_t*>(g->status_word.ptr);
            launched = launch_attend_chunk_umma(c, chunk_ctas, ctx->stream);
        }
        // an arena the TMA unit cannot address (alignment, size) keeps the mma.sync kernel
        if (launched == cudaErrorNotSupported) {
            launched = launch_attend_chunk(c, chunk_ctas, ctx->stream);
            g->chunk_launches[1] += 1;
        } else {
            g->chunk_launches[0] += 1;
        }
        cuda_check(launched, "attend (chunk) launch");
    }
    // The mma kernel merges a unit's partials in the CTA that delivers the last one; the generic kernel needs the
    // separate reduce pass.
    const uint32_t num_reduces = g->kernel == PSI_KERNEL_MMA
                                     ? 0u
                                     : static_cast<uint32_t>(fixed ? g->cap_reduces : g->plan.reduces.size());
    if (num_reduces > 0) {
        LaunchScope scope(ctx, PSI_KERNEL_CLASS_ATTEND_REDUCE);
        cuda_check(launch_attend_reduce(p, num_reduces, ctx->stream), "attend reduce launch");
    }
}

void run_append(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k, const void* v) {
    require(g->prepared, "GQA batch metadata must be updated before recording");
    require(k != nullptr && v != nullptr, "k and v must not be null");
    AppendParams p{};
    p.geo = page_geometry(g, pages, table, layer);
    p.flat_k = k;
    p.flat_v = v;
    p.req_slots = block_words(g, g->off_req_slots);
    p.flat_token_indices = block_words(g, g->off_token_indices);
    p.scalars = block_words(g, 0);
    p.num_total_tokens = g->shape.num_total_tokens;
    LaunchScope scope(g->ctx, PSI_KERNEL_CLASS_APPEND);
    cuda_check(launch_kv_append(p, g->ctx->stream), "kv append launch");
}

// Device-side address of a pinned, device-mapped host buffer (16-byte aligned), or nullptr for any other memory.
void* mapped_device_pointer(const void* host) {
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, host) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
        attr.devicePointer != nullptr && (reinterpret_cast<uintptr_t>(attr.devicePointer) & 15u) == 0) {
        return attr.devicePointer;
    }
    (void)cudaGetLastError();
    return nullptr;
}

// A prepared step through pageable host buffers: inputs staged by copy-engine transfers, output copied back, waited for.
void run_staged_host_step(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k_host,
                          const void* v_host, const void* q_host, void* out_host, uint64_t kv_bytes, uint64_t q_bytes,
                          uint64_t q_cap) {
    psi_ctx* ctx = g->ctx;
    g->step_out.ensure(ctx, q_cap, false);
    cuda_check(cudaMemcpyAsync(g->step_k.ptr, k_host, kv_bytes, cudaMemcpyHostToDevice, ctx->stream), "H2D k");
    cuda_check(cudaMemcpyAsync(g->step_v.ptr, v_host, kv_bytes, cudaMemcpyHostToDevice, ctx->stream), "H2D v");
    cuda_check(cudaMemcpyAsync(g->step_q.ptr, q_host, q_bytes, cudaMemcpyHostToDevice, ctx->stream), "H2D q");
    AttendParams p = attend_params(g, pages, table, layer, g->step_q.ptr);
    p.out = g->step_out.ptr;
    if (g->kernel == PSI_KERNEL_MMA) {
        p.new_k = g->step_k.ptr;
        p.new_v = g->step_v.ptr;
    } else {
        run_append(g, pages, table, layer, g->step_k.ptr, g->step_v.ptr);
    }
    run_attend(g, p);
    cuda_check(cudaMemcpyAsync(out_host, g->step_out.ptr, q_bytes, cudaMemcpyDeviceToHost, ctx->stream), "D2H out");
    cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------------
// context
// ---------------------------------------------------------------------------------------------------------------------
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

// ---------------------------------------------------------------------------------------------------------------------
// page arena
// ---------------------------------------------------------------------------------------------------------------------
static void pages_allocate(psi_pages* pages) {
    require(pages->ptr == nullptr, "page arena state is already loaded");
    const uint64_t bytes = pages->num_pages * pages->page_bytes;
    cudaError_t err = cudaMalloc(&pages->ptr, bytes);
    if (err == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        pages->ptr = nullptr;
        throw ExhaustedError("out of device memory for the page arena");
    }
    cuda_check(err, "cudaMalloc");
    cuda_check(cudaMemsetAsync(pages->ptr, 0, bytes, pages->ctx->stream), "cudaMemsetAsync");
}

int32_t psi_pages_create(psi_ctx* ctx, uint64_t num_pages, uint32_t page_bytes, psi_pages** out) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        require(out != nullptr, "out must not be null");
        *out = nullptr;
        require(num_pages > 0, "page arena requires pages");
        require(page_bytes > 0, "page arena requires nonzero page size");
        require(num_pages <= (uint64_t(1) << 62) / page_bytes, "page arena byte length must fit usize");
        ctx->bind();
        auto pages = std::make_unique<psi_pages>();
        pages->ctx = ctx;
        pages->owned = true;
        pages->num_pages = num_pages;
        pages->page_bytes = page_bytes;
        pages_allocate(pages.get());
        *out = pages.release();
    });
}

int32_t psi_pages_wrap(psi_ctx* ctx, void* device_ptr, uint64_t num_pages, uint32_t page_bytes, psi_pages** out) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        require(out != nullptr && device_ptr != nullptr, "out and device_ptr must not be null");
        require(num_pages > 0 && page_bytes > 0, "page arena requires pages of nonzero size");
        auto pages = std::make_unique<psi_pages>();
        pages->ctx = ctx;
        pages->ptr = device_ptr;
        pages->owned = false;
        pages->num_pages = num_pages;
        pages->page_bytes = page_bytes;
        *out = pages.release();
    });
}

int32_t psi_pages_destroy(psi_pages* pages) {
    if (pages == nullptr) return PSI_OK;
    int32_t status = guarded(pages->ctx, [&] {
        pages->ctx->bind();
        if (pages->owned && pages->ptr != nullptr) {
            (void)cudaStreamSynchronize(pages->ctx->stream);
            cuda_check(cudaFree(pages->ptr), "cudaFree");
        }
    });
    delete pages;
    return status;
}

int32_t psi_pages_device_ptr(psi_pages* pages, void** out) {
    if (pages == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(pages->ctx, [&] {
        require(pages->ptr != nullptr, "page arena state must be loaded before execution");
        *out = pages->ptr;
    });
}

int32_t psi_pages_release(psi_pages* pages) {
    if (pages == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(pages->ctx, [&] {
        require(pages->owned, "a wrapped page arena does not own its memory");
        require(pages->ptr != nullptr, "page arena state is not loaded");
        pages->ctx->bind();
        cuda_check(cudaStreamSynchronize(pages->ctx->stream), "cudaStreamSynchronize");
        cuda_check(cudaFree(pages->ptr), "cudaFree");
        pages->ptr = nullptr;
    });
}

int32_t psi_pages_allocate(psi_pages* pages) {
    if (pages == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(pages->ctx, [&] {
        require(pages->owned, "a wrapped page arena does not own its memory");
        pages->ctx->bind();
        pages_allocate(pages);
    });
}

static int32_t pages_copy_range(psi_pages* pages, uint64_t begin, uint64_t end, void* host, bool to_host) {
    if (pages == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(pages->ctx, [&] {
        require(host != nullptr, "host buffer must not be null");
        require(pages->ptr != nullptr, "page arena state must be loaded before execution");
        require(begin <= end && end <= pages->num_pages, "page-ID range outside the page arena");
        pages->ctx->bind();
        auto* dev = static_cast<unsigned char*>(pages->ptr) + begin * pages->page_bytes;
        const uint64_t bytes = (end - begin) * pages->page_bytes;
        if (bytes == 0) return;
        if (to_host) {
            cuda_check(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, pages->ctx->stream), "cudaMemcpyAsync");
        } else {
            cuda_check(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, pages->ctx->stream), "cudaMemcpyAsync");
        }
        cuda_check(cudaStreamSynchronize(pages->ctx->stream), "cudaStreamSynchronize");
    });
}

int32_t psi_pages_export_range(psi_pages* pages, uint64_t page_begin, uint64_t page_end, void* host_out) {
    return pages_copy_range(pages, page_begin, page_end, host_out, true);
}

int32_t psi_pages_import_range(psi_pages* pages, uint64_t page_begin, uint64_t page_end, const void* host_in) {
    return pages_copy_range(pages, page_begin, page_end, const_cast<void*>(host_in), false);
}

// ---------------------------------------------------------------------------------------------------------------------
// hibernation snapshots
// ---------------------------------------------------------------------------------------------------------------------
static SnapshotPlan snapshot_plan(const psi_hibernation_plan* plan) {
    require(plan != nullptr, "plan must not be null");
    SnapshotPlan out;
    out.selected = plan->selected != 0;
    if (out.selected) {
        require(plan->num_request_slot_ranges == 0 || plan->request_slot_ranges != nullptr, "request slot ranges must not be null");
        require(plan->num_page_id_ranges == 0 || plan->page_id_ranges != nullptr, "page ID ranges must not be null");
        for (uint64_t i = 0; i < plan->num_request_slot_ranges; ++i)
            out.request_slot_ranges.emplace_back(plan->request_slot_ranges[i].begin, plan->request_slot_ranges[i].end);
        for (uint64_t i = 0; i < plan->num_page_id_ranges; ++i)
            out.page_id_ranges.emplace_back(plan->page_id_ranges[i].begin, plan->page_id_ranges[i].end);
    }
    return out;
}

static std::vector<U32Range> snapshot_ranges(const psi_u32_range* ranges, uint64_t n) {
    std::vector<U32Range> out;
    for (uint64_t i = 0; i < n; ++i) out.emplace_back(ranges[i].begin, ranges[i].end);
    return out;
}

static SnapshotBuffer pages_buffer(psi_pages* pages) {
    require(pages != nullptr, "pages must not be null");
    require(pages->ptr != nullptr, "page arena resources are released");
    pages->ctx->bind();
    cuda_check(cudaStreamSynchronize(pages->ctx->stream), "cudaStreamSynchronize");
    return SnapshotBuffer{pages->ptr, pages->num_pages * pages->page_bytes, true};
}

static uint64_t table_slot_bytes(const psi_table* table) {
    return uint64_t(table->layout.num_gqa_layers) * table->row_words() * sizeof(uint32_t);
}

int32_t psi_snapshot_writer_create(const char* destination, const uint32_t* expected_files, uint64_t num_files,
                                   const psi_hibernation_plan* plan, psi_snapshot_writer** out) {
    return guarded(nullptr, [&] {
        require(out != nullptr && destination != nullptr, "out and destination must not be null");
        *out = nullptr;
        require(num_files == 0 || expected_files != nullptr, "expected files must not be null");
        const std::vector<uint32_t> files(expected_files, expected_files + num_files);
        *out = new psi_snapshot_writer(destination, files, snapshot_plan(plan));
    });
}

int32_t psi_snapshot_write_pages(psi_snapshot_writer* writer, uint32_t file, psi_pages* pages) {
    if (writer == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(pages != nullptr ? pages->ctx : nullptr, [&] {
        const SnapshotBuffer buffer = pages_buffer(pages);
        if (writer->impl.plan().selected) {
            writer->impl.write_selected_buffer(file, buffer, writer->impl.plan().page_id_ranges, pages->page_bytes);
        } else {
            writer->impl.write_full_buffer(file, buffer);
        }
    });
}

int32_t psi_snapshot_write_table(psi_snapshot_writer* writer, uint32_t file, psi_table* table) {
    if (writer == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table != nullptr ? table->ctx : nullptr, [&] {
        require(table != nullptr, "table must not be null");
        // the host mirror holds exactly what the device table holds: every write goes through both
        const SnapshotBuffer buffer{table->host.data(), table->host.size() * sizeof(uint32_t), false};
        if (writer->impl.plan().selected) {
            writer->impl.write_selected_buffer(file, buffer, writer->impl.plan().request_slot_ranges, table_slot_bytes(table));
        } else {
            writer->impl.write_full_buffer(file, buffer);
        }
    });
}

int32_t psi_snapshot_write_host_buffer(psi_snapshot_writer* writer, uint32_t file, const void* host, uint64_t bytes,
                                       const psi_u32_range* entry_ranges, uint64_t num_ranges, uint64_t entry_bytes) {
    if (writer == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        require(host != nullptr || bytes == 0, "host buffer must not be null");
        const SnapshotBuffer buffer{const_cast<void*>(host), bytes, false};
        if (entry_ranges == nullptr && num_ranges == 0 && entry_bytes == 0) {
            writer->impl.write_full_buffer(file, buffer);
        } else {
            writer->impl.write_selected_buffer(file, buffer, snapshot_ranges(entry_ranges, num_ranges), entry_bytes);
        }
    });
}

int32_t psi_snapshot_write_metadata(psi_snapshot_writer* writer, uint32_t file, const void* bytes, uint64_t n) {
    if (writer == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        require(bytes != nullptr || n == 0, "metadata must not be null");
        writer->impl.write_metadata(file, bytes, n);
    });
}

int32_t psi_snapshot_writer_commit(psi_snapshot_writer* writer) {
    if (writer == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] { writer->impl.commit(); });
}

int32_t psi_snapshot_writer_destroy(psi_snapshot_writer* writer) {
    return guarded(nullptr, [&] { delete writer; });
}

int32_t psi_snapshot_reader_open(const char* path, const uint32_t* expected_files, uint64_t num_files,
                                 const psi_hibernation_plan* plan, psi_snapshot_reader** out) {
    return guarded(nullptr, [&] {
        require(out != nullptr && path != nullptr, "out and path must not be null");
        *out = nullptr;
        require(num_files == 0 || expected_files != nullptr, "expected files must not be null");
        const std::vector<uint32_t> files(expected_files, expected_files + num_files);
        *out = new psi_snapshot_reader(path, files, snapshot_plan(plan));
    });
}

int32_t psi_snapshot_read_pages(psi_snapshot_reader* reader, uint32_t file, psi_pages* pages) {
    if (reader == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(pages != nullptr ? pages->ctx : nullptr, [&] {
        const SnapshotBuffer buffer = pages_buffer(pages);
        if (reader->impl.plan().selected) {
            reader->impl.read_selected_buffer(file, buffer, reader->impl.plan().page_id_ranges, pages->page_bytes);
        } else {
            reader->impl.read_full_buffer(file, buffer);
        }
    });
}

int32_t psi_snapshot_read_table(psi_snapshot_reader* reader, uint32_t file, psi_table* table) {
    if (reader == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table != nullptr ? table->ctx : nullptr, [&] {
        require(table != nullptr, "table must not be null");
        table->ctx->bind();
        const SnapshotBuffer buffer{table->host.data(), table->host.size() * sizeof(uint32_t), false};
        const uint64_t slot_bytes = table_slot_bytes(table);
        std::vector<U32Range> slots;
        if (reader->impl.plan().selected) {
            slots = reader->impl.plan().request_slot_ranges;
            reader->impl.read_selected_buffer(file, buffer, slots, slot_bytes);
        } else {
            slots.emplace_back(0u, table->layout.num_req_slots);
            reader->impl.read_full_buffer(file, buffer);
        }
        // the restored rows of the mirror go to the device table
        cuda_check(cudaStreamSynchronize(table->ctx->stream), "cudaStreamSynchronize");
        for (const auto& range : slots) {
            const uint64_t offset = uint64_t(range.first) * slot_bytes, n = uint64_t(range.second - range.first) * slot_bytes;
            cuda_check(cudaMemcpy(reinterpret_cast<unsigned char*>(table->dev) + offset,
                                  reinterpret_cast<const unsigned char*>(table->host.data()) + offset, n, cudaMemcpyHostToDevice),
                       "cudaMemcpy");
        }
    });
}

int32_t psi_snapshot_read_host_buffer(psi_snapshot_reader* reader, uint32_t file, void* host, uint64_t bytes,
                                      const psi_u32_range* entry_ranges, uint64_t num_ranges, uint64_t entry_bytes) {
    if (reader == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        require(host != nullptr || bytes == 0, "host buffer must not be null");
        const SnapshotBuffer buffer{host, bytes, false};
        if (entry_ranges == nullptr && num_ranges == 0 && entry_bytes == 0) {
            reader->impl.read_full_buffer(file, buffer);
        } else {
            reader->impl.read_selected_buffer(file, buffer, snapshot_ranges(entry_ranges, num_ranges), entry_bytes);
        }
    });
}

int32_t psi_snapshot_read_metadata(psi_snapshot_reader* reader, uint32_t file, void* out, uint64_t cap, uint64_t* out_n) {
    if (reader == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        require(out_n != nullptr, "out_n must not be null");
        const std::vector<uint8_t> bytes = reader->impl.read_metadata(file);
        *out_n = bytes.size();
        require(out != nullptr && cap >= bytes.size(), "metadata output capacity too small");
        std::memcpy(out, bytes.data(), bytes.size());
    });
}

int32_t psi_snapshot_reader_finish(psi_snapshot_reader* reader) {
    if (reader == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] { reader->impl.finish(); });
}

int32_t psi_snapshot_reader_destroy(psi_snapshot_reader* reader) {
    return guarded(nullptr, [&] { delete reader; });
}

// ---------------------------------------------------------------------------------------------------------------------
// request page table
// ---------------------------------------------------------------------------------------------------------------------
int32_t psi_table_create(psi_ctx* ctx, const psi_page_table_layout* layout, psi_table** out) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        require(out != nullptr && layout != nullptr, "out and layout must not be null");
        *out = nullptr;
        validate_layout(*layout);
        ctx->bind();
        auto table = std::make_unique<psi_table>();
        table->ctx = ctx;
        table->layout = *layout;
        const uint64_t words = uint64_t(layout->num_req_slots) * layout->num_gqa_layers * table->row_words();
        table->host.assign(words, 0);
        cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&table->dev), words * sizeof(uint32_t));
        if (err == cudaErrorMemoryAllocation) {
            (void)cudaGetLastError();
            throw ExhaustedError("out of device memory for the page table");
        }
        cuda_check(err, "cudaMalloc");
        cuda_check(cudaMemsetAsync(table->dev, 0, words * sizeof(uint32_t), ctx->stream), "cudaMemsetAsync");
        *out = table.release();
    });
}

int32_t psi_table_destroy(psi_table* table) {
    if (table == nullptr) return PSI_OK;
    int32_t status = guarded(table->ctx, [&] {
        table->ctx->bind();
        (void)cudaStreamSynchronize(table->ctx->stream);
        if (table->dev != nullptr) cuda_check(cudaFree(table->dev), "cudaFree");
    });
    delete table;
    return status;
}

static void table_check(const psi_table* t, uint32_t slot, uint32_t layer, uint32_t block) {
    require(slot < t->layout.num_req_slots, "GQA request page table req_slot out of range");
    require(layer < t->layout.num_gqa_layers, "GQA request page table layer out of range");
    require(block < t->layout.num_blocks, "GQA request page table block out of range");
}

static void table_upload(psi_table* t, uint64_t start, uint64_t count) {
    if (count == 0) return;
    cuda_check(cudaMemcpyAsync(t->dev + start, t->host.data() + start, count * sizeof(uint32_t),
                               cudaMemcpyHostToDevice, t->ctx->stream),
               "cudaMemcpyAsync");
}

int32_t psi_table_write(psi_table* table, uint32_t req_slot, uint32_t layer, uint32_t block, const uint32_t* page_ids,
                        uint32_t n) {
    if (table == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table->ctx, [&] {
        require(page_ids != nullptr, "page_ids must not be null");
        table_check(table, req_slot, layer, block);
        require(n == table->layout.num_page_ids_per_block,
                "GQA page-id count must match one request/GQA-layer/block entry");
        table->ctx->bind();
        const uint64_t start = table->start_index(req_slot, layer, block);
        std::copy(page_ids, page_ids + n, table->host.begin() + start);
        table_upload(table, start, n);
    });
}

int32_t psi_table_write_all_layers(psi_table* table, uint32_t req_slot, uint32_t block, const uint32_t* page_ids,
                                   uint32_t n, uint64_t num_cache_pages) {
    if (table == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table->ctx, [&] {
        require(page_ids != nullptr, "page_ids must not be null");
        table_check(table, req_slot, 0, block);
        const uint32_t per_layer = table->layout.num_page_ids_per_block;
        require(uint64_t(n) == uint64_t(table->layout.num_gqa_layers) * per_layer,
                "GQA cache block must contain all layer page IDs");
        for (uint32_t i = 0; i < n; ++i) {
            require(page_ids[i] < num_cache_pages, "runtime supplied a GQA page ID outside the cache-page buffer");
        }
        table->ctx->bind();
        for (uint32_t layer = 0; layer < table->layout.num_gqa_layers; ++layer) {
            const uint64_t start = table->start_index(req_slot, layer, block);
            std::copy(page_ids + uint64_t(layer) * per_layer, page_ids + uint64_t(layer + 1) * per_layer,
                      table->host.begin() + start);
            table_upload(table, start, per_layer);
        }
    });
}

int32_t psi_table_write_row(psi_table* table, uint32_t req_slot, uint32_t layer, const uint32_t* ids, uint32_t n) {
    if (table == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table->ctx, [&] {
        require(ids != nullptr, "ids must not be null");
        table_check(table, req_slot, layer, 0);
        require(n <= table->row_words(), "page-id count exceeds one request/GQA-layer row");
        table->ctx->bind();
        const uint64_t start = table->start_index(req_slot, layer, 0);
        std::copy(ids, ids + n, table->host.begin() + start);
        table_upload(table, start, n);
    });
}

int32_t psi_table_read(psi_table* table, uint32_t req_slot, uint32_t layer, uint32_t block, uint32_t* out, uint32_t n) {
    if (table == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table->ctx, [&] {
        require(out != nullptr, "out must not be null");
        table_check(table, req_slot, layer, block);
        require(n == table->layout.num_page_ids_per_block,
                "GQA page-id count must match one request/GQA-layer/block entry");
        table->ctx->bind();
        const uint64_t start = table->start_index(req_slot, layer, block);
        cuda_check(cudaMemcpyAsync(out, table->dev + start, n * sizeof(uint32_t), cudaMemcpyDeviceToHost,
                                   table->ctx->stream),
                   "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize(table->ctx->stream), "cudaStreamSynchronize");
    });
}

int32_t psi_table_reset_slots(psi_table* table, const uint32_t* req_slots, uint32_t n) {
    if (table == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table->ctx, [&] {
        require(req_slots != nullptr || n == 0, "req_slots must not be null");
        for (uint32_t i = 0; i < n; ++i) require(req_slots[i] < table->layout.num_req_slots,
                                                 "GQA request page table req_slot out of range");
        table->ctx->bind();
        const uint64_t per_req = table->layout.num_gqa_layers * table->row_words();
        for (uint32_t i = 0; i < n; ++i) {
            const uint64_t start = table->start_index(req_slots[i], 0, 0);
            std::fill(table->host.begin() + start, table->host.begin() + start + per_req, 0u);
            cuda_check(cudaMemsetAsync(table->dev + start, 0, per_req * sizeof(uint32_t), table->ctx->stream),
                       "cudaMemsetAsync");
        }
    });
}

int32_t psi_table_device_ptr(psi_table* table, void** out) {
    if (table == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    *out = table->dev;
    return PSI_OK;
}

// ---------------------------------------------------------------------------------------------------------------------
// host-side policy
// ---------------------------------------------------------------------------------------------------------------------
int32_t psi_replay_bucket_policy(uint32_t max_capacity, const uint32_t* boundaries, uint32_t num_boundaries,
                                 uint32_t* out, uint64_t out_cap, uint64_t* out_n) {
    return guarded(nullptr, [&] {
        require(out_n != nullptr, "out_n must not be null");
        BucketPolicy policy(max_capacity, std::vector<uint32_t>(boundaries, boundaries + num_boundaries));
        *out_n = policy.buckets().size();
        require(out != nullptr && out_cap >= policy.buckets().size(), "bucket output capacity too small");
        std::copy(policy.buckets().begin(), policy.buckets().end(), out);
    });
}

int32_t psi_replay_bucket_capacity(uint32_t max_capacity, const uint32_t* boundaries, uint32_t num_boundaries,
                                   uint32_t active, uint32_t* out) {
    return guarded(nullptr, [&] {
        require(out != nullptr, "out must not be null");
        BucketPolicy policy(max_capacity, std::vector<uint32_t>(boundaries, boundaries + num_boundaries));
        *out = policy.capacity(active);
    });
}

int32_t psi_split_kv_select(uint32_t io_dtype, uint32_t page_bytes, uint32_t num_q_heads, uint32_t num_kv_heads,
                            uint32_t head_dim, uint32_t dspark_history, uint32_t num_tokens,
                            uint32_t num_q_token_tiles, psi_split_kv_variant* out, uint32_t* out_max_q) {
    return guarded(nullptr, [&] {
        require(out != nullptr, "out must not be null");
        SplitKvSelector selector(io_dtype, page_bytes, num_q_heads, num_kv_heads, head_dim, dspark_history != 0);
        if (out_max_q != nullptr) *out_max_q = selector.max_q_tokens_per_partial_output();
        *out = selector.select(num_tokens, num_q_token_tiles);
    });
}

int32_t psi_metadata_update_host(uint32_t max_tokens, const uint32_t* req_slots, const uint32_t* token_indices,
                                 const uint32_t* cu_tokens, uint32_t num_reqs, const psi_split_kv_variant* variant,
                                 uint32_t capacity_mode, const uint32_t* boundaries, uint32_t num_boundaries,
                                 uint32_t caller_num_total_tokens, uint32_t* buf_req_slots,
                                 uint32_t* buf_flat_token_indices, uint32_t* buf_q_token_tiles, uint32_t* buf_kv_splits,
                                 uint32_t* buf_cu_kv_splits, psi_replay_shape* out_shape) {
    return guarded(nullptr, [&] {
        require(req_slots && token_indices && cu_tokens && variant && out_shape, "metadata inputs must not be null");
        require(buf_req_slots && buf_flat_token_indices && buf_q_token_tiles && buf_kv_splits && buf_cu_kv_splits,
                "metadata buffers must not be null");
        require(capacity_mode <= PSI_CAPACITY_CALLER_TOKENS, "unknown capacity mode");
        ReferenceMetadata md(max_tokens);
        const size_t t = max_tokens;
        std::copy(buf_req_slots, buf_req_slots + t, md.req_slots.begin());
        std::copy(buf_flat_token_indices, buf_flat_token_indices + t, md.flat_token_indices.begin());
        std::copy(buf_q_token_tiles, buf_q_token_tiles + 2 * t, md.q_token_tiles.begin());
        std::copy(buf_kv_splits, buf_kv_splits + 3 * t, md.kv_splits.begin());
        std::copy(buf_cu_kv_splits, buf_cu_kv_splits + t + 1, md.cu_kv_splits.begin());
        *out_shape = md.update(req_slots, token_indices, cu_tokens, num_reqs, *variant, capacity_mode,
                               std::vector<uint32_t>(boundaries, boundaries + num_boundaries), caller_num_total_tokens);
        std::copy(md.req_slots.begin(), md.req_slots.end(), buf_req_slots);
        std::copy(md.flat_token_indices.begin(), md.flat_token_indices.end(), buf_flat_token_indices);
        std::copy(md.q_token_tiles.begin(), md.q_token_tiles.end(), buf_q_token_tiles);
        std::copy(md.kv_splits.begin(), md.kv_splits.end(), buf_kv_splits);
        std::copy(md.cu_kv_splits.begin(), md.cu_kv_splits.end(), buf_cu_kv_splits);
    });
}

int32_t psi_plan_preview(uint32_t num_q_heads, uint32_t num_kv_heads, const uint32_t* token_indices,
                         const uint32_t* cu_tokens, uint32_t num_reqs, uint32_t max_ctas, uint32_t min_kv_tiles_per_cta,
                         uint32_t item_start_cost, uint32_t* out_items, uint64_t items_cap, uint32_t* out_cta_item_begin, uint64_t cta_cap,
                         uint32_t* out_counts) {
    return guarded(nullptr, [&] {
        require(token_indices && cu_tokens && out_counts, "plan inputs must not be null");
        require(num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0,
                "GQA q heads must be a positive multiple of kv heads");
        require(num_reqs > 0 && cu_tokens[0] == 0, "GQA batch cu_tokens must start at zero");
        for (uint32_t r = 0; r < num_reqs; ++r)
            require(cu_tokens[r] <= cu_tokens[r + 1], "GQA batch cu_tokens must be nondecreasing");
        const std::vector<uint32_t> slots(num_reqs, 0u);
        const WorkPlan plan = build_balanced_plan(plan_geometry(num_q_heads, num_kv_heads), slots.data(), token_indices,
                                                  cu_tokens, num_reqs, max_ctas, min_kv_tiles_per_cta, item_start_cost);
        out_counts[0] = static_cast<uint32_t>(plan.items.size());
        out_counts[1] = plan.num_ctas();
        out_counts[2] = plan.num_partial_slots;
        out_counts[3] = static_cast<uint32_t>(plan.reduces.size());
        out_counts[4] = static_cast<uint32_t>(plan.tiles.size());
        out_counts[5] = static_cast<uint32_t>(std::min<uint64_t>(plan.total_kv_tiles, kU32Max));
        if (out_items != nullptr) {
            require(items_cap >= plan.items.size(), "item output capacity too small");
            for (size_t i = 0; i < plan.items.size(); ++i) {
                const WorkItem& it = plan.items[i];
                uint32_t* o = out_items + i * 6;
                o[0] = it.tile;
                o[1] = it.head_sel;
                o[2] = it.kv_begin;
                o[3] = it.kv_end;
                o[4] = it.partial_slot;
                o[5] = plan.tiles[it.tile].flat_begin;
            }
        }
        if (out_cta_item_begin != nullptr) {
            require(cta_cap >= plan.cta_item_begin.size(), "cta output capacity too small");
            std::copy(plan.cta_item_begin.begin(), plan.cta_item_begin.end(), out_cta_item_begin);
        }
    });
}

int32_t psi_chunk_plan_preview(uint32_t num_q_heads, uint32_t num_kv_heads, const uint32_t* token_indices,
                               const uint32_t* cu_tokens, uint32_t num_reqs, uint32_t max_ctas, uint32_t equal_shares,
                               uint32_t* out_items, uint64_t items_cap, uint32_t* out_cta_item_begin, uint64_t cta_cap,
                               uint32_t* out_counts) {
    return guarded(nullptr, [&] {
        require(token_indices && cu_tokens && out_counts, "plan inputs must not be null");
        require(num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0,
                "GQA q heads must be a positive multiple of kv heads");
        require(num_reqs > 0 && cu_tokens[0] == 0, "GQA batch cu_tokens must start at zero");
        std::vector<uint32_t> slots(num_reqs), requests(num_reqs);
        for (uint32_t r = 0; r < num_reqs; ++r) {
            require(cu_tokens[r] < cu_tokens[r + 1], "every request of a long-run plan needs query tokens");
            slots[r] = r;
            requests[r] = r;
        }
        const ChunkPlan plan = build_chunk_plan(plan_geometry(num_q_heads, num_kv_heads), slots.data(), token_indices,
                                                cu_tokens, requests, max_ctas, 0, 0, equal_shares != 0);
        out_counts[0] = static_cast<uint32_t>(plan.items.size());
        out_counts[1] = plan.num_ctas();
        out_counts[2] = plan.num_partial_slots;
        out_counts[3] = plan.num_counters;
        out_counts[4] = static_cast<uint32_t>(std::min<uint64_t>(plan.total_kv_tiles, kU32Max));
        if (out_items != nullptr) {
            require(items_cap >= plan.items.size(), "item output capacity too small");
            for (size_t i = 0; i < plan.items.size(); ++i) {
                const DeviceItem& d = plan.items[i];
                uint32_t* o = out_items + i * 10;
                o[0] = d.req_slot;
                o[1] = d.kv_head;
                o[2] = d.flat_begin;
                o[3] = d.num_tokens;
                o[4] = d.kv_begin;
                o[5] = d.kv_end;
                o[6] = d.partial_slot;
                o[7] = d.partial_slot == kU32Max ? 1u : d.unit_num_items;
                o[8] = d.partial_slot == kU32Max ? kU32Max : d.unit_first_slot;
                o[9] = d.partial_slot == kU32Max ? kU32Max : d.reduce_unit;
            }
        }
        if (out_cta_item_begin != nullptr) {
            require(cta_cap >= plan.cta_item_begin.size(), "cta output capacity too small");
            std::copy(plan.cta_item_begin.begin(), plan.cta_item_begin.end(), out_cta_item_begin);
        }
    });
}

int32_t psi_id_allocator_create(uint64_t capacity, psi_id_allocator** out) {
    return guarded(nullptr, [&] {
        require(out != nullptr, "out must not be null");
        *out = new psi_id_allocator(capacity);
    });
}

int32_t psi_id_allocator_destroy(psi_id_allocator* a) {
    delete a;
    return PSI_OK;
}

int32_t psi_id_allocator_alloc_many(psi_id_allocator* a, uint64_t count, uint32_t* out_ids) {
    if (a == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        require(out_ids != nullptr || count == 0, "out_ids must not be null");
        a->impl.alloc_many(count, out_ids);
    });
}

int32_t psi_id_allocator_free_many(psi_id_allocator* a, const uint32_t* ids, uint64_t count) {
    if (a == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        require(ids != nullptr || count == 0, "ids must not be null");
        a->impl.free_many(ids, count);
    });
}

int32_t psi_id_allocator_bitmap(psi_id_allocator* a, uint64_t* out_words, uint64_t cap, uint64_t* out_n) {
    if (a == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        const auto& words = a->impl.bitmap();
        if (out_n != nullptr) *out_n = words.size();
        for (uint64_t i = 0; i < words.size() && i < cap && out_words != nullptr; ++i) out_words[i] = words[i];
    });
}

int32_t psi_id_allocator_free_count(psi_id_allocator* a, uint64_t* out) {
    if (a == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    *out = a->impl.free_count();
    return PSI_OK;
}

// ---------------------------------------------------------------------------------------------------------------------
// GQA component
// ---------------------------------------------------------------------------------------------------------------------
int32_t psi_gqa_create(psi_ctx* ctx, const psi_gqa_config* config, psi_gqa** out) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        require(out != nullptr && config != nullptr, "out and config must not be null");
        *out = nullptr;
        const psi_gqa_config& c = *config;
        require(c.num_q_heads > 0 && c.num_kv_heads > 0 && c.head_dim > 0, "GQA head counts and head_dim must be positive");
        require(c.num_q_heads % c.num_kv_heads == 0, "GQA q heads must be a multiple of kv heads");
        require(c.scale > 0.0f && std::isfinite(c.scale), "GQA scale must be positive");
        require(c.dtype <= PSI_DTYPE_F16, "unsupported GQA dtype");
        require(c.max_tokens > 0, "GQA batch metadata requires tokens");
        require(c.plan_mode <= PSI_PLAN_REFERENCE && c.kernel_mode <= PSI_KERNEL_MMA_SYNC, "unknown plan or kernel mode");
        validate_layout(c.layout);
        const uint64_t per_token = uint64_t(c.num_kv_heads) * c.head_dim * 2u * dtype_bytes(c.dtype);
        require(per_token <= kU32Max, "GQA K/V bytes per token must fit u32");
        require(c.page_bytes > 0 && c.page_bytes % per_token == 0,
                "GQA page_bytes must be divisible by the K/V bytes per token");
        require(uint64_t(c.max_tokens) * c.num_q_heads * c.head_dim <= kU32Max,
                "GQA SDPA query/output exceeds the shader u32 count domain");
        require(c.head_dim <= 256, "GQA head_dim above 256 is not supported");
        ctx->bind();

        auto g = std::make_unique<psi_gqa>();
        g->ctx = ctx;
        g->cfg = c;
        g->tokens_per_page = c.page_bytes / static_cast<uint32_t>(per_token);
        g->geo = plan_geometry(c.num_q_heads, c.num_kv_heads);
        const bool mma_ok = attend_mma_supported(c.dtype, c.head_dim, g->tokens_per_page);
        if (c.kernel_mode >= PSI_KERNEL_MMA) require(mma_ok, "the mma kernel does not support this profile");
        g->kernel = (c.kernel_mode == PSI_KERNEL_GENERIC || !mma_ok) ? PSI_KERNEL_GENERIC : PSI_KERNEL_MMA;
        const uint32_t per_sm =
            g->kernel == PSI_KERNEL_MMA ? attend_mma_ctas_per_sm(c.head_dim) : attend_generic_ctas_per_sm();
        g->grid_cap = c.max_ctas > 0 ? c.max_ctas : static_cast<uint32_t>(ctx->sm_count) * per_sm;
        g->item_start_cost = g->kernel == PSI_KERNEL_MMA ? 32u : 0u;
        g->chunk_supported = g->kernel == PSI_KERNEL_MMA && c.plan_mode == PSI_PLAN_BALANCED &&
                             attend_chunk_supported(c.dtype, c.head_dim, g->tokens_per_page);
        g->chunk_umma = g->chunk_supported && c.kernel_mode != PSI_KERNEL_MMA_SYNC;
        if (g->chunk_umma) g->status_word.ensure(ctx, sizeof(uint32_t), true);
        if (c.dtype != PSI_DTYPE_F16) {
            g->selector = std::make_unique<SplitKvSelector>(c.dtype, c.page_bytes, c.num_q_heads, c.num_kv_heads,
                                                            c.head_dim, false);
        }
        g->md = std::make_unique<ReferenceMetadata>(c.max_tokens);
        cuda_check(cudaEventCreateWithFlags(&g->upload_done, cudaEventDisableTiming), "cudaEventCreateWithFlags");
        *out = g.release();
    });
}

int32_t psi_gqa_destroy(psi_gqa* g) {
    if (g == nullptr) return PSI_OK;
    int32_t status = guarded(g->ctx, [&] {
        g->ctx->bind();
        (void)cudaStreamSynchronize(g->ctx->stream);
        g->block.release();
        g->partial_o.release();
        g->partial_ml.release();
        g->unit_counters.release();
        g->step_k.release();
        g->step_v.release();
        g->step_q.release();
        g->step_out.release();
        g->combine_ptrs.release();
        g->status_word.release();
        g->norm_rope.release();
        if (g->staging != nullptr) (void)cudaFreeHost(g->staging);
        if (g->upload_done != nullptr) (void)cudaEventDestroy(g->upload_done);
    });
    delete g;
    return status;
}

int32_t psi_gqa_set_token_topology_boundaries(psi_gqa* g, const uint32_t* boundaries, uint32_t n) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(boundaries != nullptr || n == 0, "boundaries must not be null");
        for (uint32_t i = 0; i < n; ++i) require(boundaries[i] > 0, "replay topology boundary must be positive");
        g->boundaries.assign(boundaries, boundaries + n);
    });
}

// Offsets (in words) of the device block's arrays under a replay reservation: everything sized for max_tokens, the
// arrays whose used length varies most placed last, so that an upload still moves only a prefix.
static void reserved_layout(psi_gqa* g) {
    constexpr uint64_t kItemWords = sizeof(DeviceItem) / sizeof(uint32_t);
    const uint64_t t = g->cfg.max_tokens;
    uint64_t cursor = pad_words(kScalarCount);
    g->off_req_slots = cursor;
    cursor += pad_words(t);
    g->off_token_indices = cursor;
    cursor += pad_words(t);
    g->off_cta = cursor;
    cursor += pad_words(g->grid_cap + 2);
    g->off_first_items = cursor;
    cursor += pad_words(uint64_t(g->grid_cap) * kItemWords);
    g->off_chunk_cta = cursor;
    cursor += pad_words(g->grid_cap + 2);
    g->off_items = cursor;
    cursor += pad_words(g->cap_items * kItemWords);
    g->off_chunk_items = cursor;
    cursor += pad_words(g->cap_chunk_items * kItemWords);
    g->off_reduces = cursor;
    cursor += pad_words(g->cap_reduces * 2);
    g->staging_words = cursor;
}

int32_t psi_gqa_reserve_replay(psi_gqa* g) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        if (g->replay_reserved) return;
        psi_ctx* ctx = g->ctx;
        require(!ctx->capturing, "replay capacity cannot be reserved during stream capture");
        ctx->bind();
        // worst cases for max_tokens: every token a query tile of its own, every unit cut at every CTA boundary
        const uint64_t heads = uint64_t(g->geo.num_kv_heads) * g->geo.head_tiles;
        const uint64_t units = uint64_t(g->cfg.max_tokens) * heads;
        const uint64_t cap_items = units + g->grid_cap;
        const uint64_t chunk_units = g->chunk_supported ? units / 3 + heads : 0;
        const uint64_t cap_chunk_items = g->chunk_supported ? chunk_units + 2ull * g->grid_cap + 8 : 0;
        const uint64_t slots = cap_items + cap_chunk_items * kChunkTilesPerItem;
        const uint64_t partial_bytes = slots * kMaxRows * g->cfg.head_dim * sizeof(float);
        require(partial_bytes <= (2ull << 30),
                "replay reservation needs more than 2 GiB of partial-output scratch for this max_tokens: create the "
                "component with the largest batch the replayed steps carry");
        cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
        g->cap_items = cap_items;
        g->cap_chunk_items = cap_chunk_items;
        g->cap_reduces = units;
        if (g->staging != nullptr) {
            cuda_check(cudaFreeHost(g->staging), "cudaFreeHost");
            g->staging = nullptr;
        }
        reserved_layout(g);
        cuda_check(cudaMallocHost(reinterpret_cast<void**>(&g->staging), g->staging_words * sizeof(uint32_t)), "cudaMallocHost");
        std::memset(g->staging, 0, g->staging_words * sizeof(uint32_t));
        g->block.ensure(ctx, g->staging_words * sizeof(uint32_t), true);
        g->partial_o.ensure(ctx, partial_bytes, false);
        g->partial_ml.ensure(ctx, 2 * slots * kMaxRows * sizeof(float), false);
        g->unit_counters.release();  // counters restart from zero at their new size
        g->unit_counters.ensure(ctx, slots * sizeof(uint32_t), true);
        g->partial_slots_cap = slots;
        g->status_word.ensure(ctx, sizeof(uint32_t), true);
        cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
        g->prepared = false;  // the block moved: the next step prepares again
        g->replay_reserved = true;
    });
}

}  // extern "C"

namespace {

// GQAMetadataBuffers::update plus this library's plan.  With `defer_upload` the packed block stays in the pinned
// staging buffer and its size comes back in *deferred_words: the caller brings it to the device itself.
void prepare_impl(psi_gqa* g, const uint32_t* req_slots, const uint32_t* token_indices, const uint32_t* cu_tokens,
                  uint32_t num_reqs, uint32_t capacity_mode, uint32_t caller_num_total_tokens,
                  psi_replay_shape* out_shape, bool defer_upload, uint64_t* deferred_words) {
    {
        require(req_slots != nullptr && token_indices != nullptr && cu_tokens != nullptr, "metadata inputs must not be null");
        require(capacity_mode <= PSI_CAPACITY_CALLER_TOKENS, "unknown capacity mode");
        require(num_reqs > 0, "GQA batch metadata requires tokens");
        psi_ctx* ctx = g->ctx;
        require(!ctx->capturing, "psi_gqa_prepare uploads the step's plan and stays outside captured graphs");
        ctx->bind();
        g->prepared = false;

        // Variant selection as the reference's executor does it (crates/inference-executor-metal/src/attn/gqa/mod.rs:
        // 64-94, without its measured D256/page8 work model, which tunes a different device).
        require(cu_tokens[0] == 0, "GQA batch cu_tokens must start at zero");
        uint64_t ref_q_tiles = 0;
        for (uint32_t r = 0; r < num_reqs; ++r) {
            require(cu_tokens[r] <= cu_tokens[r + 1], "GQA batch cu_tokens must be nondecreasing");
            ref_q_tiles += (uint64_t(cu_tokens[r + 1] - cu_tokens[r]) + 7) / 8;
        }
        const uint32_t num_tokens = cu_tokens[num_reqs];
        require(num_tokens > 0, "GQA batch metadata requires tokens");
        require(num_tokens <= g->cfg.max_tokens, "GQA batch exceeds the metadata token capacity");
        psi_split_kv_variant variant{};
        if (g->selector) {
            variant = g->selector->select(num_tokens, static_cast<uint32_t>(ref_q_tiles));
        } else {
            variant.kv_token_tile_size = 256;  // f16 has no reference profile: SingleQ geometry of a 256-thread block
            variant.num_threads_per_threadblock = 256;
            variant.q_head_tile_size = std::min(g->geo.group, 8u);
        }
        const psi_replay_shape shape = g->md->update(req_slots, token_indices, cu_tokens, num_reqs, variant,
                                                     capacity_mode, g->boundaries, caller_num_total_tokens);

        const uint64_t table_tokens =
            uint64_t(g->cfg.layout.num_blocks) * g->cfg.layout.num_page_ids_per_block * g->tokens_per_page;
        for (uint32_t r = 0; r < num_reqs; ++r) {
            require(req_slots[r] < g->cfg.layout.num_req_slots, "GQA request page table req_slot out of range");
            require(uint64_t(token_indices[r]) + (cu_tokens[r + 1] - cu_tokens[r]) <= table_tokens,
                    "GQA request context does not fit the request page table");
        }

        if (g->cfg.plan_mode == PSI_PLAN_REFERENCE) {
            g->plan = build_reference_plan(g->geo, *g->md, shape, variant.tiled_q != 0, token_indices, cu_tokens,
                                           num_reqs);
            g->chunk = ChunkPlan{};
        } else {
            // Requests with a long run of query tokens go to the chunk kernel (one pass over their KV for eight query
            // tiles at a time); the rest are decode rows.
            std::vector<uint32_t> decode_reqs, chunk_reqs;
            for (uint32_t r = 0; r < num_reqs; ++r) {
                const uint32_t tiles = (cu_tokens[r + 1] - cu_tokens[r] + g->geo.tokens_per_tile - 1) / g->geo.tokens_per_tile;
                if (tiles == 0) continue;
                (g->chunk_supported && tiles >= kChunkMinTiles ? chunk_reqs : decode_reqs).push_back(r);
            }
            const uint32_t min_tiles = g->kernel == PSI_KERNEL_MMA ? 16u : 4u;
            g->plan = build_balanced_plan(g->geo, req_slots, token_indices, cu_tokens, decode_reqs, g->grid_cap,
                                          min_tiles, g->item_start_cost);
            // K/V the long runs touch: below a third of the L2 the order of the work cannot cost HBM traffic, and exactly
            // equal shares beat stream order
            uint64_t chunk_kv_bytes = 0;
            for (uint32_t r : chunk_reqs)
                chunk_kv_bytes += uint64_t(token_indices[r] + (cu_tokens[r + 1] - cu_tokens[r])) * (uint64_t(g->cfg.page_bytes) / g->tokens_per_page);
            g->chunk = build_chunk_plan(g->geo, req_slots, token_indices, cu_tokens, chunk_reqs, g->grid_cap,
                                        g->plan.num_partial_slots, static_cast<uint32_t>(g->plan.reduces.size()),
                                        chunk_kv_bytes <= (40ull << 20));
        }
        const WorkPlan& plan = g->plan;
        const ChunkPlan& chunk = g->chunk;
        const std::vector<DeviceItem> device_items = flatten_plan(plan, g->geo);
        const uint32_t total_slots = plan.num_partial_slots + chunk.num_partial_slots;
        const uint32_t total_counters = static_cast<uint32_t>(plan.reduces.size()) + chunk.num_counters;

        // Pack the device block: scalars | req_slots | flat_token_indices | cta ranges | reduces | items.
        uint64_t words = 0;
        if (g->replay_reserved) {
            // fixed offsets (reserved_layout); only the used prefix is uploaded
            constexpr uint64_t kItemWords = sizeof(DeviceItem) / sizeof(uint32_t);
            require(device_items.size() <= g->cap_items && chunk.items.size() <= g->cap_chunk_items &&
                        plan.reduces.size() <= g->cap_reduces && total_slots <= g->partial_slots_cap &&
                        plan.num_ctas() <= g->grid_cap && chunk.num_ctas() <= g->grid_cap,
                    "the step exceeds the reserved replay capacity");
            words = g->off_items + device_items.size() * kItemWords;
            if (!chunk.items.empty()) words = g->off_chunk_items + chunk.items.size() * kItemWords;
            if (!plan.reduces.empty()) words = g->off_reduces + plan.reduces.size() * 2;
            cuda_check(cudaEventSynchronize(g->upload_done), "cudaEventSynchronize");  // previous upload left staging
        } else {
            uint64_t cursor = pad_words(kScalarCount);
            g->off_req_slots = cursor;
            cursor += pad_words(num_tokens);
            g->off_token_indices = cursor;
            cursor += pad_words(num_tokens);
            g->off_cta = cursor;
            cursor += pad_words(plan.cta_item_begin.size());
            g->off_reduces = cursor;
            cursor += pad_words(plan.reduces.size() * 2);
            g->off_items = cursor;
            cursor += pad_words(device_items.size() * (sizeof(DeviceItem) / sizeof(uint32_t)));
            g->off_first_items = cursor;
            cursor += pad_words(static_cast<uint64_t>(plan.num_ctas()) * (sizeof(DeviceItem) / sizeof(uint32_t)));
            g->off_chunk_cta = cursor;
            cursor += pad_words(chunk.cta_item_begin.size());
            g->off_chunk_items = cursor;
            cursor += pad_words(chunk.items.size() * (sizeof(DeviceItem) / sizeof(uint32_t)));
            words = cursor;

            if (g->staging_words < words) {
                if (g->staging != nullptr) {
                    cuda_check(cudaEventSynchronize(g->upload_done), "cudaEventSynchronize");
                    cuda_check(cudaFreeHost(g->staging), "cudaFreeHost");
                    g->staging = nullptr;
                }
                const uint64_t grown = std::max<uint64_t>(words * 2, 4096);
                cuda_check(cudaMallocHost(reinterpret_cast<void**>(&g->staging), grown * sizeof(uint32_t)), "cudaMallocHost");
                g->staging_words = grown;
            } else {
                cuda_check(cudaEventSynchronize(g->upload_done), "cudaEventSynchronize");  // previous upload left staging
            }
        }
        g->block.ensure(ctx, g->staging_words * sizeof(uint32_t), false);
        if (total_slots > g->partial_slots_cap) {
            const uint64_t slots = std::max<uint64_t>(total_slots, 2ull * g->grid_cap);
            g->partial_o.ensure(ctx, slots * kMaxRows * g->cfg.head_dim * sizeof(float), false);
            g->partial_ml.ensure(ctx, 2 * slots * kMaxRows * sizeof(float), false);
            g->unit_counters.ensure(ctx, slots * sizeof(uint32_t), true);
            g->partial_slots_cap = slots;
        }
        // Arrival counters start at zero (cleared when allocated) and every launch returns them to zero itself.
        (void)total_counters;

        uint32_t* s = g->staging;
        std::fill(s, s + kScalarCount, 0u);
        s[kScalarNumActiveTokens] = num_tokens;
        s[kScalarNumCtas] = plan.num_ctas();
        s[kScalarNumReduces] = static_cast<uint32_t>(plan.reduces.size());
        s[kScalarNumChunkCtas] = chunk.num_ctas();
        std::copy(g->md->req_slots.begin(), g->md->req_slots.begin() + num_tokens, s + g->off_req_slots);
        std::copy(g->md->flat_token_indices.begin(), g->md->flat_token_indices.begin() + num_tokens,
                  s + g->off_token_indices);
        std::copy(plan.cta_item_begin.begin(), plan.cta_item_begin.end(), s + g->off_cta);
        if (g->replay_reserved) {
            // launches run at the capacity grid: CTAs beyond the plan's find an empty range and a zero first item
            constexpr uint64_t kItemWords = sizeof(DeviceItem) / sizeof(uint32_t);
            const uint32_t items_end = static_cast<uint32_t>(device_items.size());
            for (uint64_t c = plan.cta_item_begin.size(); c < g->grid_cap + 2ull; ++c) s[g->off_cta + c] = items_end;
            if (plan.cta_item_begin.empty()) s[g->off_cta] = 0;
            std::fill(s + g->off_first_items, s + g->off_first_items + uint64_t(g->grid_cap) * kItemWords, 0u);
            const uint32_t chunk_end = static_cast<uint32_t>(chunk.items.size());
            for (uint64_t c = chunk.cta_item_begin.size(); c < g->grid_cap + 2ull; ++c) s[g->off_chunk_cta + c] = chunk_end;
            if (chunk.cta_item_begin.empty()) s[g->off_chunk_cta] = 0;
        }
        if (!plan.reduces.empty())
            std::memcpy(s + g->off_reduces, plan.reduces.data(), plan.reduces.size() * sizeof(ReduceUnit));
        if (!device_items.empty())
            std::memcpy(s + g->off_items, device_items.data(), device_items.size() * sizeof(DeviceItem));
        // a copy of every CTA's first item at a place the CTA can read without knowing its range (zeros for a CTA
        // without items, which its empty range tells it not to use)
        for (uint32_t c = 0; c < plan.num_ctas(); ++c) {
            DeviceItem first{};
            if (plan.cta_item_begin[c] < plan.cta_item_begin[c + 1]) first = device_items[plan.cta_item_begin[c]];
            std::memcpy(s + g->off_first_items + static_cast<uint64_t>(c) * (sizeof(DeviceItem) / sizeof(uint32_t)), &first,
                        sizeof(DeviceItem));
        }
        std::copy(chunk.cta_item_begin.begin(), chunk.cta_item_begin.end(), s + g->off_chunk_cta);
        if (!chunk.items.empty())
            std::memcpy(s + g->off_chunk_items, chunk.items.data(), chunk.items.size() * sizeof(DeviceItem));
        if (defer_upload) {
            *deferred_words = words;
        } else {
            cuda_check(cudaMemcpyAsync(g->block.ptr, s, words * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream),
                       "cudaMemcpyAsync");
            cuda_check(cudaEventRecord(g->upload_done, ctx->stream), "cudaEventRecord");
        }

        g->shape = shape;
        g->variant = variant;
        g->prepared = true;
        if (out_shape != nullptr) *out_shape = shape;
    }
}

}  // namespace

extern "C" {

int32_t psi_gqa_prepare(psi_gqa* g, const uint32_t* req_slots, const uint32_t* token_indices, const uint32_t* cu_tokens,
                        uint32_t num_reqs, uint32_t capacity_mode, uint32_t caller_num_total_tokens,
                        psi_replay_shape* out_shape) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        prepare_impl(g, req_slots, token_indices, cu_tokens, num_reqs, capacity_mode, caller_num_total_tokens, out_shape,
                     false, nullptr);
    });
}

int32_t psi_gqa_split_kv_variant(psi_gqa* g, psi_split_kv_variant* out) {
    if (g == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(g->prepared, "GQA batch metadata must be updated before recording");
        *out = g->variant;
    });
}

static std::vector<uint32_t>* metadata_array(psi_gqa* g, uint32_t which) {
    switch (which) {
        case PSI_MD_REQ_SLOTS: return &g->md->req_slots;
        case PSI_MD_FLAT_TOKEN_INDICES: return &g->md->flat_token_indices;
        case PSI_MD_Q_TOKEN_TILES: return &g->md->q_token_tiles;
        case PSI_MD_KV_SPLITS: return &g->md->kv_splits;
        case PSI_MD_CU_KV_SPLITS: return &g->md->cu_kv_splits;
        default: return nullptr;
    }
}

int32_t psi_gqa_metadata_read(psi_gqa* g, uint32_t which, uint64_t offset, uint32_t* out, uint64_t n) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        auto* array = metadata_array(g, which);
        require(array != nullptr && out != nullptr, "unknown metadata array or null output");
        require(offset <= array->size() && n <= array->size() - offset, "metadata range out of bounds");
        std::copy(array->begin() + offset, array->begin() + offset + n, out);
    });
}

int32_t psi_gqa_metadata_write(psi_gqa* g, uint32_t which, uint64_t offset, const uint32_t* in, uint64_t n) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        auto* array = metadata_array(g, which);
        require(array != nullptr && in != nullptr, "unknown metadata array or null input");
        require(offset <= array->size() && n <= array->size() - offset, "metadata range out of bounds");
        std::copy(in, in + n, array->begin() + offset);
    });
}

int32_t psi_gqa_plan_stats(psi_gqa* g, uint32_t* out, uint32_t n) {
    if (g == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(g->prepared, "GQA batch metadata must be updated before recording");
        const uint32_t stats[12] = {g->plan.num_ctas(),
                                   static_cast<uint32_t>(g->plan.items.size()),
                                   g->plan.num_partial_slots,
                                   static_cast<uint32_t>(g->plan.reduces.size()),
                                   static_cast<uint32_t>(g->plan.tiles.size()),
                                   g->kernel,
                                   static_cast<uint32_t>(std::min<uint64_t>(g->plan.total_kv_tiles, kU32Max)),
                                   g->geo.tokens_per_tile * g->geo.heads_per_tile,
                                   g->chunk.num_ctas(),
                                   static_cast<uint32_t>(g->chunk.items.size()),
                                   g->chunk_launches[0],
                                   g->chunk_launches[1]};
        for (uint32_t i = 0; i < n && i < 12; ++i) out[i] = stats[i];
    });
}

int32_t psi_gqa_kv_append(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k, const void* v) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        g->ctx->bind();
        run_append(g, pages, table, layer, k, v);
    });
}

int32_t psi_gqa_attend(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* q, void* out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(out != nullptr, "out must not be null");
        g->ctx->bind();
        AttendParams p = attend_params(g, pages, table, layer, q);
        p.out = out;
        run_attend(g, p);
    });
}

int32_t psi_gqa_append_attend(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k,
                              const void* v, const void* q, void* out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(out != nullptr && k != nullptr && v != nullptr, "k, v and out must not be null");
        g->ctx->bind();
        if (g->kernel != PSI_KERNEL_MMA) {  // the generic kernel has no fused form: two launches in stream order
            run_append(g, pages, table, layer, k, v);
            AttendParams p = attend_params(g, pages, table, layer, q);
            p.out = out;
            run_attend(g, p);
            return;
        }
        require((reinterpret_cast<uintptr_t>(k) & 15u) == 0 && (reinterpret_cast<uintptr_t>(v) & 15u) == 0,
                "k and v must be 16-byte aligned");
        AttendParams p = attend_params(g, pages, table, layer, q);
        p.out = out;
        p.new_k = k;
        p.new_v = v;
        run_attend(g, p);
    });
}

int32_t psi_rope_parameters(const psi_norm_rope_config* config, float* out_inverse_frequencies,
                            float* out_attention_factor, float* out_correction_low, float* out_correction_high) {
    return guarded(nullptr, [&] {
        require(config != nullptr && out_inverse_frequencies != nullptr && out_attention_factor != nullptr,
                "rope parameter outputs must not be null");
        const RopeParameters params = rope_parameters(*config);
        std::copy(params.inverse_frequencies.begin(), params.inverse_frequencies.end(), out_inverse_frequencies);
        *out_attention_factor = params.attention_factor;
        if (out_correction_low != nullptr) *out_correction_low = params.correction_low;
        if (out_correction_high != nullptr) *out_correction_high = params.correction_high;
    });
}

int32_t psi_gqa_set_norm_rope(psi_gqa* g, const psi_norm_rope_config* config, const uint16_t* q_weight,
                              const uint16_t* k_weight) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(config != nullptr && q_weight != nullptr && k_weight != nullptr, "norm/rope arguments must not be null");
        require(config->rope_dim <= g->cfg.head_dim, "RoPE dimension exceeds head_dim");
        require(std::isfinite(config->eps) && config->eps >= 0.0f, "RMSNorm eps must be finite and non-negative");
        const RopeParameters params = rope_parameters(*config);
        psi_ctx* ctx = g->ctx;
        ctx->bind();
        const uint32_t d = g->cfg.head_dim;
        const uint64_t weight_bytes = (uint64_t(d) * 2 + 15) / 16 * 16;
        std::vector<unsigned char> host(2 * weight_bytes + params.inverse_frequencies.size() * sizeof(float), 0);
        std::memcpy(host.data(), q_weight, size_t(d) * 2);
        std::memcpy(host.data() + weight_bytes, k_weight, size_t(d) * 2);
        std::memcpy(host.data() + 2 * weight_bytes, params.inverse_frequencies.data(),
                    params.inverse_frequencies.size() * sizeof(float));
        g->norm_rope.ensure(ctx, host.size(), false);
        cuda_check(cudaMemcpyAsync(g->norm_rope.ptr, host.data(), host.size(), cudaMemcpyHostToDevice, ctx->stream),
                   "cudaMemcpyAsync");  // pageable source: staged before the call returns
        g->norm_rope_cfg = *config;
        g->norm_rope_attention_factor = params.attention_factor;
        g->has_norm_rope = true;
    });
}

namespace {

// Fills everything of the front-stage launch that does not depend on where q, k, v and the gates come from.
PrepParams norm_rope_params(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer) {
    PrepParams p{};
    p.geo = page_geometry(g, pages, table, layer);
    const uint64_t weight_bytes = (uint64_t(g->cfg.head_dim) * 2 + 15) / 16 * 16;
    const auto* base = static_cast<const unsigned char*>(g->norm_rope.ptr);
    p.q_weight = base;
    p.k_weight = base + weight_bytes;
    p.inverse_frequencies = reinterpret_cast<const float*>(base + 2 * weight_bytes);
    p.attention_factor = g->norm_rope_attention_factor;
    p.eps = g->norm_rope_cfg.eps;
    p.rope_dim = g->norm_rope_cfg.rope_dim;
    p.num_q_heads = g->cfg.num_q_heads;
    p.dtype = g->cfg.dtype;
    p.req_slots = block_words(g, g->off_req_slots);
    p.flat_token_indices = block_words(g, g->off_token_indices);
    p.scalars = block_words(g, 0);
    p.num_total_tokens = g->shape.num_total_tokens;
    return p;
}

}  // namespace

int32_t psi_gqa_norm_rope_append(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* q_in,
                                 const void* k_in, const void* v_in, void* q_out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(g->prepared, "GQA batch metadata must be updated before recording");
        require(g->has_norm_rope, "psi_gqa_set_norm_rope must be called before psi_gqa_norm_rope_append");
        require(q_in != nullptr && k_in != nullptr && v_in != nullptr && q_out != nullptr, "buffers must not be null");
        g->ctx->bind();
        PrepParams p = norm_rope_params(g, pages, table, layer);
        p.q_in = q_in;
        p.k_in = k_in;
        p.v_in = v_in;
        p.q_out = q_out;
        p.q_head_stride = g->cfg.head_dim;
        p.q_token_stride = uint64_t(g->cfg.num_q_heads) * g->cfg.head_dim;
        p.kv_token_stride = uint64_t(g->cfg.num_kv_heads) * g->cfg.head_dim;
        LaunchScope scope(g->ctx, PSI_KERNEL_CLASS_NORM_ROPE_APPEND);
        cuda_check(launch_norm_rope_append(p, g->ctx->stream), "norm/rope/append launch");
    });
}

int32_t psi_gqa_projection_norm_rope_append(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer,
                                            const void* projection, uint32_t gated, void* q_out, void* gates_out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(g->prepared, "GQA batch metadata must be updated before recording");
        require(g->has_norm_rope, "psi_gqa_set_norm_rope must be called before psi_gqa_projection_norm_rope_append");
        require(projection != nullptr && q_out != nullptr, "buffers must not be null");
        require(gated <= 1, "gated must be 0 or 1");
        require(gated == 0 || gates_out != nullptr, "a gated projection needs gates_out");
        const uint64_t d = g->cfg.head_dim, hq = g->cfg.num_q_heads, hkv = g->cfg.num_kv_heads;
        const uint64_t q_width = (gated ? 2 : 1) * hq * d, width = q_width + 2 * hkv * d;
        // the reference's split shaders index one projection element per thread with a u32
        // (crates/inference-backend-metal/src/components/gqa_qgkv_split.rs:121-125, gqa_qkv_split.rs)
        require(uint64_t(g->shape.num_total_tokens) * width <= 0xFFFFFFFFull,
                gated ? "GQA projection elements exceeds the shader u32 count domain"
                      : "ungated GQA projection elements exceeds the shader u32 count domain");
        g->ctx->bind();
        PrepParams p = norm_rope_params(g, pages, table, layer);
        const uint64_t esz = dtype_bytes(g->cfg.dtype);
        const auto* base = static_cast<const unsigned char*>(projection);
        p.q_in = base;
        p.q_head_stride = gated ? 2 * d : d;
        p.q_token_stride = width;
        p.kv_token_stride = width;
        p.k_in = base + q_width * esz;
        p.v_in = base + (q_width + hkv * d) * esz;
        p.q_out = q_out;
        if (gated) {
            p.g_in = base + d * esz;  // head h of a token: q at h * 2D, its gate at h * 2D + D
            p.g_out = gates_out;
        }
        LaunchScope scope(g->ctx, PSI_KERNEL_CLASS_NORM_ROPE_APPEND);
        cuda_check(launch_norm_rope_append(p, g->ctx->stream), "projection split/norm/rope/append launch");
    });
}

int32_t psi_gqa_attend_gated(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* q,
                             const void* gates, void* out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(out != nullptr && gates != nullptr, "gates and out must not be null");
        require((reinterpret_cast<uintptr_t>(gates) & 7u) == 0, "gates must be 8-byte aligned");
        g->ctx->bind();
        AttendParams p = attend_params(g, pages, table, layer, q);
        p.out = out;
        p.gates = gates;
        run_attend(g, p);
    });
}

int32_t psi_gqa_attend_partial(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* q, float* o,
                               float* m, float* l) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(o != nullptr && m != nullptr && l != nullptr, "partial outputs must not be null");
        require((reinterpret_cast<uintptr_t>(o) & 15u) == 0, "partial output o must be 16-byte aligned");
        g->ctx->bind();
        AttendParams p = attend_params(g, pages, table, layer, q);
        p.ext_o = o;
        p.ext_m = m;
        p.ext_l = l;
        run_attend(g, p);
    });
}

static int32_t combine_impl(psi_gqa* g, const float* const* o, const float* const* m, const float* const* l, uint32_t n,
                            uint32_t num_tokens, void* out, const uint32_t* flags, uint32_t flag_value,
                            uint32_t max_polls) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(o != nullptr && m != nullptr && l != nullptr && out != nullptr, "combine arguments must not be null");
        require(n > 0 && n <= 64, "combine takes between 1 and 64 partials");
        require(num_tokens > 0 && num_tokens <= g->cfg.max_tokens, "combine token count out of range");
        psi_ctx* ctx = g->ctx;
        ctx->bind();
        g->combine_ptrs.ensure(ctx, 3 * 64 * sizeof(void*), false);
        std::vector<const float*> host(3 * 64, nullptr);
        for (uint32_t i = 0; i < n; ++i) {
            require(o[i] != nullptr && m[i] != nullptr && l[i] != nullptr, "combine partial pointers must not be null");
            host[i] = o[i];
            host[64 + i] = m[i];
            host[128 + i] = l[i];
        }
        // Pageable source: the runtime stages the bytes before the call returns, so `host` may go out of scope.
        cuda_check(cudaMemcpyAsync(g->combine_ptrs.ptr, host.data(), host.size() * sizeof(void*),
                                   cudaMemcpyHostToDevice, ctx->stream),
                   "cudaMemcpyAsync");
        CombineParams p{};
        auto* base = static_cast<const float* const*>(g->combine_ptrs.ptr);
        p.o = base;
        p.m = base + 64;
        p.l = base + 128;
        p.n = n;
        p.num_rows = num_tokens * g->cfg.num_q_heads;
        p.head_dim = g->cfg.head_dim;
        p.dtype = g->cfg.dtype;
        p.out = out;
        if (flags != nullptr) {
            g->status_word.ensure(ctx, sizeof(uint32_t), true);
            p.flags = flags;
            p.flag_value = flag_value;
            p.max_polls = max_polls == 0 ? 2000000u : max_polls;  // ~100 ns per poll: a fraction of a second by default
            p.status = static_cast<uint32_t*>(g->status_word.ptr);
        }
        LaunchScope scope(ctx, PSI_KERNEL_CLASS_COMBINE);
        cuda_check(launch_combine(p, ctx->stream), "combine launch");
    });
}

int32_t psi_gqa_block_partial(psi_gqa* g, const void* q, const void* local_k, const void* local_v, uint32_t num_tokens,
                              uint32_t block_size, const uint32_t* slot_indices, float* o, float* m, float* l) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(q != nullptr && local_k != nullptr && local_v != nullptr, "q, local_k and local_v must not be null");
        require(o != nullptr && m != nullptr && l != nullptr, "partial outputs must not be null");
        require(block_size > 0 && block_size <= 256, "GQA block SDPA block size must be in 1..=256");
        require(num_tokens > 0, "GQA block SDPA requires tokens");
        require(num_tokens % block_size == 0, "GQA block SDPA tokens must contain complete request blocks");
        g->ctx->bind();
        BlockPartialParams p{};
        p.q = q;
        p.local_k = local_k;
        p.local_v = local_v;
        p.slot_indices = slot_indices;
        p.o = o;
        p.m = m;
        p.l = l;
        p.num_tokens = num_tokens;
        p.block_size = block_size;
        p.num_q_heads = g->cfg.num_q_heads;
        p.num_kv_heads = g->cfg.num_kv_heads;
        p.head_dim = g->cfg.head_dim;
        p.dtype = g->cfg.dtype;
        p.scale = g->cfg.scale;
        g->ctx->launches += 1;
        cuda_check(launch_block_partial(p, g->ctx->stream), "block partial launch");
    });
}

int32_t psi_gqa_combine(psi_gqa* g, const float* const* o, const float* const* m, const float* const* l, uint32_t n,
                        uint32_t num_tokens, void* out) {
    return combine_impl(g, o, m, l, n, num_tokens, out, nullptr, 0, 0);
}

int32_t psi_gqa_combine_wait(psi_gqa* g, const float* const* o, const float* const* m, const float* const* l,
                             uint32_t n, uint32_t num_tokens, void* out, const uint32_t* flags, uint32_t flag_value,
                             uint32_t max_polls) {
    if (flags == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return combine_impl(g, o, m, l, n, num_tokens, out, flags, flag_value, max_polls);
}

int32_t psi_gqa_signal(psi_gqa* g, uint32_t* flag, uint32_t value) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(flag != nullptr, "flag must not be null");
        g->ctx->bind();
        g->ctx->launches += 1;
        cuda_check(launch_signal(flag, value, g->ctx->stream), "signal launch");
    });
}

int32_t psi_gqa_device_status(psi_gqa* g, int32_t* out) {
    if (g == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        g->ctx->bind();
        cuda_check(cudaStreamSynchronize(g->ctx->stream), "cudaStreamSynchronize");
        uint32_t word = 0;
        if (g->status_word.ptr != nullptr) {
            cuda_check(cudaMemcpy(&word, g->status_word.ptr, sizeof(word), cudaMemcpyDeviceToHost), "cudaMemcpy");
            if (word != 0) cuda_check(cudaMemset(g->status_word.ptr, 0, sizeof(word)), "cudaMemset");
        }
        *out = static_cast<int32_t>(word);
    });
}

int32_t psi_gqa_decode_step_host(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k_host,
                                 const void* v_host, const void* q_host, void* out_host) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(k_host != nullptr && v_host != nullptr && q_host != nullptr && out_host != nullptr,
                "host buffers must not be null");
        require(g->prepared, "GQA batch metadata must be updated before recording");
        psi_ctx* ctx = g->ctx;
        ctx->bind();
        const uint64_t esz = dtype_bytes(g->cfg.dtype);
        const uint64_t kv_cap = uint64_t(g->cfg.max_tokens) * g->cfg.num_kv_heads * g->cfg.head_dim * esz;
        const uint64_t q_cap = uint64_t(g->cfg.max_tokens) * g->cfg.num_q_heads * g->cfg.head_dim * esz;
        const uint64_t kv_bytes = uint64_t(g->shape.num_tokens) * g->cfg.num_kv_heads * g->cfg.head_dim * esz;
        const uint64_t q_bytes = uint64_t(g->shape.num_tokens) * g->cfg.num_q_heads * g->cfg.head_dim * esz;
        g->step_k.ensure(ctx, kv_cap, false);
        g->step_v.ensure(ctx, kv_cap, false);
        g->step_q.ensure(ctx, q_cap, false);
        // Pinned, device-mapped host buffers: one launch pulls q/k/v over the host link into device staging (small
        // steps: every work item waits for its query rows, which come sooner from HBM than from the host), and the
        // attention launch stores `out` straight into the host buffer.  Two launches and one wait, no copy engine
        // round trips.
        if (g->kernel == PSI_KERNEL_MMA && kv_bytes % 16 == 0 && q_bytes % 16 == 0) {
            void* dk = mapped_device_pointer(k_host);
            void* dv = mapped_device_pointer(v_host);
            void* dq = mapped_device_pointer(q_host);
            void* dout = mapped_device_pointer(out_host);
            if (dk != nullptr && dv != nullptr && dq != nullptr && dout != nullptr) {
                // the size rule of psi_gqa_step_host: large steps without long query runs are read in place
                const bool direct = q_bytes + 2 * kv_bytes >= kDirectHostBytes && !g->replay_reserved &&
                                    g->chunk.num_ctas() == 0;
                if (!direct) {
                    const void* const src[kPullBuffers] = {dq, dk, dv, nullptr};
                    void* const dst[kPullBuffers] = {g->step_q.ptr, g->step_k.ptr, g->step_v.ptr, nullptr};
                    const uint64_t bytes[kPullBuffers] = {q_bytes, kv_bytes, kv_bytes, 0};
                    ctx->launches += 1;
                    cuda_check(launch_host_pull(src, dst, bytes, ctx->stream), "host pull launch");
                }
                AttendParams p = attend_params(g, pages, table, layer, direct ? dq : g->step_q.ptr);
                p.out = dout;
                p.new_k = direct ? dk : g->step_k.ptr;
                p.new_v = direct ? dv : g->step_v.ptr;
                run_attend(g, p);
                cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
                return;
            }
        }
        run_staged_host_step(g, pages, table, layer, k_host, v_host, q_host, out_host, kv_bytes, q_bytes, q_cap);
    });
}

int32_t psi_gqa_step_host(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const uint32_t* req_slots,
                          const uint32_t* token_indices, const uint32_t* cu_tokens, uint32_t num_reqs, const void* k_host,
                          const void* v_host, const void* q_host, void* out_host) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(k_host != nullptr && v_host != nullptr && q_host != nullptr && out_host != nullptr,
                "host buffers must not be null");
        require(req_slots != nullptr && token_indices != nullptr && cu_tokens != nullptr, "metadata inputs must not be null");
        require(num_reqs > 0, "GQA batch metadata requires tokens");
        psi_ctx* ctx = g->ctx;
        require(!ctx->capturing, "psi_gqa_step_host waits for its result and stays outside captured graphs");
        ctx->bind();
        const uint32_t num_tokens = cu_tokens[num_reqs];
        require(num_tokens > 0, "GQA batch metadata requires tokens");
        require(num_tokens <= g->cfg.max_tokens, "GQA batch exceeds the metadata token capacity");
        const uint64_t esz = dtype_bytes(g->cfg.dtype);
        const uint64_t kv_cap = uint64_t(g->cfg.max_tokens) * g->cfg.num_kv_heads * g->cfg.head_dim * esz;
        const uint64_t q_cap = uint64_t(g->cfg.max_tokens) * g->cfg.num_q_heads * g->cfg.head_dim * esz;
        const uint64_t kv_bytes = uint64_t(num_tokens) * g->cfg.num_kv_heads * g->cfg.head_dim * esz;
        const uint64_t q_bytes = uint64_t(num_tokens) * g->cfg.num_q_heads * g->cfg.head_dim * esz;
        g->step_k.ensure(ctx, kv_cap, false);
        g->step_v.ensure(ctx, kv_cap, false);
        g->step_q.ensure(ctx, q_cap, false);
        void *dk = nullptr, *dv = nullptr, *dq = nullptr, *dout = nullptr;
        bool in_place = g->kernel == PSI_KERNEL_MMA && kv_bytes % 16 == 0 && q_bytes % 16 == 0;
        if (in_place) {
            dk = mapped_device_pointer(k_host);
            dv = mapped_device_pointer(v_host);
            dq = mapped_device_pointer(q_host);
            dout = mapped_device_pointer(out_host);
            in_place = dk != nullptr && dv != nullptr && dq != nullptr && dout != nullptr;
        }
        if (!in_place) {  // pageable buffers or the generic kernel: the two calls this one stands for
            prepare_impl(g, req_slots, token_indices, cu_tokens, num_reqs, PSI_CAPACITY_EXACT, 0, nullptr, false, nullptr);
            run_staged_host_step(g, pages, table, layer, k_host, v_host, q_host, out_host, kv_bytes, q_bytes, q_cap);
            return;
        }
        // Small steps pull q/k/v into device staging.  From
        // kDirectHostBytes on, that pull would sit in front of the attention for longer than the attention loses by
        // fetching each item's query rows and the step's K/V rows over the host link itself, so the launch reads the
        // host buffers in place and the transfer hides under the K/V stream (256 verify tokens of 24/4 heads, 5.2 MB:
        // 853 -> 778 us per step; 32 decode tokens, 0.33 MB: no difference).  Long query runs keep the staged path:
        // their kernel takes q and the appended rows through device memory.
        bool direct = q_bytes + 2 * kv_bytes >= kDirectHostBytes && !g->replay_reserved;
        if (direct && g->chunk_supported) {
            for (uint32_t r = 0; r < num_reqs && direct; ++r) {
                const uint32_t tiles = (cu_tokens[r + 1] - cu_tokens[r] + g->geo.tokens_per_tile - 1) / g->geo.tokens_per_tile;
                if (tiles >= kChunkMinTiles) direct = false;
            }
        }
        // The step is planned first; then ONE launch pulls the packed plan from its pinned staging buffer together with
        // q/k/v (or the plan alone when q/k/v are read in place), and the attention launch stores `out` straight into
        // the host buffer.
        uint64_t words = 0;
        prepare_impl(g, req_slots, token_indices, cu_tokens, num_reqs, PSI_CAPACITY_EXACT, 0, nullptr, true, &words);
        const uint64_t padded_words = (words + 3) / 4 * 4;
        void* staging_dev = nullptr;
        const bool plan_mapped = padded_words <= g->staging_words &&
                                 cudaHostGetDevicePointer(&staging_dev, g->staging, 0) == cudaSuccess &&
                                 staging_dev != nullptr && (reinterpret_cast<uintptr_t>(staging_dev) & 15u) == 0;
        if (!plan_mapped) {
            (void)cudaGetLastError();
            cuda_check(cudaMemcpyAsync(g->block.ptr, g->staging, words * sizeof(uint32_t), cudaMemcpyHostToDevice,
                                       ctx->stream), "cudaMemcpyAsync");
        }
        if (plan_mapped || !direct) {
            const void* const src[kPullBuffers] = {direct ? nullptr : dq, direct ? nullptr : dk, direct ? nullptr : dv,
                                                   plan_mapped ? staging_dev : nullptr};
            void* const dst[kPullBuffers] = {g->step_q.ptr, g->step_k.ptr, g->step_v.ptr, g->block.ptr};
            const uint64_t bytes[kPullBuffers] = {direct ? 0 : q_bytes, direct ? 0 : kv_bytes, direct ? 0 : kv_bytes,
                                                  plan_mapped ? padded_words * sizeof(uint32_t) : 0};
            ctx->launches += 1;
            cuda_check(launch_host_pull(src, dst, bytes, ctx->stream), "host pull launch");
        }
        cuda_check(cudaEventRecord(g->upload_done, ctx->stream), "cudaEventRecord");
        AttendParams p = attend_params(g, pages, table, layer, direct ? dq : g->step_q.ptr);
        p.out = dout;
        p.new_k = direct ? dk : g->step_k.ptr;
        p.new_v = direct ? dv : g->step_v.ptr;
        run_attend(g, p);
        cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
    });
}

int32_t psi_page_gather(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t req_slot, uint32_t layer,
                        uint32_t tok_begin, uint32_t tok_end, void* k_out, void* v_out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(k_out != nullptr && v_out != nullptr, "gather outputs must not be null");
        require(tok_begin <= tok_end, "gather token range is reversed");
        g->ctx->bind();
        GatherParams p{};
        p.geo = page_geometry(g, pages, table, layer);
        require(req_slot < g->cfg.layout.num_req_slots, "GQA request page table req_slot out of range");
        require(uint64_t(tok_end) <= uint64_t(p.geo.pages_per_req) * g->tokens_per_page,
                "gather token range does not fit the request page table");
        p.req_slot = req_slot;
        p.tok_begin = tok_begin;
        p.tok_end = tok_end;
        p.k_out = k_out;
        p.v_out = v_out;
        if (tok_end > tok_begin) {
            LaunchScope scope(g->ctx, PSI_KERNEL_CLASS_GATHER);
            cuda_check(launch_page_gather(p, g->ctx->stream), "page gather launch");
        }
    });
}

}  // extern "C"
