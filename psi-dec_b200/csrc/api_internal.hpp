// Internals shared by the files that implement the C ABI (api_*.cu): the opaque objects behind the handles, the
// exception-to-status guard, and the launch helpers every attention entry point goes through.
#pragma once

#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <new>
#include <stdexcept>
#include <string>
#include <vector>

#include "host_logic.hpp"
#include "kernels.cuh"
#include "psi_cuda.h"
#include "snapshot.hpp"

namespace psi {

struct CudaError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

extern thread_local std::string g_thread_error;

inline void cuda_check(cudaError_t err, const char* what) {
    if (err != cudaSuccess) {
        throw CudaError(std::string(what) + ": " + cudaGetErrorName(err) + " (" + cudaGetErrorString(err) + ")");
    }
}

constexpr uint32_t kWordAlign = 8;  // sections of the device metadata block start on 32-byte boundaries
inline uint64_t pad_words(uint64_t n) { return (n + kWordAlign - 1) / kWordAlign * kWordAlign; }

constexpr uint32_t kKernelClasses = 7;

}  // namespace psi

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
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> timed[psi::kKernelClasses];
    void bind() const { psi::cuda_check(cudaSetDevice(device), "cudaSetDevice"); }
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

namespace psi {

// Counts one launch, names it for a timeline profiler (an NVTX range per launch: a no-op costing a few nanoseconds
// when no tool is attached), and, while timing is on, brackets it with events on the context's stream.
struct LaunchScope {
    psi_ctx* ctx;
    cudaEvent_t end = nullptr;
    LaunchScope(psi_ctx* c, uint32_t kernel_class) : ctx(c) {
        ctx->launches += 1;
        if (ctx->timing && !ctx->capturing) {
            cudaEvent_t begin = nullptr;
            cuda_check(cudaEventCreate(&begin), "cudaEventCreate");
            cuda_check(cudaEventCreate(&end), "cudaEventCreate");
            ctx->timed[kernel_class].emplace_back(begin, end);
            cuda_check(cudaEventRecord(begin, ctx->stream), "cudaEventRecord");
        }
        // last, so that nothing that can throw stands between the push and the destructor's pop
        static const char* const kNames[kKernelClasses] = {"psi kv_append",     "psi attend_map", "psi attend_reduce",
                                                           "psi combine",       "psi page_gather", "psi attend_chunk",
                                                           "psi norm_rope_append"};
        nvtxRangePushA(kernel_class < kKernelClasses ? kNames[kernel_class] : "psi launch");
    }
    ~LaunchScope() {
        if (end != nullptr) (void)cudaEventRecord(end, ctx->stream);
        nvtxRangePop();
    }
};

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

}  // namespace psi

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
    uint64_t page_bound = 0;  // 0: none declared; else every stored page ID must be below it
    void check_ids(const uint32_t* ids, uint64_t n) const {
        if (page_bound == 0) return;
        for (uint64_t i = 0; i < n; ++i) {
            psi::require(ids[i] < page_bound, "runtime supplied a GQA page ID outside the cache-page buffer");
        }
    }
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
    psi::SnapshotWriter impl;
    psi_snapshot_writer(const std::string& d, const std::vector<uint32_t>& f, const psi::SnapshotPlan& p) : impl(d, f, p) {}
};

struct psi_snapshot_reader {
    psi::SnapshotReader impl;
    psi_snapshot_reader(const std::string& d, const std::vector<uint32_t>& f, const psi::SnapshotPlan& p) : impl(d, f, p) {}
};

struct psi_id_allocator {
    psi::IdAllocator impl;
    explicit psi_id_allocator(uint64_t capacity) : impl(capacity) {}
};

struct psi_gqa {
    psi_ctx* ctx = nullptr;
    psi_gqa_config cfg{};
    uint32_t tokens_per_page = 0;
    uint32_t kernel = PSI_KERNEL_GENERIC;  // resolved kernel
    uint32_t grid_cap = 1;
    uint32_t item_start_cost = 0;  // KV tiles one item switch is worth when shares are balanced
    psi::PlanGeometry geo{};
    std::unique_ptr<psi::SplitKvSelector> selector;  // null when the profile is outside the reference selector's domain
    std::unique_ptr<psi::ReferenceMetadata> md;
    std::vector<uint32_t> boundaries;
    psi_replay_shape shape{};
    psi_split_kv_variant variant{};
    psi::WorkPlan plan;
    psi::ChunkPlan chunk;            // long query runs (balanced plan + mma kernel only)
    bool chunk_supported = false;
    bool prepared = false;

    psi::DeviceBuffer block;       // device metadata block
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

    psi::DeviceBuffer partial_o, partial_ml;  // [slots][16][D] and [2][slots][16]
    psi::DeviceBuffer unit_counters;          // [slots] u32, zero between launches
    uint64_t partial_slots_cap = 0;
    psi::DeviceBuffer step_k, step_v, step_q, step_out;  // psi_gqa_decode_step_host staging
    psi::DeviceBuffer combine_ptrs;
    psi::DeviceBuffer status_word;  // u32 written by bounded device-side waits
    psi::DeviceBuffer sync_words;   // SyncWord counters of launches that wait or exchange; zero between launches
    psi::DeviceBuffer xchg_local;   // KV-range exchange without the fused launch: this rank's partial before the push
    // psi_gqa_step_host on large pinned buffers: copy streams and per-group events of the pipelined step
    cudaStream_t pipe_h2d = nullptr, pipe_d2h = nullptr;
    std::vector<cudaEvent_t> pipe_events;
    bool chunk_umma = false;   // long query runs on the tcgen05 kernel (else the mma.sync chunk kernel)
    uint32_t chunk_launches[2] = {0, 0};  // tcgen05, mma.sync
    psi::DeviceBuffer norm_rope;    // q weight bf16[D] | k weight bf16[D] | inverse frequencies f32[rope_dim/2]
    psi_norm_rope_config norm_rope_cfg{};
    float norm_rope_attention_factor = 1.0f;
    bool has_norm_rope = false;
};

namespace psi {

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


int32_t copy_message(const std::string& message, char* buf, size_t n);
void validate_layout(const psi_page_table_layout& l);
PageGeometry page_geometry(const psi_gqa* g, const psi_pages* pages, const psi_table* table, uint32_t layer);
const uint32_t* block_words(const psi_gqa* g, uint64_t offset);

// Requests whose query run spans at least this many query tiles go to the chunk kernels.
constexpr uint32_t kChunkMinTiles = 5;
// psi_gqa_step_host: from this many bytes of q + k + v the attention launch reads pinned host buffers in place.
constexpr uint64_t kDirectHostBytes = 1ull << 20;
// psi_gqa_step_host: from this many bytes of q + k + v in pinned buffers a step with long query runs is cut into groups
// of requests whose transfers and launches overlap; a group carries about kPipelineGroupBytes of them.
constexpr uint64_t kPipelineHostBytes = 64ull << 20;
constexpr uint64_t kPipelineGroupBytes = 48ull << 20;
constexpr uint32_t kPipelineMaxGroups = 8;

AttendParams attend_params(psi_gqa* g, const psi_pages* pages, const psi_table* table, uint32_t layer, const void* q);
void run_attend(psi_gqa* g, const AttendParams& params);
void run_append(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k, const void* v);
// Device-side address of a pinned, device-mapped host buffer (16-byte aligned), or nullptr for any other memory.
void* mapped_device_pointer(const void* host);
// A prepared step through pageable host buffers: inputs staged by copy-engine transfers, output copied back, waited for.
void run_staged_host_step(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k_host,
                          const void* v_host, const void* q_host, void* out_host, uint64_t kv_bytes, uint64_t q_bytes,
                          uint64_t q_cap);
// GQAMetadataBuffers::update plus this library's plan.  With `defer_upload` the packed block stays in the pinned
// staging buffer and its size comes back in *deferred_words: the caller brings it to the device itself.
// `plan_only` (balanced plan mode): the reference-format split plan is not computed, only the per-token arrays and this
// library's plan; the replay shape then names the token count alone.
void prepare_impl(psi_gqa* g, const uint32_t* req_slots, const uint32_t* token_indices, const uint32_t* cu_tokens,
                  uint32_t num_reqs, uint32_t capacity_mode, uint32_t caller_num_total_tokens,
                  psi_replay_shape* out_shape, bool defer_upload, uint64_t* deferred_words, bool plan_only = false);

}  // namespace psi
