// Attention over the paged cache for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc once they are running: a serving process that handed every free
// byte of HBM to its KV arena at start-up has nothing left to allocate from, a runtime that routes all device memory
// through its own pool must not see allocations it does not own, and a latency-critical decode loop cannot afford
// the device-wide synchronisation an allocation implies.  psi_gqa_attend_static is the split-KV attention of
// psi_gqa_attend for those callers: the plan, the arrival counters and the partial outputs live in one fixed
// file-scope device array that every GPU loading the library holds until exit, and the call makes no cudaMalloc,
// cudaFree or other allocating call.  The kernels are the library's ordinary attention kernels; only where their
// scratch comes from differs.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "host_logic.hpp"
#include "kernels.cuh"
#include "psi_cuda.h"

using namespace psi;

namespace {

// Capacity of the fixed scratch.  A step that needs more is rejected before anything is enqueued.
constexpr uint32_t kStaticMaxCtas = PSI_STATIC_MAX_CTAS;
constexpr uint32_t kStaticMaxItems = PSI_STATIC_MAX_ITEMS;
constexpr uint32_t kStaticMaxSlots = 2 * kStaticMaxCtas;  // a CTA share cuts at most two units
constexpr uint32_t kStaticMaxHeadDim = 256;

constexpr uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// Byte layout of the scratch: plan block | arrival counters | partial max/sum | partial outputs.
constexpr uint64_t kOffScalars = 0;
constexpr uint64_t kOffCta = align_up(kOffScalars + kScalarCount * 4, 256);
constexpr uint64_t kOffReduces = align_up(kOffCta + (kStaticMaxCtas + 1) * 4, 256);
constexpr uint64_t kOffItems = align_up(kOffReduces + kStaticMaxSlots * sizeof(ReduceUnit), 256);
constexpr uint64_t kPlanBytes = align_up(kOffItems + kStaticMaxItems * sizeof(DeviceItem), 256);
constexpr uint64_t kOffCounters = kPlanBytes;
constexpr uint64_t kOffPartialMl = align_up(kOffCounters + kStaticMaxSlots * 4, 256);
constexpr uint64_t kOffPartialO = align_up(kOffPartialMl + 2ull * kStaticMaxSlots * kMaxRows * 4, 256);
constexpr uint64_t kScratchBytes = kOffPartialO + 1ull * kStaticMaxSlots * kMaxRows * kStaticMaxHeadDim * 4;
static_assert(kScratchBytes == PSI_STATIC_SCRATCH_BYTES, "the header states the scratch size");

// The scratch itself.  In host code this name is only a handle for the runtime, not a device address: the address
// the kernels need comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned char* g_scratch_address[kMaxDevices] = {};

// Device address of the scratch on the current device (which must be `device`), resolved on first use.
cudaError_t scratch_address(int device, unsigned char** out) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* address = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&address, g_static_scratch);
        if (err != cudaSuccess) return err;
        g_scratch_address[device] = static_cast<unsigned char*>(address);
    }
    *out = g_scratch_address[device];
    return cudaSuccess;
}

int32_t fail(int32_t status, const std::string& message, char* error, size_t error_len) {
    if (error != nullptr && error_len > 0) std::snprintf(error, error_len, "%s", message.c_str());
    return status;
}

// Makes `device` current for the call and puts the caller's device back on every way out.
struct DeviceGuard {
    int previous = -1;
    bool switched = false;
    cudaError_t enter(int device) {
        cudaError_t err = cudaGetDevice(&previous);
        if (err != cudaSuccess) return err;
        if (previous == device) return cudaSuccess;
        err = cudaSetDevice(device);
        switched = err == cudaSuccess;
        return err;
    }
    ~DeviceGuard() {
        if (switched) (void)cudaSetDevice(previous);
    }
};

}  // namespace

extern "C" int32_t psi_gqa_attend_static(int32_t device, void* cuda_stream, const psi_gqa_config* config,
                                         const void* pages, const uint32_t* page_table, const uint32_t* req_slots,
                                         const uint32_t* token_indices, const uint32_t* cu_tokens, uint32_t num_reqs,
                                         uint32_t layer, const void* q, void* out, char* error, size_t error_len) {
    try {
        require(config != nullptr && pages != nullptr && page_table != nullptr && q != nullptr && out != nullptr,
                "config, pages, page_table, q and out must not be null");
        require(req_slots != nullptr && token_indices != nullptr && cu_tokens != nullptr && num_reqs > 0,
                "the batch description must not be empty");
        const psi_gqa_config& c = *config;
        require(c.num_q_heads > 0 && c.num_kv_heads > 0 && c.num_q_heads % c.num_kv_heads == 0,
                "GQA q heads must be a positive multiple of kv heads");
        require(c.head_dim > 0 && c.head_dim <= kStaticMaxHeadDim,
                "head_dim exceeds the static scratch (PSI_STATIC_MAX_HEAD_DIM)");
        require(c.dtype <= PSI_DTYPE_F16 && c.scale > 0.0f && std::isfinite(c.scale), "unsupported dtype or scale");
        require(c.kernel_mode <= PSI_KERNEL_MMA_SYNC, "unknown kernel mode (the TMA feed needs a psi_pages arena)");
        const uint64_t per_token = uint64_t(c.num_kv_heads) * c.head_dim * 2u * dtype_bytes(c.dtype);
        require(c.page_bytes > 0 && c.page_bytes % per_token == 0,
                "GQA page_bytes must be divisible by the K/V bytes per token");
        require(layer < c.layout.num_gqa_layers, "GQA page-table index exceeds layer count");
        require(device >= 0 && device < kMaxDevices, "device index out of range");
        const uint32_t tokens_per_page = c.page_bytes / static_cast<uint32_t>(per_token);
        const uint64_t table_tokens = uint64_t(c.layout.num_blocks) * c.layout.num_page_ids_per_block * tokens_per_page;
        require(cu_tokens[0] == 0, "GQA batch cu_tokens must start at zero");
        for (uint32_t r = 0; r < num_reqs; ++r) {
            require(cu_tokens[r] <= cu_tokens[r + 1], "GQA batch cu_tokens must be nondecreasing");
            require(req_slots[r] < c.layout.num_req_slots, "GQA request page table req_slot out of range");
            require(uint64_t(token_indices[r]) + (cu_tokens[r + 1] - cu_tokens[r]) <= table_tokens,
                    "GQA request context does not fit the request page table");
        }
        require(cu_tokens[num_reqs] > 0, "GQA batch metadata requires tokens");

        DeviceGuard guard;
        if (guard.enter(device) != cudaSuccess) return fail(PSI_ERR_CUDA, "cudaSetDevice failed", error, error_len);
        cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
        // The plan is uploaded from a buffer that lives only for this call, so the call cannot be part of a captured
        // graph: a replay would read freed host memory.
        cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(PSI_ERR_CUDA, "cudaStreamIsCapturing failed", error, error_len);
        }
        if (capture != cudaStreamCaptureStatusNone) {
            return fail(PSI_ERR_INVALID_ARGUMENT, "psi_gqa_attend_static cannot be recorded into a stream capture", error,
                        error_len);
        }
        unsigned char* scratch = nullptr;
        cudaError_t err = scratch_address(device, &scratch);
        if (err != cudaSuccess) {
            return fail(PSI_ERR_CUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(err), error, error_len);
        }
        int sm_count = 0;
        err = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
        if (err != cudaSuccess) return fail(PSI_ERR_CUDA, cudaGetErrorString(err), error, error_len);

        // Plan on the host as psi_gqa_prepare does in PSI_PLAN_BALANCED (same kernel choice, same balance costs), with
        // the CTA count capped by the scratch.  Long query runs stay on this kernel: the chunk kernels are not used.
        const PlanGeometry geo = plan_geometry(c.num_q_heads, c.num_kv_heads);
        const bool mma = c.kernel_mode != PSI_KERNEL_GENERIC && attend_mma_supported(c.dtype, c.head_dim, tokens_per_page);
        require(mma || c.kernel_mode < PSI_KERNEL_MMA, "the mma kernel does not support this profile");
        const uint32_t per_sm = mma ? attend_mma_ctas_per_sm(c.head_dim) : attend_generic_ctas_per_sm(c.head_dim, c.dtype);
        uint32_t max_ctas = std::min<uint32_t>(kStaticMaxCtas, static_cast<uint32_t>(sm_count) * per_sm);
        if (c.max_ctas > 0) max_ctas = std::min(max_ctas, c.max_ctas);
        const WorkPlan plan = build_balanced_plan(geo, req_slots, token_indices, cu_tokens, num_reqs, max_ctas,
                                                  mma ? 16u : 4u, mma ? 32u : 0u);
        if (plan.items.size() > kStaticMaxItems) {
            return fail(PSI_ERR_INVALID_ARGUMENT,
                        "the step needs " + std::to_string(plan.items.size()) + " work items; the static scratch holds " +
                            std::to_string(kStaticMaxItems) + " (PSI_STATIC_MAX_ITEMS)",
                        error, error_len);
        }
        if (plan.num_partial_slots > kStaticMaxSlots || plan.num_ctas() > kStaticMaxCtas) {
            return fail(PSI_ERR_INVALID_ARGUMENT, "the step's plan exceeds the static scratch", error, error_len);
        }

        std::vector<unsigned char> block(kPlanBytes, 0);
        auto* scalars = reinterpret_cast<uint32_t*>(block.data() + kOffScalars);
        scalars[kScalarNumActiveTokens] = cu_tokens[num_reqs];
        scalars[kScalarNumCtas] = plan.num_ctas();
        scalars[kScalarNumReduces] = static_cast<uint32_t>(plan.reduces.size());
        std::memcpy(block.data() + kOffCta, plan.cta_item_begin.data(), plan.cta_item_begin.size() * 4);
        if (!plan.reduces.empty()) {
            std::memcpy(block.data() + kOffReduces, plan.reduces.data(), plan.reduces.size() * sizeof(ReduceUnit));
        }
        const std::vector<DeviceItem> items = flatten_plan(plan, geo);
        if (!items.empty()) std::memcpy(block.data() + kOffItems, items.data(), items.size() * sizeof(DeviceItem));

        const uint64_t used = kOffItems + items.size() * sizeof(DeviceItem);
        // Pageable source: the runtime stages the bytes before the call returns.  Everything below is stream-ordered
        // after it, and overwrites what the previous call left in the scratch.
        err = cudaMemcpyAsync(scratch, block.data(), used, cudaMemcpyHostToDevice, stream);
        if (err == cudaSuccess) {
            // The arrival counters are the one part of the scratch that must start at zero.
            err = cudaMemsetAsync(scratch + kOffCounters, 0, kStaticMaxSlots * 4, stream);
        }
        if (err != cudaSuccess) return fail(PSI_ERR_CUDA, cudaGetErrorString(err), error, error_len);

        AttendParams p{};
        p.geo.pages = pages;
        p.geo.page_ids = page_table;
        p.geo.elem_bytes = dtype_bytes(c.dtype);
        p.geo.page_elems = c.page_bytes / p.geo.elem_bytes;
        p.geo.layer = layer;
        p.geo.num_layers = c.layout.num_gqa_layers;
        p.geo.pages_per_req = c.layout.num_blocks * c.layout.num_page_ids_per_block;
        p.geo.tokens_per_page = tokens_per_page;
        p.geo.num_kv_heads = c.num_kv_heads;
        p.geo.head_dim = c.head_dim;
        p.q = q;
        p.out = out;
        p.items = reinterpret_cast<const DeviceItem*>(scratch + kOffItems);
        p.cta_item_begin = reinterpret_cast<const uint32_t*>(scratch + kOffCta);
        p.reduces = reinterpret_cast<const ReduceUnit*>(scratch + kOffReduces);
        p.partial_o = reinterpret_cast<float*>(scratch + kOffPartialO);
        p.partial_m = reinterpret_cast<float*>(scratch + kOffPartialMl);
        p.partial_l = p.partial_m + kStaticMaxSlots * kMaxRows;
        p.unit_counters = reinterpret_cast<uint32_t*>(scratch + kOffCounters);
        p.scalars = reinterpret_cast<const uint32_t*>(scratch + kOffScalars);
        p.num_q_heads = c.num_q_heads;
        p.tokens_per_tile = geo.tokens_per_tile;
        p.dtype = c.dtype;
        p.scale_log2 = c.scale * 1.4426950408889634f;
        if (mma) {
            err = launch_attend_mma(p, plan.num_ctas(), stream);
        } else {
            err = launch_attend_generic(p, plan.num_ctas(), stream);
            if (err == cudaSuccess) err = launch_attend_reduce(p, static_cast<uint32_t>(plan.reduces.size()), stream);
        }
        if (err != cudaSuccess) {
            return fail(PSI_ERR_CUDA, std::string("attend launch: ") + cudaGetErrorString(err), error, error_len);
        }
        return PSI_OK;
    } catch (const ContractError& e) {
        return fail(PSI_ERR_INVALID_ARGUMENT, e.what(), error, error_len);
    } catch (const std::bad_alloc&) {
        return fail(PSI_ERR_RESOURCE_EXHAUSTED, "out of host memory", error, error_len);
    } catch (const std::exception& e) {
        return fail(PSI_ERR_INTERNAL, e.what(), error, error_len);
    }
}
