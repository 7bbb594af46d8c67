// KV append (per-token slot scatter into fixed-size pages) and its inverse, the block-table page gather.
//
// Both kernels move whole K/V head rows.  When a row is a multiple of 16 bytes and the caller's buffers are 16-byte
// aligned, one thread moves one 16-byte chunk (a warp covers 512 contiguous bytes on both sides); otherwise one thread
// moves one element.  The address algebra follows the reference shader
// crates/inference-backend-metal/src/components/metal/gqa_kv_page_write.metal:20-52.
#include <algorithm>

#include "device_common.cuh"

namespace psi {

namespace {

template <typename Unit>
__global__ void kv_append_kernel(AppendParams p, uint32_t units_per_row) {
    const uint32_t num_active = min(p.scalars[kScalarNumActiveTokens], p.num_total_tokens);
    const uint64_t rows = static_cast<uint64_t>(num_active) * p.geo.num_kv_heads;
    const uint64_t total = rows * units_per_row;
    const uint64_t gid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= total) return;
    const uint32_t unit = static_cast<uint32_t>(gid % units_per_row);
    const uint64_t row = gid / units_per_row;
    const uint32_t head = static_cast<uint32_t>(row % p.geo.num_kv_heads);
    const uint32_t write = static_cast<uint32_t>(row / p.geo.num_kv_heads);

    const uint32_t token = p.flat_token_indices[write];
    const uint32_t page_index = token / p.geo.tokens_per_page;
    uint32_t page_id;
    if (!checked_page_id(p.geo, table_row(p.geo, p.req_slots[write]), page_index, page_id)) return;  // write skipped
    const uint64_t dst_elem = kv_row_offset(p.geo, page_id, head, token % p.geo.tokens_per_page);
    const uint64_t src_elem = (static_cast<uint64_t>(write) * p.geo.num_kv_heads + head) * p.geo.head_dim;
    const uint64_t scale = p.geo.elem_bytes;  // element offsets -> byte offsets -> Unit offsets
    const uint64_t dst_k = dst_elem * scale / sizeof(Unit) + unit;
    const uint64_t dst_v = (dst_elem + v_region_offset(p.geo)) * scale / sizeof(Unit) + unit;
    const uint64_t src = src_elem * scale / sizeof(Unit) + unit;
    Unit* pages = static_cast<Unit*>(const_cast<void*>(p.geo.pages));
    pages[dst_k] = static_cast<const Unit*>(p.flat_k)[src];
    pages[dst_v] = static_cast<const Unit*>(p.flat_v)[src];
}

template <typename Unit>
__global__ void page_gather_kernel(GatherParams p, uint32_t units_per_row) {
    const uint64_t rows = static_cast<uint64_t>(p.tok_end - p.tok_begin) * p.geo.num_kv_heads;
    const uint64_t total = rows * units_per_row;
    const uint64_t gid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= total) return;
    const uint32_t unit = static_cast<uint32_t>(gid % units_per_row);
    const uint64_t row = gid / units_per_row;
    const uint32_t head = static_cast<uint32_t>(row % p.geo.num_kv_heads);
    const uint32_t local = static_cast<uint32_t>(row / p.geo.num_kv_heads);
    const uint32_t token = p.tok_begin + local;
    const uint32_t page_index = token / p.geo.tokens_per_page;
    uint32_t page_id;
    if (!checked_page_id(p.geo, table_row(p.geo, p.req_slot), page_index, page_id)) return;  // row left untouched
    const uint64_t src_elem = kv_row_offset(p.geo, page_id, head, token % p.geo.tokens_per_page);
    const uint64_t dst_elem = (static_cast<uint64_t>(local) * p.geo.num_kv_heads + head) * p.geo.head_dim;
    const uint64_t scale = p.geo.elem_bytes;
    const Unit* pages = static_cast<const Unit*>(p.geo.pages);
    static_cast<Unit*>(p.k_out)[dst_elem * scale / sizeof(Unit) + unit] = pages[src_elem * scale / sizeof(Unit) + unit];
    static_cast<Unit*>(p.v_out)[dst_elem * scale / sizeof(Unit) + unit] =
        pages[(src_elem + v_region_offset(p.geo)) * scale / sizeof(Unit) + unit];
}

// Pulls up to four host-mapped buffers into device memory in one launch (16-byte chunks, grid-stride).
struct PullParams {
    const uint4* src[kPullBuffers];
    uint4* dst[kPullBuffers];
    uint64_t chunks[kPullBuffers];
};

__global__ void host_pull_kernel(PullParams p) {
    // A thread's loads from all buffers go out together: a load over the host link takes a microsecond or two, and
    // one buffer after the other would put those round trips in a row.
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    uint64_t most = 0;
#pragma unroll
    for (int b = 0; b < kPullBuffers; ++b) most = max(most, p.chunks[b]);
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < most; i += stride) {
        uint4 value[kPullBuffers];
#pragma unroll
        for (int b = 0; b < kPullBuffers; ++b)
            if (i < p.chunks[b]) value[b] = p.src[b][i];
#pragma unroll
        for (int b = 0; b < kPullBuffers; ++b)
            if (i < p.chunks[b]) p.dst[b][i] = value[b];
    }
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

constexpr int kCopyThreads = 256;

}  // namespace

cudaError_t launch_kv_append(const AppendParams& p, cudaStream_t stream) {
    const uint32_t row_bytes = p.geo.head_dim * p.geo.elem_bytes;
    const uint64_t rows = static_cast<uint64_t>(p.num_total_tokens) * p.geo.num_kv_heads;
    if (rows == 0) return cudaSuccess;
    const bool wide = row_bytes % 16 == 0 && aligned16(p.flat_k) && aligned16(p.flat_v) && aligned16(p.geo.pages);
    const uint32_t units = wide ? row_bytes / 16 : p.geo.head_dim;
    const uint64_t blocks = (rows * units + kCopyThreads - 1) / kCopyThreads;
    if (wide) {
        kv_append_kernel<uint4><<<static_cast<unsigned>(blocks), kCopyThreads, 0, stream>>>(p, units);
    } else if (p.geo.elem_bytes == 4) {
        kv_append_kernel<uint32_t><<<static_cast<unsigned>(blocks), kCopyThreads, 0, stream>>>(p, units);
    } else {
        kv_append_kernel<uint16_t><<<static_cast<unsigned>(blocks), kCopyThreads, 0, stream>>>(p, units);
    }
    return cudaGetLastError();
}

cudaError_t launch_page_gather(const GatherParams& p, cudaStream_t stream) {
    const uint32_t row_bytes = p.geo.head_dim * p.geo.elem_bytes;
    const uint64_t rows = static_cast<uint64_t>(p.tok_end - p.tok_begin) * p.geo.num_kv_heads;
    if (rows == 0) return cudaSuccess;
    const bool wide = row_bytes % 16 == 0 && aligned16(p.k_out) && aligned16(p.v_out) && aligned16(p.geo.pages);
    const uint32_t units = wide ? row_bytes / 16 : p.geo.head_dim;
    const uint64_t blocks = (rows * units + kCopyThreads - 1) / kCopyThreads;
    if (wide) {
        page_gather_kernel<uint4><<<static_cast<unsigned>(blocks), kCopyThreads, 0, stream>>>(p, units);
    } else if (p.geo.elem_bytes == 4) {
        page_gather_kernel<uint32_t><<<static_cast<unsigned>(blocks), kCopyThreads, 0, stream>>>(p, units);
    } else {
        page_gather_kernel<uint16_t><<<static_cast<unsigned>(blocks), kCopyThreads, 0, stream>>>(p, units);
    }
    return cudaGetLastError();
}

cudaError_t launch_host_pull(const void* const src[kPullBuffers], void* const dst[kPullBuffers],
                             const uint64_t bytes[kPullBuffers], cudaStream_t stream) {
    PullParams p{};
    uint64_t total = 0;
    for (int b = 0; b < kPullBuffers; ++b) {
        p.src[b] = static_cast<const uint4*>(src[b]);
        p.dst[b] = static_cast<uint4*>(dst[b]);
        p.chunks[b] = bytes[b] / 16;
        total += p.chunks[b];
    }
    if (total == 0) return cudaSuccess;
    const uint64_t blocks = std::min<uint64_t>((total + kCopyThreads - 1) / kCopyThreads, 592);
    host_pull_kernel<<<static_cast<unsigned>(blocks), kCopyThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace psi
