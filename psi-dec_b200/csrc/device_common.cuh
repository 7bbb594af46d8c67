// Device helpers shared by the kernels: dtype conversion, page addressing, warp reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.cuh"

namespace psi {

__device__ __forceinline__ float load_as_float(const void* base, uint64_t index, uint32_t dtype) {
    if (dtype == PSI_DTYPE_F32) return static_cast<const float*>(base)[index];
    if (dtype == PSI_DTYPE_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[index]);
    return __half2float(static_cast<const __half*>(base)[index]);
}

__device__ __forceinline__ void store_from_float(void* base, uint64_t index, uint32_t dtype, float value) {
    if (dtype == PSI_DTYPE_F32) {
        static_cast<float*>(base)[index] = value;
    } else if (dtype == PSI_DTYPE_BF16) {
        static_cast<__nv_bfloat16*>(base)[index] = __float2bfloat16_rn(value);
    } else {
        static_cast<__half*>(base)[index] = __float2half_rn(value);
    }
}

// Loads under an L2 cache policy (createpolicy).
__device__ __forceinline__ uint32_t ld_u32_hinted(const uint32_t* src, uint64_t policy) {
    uint32_t value;
    asm volatile("ld.global.L2::cache_hint.u32 %0, [%1], %2;\n" : "=r"(value) : "l"(src), "l"(policy));
    return value;
}

__device__ __forceinline__ uint4 ld_u128_hinted(const void* src, uint64_t policy) {
    uint4 v;
    asm volatile("ld.global.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(src), "l"(policy));
    return v;
}

// First element of the (slot, layer) row of the page table.
__device__ __forceinline__ const uint32_t* table_row(const PageGeometry& g, uint32_t req_slot) {
    return g.page_ids + (static_cast<uint64_t>(req_slot) * g.num_layers + g.layer) * g.pages_per_req;
}

// Bounds-checked page-table reads.  The reference checks page IDs where they enter the table
// (crates/inference-executor-metal/src/state/gqa.rs:97-102) and table indices with debug assertions
// (crates/inference-executor-metal/src/attn/gqa/request_page_table.rs:75,115); its shaders trust the table.  Here
// the checked build of the library (libpsi_cuda_checked.so, compiled with -DPSI_CUDA_CHECKED=1) makes every kernel
// compare the index with the row length and the ID with the arena's page count before forming an address, and on a
// miss record PSI_ERR_PAGE_ID in the status word instead of touching memory outside the arena.  It stands where a
// memory checker would: for bringing up a new caller, and in the tests.  The production build leaves the device
// checks out, as the reference's shaders do: in the decode kernel's inner loop they measured 1.2 % (head_dim 256) to
// 12.7 % (head_dim 64) of the step.  The host-side checks (psi_table_set_page_bound, psi_table_write_all_layers,
// the context-fits-the-table check of psi_gqa_prepare) are part of both builds.
#ifndef PSI_CUDA_CHECKED
#define PSI_CUDA_CHECKED 0
#endif

__device__ __forceinline__ void record_page_fault(const PageGeometry& g) {
    if (g.fault != nullptr) *reinterpret_cast<volatile uint32_t*>(g.fault) = static_cast<uint32_t>(PSI_ERR_PAGE_ID);
}

// Page ID at `index` of a (slot, layer) table row; false (and id = 0) when the index or the ID is out of bounds: the
// caller skips its write.
__device__ __forceinline__ bool checked_page_id(const PageGeometry& g, const uint32_t* row_ids, uint32_t index,
                                                uint32_t& id) {
#if PSI_CUDA_CHECKED
    id = 0;
    if (index >= g.pages_per_req) {
        record_page_fault(g);
        return false;
    }
    const uint32_t raw = row_ids[index];
    if (g.num_pages != 0 && raw >= g.num_pages) {
        record_page_fault(g);
        return false;
    }
    id = raw;
    return true;
#else
    id = row_ids[index];
    return true;
#endif
}

// The form for a kernel's inner loop: the bounds are held as two 32-bit values, a miss turns into page 0 with two
// compares and a select, and the launch is flagged once, at the end, from the `bad` word the thread has gathered.
struct PageBounds {
    uint32_t ids;      // page IDs must be below this (0xFFFFFFFF when the arena's size is not known)
    uint32_t indices;  // table indices must be below this
    __device__ __forceinline__ explicit PageBounds(const PageGeometry& g)
#if PSI_CUDA_CHECKED
        : ids(g.num_pages == 0 || g.num_pages > 0xFFFFFFFFull ? 0xFFFFFFFFu : static_cast<uint32_t>(g.num_pages)),
          indices(g.pages_per_req) {}
#else
        : ids(0xFFFFFFFFu), indices(0xFFFFFFFFu) {}
#endif
    __device__ __forceinline__ uint32_t read(const uint32_t* row_ids, uint32_t index, uint32_t& bad) const {
#if PSI_CUDA_CHECKED
        const bool index_ok = index < indices;
        const uint32_t raw = row_ids[index_ok ? index : 0u];
        const bool ok = index_ok && raw < ids;
        bad |= ok ? 0u : 1u;
        return ok ? raw : 0u;
#else
        (void)bad;
        return row_ids[index];
#endif
    }
    // The same read under an L2 cache policy.
    __device__ __forceinline__ uint32_t read_hinted(const uint32_t* row_ids, uint32_t index, uint32_t& bad,
                                                    uint64_t policy) const {
#if PSI_CUDA_CHECKED
        const bool index_ok = index < indices;
        const uint32_t raw = ld_u32_hinted(row_ids + (index_ok ? index : 0u), policy);
        const bool ok = index_ok && raw < ids;
        bad |= ok ? 0u : 1u;
        return ok ? raw : 0u;
#else
        (void)bad;
        return ld_u32_hinted(row_ids + index, policy);
#endif
    }
};

// The same for reads: an out-of-bounds entry reads page 0 (valid memory) and the launch is flagged.
__device__ __forceinline__ uint32_t page_id_or_zero(const PageGeometry& g, const uint32_t* row_ids, uint32_t index) {
    uint32_t id;
    (void)checked_page_id(g, row_ids, index, id);
    return id;
}

// Element offset of K row (kv_head, token) inside the arena; V is `v_region` further.  Within one (slot, layer) row
// the two-level (block, page_id_index) address of the reference collapses to token / tokens_per_page.
__device__ __forceinline__ uint64_t kv_row_offset(const PageGeometry& g, uint32_t page_id, uint32_t kv_head,
                                                  uint32_t page_token) {
    return static_cast<uint64_t>(page_id) * g.page_elems +
           (static_cast<uint64_t>(kv_head) * g.tokens_per_page + page_token) * g.head_dim;
}

__device__ __forceinline__ uint64_t v_region_offset(const PageGeometry& g) {
    return static_cast<uint64_t>(g.num_kv_heads) * g.tokens_per_page * g.head_dim;
}

// sigmoid as the reference's gate computes it: 1 / (1 + exp(-|x|)), mirrored for negative x
// (crates/inference-backend-metal/src/components/metal/gqa_activation_gate.metal:13-16).
__device__ __forceinline__ float gate_sigmoid(float x) {
    const float y = 1.0f / (1.0f + __expf(-fabsf(x)));
    return x < 0.0f ? 1.0f - y : y;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, offset);
    return v;
}

}  // namespace psi

namespace psi {

// A work item as the kernels see it; `rows` = num_tokens * num_heads (<= 16).
struct ItemView : DeviceItem {
    uint32_t rows;
};

__device__ __forceinline__ ItemView view_item(const DeviceItem* item) {
    ItemView v;
    const uint4* src = reinterpret_cast<const uint4*>(item);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<DeviceItem*>(&v));
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = src[i];
    v.rows = v.num_tokens * v.num_heads;
    return v;
}

__device__ __forceinline__ ItemView view_item_hinted(const DeviceItem* item, uint64_t policy) {
    ItemView v;
    uint4* dst = reinterpret_cast<uint4*>(static_cast<DeviceItem*>(&v));
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = ld_u128_hinted(reinterpret_cast<const uint4*>(item) + i, policy);
    v.rows = v.num_tokens * v.num_heads;
    return v;
}

__device__ __forceinline__ ItemView view_item(const AttendParams& p, uint32_t index) {
    ItemView v;
    const uint4* src = reinterpret_cast<const uint4*>(p.items + index);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<DeviceItem*>(&v));
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = src[i];
    v.rows = v.num_tokens * v.num_heads;
    return v;
}

// Flat (token, head) row of q / out / ext_* that item row r stands for.
__device__ __forceinline__ uint64_t item_row_index(const AttendParams& p, const ItemView& v, uint32_t r) {
    return static_cast<uint64_t>(v.flat_begin + r / v.num_heads) * p.num_q_heads + v.head0 + r % v.num_heads;
}

// Keys row r may see: [0, first_pos + token(r)] clipped to the item's range end.
__device__ __forceinline__ uint32_t item_row_limit(const ItemView& v, uint32_t r) {
    return min(v.kv_end, v.first_pos + r / v.num_heads + 1);
}

constexpr float kLn2 = 0.6931471805599453f;

}  // namespace psi

namespace psi {

// sigmoid(gate) of output element `index`, or 1 when the launch has no gate.
__device__ __forceinline__ float gate_factor(const AttendParams& p, uint64_t index) {
    return p.gates == nullptr ? 1.0f : gate_sigmoid(load_as_float(p.gates, index, p.dtype));
}

}  // namespace psi
