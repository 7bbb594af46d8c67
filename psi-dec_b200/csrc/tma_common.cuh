// TMA and mbarrier building blocks shared by the kernels that bring K/V tiles from the page arena with
// cp.async.bulk.tensor: the tensor map of the arena (host), bounded mbarrier waits, the box copy, and the
// shared-memory layout a box lands in.  No multicast anywhere: a map covers this GPU's own memory only.
#pragma once

#include <cuda.h>

#include "device_common.cuh"

namespace psi {

constexpr uint32_t kMaxPolls = 200000;  // bound of every mbarrier wait (a try_wait each)

// The page arena as a TMA tensor [page][8-row group][element block][row in group][64 elements]: a page holds
// 2 * Hkv * tokens_per_page K and V rows of head_dim elements, a box is `box_rows / 8` consecutive groups with all their
// element blocks, written with the 128-byte swizzle.  False when the arena cannot be described to the TMA unit
// (alignment, size, driver entry point missing).
bool make_kv_map(const AttendParams& p, uint32_t box_rows, CUtensorMap* map);

__device__ __forceinline__ uint32_t smem_u32(const void* ptr) { return static_cast<uint32_t>(__cvta_generic_to_shared(ptr)); }

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Bounded wait on one phase of an mbarrier; false when the bound ran out.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Non-blocking test of one phase.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kMaxPolls; ++i) {
        if (mbar_try(bar, parity)) return true;
    }
    return false;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// One TMA box of the page arena into shared memory; completion is counted in bytes on `bar`.  The arena is viewed as
// [page][8-row group][element block][row in group][64 elements], a box takes whole groups of one page (all element
// blocks), so the only coordinates that vary are the group and the page; the innermost one is always 0.
// Executed by a whole converged warp; one elected lane issues the copy.
__device__ __forceinline__ void tma_load_groups(uint32_t dst, const CUtensorMap* map, uint32_t bar, uint32_t group, uint32_t page) {
    asm volatile(
        "{\n\t.reg .pred e;\n\telect.sync _|e, 0xFFFFFFFF;\n\t"
        "@e cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %3, %3, %4, %5}], [%2];\n\t}\n" ::"r"(dst),
        "l"(map), "r"(bar), "r"(0u), "r"(group), "r"(page)
        : "memory");
}

// The same under an L2 cache policy (createpolicy): a K/V stream that is read once goes in as evict-first.
__device__ __forceinline__ void tma_load_groups_hinted(uint32_t dst, const CUtensorMap* map, uint32_t bar, uint32_t group,
                                                       uint32_t page, uint64_t policy) {
    asm volatile(
        "{\n\t.reg .pred e;\n\telect.sync _|e, 0xFFFFFFFF;\n\t"
        "@e cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %3, %3, %4, %5}], [%2], %6;\n\t}\n" ::"r"(dst),
        "l"(map), "r"(bar), "r"(0u), "r"(group), "r"(page), "l"(policy)
        : "memory");
}

// Byte offset of the 16-byte chunk `chunk` (8 elements) of token row `row` in a K or V tile.  A tile is a stack of
// [row / 8][element block of 64][row % 8][64 elements]: every (8 rows x 128 bytes) block is one swizzle atom (chunk
// index XOR row % 8), the `blocks` atoms of an 8-row group follow one another, groups are blocks * 1024 bytes apart.
__device__ __forceinline__ uint32_t operand_offset(uint32_t blocks, uint32_t row, uint32_t chunk) {
    return ((row >> 3) * blocks + (chunk >> 3)) * 1024 + (row & 7) * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

}  // namespace psi
