// Multi-query attention for long query runs on the 5th-generation tensor cores (tcgen05 / TMEM), K/V staged by TMA.
//
// Same work items as attend_chunk.cu (a super-tile of up to eight 16-row query tiles of one request and KV head: 128
// rows = one native UMMA M tile), different engine.  Per CTA (224 threads, 512 TMEM columns, a shared-memory ring of
// K/V tiles of 64 tokens):
//   warps 0-3 (128 threads): one accumulator row each.  Stage their query row in TMEM as an MMA A operand (the next
//       item's row goes in before the current item's output is written), read the S row from TMEM (tcgen05.ld), apply
//       the causal limit and the online softmax without any cross-thread traffic, write P back over the S buffer as
//       the A operand of P V, rescale their O row in TMEM only when the running max ran away from the reference the
//       exponentials are taken against; epilogue, partial slots and last-arriver merge as in attend_chunk.cu.
//   warp 4: issues the MMAs from converged code with one elected lane (operands then stay in uniform registers)
//         S[128x64]  = Q[128xD] . K^T    (Q from TMEM, K as a K-major shared-memory operand, two S buffers)
//         O[128xD]  += P[128x64] . V     (P from TMEM, V as an MN-major shared-memory operand)
//       so that Q K^T of tile i+1 runs under the softmax of tile i and P V of tile i under the softmax of tile i+1.
//   warps 5 and 6: bring the K and the V tiles from their pages by TMA, one 5-D box per page segment that lands in
//       exactly the order the MMA descriptors read ([8-row group][64-element block][8 rows][64 elements], 128-byte
//       swizzle); an item's last, ragged tile is copied with zero-filling 16-byte cp.async instead.
// All hand-offs are mbarriers (TMA byte counts, tcgen05.commit, thread arrivals); every wait is bounded and reports
// PSI_ERR_TIMEOUT through the status word instead of hanging, and the kernel frees its TMEM on every path.  The kernel
// reads pages only: a step that appends and attends runs the append launch first.
//
// Arithmetic replaced: crates/inference-backend-metal/src/components/metal/gqa_split_kv_tiled_q.metal:49-378.
#include <cuda.h>

#include <mutex>
#include <type_traits>

#include "launch_util.hpp"
#include "mma_common.cuh"
#include "tma_common.cuh"

namespace psi {


namespace {

constexpr uint32_t kRowThreads = 128;   // warps 0-3: one accumulator row per thread
constexpr uint32_t kUmmaThreads = 224;  // + warp 4: MMA issue, warps 5 and 6: K and V tiles into the shared-memory ring
constexpr uint32_t kUmmaM = 128;   // query rows per CTA = TMEM lanes
constexpr uint32_t kUmmaN = 64;    // KV tokens per tile

// Shared-memory matrix descriptor of a 128-byte-swizzled operand: start address, leading / stride byte offsets in
// 16-byte units, descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>((leading_bytes >> 4) & 0x3FFFu) << 16) |
           (static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor of kind::f16: f32 accumulator, A/B element format (0 = f16, 1 = bf16), B major (0 = K,
// 1 = MN), N >> 3 and M >> 4.
template <typename T>
__device__ __forceinline__ uint32_t umma_idesc(uint32_t n, bool b_mn_major) {
    const uint32_t format = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
    return (1u << 4) | (format << 7) | (format << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((n >> 3) << 17) |
           ((kUmmaM >> 4) << 24);
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred e;\n\telect.sync _|e, 0xFFFFFFFF;\n\t"
        "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}\n" ::"r"(bar)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive f32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_load32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_store32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}

__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }




__device__ __forceinline__ void row_threads_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Executed by a whole converged warp; one elected lane (always the same one for a full warp) issues.
__device__ __forceinline__ void umma_issue_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, e;\n\tsetp.ne.b32 p, %4, 0;\n\telect.sync _|e, 0xFFFFFFFF;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tmem_store32_bits(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
        "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]),
        "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]),
        "r"(v[31])
        : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Shared-memory ring slots of one K or V tile, and how far the lazily kept softmax reference may lag the running max
// (log2 domain): P then stays below 2^8, well inside bf16/f16, and O is rescaled only on a real jump.
template <int D>
struct Ring {
    static constexpr uint32_t kSlots = D == 256 ? 7u : 12u;
};
constexpr float kRescaleThreshold = 8.0f;

template <typename T, int D>
__global__ void __launch_bounds__(kUmmaThreads, 1)
    attend_chunk_umma_kernel(const AttendParams p, const __grid_constant__ CUtensorMap kv_map, const uint32_t box_rows) {
    constexpr uint32_t kChunks = D / 8;               // 16-byte chunks per row of K / V
    constexpr uint32_t kBlocks = D / 64;              // 64-element (128-byte) blocks per row
    constexpr uint32_t kTileBytes = D * 2 * kUmmaN;   // one K or V tile: [D/64][64][64]
    constexpr uint32_t kSlots = Ring<D>::kSlots;
    constexpr uint32_t kTmemColumns = 512;
    // TMEM columns: Q as an MMA A operand (two 16-bit elements per column), two S buffers whose first half is
    // overwritten by P (again two elements per column), O
    constexpr uint32_t kColQ = 0, kColS = D / 2, kColO = D / 2 + 2 * kUmmaN;
    static_assert(kColO + D <= kTmemColumns, "Q, S and O share one TMEM allocation");
    // barriers
    constexpr uint32_t kBarFull = 0, kBarEmpty = kSlots, kBarS = 2 * kSlots, kBarO = kBarS + 2, kBarP = kBarO + 2,
                       kBarQ = kBarP + 2, kNumBarriers = kBarQ + 1;

    const uint32_t cta = blockIdx.x;
    if (cta >= p.scalars[kScalarNumChunkCtas]) return;

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[kNumBarriers];
    __shared__ uint32_t tmem_base_s, abort_s, last_s[8];

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // the swizzled operand layouts repeat every 1024 bytes: place them on that boundary whatever the toolchain did
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](uint32_t which) { return bar0 + which * 8; };

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                     "r"(kTmemColumns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        for (uint32_t b = 0; b < kBarP; ++b) mbar_init(bar(b), 1);
        for (uint32_t b = kBarP; b < kNumBarriers; ++b) mbar_init(bar(b), kRowThreads);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        abort_s = 0;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;

    const uint32_t page_mask = p.geo.tokens_per_page - 1;
    const uint32_t page_shift = 31 - __clz(p.geo.tokens_per_page);
    const unsigned char* pages = static_cast<const unsigned char*>(p.geo.pages);
    const uint64_t page_bytes = p.geo.page_elems * 2;
    const uint64_t v_region_bytes = v_region_offset(p.geo) * 2;

    // A wait that ran out flags the launch and lets every later wait fall through: results are then garbage, the
    // status word says so, and the kernel still frees its TMEM and returns.
    auto wait = [&](uint32_t which, uint32_t parity) {
        if (mbar_test(bar(which), parity & 1)) return;  // the usual case: already complete
        if (*reinterpret_cast<volatile uint32_t*>(&abort_s) == 0 && !mbar_wait(bar(which), parity & 1)) {
            abort_s = 1;
            if (p.status != nullptr) atomicExch(p.status, static_cast<uint32_t>(PSI_ERR_TIMEOUT));
        }
    };

    // Tiles, ring fills (K of tile t = fill 2t, V = fill 2t + 1) and items are counted over the whole launch, the
    // same way in every role: ring slot = fill % kSlots with barrier phase fill / kSlots; the S, O and P barriers come
    // in pairs indexed by tile % 2 with phase tile / 2, so that a barrier cannot complete a second time before its
    // waiter has seen the first (a parity wait cannot tell two completions from none); Q takes the item count.
    uint32_t tile_base = 0, item_count = 0;
    const uint32_t item_begin = p.cta_item_begin[cta], item_end = p.cta_item_begin[cta + 1];

    if (warp >= 5) {
        // ================================ producers: K (warp 5) and V (warp 6) tiles into the ring ====================
        const uint32_t v_groups = p.geo.num_kv_heads * p.geo.tokens_per_page / 8;  // 8-row groups of a page's K region
        for (uint32_t index = item_begin; index < item_end; ++index) {
            const ItemView v = view_item(p, index);
            const uint32_t* row_ids = table_row(p.geo, v.req_slot);
            const uint64_t head_bytes = static_cast<uint64_t>(v.kv_head) * p.geo.tokens_per_page * (D * 2);
            const uint32_t head_group = v.kv_head * p.geo.tokens_per_page / 8;
            const uint32_t first_tile = v.kv_begin / kUmmaN;
            const uint32_t num_tiles = (v.kv_end + kUmmaN - 1) / kUmmaN - first_tile;
            const uint32_t last_page = (v.kv_end - 1) >> page_shift;
            uint32_t window_base = kU32Max, window_ids = 0;  // 32 page ids of the request, one per lane
            for (uint32_t i = 0; i < num_tiles; ++i) {
                const uint32_t token0 = (first_tile + i) * kUmmaN;
                const bool whole = token0 + kUmmaN <= v.kv_end;
                {
                    const uint32_t first_page = token0 >> page_shift;
                    const uint32_t end_page = min(last_page, (token0 + kUmmaN - 1) >> page_shift);
                    if (first_page < window_base || end_page >= window_base + 32) {
                        window_base = first_page;
                        window_ids = first_page + lane <= last_page ? page_id_or_zero(p.geo, row_ids, first_page + lane) : 0u;
                    }
                }
                {
                    const uint32_t which = warp - 5;  // warp 5 brings the K tiles, warp 6 the V tiles
                    const uint32_t fill = 2 * (tile_base + i) + which, slot = fill % kSlots, use = fill / kSlots;
                    const uint32_t dst = smem_base + slot * kTileBytes;
                    if (use > 0) wait(kBarEmpty + slot, use - 1);  // the MMAs that read the slot's previous tile are done
                    __syncwarp();
                    if (whole) {
                        if (lane == 0) mbar_expect_tx(bar(kBarFull + slot), kTileBytes);
                        for (uint32_t row = 0; row < kUmmaN; row += box_rows) {
                            const uint32_t token = token0 + row;
                            const uint32_t page = __shfl_sync(0xFFFFFFFFu, window_ids, (token >> page_shift) - window_base);
                            const uint32_t group = which * v_groups + head_group + (token & page_mask) / 8;
                            tma_load_groups(dst + (row / 8) * (kBlocks * 1024), &kv_map, bar(kBarFull + slot), group, page);
                        }
                    } else {
                        // the item's last tile: rows at and beyond its end are zero
                        for (uint32_t c = lane; c < kUmmaN * kChunks; c += 32) {
                            const uint32_t row = c / kChunks, chunk = c % kChunks;
                            const uint32_t token = token0 + row;
                            const bool valid = token < v.kv_end;
                            const uint32_t page =
                                __shfl_sync(0xFFFFFFFFu, window_ids, valid ? (token >> page_shift) - window_base : 0u);
                            const unsigned char* src = pages + static_cast<uint64_t>(page) * page_bytes + head_bytes +
                                                       (which ? v_region_bytes : 0) + (token & page_mask) * (D * 2) + chunk * 16;
                            cp_async_16(dst + operand_offset(kBlocks, row, chunk), valid ? src : pages, valid ? 16u : 0u);
                        }
                        cp_async_commit();
                        cp_async_wait<0>();
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(kBarFull + slot));
                    }
                    __syncwarp();
                }
            }
            tile_base += num_tiles;
        }
        // the CTA does not go away with its own bulk copies in flight: every slot's last fill has landed (a bounded
        // wait of its own, also after an earlier wait gave up)
        const uint32_t fills = 2 * tile_base;
        for (uint32_t back = 1; back <= kSlots && back <= fills; ++back) {
            const uint32_t fill = fills - back;
            mbar_wait(bar(kBarFull + fill % kSlots), (fill / kSlots) & 1);
        }
    } else if (warp == 4) {
        // ================================ MMA issue (converged warp, one elected lane) ================================
        {
            const uint32_t idesc_qk = umma_idesc<T>(kUmmaN, false);
            const uint32_t idesc_pv = umma_idesc<T>(D, true);
            for (uint32_t index = item_begin; index < item_end; ++index, ++item_count) {
                const ItemView v = view_item(p, index);
                const uint32_t first_tile = v.kv_begin / kUmmaN;
                const uint32_t num_tiles = (v.kv_end + kUmmaN - 1) / kUmmaN - first_tile;

                // S[tile % 2] = Q K^T of local tile i; frees the K slot when done
                auto issue_qk = [&](uint32_t i) {
                    const uint32_t tile = tile_base + i, fill = 2 * tile, slot = fill % kSlots;
                    wait(kBarFull + slot, fill / kSlots);
                    tc_fence_after();
                    // K-major operand: 8-row groups kBlocks KiB apart; per k-step the start moves to element block ks / 4
                    // and 32 bytes on inside it (the start-address field counts 16-byte units)
                    const uint64_t k_desc = umma_desc(smem_base + slot * kTileBytes, 16, kBlocks * 1024);
                    const uint32_t s_tmem = tmem + kColS + (tile & 1) * kUmmaN;
#pragma unroll
                    for (uint32_t ks = 0; ks < uint32_t(D) / 16; ++ks)
                        umma_issue_ts(s_tmem, tmem + kColQ + ks * 8, k_desc + ((ks >> 2) * 1024 + (ks & 3) * 32) / 16, idesc_qk, ks > 0);
                    umma_commit(bar(kBarS + (tile & 1)));
                    umma_commit(bar(kBarEmpty + slot));
                };

                wait(kBarQ, item_count);  // the item's query rows are in TMEM; the rows are done with the previous item
                if (num_tiles > 0) issue_qk(0);
                for (uint32_t i = 0; i < num_tiles; ++i) {
                    const uint32_t tile = tile_base + i, fill = 2 * tile + 1, slot = fill % kSlots;
                    if (i + 1 < num_tiles) issue_qk(i + 1);  // runs under the softmax of tile i
                    wait(kBarFull + slot, fill / kSlots);
                    wait(kBarP + (tile & 1), tile >> 1);      // P of tile i is in TMEM (over the first half of its S buffer)
                    tc_fence_after();
                    // MN-major operand: 64-element blocks 1 KiB apart, 8-token groups kBlocks KiB apart, two groups per
                    // k-step
                    const uint64_t v_desc = umma_desc(smem_base + slot * kTileBytes, 1024, kBlocks * 1024);
                    const uint32_t p_tmem = tmem + kColS + (tile & 1) * kUmmaN;
#pragma unroll
                    for (uint32_t ks = 0; ks < kUmmaN / 16; ++ks)
                        umma_issue_ts(tmem + kColO, p_tmem + ks * 8, v_desc + ks * 2 * (kBlocks * 1024) / 16, idesc_pv,
                                      (i > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(bar(kBarO + (tile & 1)));
                    umma_commit(bar(kBarEmpty + slot));
                }
                tile_base += num_tiles;
            }
        }
    } else {
        // ================================ one accumulator row per thread ===============================================
        const uint32_t lane_base = (warp * 32u) << 16;  // this warp's TMEM lanes
        const uint32_t tmem_o = tmem + kColO;
        // Row of this thread in an item: 16-row tile w = tid / 16, row rr inside it -> (token, head) of the super-tile.
        const uint32_t w = tid >> 4, rr = tid & 15;
        auto row_of = [&](const ItemView& v, bool& valid) {
            const uint32_t token_off = w * p.tokens_per_tile + rr / v.num_heads;
            valid = rr < p.tokens_per_tile * v.num_heads && token_off < v.num_tokens;
            return static_cast<uint64_t>(v.flat_begin + (valid ? token_off : 0)) * p.num_q_heads + v.head0 + rr % v.num_heads;
        };
        // This thread's query row of an item into its TMEM lane (zero for rows the super-tile does not have).  Called
        // when every Q K^T of the previous item has completed; 16 loads in flight at a time.
        auto load_q = [&](const ItemView& v) {
            bool valid;
            const uint64_t row = row_of(v, valid);
            const uint4* q_row = reinterpret_cast<const uint4*>(static_cast<const T*>(p.q) + row * D);
#pragma unroll 1
            for (uint32_t c = 0; c < uint32_t(D) / 2; c += 64) {
                uint32_t regs[2][32];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const uint4 value = valid ? q_row[c / 4 + j] : make_uint4(0, 0, 0, 0);
                    regs[j / 8][4 * (j % 8)] = value.x;
                    regs[j / 8][4 * (j % 8) + 1] = value.y;
                    regs[j / 8][4 * (j % 8) + 2] = value.z;
                    regs[j / 8][4 * (j % 8) + 3] = value.w;
                }
                __syncwarp();
                tmem_store32_bits(tmem + kColQ + lane_base + c, regs[0]);
                tmem_store32_bits(tmem + kColQ + lane_base + c + 32, regs[1]);
            }
            tmem_store_wait();
            tc_fence_before();
            mbar_arrive(bar(kBarQ));
        };

        if (item_begin < item_end) load_q(view_item(p, item_begin));
        for (uint32_t index = item_begin; index < item_end; ++index, ++item_count) {
            const ItemView v = view_item(p, index);
            bool row_valid;
            const uint64_t out_row = row_of(v, row_valid);
            const uint32_t token_off = w * p.tokens_per_tile + rr / v.num_heads;
            const uint32_t limit = row_valid ? min(v.kv_end, v.first_pos + token_off + 1) : v.kv_end;
            const uint32_t min_limit = min(v.kv_end, v.first_pos + 1);
            const uint32_t first_tile = v.kv_begin / kUmmaN;
            const uint32_t num_tiles = (v.kv_end + kUmmaN - 1) / kUmmaN - first_tile;

            // softmax state in the log2 domain: `row_ref` is the reference the exponentials are taken against (it
            // trails the true running max `row_max` by at most kRescaleThreshold), `row_sum` is relative to it
            float row_ref = -INFINITY, row_max = -INFINITY, row_sum = 0.0f;
            for (uint32_t i = 0; i < num_tiles; ++i) {
                const uint32_t tile = tile_base + i, buf = tile & 1;
                const uint32_t token0 = (first_tile + i) * kUmmaN;
                const uint32_t tmem_s = tmem + kColS + buf * kUmmaN + lane_base;
                wait(kBarS + buf, tile >> 1);
                __syncwarp();  // the TMEM accesses below are warp-collective
                tc_fence_after();

                float s[kUmmaN];
                {
                    float part[32];
                    tmem_load32(tmem_s, part);
#pragma unroll
                    for (int c = 0; c < 32; ++c) s[c] = part[c];
                    tmem_load32(tmem_s + 32, part);
#pragma unroll
                    for (int c = 0; c < 32; ++c) s[32 + c] = part[c];
                }
                if (token0 < v.kv_begin || token0 + kUmmaN > min_limit) {
#pragma unroll
                    for (int c = 0; c < int(kUmmaN); ++c) {
                        const uint32_t token = token0 + c;
                        if (token >= limit || token < v.kv_begin) s[c] = -INFINITY;
                    }
                }
                float m4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
                for (int c = 4; c < int(kUmmaN); c += 4) {
                    m4[0] = fmaxf(m4[0], s[c]);
                    m4[1] = fmaxf(m4[1], s[c + 1]);
                    m4[2] = fmaxf(m4[2], s[c + 2]);
                    m4[3] = fmaxf(m4[3], s[c + 3]);
                }
                const float tile_max = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;  // scale > 0
                row_max = fmaxf(row_max, tile_max);
                const bool moved = row_max > row_ref + kRescaleThreshold;  // also the first visible key (-inf reference)
                float corr = 1.0f;
                if (moved) {
                    corr = row_ref == -INFINITY ? 0.0f : fast_exp2(row_ref - row_max);
                    row_ref = row_max;
                }
                const float base = row_ref == -INFINITY ? 0.0f : row_ref;
                float sum4[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t packed[kUmmaN / 2];
#pragma unroll
                for (int c = 0; c < int(kUmmaN); c += 4) {
                    const float e0 = fast_exp2(fmaf(s[c], p.scale_log2, -base));
                    const float e1 = fast_exp2(fmaf(s[c + 1], p.scale_log2, -base));
                    const float e2 = fast_exp2(fmaf(s[c + 2], p.scale_log2, -base));
                    const float e3 = fast_exp2(fmaf(s[c + 3], p.scale_log2, -base));
                    sum4[0] += e0;
                    sum4[1] += e1;
                    sum4[2] += e2;
                    sum4[3] += e3;
                    packed[c / 2] = Mma<T>::pack(e0, e1);
                    packed[c / 2 + 1] = Mma<T>::pack(e2, e3);
                }
                row_sum = row_sum * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));

                // O is touched only when a reference moved (per warp: each warp owns its 32 rows), and only then does
                // P wait for the previous P V; otherwise P goes out first and the wait just keeps the phases in step
                const bool rescale = i > 0 && __any_sync(0xFFFFFFFFu, moved);
                if (rescale) {
                    wait(kBarO + ((tile - 1) & 1), (tile - 1) >> 1);
                    __syncwarp();
                    tc_fence_after();
#pragma unroll 1
                    for (uint32_t c = 0; c < uint32_t(D); c += 32) {
                        float o[32];
                        tmem_load32(tmem_o + lane_base + c, o);
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] *= corr;
                        tmem_store32(tmem_o + lane_base + c, o);
                    }
                }
                __syncwarp();
                tmem_store32_bits(tmem_s, packed);  // P over the first 32 columns of this S buffer
                tmem_store_wait();
                tc_fence_before();
                mbar_arrive(bar(kBarP + buf));
                if (i > 0 && !rescale) wait(kBarO + ((tile - 1) & 1), (tile - 1) >> 1);
            }
            if (num_tiles > 0) {
                const uint32_t last = tile_base + num_tiles - 1;
                wait(kBarO + (last & 1), last >> 1);
                __syncwarp();
                tc_fence_after();
            }
            tile_base += num_tiles;
            // The next item's query rows go to TMEM before this item's output is written: its first Q K^T products then
            // run under the epilogue (O is not touched before P of that item's first tile exists).
            if (index + 1 < item_end) load_q(view_item(p, index + 1));

            // ---- epilogue: every thread finishes its own row ---------------------------------------------------------------
            // back to the true max as the reference: l' = l * 2^(ref - max); O / l is unchanged by the shift
            const float inv = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;
            const float sum_at_max = row_max == -INFINITY ? row_sum : row_sum * fast_exp2(row_ref - row_max);
            const bool is_partial = v.partial_slot != kU32Max;
            const uint64_t prow = is_partial ? static_cast<uint64_t>(v.partial_slot + w) * kMaxRows + rr : 0;
#pragma unroll 1
            for (uint32_t c = 0; c < uint32_t(D); c += 32) {
                float o[32];
                if (num_tiles > 0) {
                    tmem_load32(tmem_o + lane_base + c, o);
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] = 0.0f;
                }
                if (row_valid) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] *= inv;
                    if (is_partial) {
                        // a partial slot of this kernel is stored column-major in float4 units, [D / 4][16 rows]: the
                        // 16 rows of a tile are 16 consecutive lanes here, so every store instruction writes whole
                        // 256-byte runs (the merge below reads them the same way)
                        float4* dst = reinterpret_cast<float4*>(p.partial_o + static_cast<uint64_t>(v.partial_slot + w) * kMaxRows * D) +
                                      static_cast<uint64_t>(c / 4) * kMaxRows + rr;
#pragma unroll
                        for (int e = 0; e < 32; e += 4)
                            dst[static_cast<uint64_t>(e / 4) * kMaxRows] = make_float4(o[e], o[e + 1], o[e + 2], o[e + 3]);
                    } else if (p.ext_o != nullptr) {
                        float* dst = p.ext_o + out_row * D + c;
#pragma unroll
                        for (int e = 0; e < 32; e += 4)
                            *reinterpret_cast<float4*>(dst + e) = make_float4(o[e], o[e + 1], o[e + 2], o[e + 3]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) store_out8<T>(p, out_row * D + c + e, o + e);
                    }
                }
                __syncwarp();  // the TMEM load of the next pass is warp-collective
            }
            if (row_valid) {
                if (is_partial) {
                    p.partial_m[prow] = row_max;
                    p.partial_l[prow] = sum_at_max;
                } else if (p.ext_o != nullptr) {
                    p.ext_m[out_row] = row_max * kLn2;
                    p.ext_l[out_row] = sum_at_max;
                }
            }
            tc_fence_before();

            // ---- units shared with other CTAs: whoever delivers a tile's last partial merges it ---------------------------
            if (is_partial) {
                __threadfence();
                row_threads_sync();
                if (tid < 8) {
                    const bool has_rows = tid * p.tokens_per_tile < v.num_tokens;
                    last_s[tid] = has_rows && atomicAdd(p.unit_counters + v.reduce_unit + tid, 1u) == v.unit_num_items - 1;
                    __threadfence();  // the other pieces' partials are read (from L2) only after their arrivals were seen
                }
                row_threads_sync();
                for (uint32_t tile = 0; tile < 8; ++tile) {
                    if (!last_s[tile]) continue;
                    // 16 rows x D / 4 float4 outputs per tile: a thread takes row tid % 16 and the float4 columns
                    // tid / 16 + 8 j (16 consecutive lanes read 256 consecutive bytes of the column-major slots)
                    const uint32_t tile_tokens = min(p.tokens_per_tile, v.num_tokens - tile * p.tokens_per_tile);
                    const uint32_t tile_rows = tile_tokens * v.num_heads;
                    constexpr uint32_t kPerThread = kMaxRows * (D / 4) / kRowThreads;
                    constexpr uint32_t kColumnStep = kRowThreads / kMaxRows;  // float4 columns between a thread's outputs
                    // a row beyond the tile's last one is computed on the last row and dropped at the end: the loops
                    // below are then straight-line code whose loads all go out before the first one is used
                    const uint32_t r = min(tid % kMaxRows, tile_rows - 1), c4_0 = tid / kMaxRows;
                    const bool row_present = tid % kMaxRows < tile_rows;
                    const uint64_t slot_rows = static_cast<uint64_t>(v.unit_first_slot + tile) * kMaxRows;
                    // one pass over the pieces with the running max of a row carried along (sums are rescaled when
                    // a later piece raises it); the loads of piece s + 1 are in flight while piece s is folded in
                    float4 acc[kPerThread];
#pragma unroll
                    for (uint32_t j = 0; j < kPerThread; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    constexpr uint64_t kPieceRows = 8 * kMaxRows;  // rows between the same tile of consecutive pieces
                    float pm[2], pl[2];
                    float4 part[2][kPerThread];
                    auto fetch = [&](uint32_t piece, float& m_out, float& l_out, float4 (&o_out)[kPerThread]) {
                        const uint64_t rows = slot_rows + piece * kPieceRows;
                        m_out = __ldcg(p.partial_m + rows + r);
                        l_out = __ldcg(p.partial_l + rows + r);
                        const float4* slot = reinterpret_cast<const float4*>(p.partial_o + rows * D) + r;
#pragma unroll
                        for (uint32_t j = 0; j < kPerThread; ++j)
                            o_out[j] = __ldcg(slot + static_cast<uint64_t>(c4_0 + j * kColumnStep) * kMaxRows);
                    };
                    // one row per thread: a single running max, sum and carry for all of its columns
                    float top_all = -INFINITY, sum_all = 0.0f;
                    auto fold = [&](float m_in, float l_in, const float4 (&o_in)[kPerThread]) {
                        const float top = fmaxf(top_all, m_in);
                        const float carry = top_all == -INFINITY ? 0.0f : fast_exp2(top_all - top);
                        const float w = m_in == -INFINITY ? 0.0f : fast_exp2(m_in - top) * l_in;
                        sum_all = sum_all * carry + w;
#pragma unroll
                        for (uint32_t j = 0; j < kPerThread; ++j) {
                            acc[j].x = acc[j].x * carry + w * o_in[j].x;
                            acc[j].y = acc[j].y * carry + w * o_in[j].y;
                            acc[j].z = acc[j].z * carry + w * o_in[j].z;
                            acc[j].w = acc[j].w * carry + w * o_in[j].w;
                        }
                        top_all = top;
                    };
                    fetch(0, pm[0], pl[0], part[0]);
                    for (uint32_t s0 = 0; s0 < v.unit_num_items; s0 += 2) {
                        if (s0 + 1 < v.unit_num_items) fetch(s0 + 1, pm[1], pl[1], part[1]);
                        fold(pm[0], pl[0], part[0]);
                        if (s0 + 1 < v.unit_num_items) {
                            if (s0 + 2 < v.unit_num_items) fetch(s0 + 2, pm[0], pl[0], part[0]);
                            fold(pm[1], pl[1], part[1]);
                        }
                    }
                    if (row_present) {
                        const float scale = sum_all > 0.0f ? 1.0f / sum_all : 0.0f;
                        const uint64_t row =
                            static_cast<uint64_t>(v.flat_begin + tile * p.tokens_per_tile + r / v.num_heads) * p.num_q_heads +
                            v.head0 + r % v.num_heads;
#pragma unroll
                        for (uint32_t j = 0; j < kPerThread; ++j) {
                            const uint32_t c4 = c4_0 + j * kColumnStep;
                            const float4 value = make_float4(acc[j].x * scale, acc[j].y * scale, acc[j].z * scale, acc[j].w * scale);
                            if (p.ext_o != nullptr) {
                                *reinterpret_cast<float4*>(p.ext_o + row * D + 4 * c4) = value;
                            } else {
                                store_out4<T>(p, row * D + 4 * c4, value);
                            }
                        }
                        if (p.ext_o != nullptr && c4_0 == 0) {
                            p.ext_m[row] = top_all * kLn2;
                            p.ext_l[row] = sum_all;
                        }
                    }
                    if (tid == 0) p.unit_counters[v.reduce_unit + tile] = 0;  // ready for the next launch
                }
                row_threads_sync();  // the flags are read before the next item overwrites them
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns) : "memory");
    }
}

template <typename T, int D>
cudaError_t launch_one(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    constexpr uint32_t kSmem = Ring<D>::kSlots * (D * 2 * kUmmaN) + 1024;
    const uint32_t box_rows = p.geo.tokens_per_page < kUmmaN ? p.geo.tokens_per_page : kUmmaN;
    CUtensorMap map;
    if (!make_kv_map(p, box_rows, &map)) return cudaErrorNotSupported;
    auto kernel = attend_chunk_umma_kernel<T, D>;
    static std::atomic<uint64_t> configured{0};  // per instantiation, one bit per device
    cudaError_t err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), static_cast<int>(kSmem), configured);
    if (err != cudaSuccess) return err;
    kernel<<<num_ctas, kUmmaThreads, kSmem, stream>>>(p, map, box_rows);
    return cudaGetLastError();
}

template <typename T>
cudaError_t launch_for_dim(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    switch (p.geo.head_dim) {
        case 128: return launch_one<T, 128>(p, num_ctas, stream);
        case 256: return launch_one<T, 256>(p, num_ctas, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

// cudaErrorNotSupported: the arena cannot be described to the TMA unit (alignment, size); nothing was launched and
// the caller takes launch_attend_chunk instead.

cudaError_t launch_attend_chunk_umma(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    if (num_ctas == 0) return cudaSuccess;
    return p.dtype == PSI_DTYPE_BF16 ? launch_for_dim<__nv_bfloat16>(p, num_ctas, stream)
                                     : launch_for_dim<__half>(p, num_ctas, stream);
}

}  // namespace psi
