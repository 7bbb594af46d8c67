// Split-KV flash-decode map kernel for bf16 / f16 on sm_100a.
//
// One CTA per device CTA slot walks a contiguous share of the step's work items.  A work item is all query rows of
// one (q tile, KV head) - the tokens of the tile times the heads of the GQA group, at most 16 rows - against a range
// of KV tokens, so every KV byte of the step is read from HBM exactly once.
//
// Inside a CTA each of the eight warps owns every eighth 16-token KV tile of the item and streams it through its own
// ring of shared-memory slots (K tile, V tile, K tile, ...) with 16-byte cp.async copies (a warp-wide copy covers 512
// contiguous bytes of one page), so the steady state has no CTA-wide barrier: a warp waits only for its own oldest
// slot, and two warps per scheduler hide each other's instruction latencies.  The 16 query rows are one m16 MMA
// tile: S = Q K^T and O += P V run as mma.sync.m16n8k16 with f32 accumulators, operands fetched by ldmatrix from
// XOR-swizzled rows; the online softmax runs on the accumulator fragments with quad shuffles in the log2 domain, and
// O is rescaled only when a row's running max moved.  At the end of an item the warps merge their (O, m, l) through
// shared memory and write either the final output or one partial slot; the CTA that delivers the last partial of a
// (q tile, KV head) unit merges the unit's partials itself (arrival counter, no waiting), so no second kernel runs.
//
// The arithmetic this replaces: crates/inference-backend-metal/src/components/metal/gqa_split_kv_single_q_map.metal
// (decode rows) and metal/gqa_split_kv_tiled_q.metal:161-319 (several query tokens of one request with the in-kernel
// causal limit).
#include "exchange.cuh"
#include "launch_util.hpp"
#include "mma_common.cuh"
#include "tma_common.cuh"

namespace psi {

namespace {

template <int D, int NSLOT>
struct SmemLayout {
    static constexpr uint32_t kRowBytes = D * 2;
    static constexpr uint32_t kTileBytes = kTile * kRowBytes;        // one K or V tile = one ring slot
    static constexpr uint32_t kQBytes = kTile * kRowBytes;
    static constexpr uint32_t kRingOffset = kQBytes;
    static constexpr uint32_t kMergeStride = D + 8;                  // floats per merged row
    static constexpr uint32_t kMergeBytes = kWarps * kTile * kMergeStride * 4;
    static constexpr uint32_t kRingBytes = kWarps * NSLOT * kTileBytes;
    static constexpr uint32_t kTotal = kRingOffset + (kRingBytes > kMergeBytes ? kRingBytes : kMergeBytes);
};


// kExchange: the launch is one rank's part of a KV-range exchange (exchange.cuh); the outputs go to the rank's slot of
// the owner's receive area (ext_*), and the launch ends with the flag publication and, on the owner, the merge.
//
// kTma: whole K/V tiles come from their pages as TMA boxes (cp.async.bulk.tensor, one instruction per 16-token tile
// and warp, completion on one mbarrier per ring slot) instead of 16-byte cp.async copies; the tiles then lie in the
// box layout of tma_common.cuh.  An item's ragged last tile and this step's own rows still come by cp.async.
template <typename T, int D, int NSLOT, bool kExchange, bool kTma>
__global__ void __launch_bounds__(kThreads, 1) attend_mma_kernel(AttendParams p, const __grid_constant__ CUtensorMap kv_map,
                                                                uint32_t box_rows) {
    using L = SmemLayout<D, NSLOT>;
    constexpr uint32_t kBlocks = D / 64;                     // 128-byte element blocks per row (TMA box layout)
    constexpr uint32_t kChunks = D / 8;                      // 16-byte chunks per row
    constexpr uint32_t kRowsPerCopy = 32 / (kChunks < 32 ? kChunks : 32);

    const uint32_t cta = blockIdx.x;
    // The plan and the page table are read again by the next launch of the step (one launch per layer) while hundreds
    // of megabytes of K/V pass through the L2 in between: their lines are loaded to be evicted last.
    const uint64_t keep = l2_evict_last_policy();
    // One round trip for everything the first tile copies depend on: the CTA count, this CTA's item range and a copy
    // of its first item all go out before the first of them is needed.
    const uint32_t num_ctas = ld_u32_hinted(p.scalars + kScalarNumCtas, keep);
    const uint32_t item_begin = ld_u32_hinted(p.cta_item_begin + cta, keep);
    const uint32_t item_end = ld_u32_hinted(p.cta_item_begin + cta + 1, keep);
    const bool have_first = p.cta_first_items != nullptr;
    const ItemView first_item = view_item_hinted(have_first ? p.cta_first_items + cta : p.items, keep);
    if (cta >= num_ctas) return;

    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint32_t limit_s[kTile];
    __shared__ float merge_m[kWarps][kTile];
    __shared__ float merge_l[kWarps][kTile];
    __shared__ uint32_t arrival_s;
    __shared__ uint32_t slot_free_s;  // exchange launches: this CTA may store into the rank's slot
    __shared__ __align__(8) uint64_t ring_bar_s[kTma ? kWarps : 1][kTma ? NSLOT : 1];  // one mbarrier per ring slot

    const uint32_t tid = threadIdx.x;
    // The consumed word lives on the owner: its value is requested now and looked at before the first store.
    uint32_t consumed_early = 0;
    if (kExchange && tid == 0 && p.xchg.step >= 3) consumed_early = ld_relaxed_sys(p.xchg.consumed);
    const uint32_t warp = tid >> 5;
    const uint32_t lane = tid & 31;
    const uint32_t quad_row = lane >> 2;  // accumulator rows quad_row and quad_row + 8
    const uint32_t quad_col = lane & 3;

    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const uint32_t q_base = smem_base;
    const uint32_t ring_base = smem_base + L::kRingOffset + warp * NSLOT * L::kTileBytes;
    float* merge_o = reinterpret_cast<float*>(smem + L::kRingOffset);

    const uint32_t page_mask = p.geo.tokens_per_page - 1;          // tokens_per_page is a power of two
    const uint32_t page_shift = 31 - __clz(p.geo.tokens_per_page);
    const unsigned char* pages = static_cast<const unsigned char*>(p.geo.pages);
    const uint64_t page_bytes = p.geo.page_elems * 2;
    const uint64_t v_region_bytes = v_region_offset(p.geo) * 2;

    const FragmentLanes frag(lane, L::kRowBytes, kTma ? kBlocks * 1024u : 0u);
    uint32_t tma_bits = 0;    // ring slots of this warp whose current fill is a TMA box (waited for on the slot's mbarrier)
    uint32_t phase_bits = 0;  // parity of each slot's mbarrier phase that the next wait is for
    bool ring_ok = true;      // false once a bounded mbarrier wait ran out: later waits are skipped
    if (kTma) {
        if (tid < kWarps * NSLOT) mbar_init(smem_u32(&ring_bar_s[tid / NSLOT][tid % NSLOT]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const uint32_t v_groups = p.geo.num_kv_heads * p.geo.tokens_per_page / 8;  // 8-row groups of a page's K region
    const uint64_t stream_policy = l2_evict_first_policy();  // full K/V tiles are read once per launch

    // copy lane roles: this lane moves chunk copy_chunk of rows copy_row, copy_row + kRowsPerCopy, ...
    const uint32_t copy_row = lane / kChunks, copy_chunk = lane % kChunks;
    const uint32_t copy_src = copy_row * L::kRowBytes + copy_chunk * 16;
    const uint32_t copy_x = copy_chunk ^ copy_row;                  // copy_row < 8: XOR-able with the row step below

    const bool fused = p.new_k != nullptr;
    const PageBounds bounds(p.geo);
    uint32_t bad_page = 0;  // set when a table index or page ID was out of bounds (that read went to page 0 instead)
    for (uint32_t index = item_begin; index < item_end; ++index) {
        const ItemView v = (have_first && index == item_begin) ? first_item : view_item_hinted(p.items + index, keep);
        __syncthreads();  // the previous item's merge is done with the ring, with q and with limit_s
        if (kTma) fence_async_smem();  // ... before TMA boxes (another proxy) overwrite what the merge wrote there

        // Keys at or beyond `paged_end` are this step's own tokens: in the fused step they are read from new_k/new_v.
        const uint32_t paged_end = fused ? min(v.kv_end, v.new_begin) : v.kv_end;

        // ---- this warp's share of the item's KV tiles ----------------------------------------------------------------
        const uint32_t first_tile = v.kv_begin / kTile;
        const uint32_t end_tile = (v.kv_end + kTile - 1) / kTile;
        const uint32_t item_tiles = end_tile - first_tile;
        const uint32_t my_tiles = item_tiles > warp ? (item_tiles - warp + kWarps - 1) / kWarps : 0;
        const uint32_t my_halves = 2 * my_tiles;  // K tile, V tile, K tile, ...
        auto tile_of = [&](uint32_t j) { return first_tile + warp + j * kWarps; };
        const uint32_t* row_ids = table_row(p.geo, v.req_slot);
        const uint64_t head_bytes = static_cast<uint64_t>(v.kv_head) * p.geo.tokens_per_page * L::kRowBytes;
        const uint32_t head_group = v.kv_head * p.geo.tokens_per_page / 8;

        // Page ids of the two 8-token halves of local tile i (equal when a page holds 16 tokens or more).
        auto lookup = [&](uint32_t i, uint32_t& id_lo, uint32_t& id_hi) {
            const uint32_t token = tile_of(i) * kTile;
            id_lo = token < paged_end ? bounds.read_hinted(row_ids, token >> page_shift, bad_page, keep) : 0u;
            id_hi = token + 8 < paged_end ? bounds.read_hinted(row_ids, (token + 8) >> page_shift, bad_page, keep) : 0u;
        };
        // Issues the copies of half-tile h (K of tile h/2 when h is even, else V) into ring slot `slot`.
        auto issue = [&](uint32_t h, uint32_t slot, uint32_t id_lo, uint32_t id_hi) {
            const uint32_t token0 = tile_of(h >> 1) * kTile;
            const uint32_t dst0 = ring_base + slot * L::kTileBytes + copy_row * L::kRowBytes;
            const uint64_t region = head_bytes + ((h & 1) ? v_region_bytes : 0) + copy_src;
            const unsigned char* src_lo =
                pages + static_cast<uint64_t>(id_lo) * page_bytes + region + (token0 & page_mask) * L::kRowBytes;
            const unsigned char* src_hi =
                pages + static_cast<uint64_t>(id_hi) * page_bytes + region + ((token0 + 8) & page_mask) * L::kRowBytes;
            if (kTma && token0 + kTile <= paged_end) {
                // one box of 16 rows, or two of 8 when a page holds 8 tokens; the elected lane issues
                const uint32_t bar = smem_u32(&ring_bar_s[kTma ? warp : 0][kTma ? slot : 0]);
                const uint32_t tile_base = ring_base + slot * L::kTileBytes;
                const uint32_t group0 = ((h & 1) ? v_groups : 0u) + head_group;
                if (lane == 0) mbar_expect_tx(bar, L::kTileBytes);
                __syncwarp();
                tma_load_groups_hinted(tile_base, &kv_map, bar, group0 + (token0 & page_mask) / 8, id_lo, stream_policy);
                if (box_rows < kTile) {
                    tma_load_groups_hinted(tile_base + kBlocks * 1024u, &kv_map, bar, group0 + ((token0 + 8) & page_mask) / 8,
                                           id_hi, stream_policy);
                }
                tma_bits |= 1u << slot;
            } else if (token0 + kTile <= paged_end) {
#pragma unroll
                for (uint32_t it = 0; it < kTile / kRowsPerCopy; ++it) {
                    const uint32_t row0 = it * kRowsPerCopy;  // this lane's row is row0 + copy_row
                    const unsigned char* src = row0 < 8 ? src_lo + row0 * L::kRowBytes : src_hi + (row0 - 8) * L::kRowBytes;
                    cp_async_16_hinted(dst0 + row0 * L::kRowBytes + ((copy_x ^ (row0 & 7)) << 4), src, 16u, stream_policy);
                }
            } else {
                // The item's last tile (ragged end, or this step's own tokens) is rare: a rolled loop keeps its code to
                // a few instruction-cache lines, which are fetched in mid-stream behind the K/V traffic of all SMs.
                const unsigned char* fresh = static_cast<const unsigned char*>((h & 1) ? p.new_v : p.new_k);
#pragma unroll 1
                for (uint32_t it = 0; it < kTile / kRowsPerCopy; ++it) {
                    const uint32_t row0 = it * kRowsPerCopy;
                    const uint32_t token = token0 + row0 + copy_row;
                    const unsigned char* src = row0 < 8 ? src_lo + row0 * L::kRowBytes : src_hi + (row0 - 8) * L::kRowBytes;
                    uint32_t bytes = 16u;
                    if (token >= v.kv_end) {
                        src = pages;  // beyond the item: zero-fill
                        bytes = 0u;
                    } else if (token >= paged_end) {
                        // one of this step's tokens: row (flat token, kv head) of the new K / V
                        src = fresh + (static_cast<uint64_t>(v.flat_req_begin + (token - v.new_begin)) * p.geo.num_kv_heads +
                                       v.kv_head) * L::kRowBytes + copy_chunk * 16;
                    }
                    const uint32_t dst = kTma ? ring_base + slot * L::kTileBytes + operand_offset(kBlocks, row0 + copy_row, copy_chunk)
                                              : dst0 + row0 * L::kRowBytes + ((copy_x ^ (row0 & 7)) << 4);
                    cp_async_16(dst, src, bytes);
                }
                tma_bits &= ~(1u << slot);
            }
        };

        RowState<D> st;
        st.clear();

        // The query rows go straight into shared memory (zero rows beyond the item's) as the item's oldest copy group:
        // they need nothing but the item, so they are under way before the first page id is known.
        for (uint32_t i = tid; i < kTile * kChunks; i += kThreads) {
            const uint32_t r = i / kChunks, c = i % kChunks;
            const bool present = r < v.rows;
            const T* src = static_cast<const T*>(p.q) + (present ? item_row_index(p, v, r) * D + c * 8 : 0);
            cp_async_16(q_base + swizzled(r, c, L::kRowBytes), src, present ? 16u : 0u);
        }
        cp_async_commit();

        // ids of the tile whose halves are issued next, and of the tile after it
        uint32_t cur_lo = 0, cur_hi = 0, next_lo = 0, next_hi = 0;
        if (my_tiles > 0) lookup(0, cur_lo, cur_hi);
        if (my_tiles > 1) lookup(1, next_lo, next_hi);
#pragma unroll
        for (uint32_t h = 0; h < NSLOT - 1; ++h) {
            if (h < my_halves) {
                issue(h, h, cur_lo, cur_hi);
                if (h & 1) {  // the tile is fully issued: advance the id window
                    cur_lo = next_lo;
                    cur_hi = next_hi;
                    if ((h >> 1) + 2 < my_tiles) lookup((h >> 1) + 2, next_lo, next_hi);
                }
            }
            cp_async_commit();
        }

        // ---- with the first tiles in flight: the per-row causal limits, and in the fused step this item's share of the
        // step's K/V rows into their pages -------------------------------------------------------------------------------
        if (tid < kTile) limit_s[tid] = tid < v.rows ? item_row_limit(v, tid) : v.kv_end;
        if (fused && v.writes_kv) {
            for (uint32_t i = tid; i < v.num_tokens * 2 * kChunks; i += kThreads) {
                const uint32_t c = i % kChunks, which = (i / kChunks) & 1, j = i / (2 * kChunks);
                const uint32_t pos = v.first_pos + j;
                uint32_t write_id = 0;
                if (pos >= v.kv_begin && pos < v.kv_end && checked_page_id(p.geo, row_ids, pos >> page_shift, write_id)) {
                    const unsigned char* fresh = static_cast<const unsigned char*>(which ? p.new_v : p.new_k);
                    const uint4 value = *reinterpret_cast<const uint4*>(
                        fresh + (static_cast<uint64_t>(v.flat_begin + j) * p.geo.num_kv_heads + v.kv_head) * L::kRowBytes + c * 16);
                    unsigned char* dst = const_cast<unsigned char*>(pages) +
                                         static_cast<uint64_t>(write_id) * page_bytes + head_bytes +
                                         (which ? v_region_bytes : 0) + (pos & page_mask) * L::kRowBytes + c * 16;
                    *reinterpret_cast<uint4*>(dst) = value;
                }
            }
        }
        cp_async_wait<NSLOT - 1>();  // the query rows (the oldest group) have landed; the K/V tiles stay in flight
        __syncthreads();

        const uint32_t limit0 = limit_s[quad_row], limit1 = limit_s[quad_row + 8];
        uint32_t limit_min = v.kv_end;
        for (uint32_t r = 0; r < v.rows; ++r) limit_min = min(limit_min, limit_s[r]);

        uint32_t pa[4];
        for (uint32_t h = 0; h < my_halves; ++h) {
            cp_async_wait<NSLOT - 2>();
            __syncwarp();
            if (kTma) {
                const uint32_t s = h % NSLOT;
                if ((tma_bits >> s) & 1u) {
                    const uint32_t bar = smem_u32(&ring_bar_s[kTma ? warp : 0][kTma ? s : 0]);
                    const uint32_t parity = (phase_bits >> s) & 1u;
                    if (ring_ok && !mbar_test(bar, parity) && !mbar_wait(bar, parity)) {
                        ring_ok = false;  // the box never arrived: report it and stop waiting (the results are not valid)
                        if (lane == 0 && p.status != nullptr) atomicExch(p.status, static_cast<uint32_t>(PSI_ERR_TIMEOUT));
                    }
                    phase_bits ^= 1u << s;
                }
            }
            const uint32_t ahead = h + NSLOT - 1;
            if (ahead < my_halves) {
                issue(ahead, ahead % NSLOT, cur_lo, cur_hi);
                if (ahead & 1) {
                    cur_lo = next_lo;
                    cur_hi = next_hi;
                    if ((ahead >> 1) + 2 < my_tiles) lookup((ahead >> 1) + 2, next_lo, next_hi);
                }
            }
            cp_async_commit();

            const uint32_t slot_base = ring_base + (h % NSLOT) * L::kTileBytes;
            if ((h & 1) == 0) {
                const uint32_t token0 = tile_of(h >> 1) * kTile;
                const bool masked = token0 < v.kv_begin || token0 + kTile > limit_min;
                TileMath<T, D, kTma>::scores(frag, q_base, slot_base, p.scale_log2, masked, token0, limit0, limit1,
                                             v.kv_begin, st, pa);
            } else {
                TileMath<T, D, kTma>::values(frag, slot_base, pa, st);
            }
        }

        // ---- merge the warps' partial results --------------------------------------------------------------------------
        const bool is_partial = v.partial_slot != kU32Max;
        cp_async_wait<0>();
        if (kExchange && index == item_begin && tid == 0) slot_free_s = slot_is_free(p.xchg, consumed_early) ? 1u : 0u;
        __syncthreads();  // every warp is done with its ring: the merge buffer may overwrite it
        st.l0 += __shfl_xor_sync(0xFFFFFFFFu, st.l0, 1);
        st.l0 += __shfl_xor_sync(0xFFFFFFFFu, st.l0, 2);
        st.l1 += __shfl_xor_sync(0xFFFFFFFFu, st.l1, 1);
        st.l1 += __shfl_xor_sync(0xFFFFFFFFu, st.l1, 2);
        if (quad_col == 0) {
            merge_m[warp][quad_row] = st.m0;
            merge_m[warp][quad_row + 8] = st.m1;
            merge_l[warp][quad_row] = st.l0;
            merge_l[warp][quad_row + 8] = st.l1;
        }
        {
            // Rows 8..15 are padding when the item carries at most eight query rows (decode rows of a GQA group of
            // eight): the merge below never reads them, so they are not written.
            float* mine = merge_o + warp * kTile * L::kMergeStride + 2 * quad_col;
#pragma unroll
            for (int j = 0; j < D / 8; ++j)
                *reinterpret_cast<float2*>(mine + quad_row * L::kMergeStride + 8 * j) = make_float2(st.o[j][0], st.o[j][1]);
            if (v.rows > 8) {
#pragma unroll
                for (int j = 0; j < D / 8; ++j)
                    *reinterpret_cast<float2*>(mine + (quad_row + 8) * L::kMergeStride + 8 * j) = make_float2(st.o[j][2], st.o[j][3]);
            }
        }
        __syncthreads();

        for (uint32_t i = tid; i < v.rows * (D / 4); i += kThreads) {
            const uint32_t r = i / (D / 4), c4 = i % (D / 4);
            float row_max = -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) row_max = fmaxf(row_max, merge_m[w][r]);
            float sum = 0.0f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float wm = merge_m[w][r];
                const float weight = wm == -INFINITY ? 0.0f : exp2f(wm - row_max);
                sum += weight * merge_l[w][r];
                const float4 part =
                    *reinterpret_cast<const float4*>(merge_o + (w * kTile + r) * L::kMergeStride + 4 * c4);
                acc.x += weight * part.x;
                acc.y += weight * part.y;
                acc.z += weight * part.z;
                acc.w += weight * part.w;
            }
            const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
            acc.x *= inv;
            acc.y *= inv;
            acc.z *= inv;
            acc.w *= inv;
            if (is_partial) {
                const uint64_t prow = static_cast<uint64_t>(v.partial_slot) * kMaxRows + r;
                *reinterpret_cast<float4*>(p.partial_o + prow * D + 4 * c4) = acc;
                if (c4 == 0) {
                    p.partial_m[prow] = row_max;
                    p.partial_l[prow] = sum;
                }
            } else {
                const uint64_t row = item_row_index(p, v, r);
                if (kExchange && !slot_free_s) {
                    // the slot still holds a step the owner has not merged: nothing is stored, the flag stays back
                } else if (p.ext_o != nullptr) {
                    *reinterpret_cast<float4*>(p.ext_o + row * D + 4 * c4) = acc;
                    if (c4 == 0) {
                        p.ext_m[row] = row_max * kLn2;
                        p.ext_l[row] = sum;
                    }
                } else {
                    store_out4<T>(p, row * D + 4 * c4, acc);
                }
            }
        }

        // ---- the CTA that delivers a unit's last partial merges the unit -------------------------------------------------
        if (is_partial) {
            // The barrier orders every thread's partial stores before thread 0's fence, and the fence (cumulative)
            // makes them visible device-wide before the arrival is counted; the second fence orders the count before
            // the reads of the other pieces' partials that follow the next barrier.
            __syncthreads();
            if (tid == 0) {
                __threadfence();
                arrival_s = atomicAdd(p.unit_counters + v.reduce_unit, 1u);
                __threadfence();
            }
            __syncthreads();
            if (arrival_s == v.unit_num_items - 1) {
                // Every thread merges its own outputs (row r, four columns in each half of the row) from all pieces:
                // the pieces' statistics of row r and their O values go out together, four pieces at a time, so a
                // unit of up to four pieces and eight rows costs every thread one round trip.  The two column groups
                // are half a row apart, which keeps each store instruction of a warp contiguous (the output may be a
                // buffer in host memory, where partly written lines cross the host link one by one).
                const uint32_t n = v.unit_num_items, rows = v.rows;
                constexpr uint32_t kHalf = D / 8;  // float4 columns per half row
                for (uint32_t i = tid; i < rows * kHalf; i += kThreads) {
                    const uint32_t r = i / kHalf, c4 = i % kHalf;
                    const uint64_t prow0 = static_cast<uint64_t>(v.unit_first_slot) * kMaxRows + r;
                    float run_max = -INFINITY, sum = 0.0f;
                    float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
                    for (uint32_t s0 = 0; s0 < n; s0 += 4) {
                        float pm[4], pl[4];
                        float4 part0[4], part1[4];
#pragma unroll
                        for (uint32_t k = 0; k < 4; ++k) {
                            const uint64_t prow = prow0 + static_cast<uint64_t>(min(s0 + k, n - 1)) * kMaxRows;
                            pm[k] = __ldcg(p.partial_m + prow);
                            pl[k] = __ldcg(p.partial_l + prow);
                            const float4* src = reinterpret_cast<const float4*>(p.partial_o + prow * D) + c4;
                            part0[k] = __ldcg(src);
                            part1[k] = __ldcg(src + kHalf);
                        }
                        float group_max = run_max;
#pragma unroll
                        for (uint32_t k = 0; k < 4; ++k)
                            if (s0 + k < n) group_max = fmaxf(group_max, pm[k]);
                        const float carry = run_max == -INFINITY ? 0.0f : exp2f(run_max - group_max);
                        sum *= carry;
                        acc0.x *= carry;
                        acc0.y *= carry;
                        acc0.z *= carry;
                        acc0.w *= carry;
                        acc1.x *= carry;
                        acc1.y *= carry;
                        acc1.z *= carry;
                        acc1.w *= carry;
#pragma unroll
                        for (uint32_t k = 0; k < 4; ++k) {
                            const float weight =
                                (s0 + k < n && pm[k] != -INFINITY) ? exp2f(pm[k] - group_max) * pl[k] : 0.0f;
                            sum += weight;
                            acc0.x += weight * part0[k].x;
                            acc0.y += weight * part0[k].y;
                            acc0.z += weight * part0[k].z;
                            acc0.w += weight * part0[k].w;
                            acc1.x += weight * part1[k].x;
                            acc1.y += weight * part1[k].y;
                            acc1.z += weight * part1[k].z;
                            acc1.w += weight * part1[k].w;
                        }
                        run_max = group_max;
                    }
                    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
                    acc0.x *= inv;
                    acc0.y *= inv;
                    acc0.z *= inv;
                    acc0.w *= inv;
                    acc1.x *= inv;
                    acc1.y *= inv;
                    acc1.z *= inv;
                    acc1.w *= inv;
                    const uint64_t row = item_row_index(p, v, r);
                    if (kExchange && !slot_free_s) {
                        // as above: no store into a slot that is not free
                    } else if (p.ext_o != nullptr) {
                        *reinterpret_cast<float4*>(p.ext_o + row * D + 4 * c4) = acc0;
                        *reinterpret_cast<float4*>(p.ext_o + row * D + 4 * (c4 + kHalf)) = acc1;
                        if (c4 == 0) {
                            p.ext_m[row] = run_max * kLn2;
                            p.ext_l[row] = sum;
                        }
                    } else {
                        store_out4<T>(p, row * D + 4 * c4, acc0);
                        store_out4<T>(p, row * D + 4 * (c4 + kHalf), acc1);
                    }
                }
                if (tid == 0) p.unit_counters[v.reduce_unit] = 0;  // ready for the next launch
            }
        }
    }
    if (bad_page != 0) record_page_fault(p.geo);
    if (kExchange) {
        exchange_publish(p.xchg, p.status, num_ctas, item_begin < item_end && slot_free_s == 0);
        if (p.xchg.recv != nullptr) exchange_merge<kThreads>(p.xchg, p.status, p.out, p.dtype, D, cta, num_ctas);
    }
}

template <int D>
constexpr int stages_for() {
    return D == 256 ? 3 : (D == 128 ? 6 : 8);  // ring slots (one K or V tile each) per warp
}

template <typename T, int D, bool kExchange, bool kTma>
cudaError_t launch_one(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream, const CUtensorMap& map,
                       uint32_t box_rows) {
    constexpr int NSLOT = stages_for<D>();
    using L = SmemLayout<D, NSLOT>;
    auto kernel = attend_mma_kernel<T, D, NSLOT, kExchange, kTma>;
    static std::atomic<uint64_t> configured{0};  // per instantiation, one bit per device
    cudaError_t err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), static_cast<int>(L::kTotal), configured);
    if (err != cudaSuccess) return err;
    kernel<<<num_ctas, kThreads, L::kTotal, stream>>>(p, map, box_rows);
    return cudaGetLastError();
}

template <typename T, bool kExchange>
cudaError_t launch_for_dim(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    // The TMA feed when the component asks for it and the arena can be described to the TMA unit (page count known,
    // alignment); otherwise, and for the exchange launches, the cp.async feed.
    CUtensorMap map{};
    const uint32_t box_rows = p.geo.tokens_per_page < static_cast<uint32_t>(kTile) ? p.geo.tokens_per_page : kTile;
    const bool tma = !kExchange && p.tma_feed != 0 && make_kv_map(p, box_rows, &map);
    if (tma) {
        if constexpr (!kExchange) {
            switch (p.geo.head_dim) {
                case 64: return launch_one<T, 64, false, true>(p, num_ctas, stream, map, box_rows);
                case 128: return launch_one<T, 128, false, true>(p, num_ctas, stream, map, box_rows);
                case 256: return launch_one<T, 256, false, true>(p, num_ctas, stream, map, box_rows);
                default: return cudaErrorInvalidValue;
            }
        }
    }
    switch (p.geo.head_dim) {
        case 64: return launch_one<T, 64, kExchange, false>(p, num_ctas, stream, map, box_rows);
        case 128: return launch_one<T, 128, kExchange, false>(p, num_ctas, stream, map, box_rows);
        case 256: return launch_one<T, 256, kExchange, false>(p, num_ctas, stream, map, box_rows);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

bool attend_mma_supported(uint32_t dtype, uint32_t head_dim, uint32_t tokens_per_page) {
    const bool dtype_ok = dtype == PSI_DTYPE_BF16 || dtype == PSI_DTYPE_F16;
    const bool dim_ok = head_dim == 64 || head_dim == 128 || head_dim == 256;
    const bool page_ok = tokens_per_page >= 8 && (tokens_per_page & (tokens_per_page - 1)) == 0;
    return dtype_ok && dim_ok && page_ok;
}

uint32_t attend_mma_ctas_per_sm(uint32_t /*head_dim*/) { return 1; }


cudaError_t launch_attend_mma(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    if (num_ctas == 0) return cudaSuccess;
    if ((reinterpret_cast<uintptr_t>(p.q) & 15u) != 0 || (reinterpret_cast<uintptr_t>(p.geo.pages) & 15u) != 0 ||
        (p.out != nullptr && (reinterpret_cast<uintptr_t>(p.out) & 7u) != 0)) {
        return cudaErrorMisalignedAddress;
    }
    if (p.xchg.flag != nullptr) {
        if (p.ext_o == nullptr || p.xchg.sync_words == nullptr || p.xchg.consumed == nullptr) return cudaErrorInvalidValue;
        return p.dtype == PSI_DTYPE_BF16 ? launch_for_dim<__nv_bfloat16, true>(p, num_ctas, stream)
                                         : launch_for_dim<__half, true>(p, num_ctas, stream);
    }
    return p.dtype == PSI_DTYPE_BF16 ? launch_for_dim<__nv_bfloat16, false>(p, num_ctas, stream)
                                     : launch_for_dim<__half, false>(p, num_ctas, stream);
}

}  // namespace psi
