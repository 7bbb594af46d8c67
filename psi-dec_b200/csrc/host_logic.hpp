// Host-side policy of the paged GQA decode path: replay buckets, SplitKV variant selection, the reference-format
// batch metadata, the device work plan and the page-ID allocator.  Pure C++ (no CUDA), shared by the C ABI.
#pragma once

#include <cstdint>
#include <deque>
#include <stdexcept>
#include <string>
#include <vector>

#include "psi_cuda.h"

namespace psi {

// A violated caller contract (the reference panics); mapped to PSI_ERR_INVALID_ARGUMENT at the C ABI.
struct ContractError : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct ExhaustedError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

inline void require(bool ok, const char* message) {
    if (!ok) throw ContractError(message);
}

constexpr uint32_t kU32Max = 0xFFFFFFFFu;
constexpr uint32_t kKvTile = 16;    // KV tokens per device work tile
constexpr uint32_t kMaxRows = 16;   // query rows (tokens x heads) one work item carries

inline uint32_t dtype_bytes(uint32_t dtype) { return dtype == PSI_DTYPE_F32 ? 4u : 2u; }

// ---- replay buckets (crates/inference-executor-core/src/replay.rs) ------------------------------------------------
class BucketPolicy {
public:
    BucketPolicy(uint32_t max_capacity, const std::vector<uint32_t>& topology_boundaries);
    const std::vector<uint32_t>& buckets() const { return buckets_; }
    uint32_t max_capacity() const { return max_capacity_; }
    uint32_t capacity(uint32_t active) const;

private:
    uint32_t max_capacity_;
    std::vector<uint32_t> buckets_;
};

// ---- SplitKV variant selector (crates/inference-backend-metal/src/components/gqa_split_kv.rs) ---------------------
class SplitKvSelector {
public:
    SplitKvSelector(uint32_t io_dtype, uint32_t page_bytes, uint32_t num_q_heads, uint32_t num_kv_heads,
                    uint32_t head_dim, bool dspark_history);
    psi_split_kv_variant select(uint32_t num_tokens, uint32_t num_q_token_tiles) const;
    uint32_t tiled_q_token_tile_size() const { return 8; }
    uint32_t max_q_tokens_per_partial_output() const { return supports_tiled_ ? 8u : 1u; }
    uint32_t tokens_per_page() const { return tokens_per_page_; }

private:
    uint32_t group_;
    uint32_t tokens_per_page_;
    bool supports_tiled_;
    bool full_group_for_tiled_;
    uint32_t single_threads_;
};

// ---- reference-format batch metadata (crates/inference-executor-metal/src/attn/gqa/batch_metadata.rs) -------------
struct ReferenceMetadata {
    // Capacity-sized host mirrors; only the prefixes the reference writes are touched by update().
    std::vector<uint32_t> req_slots, flat_token_indices, q_token_tiles, kv_splits, cu_kv_splits;
    explicit ReferenceMetadata(uint32_t max_tokens);
    uint32_t max_tokens() const { return static_cast<uint32_t>(req_slots.size()); }
    // The per-token arrays alone (request slot and request-absolute position of every query token), with update()'s
    // checks of the batch; returns the token count.  What a launch needs when no reference-format split plan is asked for.
    uint32_t expand_tokens(const uint32_t* req_slots_by_req, const uint32_t* token_indices, const uint32_t* cu_tokens,
                           uint32_t num_reqs);
    psi_replay_shape update(const uint32_t* req_slots_by_req, const uint32_t* token_indices, const uint32_t* cu_tokens,
                            uint32_t num_reqs, const psi_split_kv_variant& variant, uint32_t capacity_mode,
                            const std::vector<uint32_t>& token_topology_boundaries, uint32_t caller_num_total_tokens);
};

// ---- device work plan ------------------------------------------------------------------------------------------------
// One query tile the kernels execute: consecutive flat tokens of one request, at most tokens_per_tile of them.
struct ExecTile {
    uint32_t flat_begin;
    uint32_t flat_end;
    uint32_t req_slot;
    uint32_t first_pos;       // request-absolute position of the tile's first token
    uint32_t new_begin;       // request-absolute position of the request's first token of this step
    uint32_t flat_req_begin;  // flat index of that token
};

// One unit of map work while the plan is being built: the rows of (tile, head_sel) against KV tokens
// [kv_begin, kv_end).
struct WorkItem {
    uint32_t tile;
    uint32_t head_sel;      // kv_head * head_tiles + head_tile
    uint32_t kv_begin;
    uint32_t kv_end;
    uint32_t partial_slot;  // kU32Max: the item covers its unit alone and writes the final output itself
    uint32_t reduce_unit;   // index into the plan's reduce list when partial_slot is set
    uint32_t unit_first_slot;  // partial slot of the unit's first item (slots of one unit are consecutive)
    uint32_t unit_num_items;   // items that share the unit
};

// The same item as the kernels read it: self-contained, 64 bytes, no further indirection.
struct DeviceItem {
    uint32_t kv_begin;
    uint32_t kv_end;
    uint32_t partial_slot;
    uint32_t reduce_unit;
    uint32_t unit_first_slot;
    uint32_t unit_num_items;
    uint32_t flat_begin;      // first flat query token of the tile
    uint32_t num_tokens;      // query tokens in the tile
    uint32_t req_slot;
    uint32_t kv_head;
    uint32_t head0;           // first q head the item carries
    uint32_t num_heads;       // q heads the item carries; row r = (token r / num_heads, head r % num_heads)
    uint32_t first_pos;       // position of the tile's first token: token j sees keys [0, first_pos + j]
    uint32_t new_begin;       // positions at or beyond this belong to this step's appended tokens
    uint32_t flat_req_begin;  // flat index of the token at position new_begin
    uint32_t writes_kv;       // 1: the item appends its tile's K/V rows that fall into its KV range (fused step)
};
static_assert(sizeof(DeviceItem) == 64, "DeviceItem is read as four 16-byte words");

struct ReduceUnit {
    uint32_t first_item;
    uint32_t num_items;
};

struct PlanGeometry {
    uint32_t group;            // q heads per kv head
    uint32_t heads_per_tile;   // q heads of one group one item carries (<= 16)
    uint32_t head_tiles;       // ceil(group / heads_per_tile)
    uint32_t tokens_per_tile;  // query tokens one item carries
    uint32_t num_kv_heads;
};

PlanGeometry plan_geometry(uint32_t num_q_heads, uint32_t num_kv_heads);

struct WorkPlan {
    std::vector<ExecTile> tiles;
    std::vector<WorkItem> items;
    std::vector<uint32_t> cta_item_begin;  // [num_ctas + 1]
    std::vector<ReduceUnit> reduces;
    uint32_t num_partial_slots = 0;
    uint64_t total_kv_tiles = 0;
    uint32_t num_ctas() const { return cta_item_begin.empty() ? 0u : static_cast<uint32_t>(cta_item_begin.size() - 1); }
};

// Equal-share plan: the (tile, head_sel) units laid end to end in 16-token KV tiles, cut into `max_ctas` (or fewer)
// contiguous shares.  `item_start_cost` (in KV tiles) is what opening one more item costs a CTA; shares are equal in
// KV tiles plus that cost per unit start.
WorkPlan build_balanced_plan(const PlanGeometry& geo, const uint32_t* req_slots, const uint32_t* token_indices,
                             const uint32_t* cu_tokens, uint32_t num_reqs, uint32_t max_ctas,
                             uint32_t min_kv_tiles_per_cta, uint32_t item_start_cost = 0);
// The same over a subset of the batch's requests (indices into the request arrays, ascending).
WorkPlan build_balanced_plan(const PlanGeometry& geo, const uint32_t* req_slots, const uint32_t* token_indices,
                             const uint32_t* cu_tokens, const std::vector<uint32_t>& requests, uint32_t max_ctas,
                             uint32_t min_kv_tiles_per_cta, uint32_t item_start_cost = 0);

// One CTA per (reference KV split, head_sel); reference q tiles wider than tokens_per_tile are cut into sub-tiles
// that share the split boundaries.
WorkPlan build_reference_plan(const PlanGeometry& geo, const ReferenceMetadata& md, const psi_replay_shape& shape,
                              bool tiled_q, const uint32_t* token_indices, const uint32_t* cu_tokens,
                              uint32_t num_reqs);

// Plan of the long-query (chunk) kernel: items are super-tiles of up to eight consecutive query tiles of one request
// and KV head; the warp w of a CTA owns tile w of the super-tile, its partial slot is `partial_slot + w` and its arrival
// counter `reduce_unit + w`; the slots of one unit lie 8 apart (`unit_first_slot + ordinal * 8 + w`).
struct ChunkPlan {
    std::vector<DeviceItem> items;
    std::vector<uint32_t> cta_item_begin;
    uint32_t num_partial_slots = 0;   // slots used beyond slot_base
    uint32_t num_counters = 0;        // counters used beyond counter_base
    uint64_t total_kv_tiles = 0;
    uint32_t num_ctas() const { return cta_item_begin.empty() ? 0u : static_cast<uint32_t>(cta_item_begin.size() - 1); }
};
constexpr uint32_t kChunkTilesPerItem = 8;  // one query tile per warp
constexpr uint32_t kChunkMinPieceTiles = 64;   // a KV piece of a cut unit is at least this many 16-token tiles
constexpr uint32_t kChunkStartCostTiles = 8;   // fixed cost of a work item (query load, epilogue) in KV tiles

// `equal_shares`: contiguous shares of exactly equal size (for working sets that stay in L2 in any order); otherwise
// units are dealt whole, in stream order, to the CTA that is free first, and only long units are cut.
ChunkPlan build_chunk_plan(const PlanGeometry& geo, const uint32_t* req_slots, const uint32_t* token_indices,
                           const uint32_t* cu_tokens, const std::vector<uint32_t>& requests, uint32_t max_ctas,
                           uint32_t slot_base, uint32_t counter_base, bool equal_shares = false);

// Device form of a finished plan.
std::vector<DeviceItem> flatten_plan(const WorkPlan& plan, const PlanGeometry& geo);

// ---- RoPE parameters (crates/inference-backend-metal/src/components/rms_norm_rope.rs:126-230) ---------------------
struct RopeParameters {
    std::vector<float> inverse_frequencies;  // rope_dim / 2
    float attention_factor = 1.0f;
    float correction_low = 0.0f, correction_high = 0.0f;  // Yarn only
};
RopeParameters rope_parameters(const psi_norm_rope_config& config);

// ---- page-ID allocator (crates/inference-runtime-core/src/memory/u32_id_allocator.rs) --------------------------------
class IdAllocator {
public:
    explicit IdAllocator(uint64_t capacity);
    void alloc_many(uint64_t count, uint32_t* out);
    void free_many(const uint32_t* ids, uint64_t count);
    const std::vector<uint64_t>& bitmap() const { return bitmap_; }
    uint64_t free_count() const { return free_ids_.size() + (capacity_ - counter_); }

private:
    void mark(uint32_t id, bool live);
    uint64_t capacity_;
    uint64_t counter_ = 0;
    std::deque<uint32_t> free_ids_;
    std::vector<uint64_t> bitmap_;
};

}  // namespace psi
