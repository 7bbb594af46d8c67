// C ABI: host-side policy objects (replay buckets, variant selector, reference metadata, plan previews).
#include "api_internal.hpp"

using namespace psi;

extern "C" {

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

}  // extern "C"
