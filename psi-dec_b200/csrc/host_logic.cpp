#include "host_logic.hpp"

#include <algorithm>
#include <cmath>
#include <limits>
#include <queue>

namespace psi {

namespace {
uint64_t div_ceil(uint64_t a, uint64_t b) { return (a + b - 1) / b; }
uint32_t sat_u32(uint64_t v) { return v > kU32Max ? kU32Max : static_cast<uint32_t>(v); }
}  // namespace

// -------------------------------------------------------------------------------------------------------------------
// Replay buckets.  Base list up to 64, then four equal steps per octave, plus `boundary - 1` for each topology
// boundary and the terminal capacity (crates/inference-executor-core/src/replay.rs:25-44,69-90).
// -------------------------------------------------------------------------------------------------------------------
BucketPolicy::BucketPolicy(uint32_t max_capacity, const std::vector<uint32_t>& topology_boundaries)
    : max_capacity_(max_capacity) {
    require(max_capacity > 0, "replay bucket capacity must be positive");
    for (uint32_t b : {1u, 2u, 4u, 6u, 8u, 12u, 16u, 20u, 24u, 32u, 40u, 48u, 56u, 64u}) {
        if (b <= max_capacity) buckets_.push_back(b);
    }
    bool open = true;
    for (uint32_t octave = 64; open && octave < max_capacity; octave = sat_u32(uint64_t(octave) * 2)) {
        for (uint32_t quarter = 1; quarter <= 4; ++quarter) {
            uint32_t candidate = sat_u32(uint64_t(octave) + uint64_t(octave / 4) * quarter);
            if (candidate >= max_capacity) {
                open = false;
                break;
            }
            buckets_.push_back(candidate);
        }
    }
    for (uint32_t boundary : topology_boundaries) {
        require(boundary > 0, "replay topology boundary must be positive");
        if (boundary > 1 && boundary <= max_capacity) buckets_.push_back(boundary - 1);
    }
    buckets_.push_back(max_capacity);
    std::sort(buckets_.begin(), buckets_.end());
    buckets_.erase(std::unique(buckets_.begin(), buckets_.end()), buckets_.end());
}

uint32_t BucketPolicy::capacity(uint32_t active) const {
    require(active > 0, "replay bucket requires active work");
    require(active <= max_capacity_, "replay active work exceeds capacity");
    return *std::lower_bound(buckets_.begin(), buckets_.end(), active);
}

// -------------------------------------------------------------------------------------------------------------------
// Variant selector (crates/inference-backend-metal/src/components/gqa_split_kv.rs:29-157).
// -------------------------------------------------------------------------------------------------------------------
SplitKvSelector::SplitKvSelector(uint32_t io_dtype, uint32_t page_bytes, uint32_t num_q_heads, uint32_t num_kv_heads,
                                 uint32_t head_dim, bool dspark_history) {
    require(io_dtype == PSI_DTYPE_F32 || io_dtype == PSI_DTYPE_BF16, "GQA SplitKV io_dtype must be f32 or bf16");
    require(page_bytes > 0 && num_q_heads > 0 && num_kv_heads > 0 && head_dim > 0, "GQA SplitKV config must be positive");
    require(num_q_heads % num_kv_heads == 0, "GQA q heads must be a multiple of kv heads");
    uint64_t per_token = uint64_t(num_kv_heads) * head_dim * 2u * dtype_bytes(io_dtype);
    require(per_token <= kU32Max, "GQA K/V bytes per token must fit u32");
    require(page_bytes % per_token == 0, "GQA page_bytes must be divisible by the K/V bytes per token");
    tokens_per_page_ = page_bytes / static_cast<uint32_t>(per_token);
    group_ = num_q_heads / num_kv_heads;
    bool profile = (head_dim == 128 && tokens_per_page_ == 8) ||
                   (head_dim == 256 && (tokens_per_page_ == 8 || tokens_per_page_ == 16));
    supports_tiled_ = !dspark_history && io_dtype == PSI_DTYPE_BF16 && profile && group_ <= 8;
    full_group_for_tiled_ = !dspark_history && head_dim == 128 && tokens_per_page_ == 8;
    uint32_t bounded = std::max(32u, std::min(head_dim, 256u));
    single_threads_ = 1;
    while (single_threads_ < bounded) single_threads_ <<= 1;
}

psi_split_kv_variant SplitKvSelector::select(uint32_t num_tokens, uint32_t num_q_token_tiles) const {
    require(num_tokens > 0, "GQA SplitKV selection requires tokens");
    require(num_q_token_tiles > 0 && num_q_token_tiles <= num_tokens, "GQA SplitKV q-token-tile count out of range");
    const uint32_t max_head_tile = 256 / (tiled_q_token_tile_size() / 8 * 32);
    psi_split_kv_variant v{};
    if (!supports_tiled_ || uint64_t(num_tokens) < 2ull * num_q_token_tiles) {
        v.tiled_q = 0;
        v.kv_token_tile_size = single_threads_;
        v.num_threads_per_threadblock = single_threads_;
        v.q_head_tile_size = std::min(group_, max_head_tile);
        return v;
    }
    bool halve = !full_group_for_tiled_ && uint64_t(num_tokens) < 4ull * num_q_token_tiles;
    v.tiled_q = 1;
    v.q_token_tile_size = tiled_q_token_tile_size();
    v.kv_token_tile_size = 16;
    v.q_head_tile_size = std::min(halve ? (group_ + 1) / 2 : group_, max_head_tile);
    return v;
}

// -------------------------------------------------------------------------------------------------------------------
// Reference-format metadata (crates/inference-executor-metal/src/attn/gqa/batch_metadata.rs:192-523).
// -------------------------------------------------------------------------------------------------------------------
ReferenceMetadata::ReferenceMetadata(uint32_t max_tokens)
    : req_slots(max_tokens, 0), flat_token_indices(max_tokens, 0), q_token_tiles(size_t(max_tokens) * 2, 0),
      kv_splits(size_t(max_tokens) * 3, 0), cu_kv_splits(size_t(max_tokens) + 1, 0) {
    require(max_tokens > 0, "GQA batch metadata requires tokens");
}

namespace {

struct SplitCandidateTile {
    uint32_t flat_begin, flat_end, context_len;
    uint64_t kv_tiles;
    uint64_t splits = 1;
};

// Greedy refinement shared by both reference planners: while budget remains, give one more split to the tile whose
// splits are currently the longest (first such tile wins ties), batch_metadata.rs:370-386,466-488.
void refine_splits(std::vector<SplitCandidateTile>& tiles, uint64_t used, uint64_t budget, bool charge_tokens) {
    while (used < budget) {
        int64_t best = -1;
        uint64_t best_len = 0;
        for (size_t i = 0; i < tiles.size(); ++i) {
            const auto& t = tiles[i];
            uint64_t cost = charge_tokens ? t.flat_end - t.flat_begin : 1;
            if (used + cost > budget || t.splits >= t.kv_tiles) continue;
            uint64_t len = div_ceil(t.kv_tiles, t.splits);
            if (best < 0 || len > best_len) {
                best = static_cast<int64_t>(i);
                best_len = len;
            }
        }
        if (best < 0) break;
        used += charge_tokens ? tiles[best].flat_end - tiles[best].flat_begin : 1;
        tiles[best].splits += 1;
    }
}

}  // namespace

uint32_t ReferenceMetadata::expand_tokens(const uint32_t* req_slots_by_req, const uint32_t* token_indices,
                                          const uint32_t* cu_tokens, uint32_t num_reqs) {
    require(num_reqs > 0, "GQA batch metadata requires tokens");
    require(cu_tokens[0] == 0, "GQA batch cu_tokens must start at zero");
    for (uint32_t r = 0; r < num_reqs; ++r) {
        require(cu_tokens[r] <= cu_tokens[r + 1], "GQA batch cu_tokens must be nondecreasing");
        require(uint64_t(token_indices[r]) + (cu_tokens[r + 1] - cu_tokens[r]) <= kU32Max,
                "GQA request context length must fit u32");
    }
    const uint32_t num_tokens = cu_tokens[num_reqs];
    require(num_tokens > 0, "GQA batch metadata requires tokens");
    require(num_tokens <= max_tokens(), "GQA batch exceeds the metadata token capacity");
    for (uint32_t r = 0, t = 0; r < num_reqs; ++r) {
        for (uint32_t i = 0; i < cu_tokens[r + 1] - cu_tokens[r]; ++i, ++t) {
            req_slots[t] = req_slots_by_req[r];
            flat_token_indices[t] = token_indices[r] + i;
        }
    }
    return num_tokens;
}

psi_replay_shape ReferenceMetadata::update(const uint32_t* req_slots_by_req, const uint32_t* token_indices,
                                           const uint32_t* cu_tokens, uint32_t num_reqs,
                                           const psi_split_kv_variant& variant, uint32_t capacity_mode,
                                           const std::vector<uint32_t>& token_topology_boundaries,
                                           uint32_t caller_num_total_tokens) {
    require(num_reqs > 0, "GQA batch metadata requires tokens");
    require(cu_tokens[0] == 0, "GQA batch cu_tokens must start at zero");
    for (uint32_t r = 0; r < num_reqs; ++r) {
        require(cu_tokens[r] <= cu_tokens[r + 1], "GQA batch cu_tokens must be nondecreasing");
        require(uint64_t(token_indices[r]) + (cu_tokens[r + 1] - cu_tokens[r]) <= kU32Max,
                "GQA request context length must fit u32");
    }
    const uint32_t num_tokens = cu_tokens[num_reqs];
    require(num_tokens > 0, "GQA batch metadata requires tokens");
    require(num_tokens <= max_tokens(), "GQA batch exceeds the metadata token capacity");
    if (capacity_mode == PSI_CAPACITY_CALLER_TOKENS) {
        require(num_tokens <= caller_num_total_tokens,
                "GQA active token count must not exceed the caller-owned token capacity");
        require(caller_num_total_tokens <= max_tokens(),
                "GQA caller-owned token capacity must not exceed the metadata capacity");
    }
    for (uint32_t r = 0, t = 0; r < num_reqs; ++r) {
        for (uint32_t i = 0; i < cu_tokens[r + 1] - cu_tokens[r]; ++i, ++t) {
            req_slots[t] = req_slots_by_req[r];
            flat_token_indices[t] = token_indices[r] + i;
        }
    }

    const bool tiled = variant.tiled_q != 0;
    require(variant.kv_token_tile_size > 0, "GQA KV-token tile size must be positive");
    std::vector<SplitCandidateTile> tiles;
    if (!tiled) {
        tiles.reserve(num_tokens);
        for (uint32_t t = 0; t < num_tokens; ++t) {
            uint32_t ctx = flat_token_indices[t] + 1;
            tiles.push_back({t, t + 1, ctx, div_ceil(ctx, variant.kv_token_tile_size)});
        }
        refine_splits(tiles, num_tokens, max_tokens(), /*charge_tokens=*/false);
    } else {
        require(variant.q_token_tile_size > 0, "GQA Q-token tile size must be positive");
        for (uint32_t r = 0; r < num_reqs; ++r) {
            for (uint32_t begin = cu_tokens[r]; begin < cu_tokens[r + 1];) {
                uint32_t end = std::min(cu_tokens[r + 1], begin + variant.q_token_tile_size);
                uint32_t ctx = token_indices[r] + (end - cu_tokens[r]);
                tiles.push_back({begin, end, ctx, div_ceil(ctx, variant.kv_token_tile_size)});
                begin = end;
            }
        }
        refine_splits(tiles, num_tokens, max_tokens(), /*charge_tokens=*/true);
    }

    std::vector<uint32_t> splits, cu{0};
    for (size_t i = 0; i < tiles.size(); ++i) {
        const auto& t = tiles[i];
        for (uint64_t s = 0; s < t.splits; ++s) {
            uint64_t begin = t.kv_tiles * s / t.splits * variant.kv_token_tile_size;
            uint64_t end = t.kv_tiles * (s + 1) / t.splits * variant.kv_token_tile_size;
            require(begin <= kU32Max, "GQA map KV split KV-token begin must fit u32");
            splits.push_back(static_cast<uint32_t>(i));
            splits.push_back(static_cast<uint32_t>(begin));
            splits.push_back(static_cast<uint32_t>(std::min<uint64_t>(end, t.context_len)));
        }
        cu.push_back(static_cast<uint32_t>(splits.size() / 3));
    }
    const uint32_t num_tiles = static_cast<uint32_t>(tiles.size());
    const uint32_t num_splits = static_cast<uint32_t>(splits.size() / 3);

    uint32_t total_tokens = num_tokens, total_tiles = num_tiles, total_splits = 0;
    if (capacity_mode == PSI_CAPACITY_EXACT) {
        uint64_t pow2 = 1;
        while (pow2 < num_splits) pow2 <<= 1;
        total_splits = static_cast<uint32_t>(std::min<uint64_t>(pow2, max_tokens()));
    } else {
        BucketPolicy plain(max_tokens(), {});
        total_tiles = plain.capacity(num_tiles);
        total_splits = plain.capacity(num_splits);
        total_tokens = capacity_mode == PSI_CAPACITY_BUCKETED
                           ? BucketPolicy(max_tokens(), token_topology_boundaries).capacity(num_tokens)
                           : caller_num_total_tokens;
    }
    require(total_splits >= num_splits, "GQA KV split capacity is below the active split count");

    if (tiled) {
        for (uint32_t i = 0; i < num_tiles; ++i) {
            q_token_tiles[size_t(i) * 2] = tiles[i].flat_begin;
            q_token_tiles[size_t(i) * 2 + 1] = tiles[i].flat_end;
        }
    }
    std::copy(splits.begin(), splits.end(), kv_splits.begin());
    std::fill(kv_splits.begin() + splits.size(), kv_splits.begin() + size_t(total_splits) * 3, kU32Max);
    std::copy(cu.begin(), cu.end(), cu_kv_splits.begin());

    psi_replay_shape shape{};
    shape.num_tokens = num_tokens;
    shape.num_total_tokens = total_tokens;
    shape.num_q_token_tiles = num_tiles;
    shape.num_total_q_token_tiles = total_tiles;
    shape.num_sdpa_map_task_templates = num_splits;
    shape.num_total_sdpa_map_task_templates = total_splits;
    shape.reduce_sdpa_partial_outputs = (tiled || num_splits > num_tokens) ? 1u : 0u;
    return shape;
}

// -------------------------------------------------------------------------------------------------------------------
// Device work plans.
// -------------------------------------------------------------------------------------------------------------------
PlanGeometry plan_geometry(uint32_t num_q_heads, uint32_t num_kv_heads) {
    PlanGeometry g{};
    g.group = num_q_heads / num_kv_heads;
    g.heads_per_tile = std::min(g.group, kMaxRows);
    g.head_tiles = static_cast<uint32_t>(div_ceil(g.group, g.heads_per_tile));
    g.tokens_per_tile = std::max(1u, kMaxRows / g.heads_per_tile);
    g.num_kv_heads = num_kv_heads;
    return g;
}

namespace {

// Closes the plan: assigns partial slots to every item whose (tile, head_sel) unit is shared with another item and
// lists those units for the reduce pass.  Items of one unit must be adjacent.
void finish_plan(WorkPlan& plan) {
    plan.num_partial_slots = 0;
    plan.reduces.clear();
    size_t i = 0;
    while (i < plan.items.size()) {
        size_t j = i + 1;
        while (j < plan.items.size() && plan.items[j].tile == plan.items[i].tile &&
               plan.items[j].head_sel == plan.items[i].head_sel) {
            ++j;
        }
        if (j - i == 1) {
            plan.items[i].partial_slot = kU32Max;
        } else {
            const uint32_t unit = static_cast<uint32_t>(plan.reduces.size());
            const uint32_t first_slot = plan.num_partial_slots;
            plan.reduces.push_back({static_cast<uint32_t>(i), static_cast<uint32_t>(j - i)});
            for (size_t k = i; k < j; ++k) {
                plan.items[k].partial_slot = plan.num_partial_slots++;
                plan.items[k].reduce_unit = unit;
                plan.items[k].unit_first_slot = first_slot;
                plan.items[k].unit_num_items = static_cast<uint32_t>(j - i);
            }
        }
        i = j;
    }
}

}  // namespace

WorkPlan build_balanced_plan(const PlanGeometry& geo, const uint32_t* req_slots, const uint32_t* token_indices,
                             const uint32_t* cu_tokens, uint32_t num_reqs, uint32_t max_ctas,
                             uint32_t min_kv_tiles_per_cta, uint32_t item_start_cost) {
    std::vector<uint32_t> all(num_reqs);
    for (uint32_t r = 0; r < num_reqs; ++r) all[r] = r;
    return build_balanced_plan(geo, req_slots, token_indices, cu_tokens, all, max_ctas, min_kv_tiles_per_cta,
                               item_start_cost);
}

WorkPlan build_balanced_plan(const PlanGeometry& geo, const uint32_t* req_slots, const uint32_t* token_indices,
                             const uint32_t* cu_tokens, const std::vector<uint32_t>& requests, uint32_t max_ctas,
                             uint32_t min_kv_tiles_per_cta, uint32_t item_start_cost) {
    WorkPlan plan;
    std::vector<uint32_t> tile_ctx;
    for (uint32_t r : requests) {
        for (uint32_t begin = cu_tokens[r]; begin < cu_tokens[r + 1];) {
            uint32_t end = std::min(cu_tokens[r + 1], begin + geo.tokens_per_tile);
            plan.tiles.push_back({begin, end, req_slots[r], token_indices[r] + (begin - cu_tokens[r]),
                                  token_indices[r], cu_tokens[r]});
            tile_ctx.push_back(token_indices[r] + (end - cu_tokens[r]));
            begin = end;
        }
    }
    const uint32_t heads = geo.num_kv_heads * geo.head_tiles;
    uint64_t total = 0;
    for (uint32_t ctx : tile_ctx) total += div_ceil(ctx, kKvTile) * heads;
    plan.total_kv_tiles = total;
    if (total == 0) return plan;

    uint64_t wanted = std::max<uint64_t>(1, total / std::max(1u, min_kv_tiles_per_cta));
    const uint64_t num_ctas = std::min<uint64_t>(std::max(1u, max_ctas), wanted);
    // Every unit is laid out as `start_cost` virtual tiles (what opening a new item costs a CTA: pipeline drain,
    // merge, first-load latency) followed by its KV tiles; share c covers positions [span*c/n, span*(c+1)/n) of that
    // line, so CTAs that open several items get correspondingly fewer KV tiles.
    const uint64_t start_cost = item_start_cost;
    const uint64_t span = total + start_cost * plan.tiles.size() * heads;
    uint64_t cursor = 0;  // position of the current unit's first (virtual) tile
    uint32_t cta = 0;
    plan.cta_item_begin.assign(1, 0);
    auto share_end = [&](uint64_t c) { return span * (c + 1) / num_ctas; };
    for (uint32_t tile = 0; tile < plan.tiles.size(); ++tile) {
        const uint64_t unit_tiles = div_ceil(tile_ctx[tile], kKvTile);
        const uint64_t unit_span = start_cost + unit_tiles;
        for (uint32_t h = 0; h < heads; ++h) {
            uint64_t done = 0;
            while (done < unit_span) {
                while (cursor + done >= share_end(cta)) {
                    ++cta;
                    plan.cta_item_begin.push_back(static_cast<uint32_t>(plan.items.size()));
                }
                const uint64_t take = std::min(unit_span - done, share_end(cta) - (cursor + done));
                const uint64_t real_begin = std::max(done, start_cost) - start_cost;
                const uint64_t real_end = std::max(done + take, start_cost) - start_cost;
                if (real_end > real_begin) {
                    WorkItem item{};
                    item.tile = tile;
                    item.head_sel = h;
                    item.kv_begin = static_cast<uint32_t>(real_begin * kKvTile);
                    item.kv_end = static_cast<uint32_t>(std::min<uint64_t>(real_end * kKvTile, tile_ctx[tile]));
                    plan.items.push_back(item);
                }
                done += take;
            }
            cursor += unit_span;
        }
    }
    while (plan.cta_item_begin.size() < num_ctas + 1) plan.cta_item_begin.push_back(static_cast<uint32_t>(plan.items.size()));
    finish_plan(plan);
    return plan;
}

WorkPlan build_reference_plan(const PlanGeometry& geo, const ReferenceMetadata& md, const psi_replay_shape& shape,
                              bool tiled_q, const uint32_t* token_indices, const uint32_t* cu_tokens,
                              uint32_t num_reqs) {
    WorkPlan plan;
    const uint32_t heads = geo.num_kv_heads * geo.head_tiles;
    uint32_t req = 0;  // reference q tiles come in flat-token order, so the owning request only moves forward
    for (uint32_t rt = 0; rt < shape.num_q_token_tiles; ++rt) {
        const uint32_t flat_begin = tiled_q ? md.q_token_tiles[size_t(rt) * 2] : rt;
        const uint32_t flat_end = tiled_q ? md.q_token_tiles[size_t(rt) * 2 + 1] : rt + 1;
        const uint32_t s_begin = md.cu_kv_splits[rt], s_end = md.cu_kv_splits[rt + 1];
        for (uint32_t begin = flat_begin; begin < flat_end;) {
            const uint32_t end = std::min(flat_end, begin + geo.tokens_per_tile);
            const uint32_t tile = static_cast<uint32_t>(plan.tiles.size());
            while (req + 1 < num_reqs && begin >= cu_tokens[req + 1]) ++req;
            plan.tiles.push_back({begin, end, md.req_slots[begin], md.flat_token_indices[begin], token_indices[req],
                                  cu_tokens[req]});
            const uint32_t ctx = md.flat_token_indices[end - 1] + 1;  // keys the sub-tile's last token sees
            for (uint32_t h = 0; h < heads; ++h) {
                for (uint32_t s = s_begin; s < s_end; ++s) {
                    const uint32_t kv_begin = md.kv_splits[size_t(s) * 3 + 1];
                    const uint32_t kv_end = std::min(md.kv_splits[size_t(s) * 3 + 2], ctx);
                    if (kv_begin >= kv_end && s != s_begin) continue;  // the split lies beyond this sub-tile's context
                    WorkItem item{};
                    item.tile = tile;
                    item.head_sel = h;
                    item.kv_begin = kv_begin;
                    item.kv_end = std::max(kv_end, kv_begin);
                    plan.items.push_back(item);
                    plan.total_kv_tiles += div_ceil(item.kv_end - item.kv_begin, kKvTile);
                }
            }
            begin = end;
        }
    }
    plan.cta_item_begin.resize(plan.items.size() + 1);
    for (size_t i = 0; i <= plan.items.size(); ++i) plan.cta_item_begin[i] = static_cast<uint32_t>(i);
    finish_plan(plan);
    return plan;
}

ChunkPlan build_chunk_plan(const PlanGeometry& geo, const uint32_t* req_slots, const uint32_t* token_indices,
                           const uint32_t* cu_tokens, const std::vector<uint32_t>& requests, uint32_t max_ctas,
                           uint32_t slot_base, uint32_t counter_base, bool equal_shares) {
    ChunkPlan plan;
    // Units in stream order: all super-tiles of one (request, KV head) follow one another, so that CTAs working on
    // neighbouring units at the same time read the same K/V pages (once from HBM, then from L2).
    struct Unit {
        uint32_t req, flat_begin, flat_end, ctx_end, head;
    };
    std::vector<Unit> units;
    const uint32_t tokens_per_item = geo.tokens_per_tile * kChunkTilesPerItem;
    const uint32_t heads = geo.num_kv_heads * geo.head_tiles;
    uint64_t total = 0;
    // longest requests first: the work dealt last, which decides how far the last CTA trails, is the cheapest
    std::vector<uint32_t> by_length(requests);
    std::stable_sort(by_length.begin(), by_length.end(), [&](uint32_t a, uint32_t b) {
        return token_indices[a] + (cu_tokens[a + 1] - cu_tokens[a]) > token_indices[b] + (cu_tokens[b + 1] - cu_tokens[b]);
    });
    for (uint32_t r : by_length) {
        for (uint32_t h = 0; h < heads; ++h) {
            for (uint32_t begin = cu_tokens[r]; begin < cu_tokens[r + 1];) {
                const uint32_t end = std::min(cu_tokens[r + 1], begin + tokens_per_item);
                units.push_back({r, begin, end, token_indices[r] + (end - cu_tokens[r]), h});
                total += div_ceil(units.back().ctx_end, kKvTile);
                begin = end;
            }
        }
    }
    plan.total_kv_tiles = total;
    if (total == 0) return plan;
    const uint64_t num_ctas = std::min<uint64_t>(std::max(1u, max_ctas), std::max<uint64_t>(1, total / 4));
    auto make_item = [&](const Unit& u, uint64_t tile_begin, uint64_t tile_end) {
        const uint32_t head_tile = u.head % geo.head_tiles;
        DeviceItem d{};
        d.kv_begin = static_cast<uint32_t>(tile_begin * kKvTile);
        d.kv_end = static_cast<uint32_t>(std::min<uint64_t>(tile_end * kKvTile, u.ctx_end));
        d.partial_slot = kU32Max;
        d.flat_begin = u.flat_begin;
        d.num_tokens = u.flat_end - u.flat_begin;
        d.req_slot = req_slots[u.req];
        d.kv_head = u.head / geo.head_tiles;
        d.head0 = d.kv_head * geo.group + head_tile * geo.heads_per_tile;
        d.num_heads = std::min(geo.heads_per_tile, geo.group - head_tile * geo.heads_per_tile);
        d.first_pos = token_indices[u.req] + (u.flat_begin - cu_tokens[u.req]);
        d.new_begin = token_indices[u.req];
        d.flat_req_begin = cu_tokens[u.req];
        d.writes_kv = head_tile == 0 ? 1u : 0u;
        return d;
    };
    // `n` consecutive items starting at `first` are the pieces of one unit cut across CTAs: partial slots 8 apart,
    // eight arrival counters
    auto share_unit = [&](std::vector<DeviceItem*>& pieces) {
        const uint32_t n = static_cast<uint32_t>(pieces.size());
        if (n <= 1) return;
        const uint32_t first_slot = slot_base + plan.num_partial_slots;
        for (uint32_t k = 0; k < n; ++k) {
            pieces[k]->partial_slot = first_slot + k * kChunkTilesPerItem;
            pieces[k]->reduce_unit = counter_base + plan.num_counters;
            pieces[k]->unit_first_slot = first_slot;
            pieces[k]->unit_num_items = n;
        }
        plan.num_partial_slots += n * kChunkTilesPerItem;
        plan.num_counters += kChunkTilesPerItem;
    };
    if (equal_shares) {
        // A working set that stays in L2 whatever the order: contiguous shares of exactly equal size, units cut where a
        // share ends (two or three pieces per cut unit instead of many), slivers below a quarter of the minimum piece
        // folded into their neighbour.
        const uint64_t sliver = kChunkMinPieceTiles / 4;
        plan.items.reserve(units.size() + num_ctas);
        std::vector<uint32_t> owner;  // CTA of every item, in item order
        uint64_t cursor = 0;
        uint32_t cta = 0;
        auto share_end = [&](uint64_t c) { return total * (c + 1) / num_ctas; };
        std::vector<std::pair<size_t, size_t>> unit_items;  // [first, last) item of every unit
        for (const Unit& u : units) {
            const uint64_t unit_tiles = div_ceil(u.ctx_end, kKvTile);
            const size_t first = plan.items.size();
            uint64_t done = 0;
            while (done < unit_tiles) {
                while (cta + 1 < num_ctas && cursor + done + (done == 0 ? sliver : 0) >= share_end(cta)) ++cta;
                uint64_t take = std::min(unit_tiles - done, std::max<uint64_t>(share_end(cta) - (cursor + done), 1));
                if (cta + 1 >= num_ctas || unit_tiles - done - take < sliver) take = unit_tiles - done;
                plan.items.push_back(make_item(u, done, done + take));
                owner.push_back(cta);
                done += take;
            }
            cursor += unit_tiles;
            unit_items.emplace_back(first, plan.items.size());
        }
        for (const auto& range : unit_items) {
            std::vector<DeviceItem*> pieces;
            for (size_t i = range.first; i < range.second; ++i) pieces.push_back(&plan.items[i]);
            share_unit(pieces);
        }
        plan.cta_item_begin.assign(num_ctas + 1, static_cast<uint32_t>(plan.items.size()));
        plan.cta_item_begin[0] = 0;
        for (size_t i = plan.items.size(); i-- > 0;) plan.cta_item_begin[owner[i]] = static_cast<uint32_t>(i);
        for (uint64_t c = num_ctas; c-- > 1;)  // CTAs without items start where the next one does
            plan.cta_item_begin[c] = std::min(plan.cta_item_begin[c], plan.cta_item_begin[c + 1]);
        return plan;
    }
    // A unit longer than half a CTA's fair share is cut along its KV range into equal pieces (partial slots, merged
    // by the last arriver), which bounds how far the last CTA can trail the others; shorter units stay whole, since
    // every piece costs a partial write and a fence, and the merge reads all of them.
    const uint64_t piece_cap = std::max<uint64_t>(kChunkMinPieceTiles, div_ceil(total, num_ctas * 2));

    // Pieces are dealt in order to whichever CTA is free first under the cost model (KV tiles + a fixed start
    // cost): the static equivalent of CTAs pulling work from a queue.
    struct Slot {
        uint64_t load;
        uint32_t cta;
        bool operator>(const Slot& o) const { return load != o.load ? load > o.load : cta > o.cta; }
    };
    std::priority_queue<Slot, std::vector<Slot>, std::greater<Slot>> free_first;
    for (uint32_t c = 0; c < num_ctas; ++c) free_first.push({0, c});
    std::vector<std::vector<DeviceItem>> per_cta(num_ctas);
    for (const Unit& u : units) {
        const uint64_t unit_tiles = div_ceil(u.ctx_end, kKvTile);
        const uint32_t n = static_cast<uint32_t>(div_ceil(unit_tiles, piece_cap));
        const uint32_t head_tile = u.head % geo.head_tiles;
        const uint32_t first_slot = slot_base + plan.num_partial_slots;
        for (uint32_t k = 0; k < n; ++k) {
            const uint64_t tile_begin = unit_tiles * k / n, tile_end = unit_tiles * (k + 1) / n;
            DeviceItem d{};
            d.kv_begin = static_cast<uint32_t>(tile_begin * kKvTile);
            d.kv_end = static_cast<uint32_t>(std::min<uint64_t>(tile_end * kKvTile, u.ctx_end));
            d.partial_slot = kU32Max;
            d.flat_begin = u.flat_begin;
            d.num_tokens = u.flat_end - u.flat_begin;
            d.req_slot = req_slots[u.req];
            d.kv_head = u.head / geo.head_tiles;
            d.head0 = d.kv_head * geo.group + head_tile * geo.heads_per_tile;
            d.num_heads = std::min(geo.heads_per_tile, geo.group - head_tile * geo.heads_per_tile);
            d.first_pos = token_indices[u.req] + (u.flat_begin - cu_tokens[u.req]);
            d.new_begin = token_indices[u.req];
            d.flat_req_begin = cu_tokens[u.req];
            d.writes_kv = head_tile == 0 ? 1u : 0u;
            if (n > 1) {  // the unit is shared between CTAs: partial slots 8 apart, eight arrival counters
                d.partial_slot = first_slot + k * kChunkTilesPerItem;
                d.reduce_unit = counter_base + plan.num_counters;
                d.unit_first_slot = first_slot;
                d.unit_num_items = n;
            }
            Slot slot = free_first.top();
            free_first.pop();
            per_cta[slot.cta].push_back(d);
            slot.load += (tile_end - tile_begin) + kChunkStartCostTiles;
            free_first.push(slot);
        }
        if (n > 1) {
            plan.num_partial_slots += n * kChunkTilesPerItem;
            plan.num_counters += kChunkTilesPerItem;
        }
    }
    plan.cta_item_begin.assign(1, 0);
    for (const auto& list : per_cta) {
        plan.items.insert(plan.items.end(), list.begin(), list.end());
        plan.cta_item_begin.push_back(static_cast<uint32_t>(plan.items.size()));
    }
    return plan;
}

std::vector<DeviceItem> flatten_plan(const WorkPlan& plan, const PlanGeometry& geo) {
    std::vector<DeviceItem> out(plan.items.size());
    for (size_t i = 0; i < plan.items.size(); ++i) {
        const WorkItem& it = plan.items[i];
        const ExecTile& tile = plan.tiles[it.tile];
        const uint32_t head_tile = it.head_sel % geo.head_tiles;
        DeviceItem& d = out[i];
        d.kv_begin = it.kv_begin;
        d.kv_end = it.kv_end;
        d.partial_slot = it.partial_slot;
        d.reduce_unit = it.reduce_unit;
        d.unit_first_slot = it.unit_first_slot;
        d.unit_num_items = it.unit_num_items;
        d.flat_begin = tile.flat_begin;
        d.num_tokens = tile.flat_end - tile.flat_begin;
        d.req_slot = tile.req_slot;
        d.kv_head = it.head_sel / geo.head_tiles;
        d.head0 = d.kv_head * geo.group + head_tile * geo.heads_per_tile;
        d.num_heads = std::min(geo.heads_per_tile, geo.group - head_tile * geo.heads_per_tile);
        d.first_pos = tile.first_pos;
        d.new_begin = tile.new_begin;
        d.flat_req_begin = tile.flat_req_begin;
        d.writes_kv = head_tile == 0 ? 1u : 0u;
    }
    return out;
}

// -------------------------------------------------------------------------------------------------------------------
// RoPE inverse frequencies, with the Yarn ramp when scaling is on.
// -------------------------------------------------------------------------------------------------------------------
RopeParameters rope_parameters(const psi_norm_rope_config& c) {
    require(c.rope_dim > 0 && c.rope_dim % 2 == 0, "RoPE dimension must be positive and even");
    require(std::isfinite(c.rope_theta) && c.rope_theta > 0.0f, "rope_theta must be finite and positive");
    RopeParameters out;
    const uint32_t rope_half = c.rope_dim / 2;
    const bool yarn = c.yarn_enabled != 0;
    if (yarn) {
        require(std::isfinite(c.yarn_factor) && c.yarn_factor >= 1.0f, "Yarn factor must be at least 1");
        require(std::isfinite(c.yarn_attention_factor) && c.yarn_attention_factor > 0.0f, "Yarn attention factor must be positive");
        require(c.yarn_beta_fast > 0.0f && c.yarn_beta_slow > 0.0f && c.yarn_beta_fast >= c.yarn_beta_slow,
                "Yarn beta_fast must be at least beta_slow, both positive");
        require(c.yarn_original_max_position_embeddings > 0, "Yarn original context length must be positive");
        require(c.rope_theta > 1.0f, "Yarn rope_theta must be greater than 1");
        auto correction = [&](float rotations) {
            const double two_pi = 6.283185307179586;
            return static_cast<float>(double(c.rope_dim) *
                                      std::log(double(c.yarn_original_max_position_embeddings) / (double(rotations) * two_pi)) /
                                      (2.0 * std::log(double(c.rope_theta))));
        };
        float low = std::max(correction(c.yarn_beta_fast), 0.0f);
        float high = std::min(correction(c.yarn_beta_slow), static_cast<float>(c.rope_dim - 1));
        if (c.yarn_truncate) {
            low = std::floor(low);
            high = std::ceil(high);
        }
        require(low <= high, "Yarn correction range must be ordered");
        if (low == high) high += 0.001f;
        out.correction_low = low;
        out.correction_high = high;
        out.attention_factor = c.yarn_attention_factor;
    }
    out.inverse_frequencies.resize(rope_half);
    for (uint32_t d = 0; d < rope_half; ++d) {
        float inv = std::pow(c.rope_theta, -(static_cast<float>(d) / static_cast<float>(rope_half)));
        if (yarn) {
            float ramp = (static_cast<float>(d) - out.correction_low) / (out.correction_high - out.correction_low);
            ramp = std::min(std::max(ramp, 0.0f), 1.0f);
            inv *= 1.0f + ramp * (1.0f / c.yarn_factor - 1.0f);
        }
        require(std::isfinite(inv) && inv > 0.0f, "RMSNorm/RoPE inverse frequency must be finite and positive");
        out.inverse_frequencies[d] = inv;
    }
    return out;
}

// -------------------------------------------------------------------------------------------------------------------
// Page-ID allocator: freed IDs are handed out first, oldest free first, then fresh IDs from the counter.
// -------------------------------------------------------------------------------------------------------------------
IdAllocator::IdAllocator(uint64_t capacity) : capacity_(capacity), bitmap_(div_ceil(capacity, 64), 0) {
    require(capacity <= kU32Max, "ID allocator capacity must fit u32");
}

void IdAllocator::mark(uint32_t id, bool live) {
    require(id < capacity_, "U32 ID allocator ID is out of range");
    uint64_t bit = 1ull << (id & 63);
    if (live) bitmap_[id >> 6] |= bit; else bitmap_[id >> 6] &= ~bit;
}

void IdAllocator::alloc_many(uint64_t count, uint32_t* out) {
    uint64_t n = 0;
    while (n < count && !free_ids_.empty()) {
        out[n++] = free_ids_.front();
        free_ids_.pop_front();
    }
    if (n < count) {
        uint64_t fresh = count - n;
        if (counter_ + fresh > capacity_) {
            for (uint64_t i = 0; i < n; ++i) free_ids_.push_back(out[i]);
            throw ExhaustedError("not enough ID");
        }
        for (uint64_t i = 0; i < fresh; ++i) out[n + i] = static_cast<uint32_t>(counter_ + i);
        counter_ += fresh;
    }
    for (uint64_t i = 0; i < count; ++i) mark(out[i], true);
}

void IdAllocator::free_many(const uint32_t* ids, uint64_t count) {
    for (uint64_t i = 0; i < count; ++i) {
        mark(ids[i], false);
        free_ids_.push_back(ids[i]);
    }
}

}  // namespace psi
