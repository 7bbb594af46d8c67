// Helpers behind the C ABI that several entry points share: layout validation, launch parameter assembly, the launch
// sequence of one attention call, and the per-step planning (prepare_impl).
#include "api_internal.hpp"

namespace psi {

thread_local std::string g_thread_error;

int32_t copy_message(const std::string& message, char* buf, size_t n) {
    if (buf == nullptr || n == 0) return PSI_ERR_INVALID_ARGUMENT;
    size_t len = std::min(message.size(), n - 1);
    std::memcpy(buf, message.data(), len);
    buf[len] = '\0';
    return PSI_OK;
}

void validate_layout(const psi_page_table_layout& l) {
    require(l.num_req_slots > 0 && l.num_blocks > 0 && l.num_gqa_layers > 0 && l.num_page_ids_per_block > 0,
            "GQA page-table layout dimensions must be positive");
    const uint64_t per_req = uint64_t(l.num_blocks) * l.num_page_ids_per_block;
    require(per_req <= kU32Max, "GQA per-request physical page count must fit u32");
    const long double total = (long double)l.num_req_slots * l.num_gqa_layers * (long double)per_req;
    require(total < 4.0e18L, "GQA page-table element count must fit usize");
}

PageGeometry page_geometry(const psi_gqa* g, const psi_pages* pages, const psi_table* table, uint32_t layer) {
    require(pages != nullptr && table != nullptr, "pages and table must not be null");
    require(pages->ctx == g->ctx && table->ctx == g->ctx, "pages, table and GQA component must share one context");
    require(pages->ptr != nullptr, "page arena state must be loaded before execution");
    require(pages->page_bytes == g->cfg.page_bytes, "page arena page_bytes differs from the GQA configuration");
    const auto& a = table->layout;
    const auto& b = g->cfg.layout;
    require(a.num_req_slots == b.num_req_slots && a.num_gqa_layers == b.num_gqa_layers &&
                a.num_blocks == b.num_blocks && a.num_page_ids_per_block == b.num_page_ids_per_block,
            "page table layout differs from the GQA configuration");
    require(layer < b.num_gqa_layers, "GQA page-table index exceeds layer count");
    PageGeometry geo{};
    geo.pages = pages->ptr;
    geo.page_ids = table->dev;
    geo.elem_bytes = dtype_bytes(g->cfg.dtype);
    geo.page_elems = g->cfg.page_bytes / geo.elem_bytes;
    geo.num_pages = pages->num_pages;
    geo.layer = layer;
    geo.num_layers = b.num_gqa_layers;
    geo.pages_per_req = static_cast<uint32_t>(table->row_words());
    geo.tokens_per_page = g->tokens_per_page;
    geo.num_kv_heads = g->cfg.num_kv_heads;
    geo.head_dim = g->cfg.head_dim;
    geo.fault = static_cast<uint32_t*>(g->status_word.ptr);
    return geo;
}

const uint32_t* block_words(const psi_gqa* g, uint64_t offset) {
    return static_cast<const uint32_t*>(g->block.ptr) + offset;
}


AttendParams attend_params(psi_gqa* g, const psi_pages* pages, const psi_table* table, uint32_t layer, const void* q) {
    require(g->prepared, "GQA batch metadata must be updated before recording");
    require(q != nullptr, "q must not be null");
    AttendParams p{};
    p.geo = page_geometry(g, pages, table, layer);
    p.q = q;
    p.items = reinterpret_cast<const DeviceItem*>(block_words(g, g->off_items));
    p.cta_item_begin = block_words(g, g->off_cta);
    if (g->kernel == PSI_KERNEL_MMA) p.cta_first_items = reinterpret_cast<const DeviceItem*>(block_words(g, g->off_first_items));
    p.reduces = reinterpret_cast<const ReduceUnit*>(block_words(g, g->off_reduces));
    p.partial_o = static_cast<float*>(g->partial_o.ptr);
    p.partial_m = static_cast<float*>(g->partial_ml.ptr);
    p.partial_l = p.partial_m == nullptr ? nullptr : p.partial_m + g->partial_slots_cap * kMaxRows;
    p.unit_counters = static_cast<uint32_t*>(g->unit_counters.ptr);
    p.scalars = block_words(g, 0);
    p.num_q_heads = g->cfg.num_q_heads;
    p.tokens_per_tile = g->geo.tokens_per_tile;
    p.dtype = g->cfg.dtype;
    p.scale_log2 = g->cfg.scale * 1.4426950408889634f;
    p.tma_feed = g->cfg.kernel_mode == PSI_KERNEL_MMA_TMA ? 1u : 0u;
    p.status = static_cast<uint32_t*>(g->status_word.ptr);
    return p;
}

void run_attend(psi_gqa* g, const AttendParams& params) {
    psi_ctx* ctx = g->ctx;
    AttendParams p = params;
    // Under a replay reservation a captured launch sequence has to be right for every later plan: always the same
    // launches (append, map, chunk, reduce where the kernel needs one), each at its capacity grid, each reading its
    // active counts from the device block.
    const bool fixed = g->replay_reserved;
    if (p.new_k != nullptr && (fixed || g->chunk.num_ctas() > 0)) {
        // A fused step that carries long query runs: their K/V tiles are fetched page-wise by TMA, so the step's rows
        // go to their pages first (one more launch, against milliseconds of attention) and both kernels read pages only.
        AppendParams a{};
        a.geo = p.geo;
        a.flat_k = p.new_k;
        a.flat_v = p.new_v;
        a.req_slots = block_words(g, g->off_req_slots);
        a.flat_token_indices = block_words(g, g->off_token_indices);
        a.scalars = block_words(g, 0);
        a.num_total_tokens = g->shape.num_total_tokens;
        {
            LaunchScope scope(ctx, PSI_KERNEL_CLASS_APPEND);
            cuda_check(launch_kv_append(a, ctx->stream), "kv append launch");
        }
        p.new_k = nullptr;
        p.new_v = nullptr;
    }
    const uint32_t num_ctas = fixed ? g->grid_cap : g->plan.num_ctas();
    if (num_ctas > 0) {
        LaunchScope scope(ctx, PSI_KERNEL_CLASS_ATTEND_MAP);
        if (g->kernel == PSI_KERNEL_MMA) {
            cuda_check(launch_attend_mma(p, num_ctas, ctx->stream), "attend (mma) launch");
        } else {
            cuda_check(launch_attend_generic(p, num_ctas, ctx->stream), "attend (generic) launch");
        }
    }
    const uint32_t chunk_ctas = fixed ? (g->chunk_supported ? g->grid_cap : 0u) : g->chunk.num_ctas();
    if (chunk_ctas > 0) {
        AttendParams c = p;
        c.items = reinterpret_cast<const DeviceItem*>(block_words(g, g->off_chunk_items));
        c.cta_item_begin = block_words(g, g->off_chunk_cta);
        LaunchScope scope(ctx, PSI_KERNEL_CLASS_ATTEND_CHUNK);
        cudaError_t launched = cudaErrorNotSupported;
        if (g->chunk_umma) {
            c.status = static_cast<uint32_t*>(g->status_word.ptr);
            launched = launch_attend_chunk_umma(c, chunk_ctas, ctx->stream);
        }
        // an arena the TMA unit cannot address (alignment, size) keeps the mma.sync kernel
        if (launched == cudaErrorNotSupported) {
            launched = launch_attend_chunk(c, chunk_ctas, ctx->stream);
            g->chunk_launches[1] += 1;
        } else {
            g->chunk_launches[0] += 1;
        }
        cuda_check(launched, "attend (chunk) launch");
    }
    // The mma kernel merges a unit's partials in the CTA that delivers the last one; the generic kernel needs the
    // separate reduce pass.
    const uint32_t num_reduces = g->kernel == PSI_KERNEL_MMA
                                     ? 0u
                                     : static_cast<uint32_t>(fixed ? g->cap_reduces : g->plan.reduces.size());
    if (num_reduces > 0) {
        LaunchScope scope(ctx, PSI_KERNEL_CLASS_ATTEND_REDUCE);
        cuda_check(launch_attend_reduce(p, num_reduces, ctx->stream), "attend reduce launch");
    }
}

void run_append(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k, const void* v) {
    require(g->prepared, "GQA batch metadata must be updated before recording");
    require(k != nullptr && v != nullptr, "k and v must not be null");
    AppendParams p{};
    p.geo = page_geometry(g, pages, table, layer);
    p.flat_k = k;
    p.flat_v = v;
    p.req_slots = block_words(g, g->off_req_slots);
    p.flat_token_indices = block_words(g, g->off_token_indices);
    p.scalars = block_words(g, 0);
    p.num_total_tokens = g->shape.num_total_tokens;
    LaunchScope scope(g->ctx, PSI_KERNEL_CLASS_APPEND);
    cuda_check(launch_kv_append(p, g->ctx->stream), "kv append launch");
}

// Device-side address of a pinned, device-mapped host buffer (16-byte aligned), or nullptr for any other memory.
void* mapped_device_pointer(const void* host) {
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, host) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
        attr.devicePointer != nullptr && (reinterpret_cast<uintptr_t>(attr.devicePointer) & 15u) == 0) {
        return attr.devicePointer;
    }
    (void)cudaGetLastError();
    return nullptr;
}

// A prepared step through pageable host buffers: inputs staged by copy-engine transfers, output copied back, waited for.
void run_staged_host_step(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k_host,
                          const void* v_host, const void* q_host, void* out_host, uint64_t kv_bytes, uint64_t q_bytes,
                          uint64_t q_cap) {
    psi_ctx* ctx = g->ctx;
    g->step_out.ensure(ctx, q_cap, false);
    cuda_check(cudaMemcpyAsync(g->step_k.ptr, k_host, kv_bytes, cudaMemcpyHostToDevice, ctx->stream), "H2D k");
    cuda_check(cudaMemcpyAsync(g->step_v.ptr, v_host, kv_bytes, cudaMemcpyHostToDevice, ctx->stream), "H2D v");
    cuda_check(cudaMemcpyAsync(g->step_q.ptr, q_host, q_bytes, cudaMemcpyHostToDevice, ctx->stream), "H2D q");
    AttendParams p = attend_params(g, pages, table, layer, g->step_q.ptr);
    p.out = g->step_out.ptr;
    if (g->kernel == PSI_KERNEL_MMA) {
        p.new_k = g->step_k.ptr;
        p.new_v = g->step_v.ptr;
    } else {
        run_append(g, pages, table, layer, g->step_k.ptr, g->step_v.ptr);
    }
    run_attend(g, p);
    cuda_check(cudaMemcpyAsync(out_host, g->step_out.ptr, q_bytes, cudaMemcpyDeviceToHost, ctx->stream), "D2H out");
    cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
}


// GQAMetadataBuffers::update plus this library's plan.  With `defer_upload` the packed block stays in the pinned
// staging buffer and its size comes back in *deferred_words: the caller brings it to the device itself.
void prepare_impl(psi_gqa* g, const uint32_t* req_slots, const uint32_t* token_indices, const uint32_t* cu_tokens,
                  uint32_t num_reqs, uint32_t capacity_mode, uint32_t caller_num_total_tokens,
                  psi_replay_shape* out_shape, bool defer_upload, uint64_t* deferred_words, bool plan_only) {
    {
        require(!plan_only || g->cfg.plan_mode == PSI_PLAN_BALANCED, "a plan-only prepare needs the balanced plan mode");
        require(req_slots != nullptr && token_indices != nullptr && cu_tokens != nullptr, "metadata inputs must not be null");
        require(capacity_mode <= PSI_CAPACITY_CALLER_TOKENS, "unknown capacity mode");
        require(num_reqs > 0, "GQA batch metadata requires tokens");
        psi_ctx* ctx = g->ctx;
        require(!ctx->capturing, "psi_gqa_prepare uploads the step's plan and stays outside captured graphs");
        ctx->bind();
        g->prepared = false;

        // Variant selection as the reference's executor does it (crates/inference-executor-metal/src/attn/gqa/mod.rs:
        // 64-94, without its measured D256/page8 work model, which tunes a different device).
        require(cu_tokens[0] == 0, "GQA batch cu_tokens must start at zero");
        uint64_t ref_q_tiles = 0;
        for (uint32_t r = 0; r < num_reqs; ++r) {
            require(cu_tokens[r] <= cu_tokens[r + 1], "GQA batch cu_tokens must be nondecreasing");
            ref_q_tiles += (uint64_t(cu_tokens[r + 1] - cu_tokens[r]) + 7) / 8;
        }
        const uint32_t num_tokens = cu_tokens[num_reqs];
        require(num_tokens > 0, "GQA batch metadata requires tokens");
        require(num_tokens <= g->cfg.max_tokens, "GQA batch exceeds the metadata token capacity");
        psi_split_kv_variant variant{};
        if (g->selector) {
            variant = g->selector->select(num_tokens, static_cast<uint32_t>(ref_q_tiles));
        } else {
            variant.kv_token_tile_size = 256;  // f16 has no reference profile: SingleQ geometry of a 256-thread block
            variant.num_threads_per_threadblock = 256;
            variant.q_head_tile_size = std::min(g->geo.group, 8u);
        }
        psi_replay_shape shape{};
        if (plan_only) {
            shape.num_tokens = shape.num_total_tokens = g->md->expand_tokens(req_slots, token_indices, cu_tokens, num_reqs);
        } else {
            shape = g->md->update(req_slots, token_indices, cu_tokens, num_reqs, variant, capacity_mode, g->boundaries,
                                  caller_num_total_tokens);
        }

        const uint64_t table_tokens =
            uint64_t(g->cfg.layout.num_blocks) * g->cfg.layout.num_page_ids_per_block * g->tokens_per_page;
        for (uint32_t r = 0; r < num_reqs; ++r) {
            require(req_slots[r] < g->cfg.layout.num_req_slots, "GQA request page table req_slot out of range");
            require(uint64_t(token_indices[r]) + (cu_tokens[r + 1] - cu_tokens[r]) <= table_tokens,
                    "GQA request context does not fit the request page table");
        }

        if (g->cfg.plan_mode == PSI_PLAN_REFERENCE) {
            g->plan = build_reference_plan(g->geo, *g->md, shape, variant.tiled_q != 0, token_indices, cu_tokens,
                                           num_reqs);
            g->chunk = ChunkPlan{};
        } else {
            // Requests with a long run of query tokens go to the chunk kernel (one pass over their KV for eight query
            // tiles at a time); the rest are decode rows.
            std::vector<uint32_t> decode_reqs, chunk_reqs;
            for (uint32_t r = 0; r < num_reqs; ++r) {
                const uint32_t tiles = (cu_tokens[r + 1] - cu_tokens[r] + g->geo.tokens_per_tile - 1) / g->geo.tokens_per_tile;
                if (tiles == 0) continue;
                (g->chunk_supported && tiles >= kChunkMinTiles ? chunk_reqs : decode_reqs).push_back(r);
            }
            const uint32_t min_tiles = g->kernel == PSI_KERNEL_MMA ? 16u : 4u;
            g->plan = build_balanced_plan(g->geo, req_slots, token_indices, cu_tokens, decode_reqs, g->grid_cap,
                                          min_tiles, g->item_start_cost);
            // K/V the long runs touch: below a third of the L2 the order of the work cannot cost HBM traffic, and exactly
            // equal shares beat stream order
            uint64_t chunk_kv_bytes = 0;
            for (uint32_t r : chunk_reqs)
                chunk_kv_bytes += uint64_t(token_indices[r] + (cu_tokens[r + 1] - cu_tokens[r])) * (uint64_t(g->cfg.page_bytes) / g->tokens_per_page);
            g->chunk = build_chunk_plan(g->geo, req_slots, token_indices, cu_tokens, chunk_reqs, g->grid_cap,
                                        g->plan.num_partial_slots, static_cast<uint32_t>(g->plan.reduces.size()),
                                        chunk_kv_bytes <= (40ull << 20));
        }
        const WorkPlan& plan = g->plan;
        const ChunkPlan& chunk = g->chunk;
        const std::vector<DeviceItem> device_items = flatten_plan(plan, g->geo);
        const uint32_t total_slots = plan.num_partial_slots + chunk.num_partial_slots;
        const uint32_t total_counters = static_cast<uint32_t>(plan.reduces.size()) + chunk.num_counters;

        // Pack the device block: scalars | req_slots | flat_token_indices | cta ranges | reduces | items.
        uint64_t words = 0;
        if (g->replay_reserved) {
            // fixed offsets (reserved_layout); only the used prefix is uploaded
            constexpr uint64_t kItemWords = sizeof(DeviceItem) / sizeof(uint32_t);
            require(device_items.size() <= g->cap_items && chunk.items.size() <= g->cap_chunk_items &&
                        plan.reduces.size() <= g->cap_reduces && total_slots <= g->partial_slots_cap &&
                        plan.num_ctas() <= g->grid_cap && chunk.num_ctas() <= g->grid_cap,
                    "the step exceeds the reserved replay capacity");
            words = g->off_items + device_items.size() * kItemWords;
            if (!chunk.items.empty()) words = g->off_chunk_items + chunk.items.size() * kItemWords;
            if (!plan.reduces.empty()) words = g->off_reduces + plan.reduces.size() * 2;
            cuda_check(cudaEventSynchronize(g->upload_done), "cudaEventSynchronize");  // previous upload left staging
        } else {
            uint64_t cursor = pad_words(kScalarCount);
            g->off_req_slots = cursor;
            cursor += pad_words(num_tokens);
            g->off_token_indices = cursor;
            cursor += pad_words(num_tokens);
            g->off_cta = cursor;
            cursor += pad_words(plan.cta_item_begin.size());
            g->off_reduces = cursor;
            cursor += pad_words(plan.reduces.size() * 2);
            g->off_items = cursor;
            cursor += pad_words(device_items.size() * (sizeof(DeviceItem) / sizeof(uint32_t)));
            g->off_first_items = cursor;
            cursor += pad_words(static_cast<uint64_t>(plan.num_ctas()) * (sizeof(DeviceItem) / sizeof(uint32_t)));
            g->off_chunk_cta = cursor;
            cursor += pad_words(chunk.cta_item_begin.size());
            g->off_chunk_items = cursor;
            cursor += pad_words(chunk.items.size() * (sizeof(DeviceItem) / sizeof(uint32_t)));
            words = cursor;

            if (g->staging_words < words) {
                if (g->staging != nullptr) {
                    cuda_check(cudaEventSynchronize(g->upload_done), "cudaEventSynchronize");
                    cuda_check(cudaFreeHost(g->staging), "cudaFreeHost");
                    g->staging = nullptr;
                }
                const uint64_t grown = std::max<uint64_t>(words * 2, 4096);
                cuda_check(cudaMallocHost(reinterpret_cast<void**>(&g->staging), grown * sizeof(uint32_t)), "cudaMallocHost");
                g->staging_words = grown;
            } else {
                cuda_check(cudaEventSynchronize(g->upload_done), "cudaEventSynchronize");  // previous upload left staging
            }
        }
        g->block.ensure(ctx, g->staging_words * sizeof(uint32_t), false);
        if (total_slots > g->partial_slots_cap) {
            const uint64_t slots = std::max<uint64_t>(total_slots, 2ull * g->grid_cap);
            g->partial_o.ensure(ctx, slots * kMaxRows * g->cfg.head_dim * sizeof(float), false);
            g->partial_ml.ensure(ctx, 2 * slots * kMaxRows * sizeof(float), false);
            g->unit_counters.ensure(ctx, slots * sizeof(uint32_t), true);
            g->partial_slots_cap = slots;
        }
        // Arrival counters start at zero (cleared when allocated) and every launch returns them to zero itself.
        (void)total_counters;

        uint32_t* s = g->staging;
        std::fill(s, s + kScalarCount, 0u);
        s[kScalarNumActiveTokens] = num_tokens;
        s[kScalarNumCtas] = plan.num_ctas();
        s[kScalarNumReduces] = static_cast<uint32_t>(plan.reduces.size());
        s[kScalarNumChunkCtas] = chunk.num_ctas();
        std::copy(g->md->req_slots.begin(), g->md->req_slots.begin() + num_tokens, s + g->off_req_slots);
        std::copy(g->md->flat_token_indices.begin(), g->md->flat_token_indices.begin() + num_tokens,
                  s + g->off_token_indices);
        std::copy(plan.cta_item_begin.begin(), plan.cta_item_begin.end(), s + g->off_cta);
        if (g->replay_reserved) {
            // launches run at the capacity grid: CTAs beyond the plan's find an empty range and a zero first item
            constexpr uint64_t kItemWords = sizeof(DeviceItem) / sizeof(uint32_t);
            const uint32_t items_end = static_cast<uint32_t>(device_items.size());
            for (uint64_t c = plan.cta_item_begin.size(); c < g->grid_cap + 2ull; ++c) s[g->off_cta + c] = items_end;
            if (plan.cta_item_begin.empty()) s[g->off_cta] = 0;
            std::fill(s + g->off_first_items, s + g->off_first_items + uint64_t(g->grid_cap) * kItemWords, 0u);
            const uint32_t chunk_end = static_cast<uint32_t>(chunk.items.size());
            for (uint64_t c = chunk.cta_item_begin.size(); c < g->grid_cap + 2ull; ++c) s[g->off_chunk_cta + c] = chunk_end;
            if (chunk.cta_item_begin.empty()) s[g->off_chunk_cta] = 0;
        }
        if (!plan.reduces.empty())
            std::memcpy(s + g->off_reduces, plan.reduces.data(), plan.reduces.size() * sizeof(ReduceUnit));
        if (!device_items.empty())
            std::memcpy(s + g->off_items, device_items.data(), device_items.size() * sizeof(DeviceItem));
        // a copy of every CTA's first item at a place the CTA can read without knowing its range (zeros for a CTA
        // without items, which its empty range tells it not to use)
        for (uint32_t c = 0; c < plan.num_ctas(); ++c) {
            DeviceItem first{};
            if (plan.cta_item_begin[c] < plan.cta_item_begin[c + 1]) first = device_items[plan.cta_item_begin[c]];
            std::memcpy(s + g->off_first_items + static_cast<uint64_t>(c) * (sizeof(DeviceItem) / sizeof(uint32_t)), &first,
                        sizeof(DeviceItem));
        }
        std::copy(chunk.cta_item_begin.begin(), chunk.cta_item_begin.end(), s + g->off_chunk_cta);
        if (!chunk.items.empty())
            std::memcpy(s + g->off_chunk_items, chunk.items.data(), chunk.items.size() * sizeof(DeviceItem));
        if (defer_upload) {
            *deferred_words = words;
        } else {
            cuda_check(cudaMemcpyAsync(g->block.ptr, s, words * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream),
                       "cudaMemcpyAsync");
            cuda_check(cudaEventRecord(g->upload_done, ctx->stream), "cudaEventRecord");
        }

        g->shape = shape;
        g->variant = variant;
        g->prepared = true;
        if (out_shape != nullptr) *out_shape = shape;
    }
}

}  // namespace psi
