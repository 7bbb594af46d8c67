// C ABI: the GQA component - creation, replay reservation, per-step prepare, KV append and attention.
#include "api_internal.hpp"

using namespace psi;

extern "C" {

int32_t psi_gqa_create(psi_ctx* ctx, const psi_gqa_config* config, psi_gqa** out) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        require(out != nullptr && config != nullptr, "out and config must not be null");
        *out = nullptr;
        const psi_gqa_config& c = *config;
        require(c.num_q_heads > 0 && c.num_kv_heads > 0 && c.head_dim > 0, "GQA head counts and head_dim must be positive");
        require(c.num_q_heads % c.num_kv_heads == 0, "GQA q heads must be a multiple of kv heads");
        require(c.scale > 0.0f && std::isfinite(c.scale), "GQA scale must be positive");
        require(c.dtype <= PSI_DTYPE_F16, "unsupported GQA dtype");
        require(c.max_tokens > 0, "GQA batch metadata requires tokens");
        require(c.plan_mode <= PSI_PLAN_REFERENCE && c.kernel_mode <= PSI_KERNEL_MMA_TMA, "unknown plan or kernel mode");
        validate_layout(c.layout);
        const uint64_t per_token = uint64_t(c.num_kv_heads) * c.head_dim * 2u * dtype_bytes(c.dtype);
        require(per_token <= kU32Max, "GQA K/V bytes per token must fit u32");
        require(c.page_bytes > 0 && c.page_bytes % per_token == 0,
                "GQA page_bytes must be divisible by the K/V bytes per token");
        require(uint64_t(c.max_tokens) * c.num_q_heads * c.head_dim <= kU32Max,
                "GQA SDPA query/output exceeds the shader u32 count domain");
        require(c.head_dim <= 256, "GQA head_dim above 256 is not supported");
        ctx->bind();

        auto g = std::make_unique<psi_gqa>();
        g->ctx = ctx;
        g->cfg = c;
        g->tokens_per_page = c.page_bytes / static_cast<uint32_t>(per_token);
        g->geo = plan_geometry(c.num_q_heads, c.num_kv_heads);
        const bool mma_ok = attend_mma_supported(c.dtype, c.head_dim, g->tokens_per_page);
        if (c.kernel_mode >= PSI_KERNEL_MMA) require(mma_ok, "the mma kernel does not support this profile");
        g->kernel = (c.kernel_mode == PSI_KERNEL_GENERIC || !mma_ok) ? PSI_KERNEL_GENERIC : PSI_KERNEL_MMA;
        const uint32_t per_sm =
            g->kernel == PSI_KERNEL_MMA ? attend_mma_ctas_per_sm(c.head_dim) : attend_generic_ctas_per_sm(c.head_dim, c.dtype);
        g->grid_cap = c.max_ctas > 0 ? c.max_ctas : static_cast<uint32_t>(ctx->sm_count) * per_sm;
        g->item_start_cost = g->kernel == PSI_KERNEL_MMA ? 32u : 0u;
        g->chunk_supported = g->kernel == PSI_KERNEL_MMA && c.plan_mode == PSI_PLAN_BALANCED &&
                             attend_chunk_supported(c.dtype, c.head_dim, g->tokens_per_page);
        g->chunk_umma = g->chunk_supported && c.kernel_mode != PSI_KERNEL_MMA_SYNC;
        g->status_word.ensure(ctx, sizeof(uint32_t), true);  // bounded waits and bounds checks report here
        if (c.dtype != PSI_DTYPE_F16) {
            g->selector = std::make_unique<SplitKvSelector>(c.dtype, c.page_bytes, c.num_q_heads, c.num_kv_heads,
                                                            c.head_dim, false);
        }
        g->md = std::make_unique<ReferenceMetadata>(c.max_tokens);
        cuda_check(cudaEventCreateWithFlags(&g->upload_done, cudaEventDisableTiming), "cudaEventCreateWithFlags");
        *out = g.release();
    });
}

int32_t psi_gqa_destroy(psi_gqa* g) {
    if (g == nullptr) return PSI_OK;
    int32_t status = guarded(g->ctx, [&] {
        g->ctx->bind();
        (void)cudaStreamSynchronize(g->ctx->stream);
        g->block.release();
        g->partial_o.release();
        g->partial_ml.release();
        g->unit_counters.release();
        g->step_k.release();
        g->step_v.release();
        g->step_q.release();
        g->step_out.release();
        g->combine_ptrs.release();
        g->status_word.release();
        g->sync_words.release();
        g->xchg_local.release();
        g->norm_rope.release();
        for (cudaEvent_t e : g->pipe_events) (void)cudaEventDestroy(e);
        if (g->pipe_h2d != nullptr) (void)cudaStreamDestroy(g->pipe_h2d);
        if (g->pipe_d2h != nullptr) (void)cudaStreamDestroy(g->pipe_d2h);
        if (g->staging != nullptr) (void)cudaFreeHost(g->staging);
        if (g->upload_done != nullptr) (void)cudaEventDestroy(g->upload_done);
    });
    delete g;
    return status;
}

int32_t psi_gqa_set_token_topology_boundaries(psi_gqa* g, const uint32_t* boundaries, uint32_t n) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(boundaries != nullptr || n == 0, "boundaries must not be null");
        for (uint32_t i = 0; i < n; ++i) require(boundaries[i] > 0, "replay topology boundary must be positive");
        g->boundaries.assign(boundaries, boundaries + n);
    });
}

// Offsets (in words) of the device block's arrays under a replay reservation: everything sized for max_tokens, the
// arrays whose used length varies most placed last, so that an upload still moves only a prefix.
static void reserved_layout(psi_gqa* g) {
    constexpr uint64_t kItemWords = sizeof(DeviceItem) / sizeof(uint32_t);
    const uint64_t t = g->cfg.max_tokens;
    uint64_t cursor = pad_words(kScalarCount);
    g->off_req_slots = cursor;
    cursor += pad_words(t);
    g->off_token_indices = cursor;
    cursor += pad_words(t);
    g->off_cta = cursor;
    cursor += pad_words(g->grid_cap + 2);
    g->off_first_items = cursor;
    cursor += pad_words(uint64_t(g->grid_cap) * kItemWords);
    g->off_chunk_cta = cursor;
    cursor += pad_words(g->grid_cap + 2);
    g->off_items = cursor;
    cursor += pad_words(g->cap_items * kItemWords);
    g->off_chunk_items = cursor;
    cursor += pad_words(g->cap_chunk_items * kItemWords);
    g->off_reduces = cursor;
    cursor += pad_words(g->cap_reduces * 2);
    g->staging_words = cursor;
}

int32_t psi_gqa_reserve_replay(psi_gqa* g) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        if (g->replay_reserved) return;
        psi_ctx* ctx = g->ctx;
        require(!ctx->capturing, "replay capacity cannot be reserved during stream capture");
        ctx->bind();
        // worst cases for max_tokens: every token a query tile of its own, every unit cut at every CTA boundary
        const uint64_t heads = uint64_t(g->geo.num_kv_heads) * g->geo.head_tiles;
        const uint64_t units = uint64_t(g->cfg.max_tokens) * heads;
        const uint64_t cap_items = units + g->grid_cap;
        const uint64_t chunk_units = g->chunk_supported ? units / 3 + heads : 0;
        const uint64_t cap_chunk_items = g->chunk_supported ? chunk_units + 2ull * g->grid_cap + 8 : 0;
        const uint64_t slots = cap_items + cap_chunk_items * kChunkTilesPerItem;
        const uint64_t partial_bytes = slots * kMaxRows * g->cfg.head_dim * sizeof(float);
        require(partial_bytes <= (2ull << 30),
                "replay reservation needs more than 2 GiB of partial-output scratch for this max_tokens: create the "
                "component with the largest batch the replayed steps carry");
        cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
        g->cap_items = cap_items;
        g->cap_chunk_items = cap_chunk_items;
        g->cap_reduces = units;
        if (g->staging != nullptr) {
            cuda_check(cudaFreeHost(g->staging), "cudaFreeHost");
            g->staging = nullptr;
        }
        reserved_layout(g);
        cuda_check(cudaMallocHost(reinterpret_cast<void**>(&g->staging), g->staging_words * sizeof(uint32_t)), "cudaMallocHost");
        std::memset(g->staging, 0, g->staging_words * sizeof(uint32_t));
        g->block.ensure(ctx, g->staging_words * sizeof(uint32_t), true);
        g->partial_o.ensure(ctx, partial_bytes, false);
        g->partial_ml.ensure(ctx, 2 * slots * kMaxRows * sizeof(float), false);
        g->unit_counters.release();  // counters restart from zero at their new size
        g->unit_counters.ensure(ctx, slots * sizeof(uint32_t), true);
        g->partial_slots_cap = slots;
        g->status_word.ensure(ctx, sizeof(uint32_t), true);
        cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
        g->prepared = false;  // the block moved: the next step prepares again
        g->replay_reserved = true;
    });
}

int32_t psi_gqa_prepare(psi_gqa* g, const uint32_t* req_slots, const uint32_t* token_indices, const uint32_t* cu_tokens,
                        uint32_t num_reqs, uint32_t capacity_mode, uint32_t caller_num_total_tokens,
                        psi_replay_shape* out_shape) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        prepare_impl(g, req_slots, token_indices, cu_tokens, num_reqs, capacity_mode, caller_num_total_tokens, out_shape,
                     false, nullptr);
    });
}

int32_t psi_gqa_split_kv_variant(psi_gqa* g, psi_split_kv_variant* out) {
    if (g == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(g->prepared, "GQA batch metadata must be updated before recording");
        *out = g->variant;
    });
}

static std::vector<uint32_t>* metadata_array(psi_gqa* g, uint32_t which) {
    switch (which) {
        case PSI_MD_REQ_SLOTS: return &g->md->req_slots;
        case PSI_MD_FLAT_TOKEN_INDICES: return &g->md->flat_token_indices;
        case PSI_MD_Q_TOKEN_TILES: return &g->md->q_token_tiles;
        case PSI_MD_KV_SPLITS: return &g->md->kv_splits;
        case PSI_MD_CU_KV_SPLITS: return &g->md->cu_kv_splits;
        default: return nullptr;
    }
}

int32_t psi_gqa_metadata_read(psi_gqa* g, uint32_t which, uint64_t offset, uint32_t* out, uint64_t n) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        auto* array = metadata_array(g, which);
        require(array != nullptr && out != nullptr, "unknown metadata array or null output");
        require(offset <= array->size() && n <= array->size() - offset, "metadata range out of bounds");
        std::copy(array->begin() + offset, array->begin() + offset + n, out);
    });
}

int32_t psi_gqa_metadata_write(psi_gqa* g, uint32_t which, uint64_t offset, const uint32_t* in, uint64_t n) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        auto* array = metadata_array(g, which);
        require(array != nullptr && in != nullptr, "unknown metadata array or null input");
        require(offset <= array->size() && n <= array->size() - offset, "metadata range out of bounds");
        std::copy(in, in + n, array->begin() + offset);
    });
}

int32_t psi_gqa_plan_stats(psi_gqa* g, uint32_t* out, uint32_t n) {
    if (g == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(g->prepared, "GQA batch metadata must be updated before recording");
        const uint32_t stats[12] = {g->plan.num_ctas(),
                                   static_cast<uint32_t>(g->plan.items.size()),
                                   g->plan.num_partial_slots,
                                   static_cast<uint32_t>(g->plan.reduces.size()),
                                   static_cast<uint32_t>(g->plan.tiles.size()),
                                   g->kernel,
                                   static_cast<uint32_t>(std::min<uint64_t>(g->plan.total_kv_tiles, kU32Max)),
                                   g->geo.tokens_per_tile * g->geo.heads_per_tile,
                                   g->chunk.num_ctas(),
                                   static_cast<uint32_t>(g->chunk.items.size()),
                                   g->chunk_launches[0],
                                   g->chunk_launches[1]};
        for (uint32_t i = 0; i < n && i < 12; ++i) out[i] = stats[i];
    });
}

int32_t psi_gqa_kv_append(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k, const void* v) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        g->ctx->bind();
        run_append(g, pages, table, layer, k, v);
    });
}

int32_t psi_gqa_attend(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* q, void* out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(out != nullptr, "out must not be null");
        g->ctx->bind();
        AttendParams p = attend_params(g, pages, table, layer, q);
        p.out = out;
        run_attend(g, p);
    });
}

int32_t psi_gqa_append_attend(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k,
                              const void* v, const void* q, void* out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(out != nullptr && k != nullptr && v != nullptr, "k, v and out must not be null");
        g->ctx->bind();
        if (g->kernel != PSI_KERNEL_MMA) {  // the generic kernel has no fused form: two launches in stream order
            run_append(g, pages, table, layer, k, v);
            AttendParams p = attend_params(g, pages, table, layer, q);
            p.out = out;
            run_attend(g, p);
            return;
        }
        require((reinterpret_cast<uintptr_t>(k) & 15u) == 0 && (reinterpret_cast<uintptr_t>(v) & 15u) == 0,
                "k and v must be 16-byte aligned");
        AttendParams p = attend_params(g, pages, table, layer, q);
        p.out = out;
        p.new_k = k;
        p.new_v = v;
        run_attend(g, p);
    });
}

int32_t psi_rope_parameters(const psi_norm_rope_config* config, float* out_inverse_frequencies,
                            float* out_attention_factor, float* out_correction_low, float* out_correction_high) {
    return guarded(nullptr, [&] {
        require(config != nullptr && out_inverse_frequencies != nullptr && out_attention_factor != nullptr,
                "rope parameter outputs must not be null");
        const RopeParameters params = rope_parameters(*config);
        std::copy(params.inverse_frequencies.begin(), params.inverse_frequencies.end(), out_inverse_frequencies);
        *out_attention_factor = params.attention_factor;
        if (out_correction_low != nullptr) *out_correction_low = params.correction_low;
        if (out_correction_high != nullptr) *out_correction_high = params.correction_high;
    });
}

int32_t psi_gqa_set_norm_rope(psi_gqa* g, const psi_norm_rope_config* config, const uint16_t* q_weight,
                              const uint16_t* k_weight) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(config != nullptr && q_weight != nullptr && k_weight != nullptr, "norm/rope arguments must not be null");
        require(config->rope_dim <= g->cfg.head_dim, "RoPE dimension exceeds head_dim");
        require(std::isfinite(config->eps) && config->eps >= 0.0f, "RMSNorm eps must be finite and non-negative");
        const RopeParameters params = rope_parameters(*config);
        psi_ctx* ctx = g->ctx;
        ctx->bind();
        const uint32_t d = g->cfg.head_dim;
        const uint64_t weight_bytes = (uint64_t(d) * 2 + 15) / 16 * 16;
        std::vector<unsigned char> host(2 * weight_bytes + params.inverse_frequencies.size() * sizeof(float), 0);
        std::memcpy(host.data(), q_weight, size_t(d) * 2);
        std::memcpy(host.data() + weight_bytes, k_weight, size_t(d) * 2);
        std::memcpy(host.data() + 2 * weight_bytes, params.inverse_frequencies.data(),
                    params.inverse_frequencies.size() * sizeof(float));
        g->norm_rope.ensure(ctx, host.size(), false);
        cuda_check(cudaMemcpyAsync(g->norm_rope.ptr, host.data(), host.size(), cudaMemcpyHostToDevice, ctx->stream),
                   "cudaMemcpyAsync");  // pageable source: staged before the call returns
        g->norm_rope_cfg = *config;
        g->norm_rope_attention_factor = params.attention_factor;
        g->has_norm_rope = true;
    });
}

namespace {

// Fills everything of the front-stage launch that does not depend on where q, k, v and the gates come from.
PrepParams norm_rope_params(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer) {
    PrepParams p{};
    p.geo = page_geometry(g, pages, table, layer);
    const uint64_t weight_bytes = (uint64_t(g->cfg.head_dim) * 2 + 15) / 16 * 16;
    const auto* base = static_cast<const unsigned char*>(g->norm_rope.ptr);
    p.q_weight = base;
    p.k_weight = base + weight_bytes;
    p.inverse_frequencies = reinterpret_cast<const float*>(base + 2 * weight_bytes);
    p.attention_factor = g->norm_rope_attention_factor;
    p.eps = g->norm_rope_cfg.eps;
    p.rope_dim = g->norm_rope_cfg.rope_dim;
    p.num_q_heads = g->cfg.num_q_heads;
    p.dtype = g->cfg.dtype;
    p.req_slots = block_words(g, g->off_req_slots);
    p.flat_token_indices = block_words(g, g->off_token_indices);
    p.scalars = block_words(g, 0);
    p.num_total_tokens = g->shape.num_total_tokens;
    return p;
}

}  // namespace

int32_t psi_gqa_norm_rope_append(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* q_in,
                                 const void* k_in, const void* v_in, void* q_out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(g->prepared, "GQA batch metadata must be updated before recording");
        require(g->has_norm_rope, "psi_gqa_set_norm_rope must be called before psi_gqa_norm_rope_append");
        require(q_in != nullptr && k_in != nullptr && v_in != nullptr && q_out != nullptr, "buffers must not be null");
        g->ctx->bind();
        PrepParams p = norm_rope_params(g, pages, table, layer);
        p.q_in = q_in;
        p.k_in = k_in;
        p.v_in = v_in;
        p.q_out = q_out;
        p.q_head_stride = g->cfg.head_dim;
        p.q_token_stride = uint64_t(g->cfg.num_q_heads) * g->cfg.head_dim;
        p.kv_token_stride = uint64_t(g->cfg.num_kv_heads) * g->cfg.head_dim;
        LaunchScope scope(g->ctx, PSI_KERNEL_CLASS_NORM_ROPE_APPEND);
        cuda_check(launch_norm_rope_append(p, g->ctx->stream), "norm/rope/append launch");
    });
}

int32_t psi_gqa_projection_norm_rope_append(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer,
                                            const void* projection, uint32_t gated, void* q_out, void* gates_out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(g->prepared, "GQA batch metadata must be updated before recording");
        require(g->has_norm_rope, "psi_gqa_set_norm_rope must be called before psi_gqa_projection_norm_rope_append");
        require(projection != nullptr && q_out != nullptr, "buffers must not be null");
        require(gated <= 1, "gated must be 0 or 1");
        require(gated == 0 || gates_out != nullptr, "a gated projection needs gates_out");
        const uint64_t d = g->cfg.head_dim, hq = g->cfg.num_q_heads, hkv = g->cfg.num_kv_heads;
        const uint64_t q_width = (gated ? 2 : 1) * hq * d, width = q_width + 2 * hkv * d;
        // the reference's split shaders index one projection element per thread with a u32
        // (crates/inference-backend-metal/src/components/gqa_qgkv_split.rs:121-125, gqa_qkv_split.rs)
        require(uint64_t(g->shape.num_total_tokens) * width <= 0xFFFFFFFFull,
                gated ? "GQA projection elements exceeds the shader u32 count domain"
                      : "ungated GQA projection elements exceeds the shader u32 count domain");
        g->ctx->bind();
        PrepParams p = norm_rope_params(g, pages, table, layer);
        const uint64_t esz = dtype_bytes(g->cfg.dtype);
        const auto* base = static_cast<const unsigned char*>(projection);
        p.q_in = base;
        p.q_head_stride = gated ? 2 * d : d;
        p.q_token_stride = width;
        p.kv_token_stride = width;
        p.k_in = base + q_width * esz;
        p.v_in = base + (q_width + hkv * d) * esz;
        p.q_out = q_out;
        if (gated) {
            p.g_in = base + d * esz;  // head h of a token: q at h * 2D, its gate at h * 2D + D
            p.g_out = gates_out;
        }
        LaunchScope scope(g->ctx, PSI_KERNEL_CLASS_NORM_ROPE_APPEND);
        cuda_check(launch_norm_rope_append(p, g->ctx->stream), "projection split/norm/rope/append launch");
    });
}

int32_t psi_gqa_attend_gated(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* q,
                             const void* gates, void* out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(out != nullptr && gates != nullptr, "gates and out must not be null");
        require((reinterpret_cast<uintptr_t>(gates) & 7u) == 0, "gates must be 8-byte aligned");
        g->ctx->bind();
        AttendParams p = attend_params(g, pages, table, layer, q);
        p.out = out;
        p.gates = gates;
        run_attend(g, p);
    });
}

int32_t psi_gqa_device_status(psi_gqa* g, int32_t* out) {
    if (g == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        g->ctx->bind();
        cuda_check(cudaStreamSynchronize(g->ctx->stream), "cudaStreamSynchronize");
        uint32_t word = 0;
        if (g->status_word.ptr != nullptr) {
            cuda_check(cudaMemcpy(&word, g->status_word.ptr, sizeof(word), cudaMemcpyDeviceToHost), "cudaMemcpy");
            if (word != 0) cuda_check(cudaMemset(g->status_word.ptr, 0, sizeof(word)), "cudaMemset");
        }
        *out = static_cast<int32_t>(word);
    });
}

int32_t psi_page_gather(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t req_slot, uint32_t layer,
                        uint32_t tok_begin, uint32_t tok_end, void* k_out, void* v_out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(k_out != nullptr && v_out != nullptr, "gather outputs must not be null");
        require(tok_begin <= tok_end, "gather token range is reversed");
        g->ctx->bind();
        GatherParams p{};
        p.geo = page_geometry(g, pages, table, layer);
        require(req_slot < g->cfg.layout.num_req_slots, "GQA request page table req_slot out of range");
        require(uint64_t(tok_end) <= uint64_t(p.geo.pages_per_req) * g->tokens_per_page,
                "gather token range does not fit the request page table");
        p.req_slot = req_slot;
        p.tok_begin = tok_begin;
        p.tok_end = tok_end;
        p.k_out = k_out;
        p.v_out = v_out;
        if (tok_end > tok_begin) {
            LaunchScope scope(g->ctx, PSI_KERNEL_CLASS_GATHER);
            cuda_check(launch_page_gather(p, g->ctx->stream), "page gather launch");
        }
    });
}

}  // extern "C"
