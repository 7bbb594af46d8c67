// C ABI: partial outputs, their merge, and the KV-range exchange between devices.
#include "api_internal.hpp"

using namespace psi;

extern "C" {

int32_t psi_gqa_attend_partial(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* q, float* o,
                               float* m, float* l) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(o != nullptr && m != nullptr && l != nullptr, "partial outputs must not be null");
        require((reinterpret_cast<uintptr_t>(o) & 15u) == 0, "partial output o must be 16-byte aligned");
        g->ctx->bind();
        AttendParams p = attend_params(g, pages, table, layer, q);
        p.ext_o = o;
        p.ext_m = m;
        p.ext_l = l;
        run_attend(g, p);
    });
}

static int32_t combine_impl(psi_gqa* g, const float* const* o, const float* const* m, const float* const* l, uint32_t n,
                            uint32_t num_tokens, void* out, const uint32_t* flags, uint32_t flag_value,
                            uint32_t max_polls) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(o != nullptr && m != nullptr && l != nullptr && out != nullptr, "combine arguments must not be null");
        require(n > 0 && n <= 64, "combine takes between 1 and 64 partials");
        require(num_tokens > 0 && num_tokens <= g->cfg.max_tokens, "combine token count out of range");
        psi_ctx* ctx = g->ctx;
        ctx->bind();
        g->combine_ptrs.ensure(ctx, 3 * 64 * sizeof(void*), false);
        std::vector<const float*> host(3 * 64, nullptr);
        for (uint32_t i = 0; i < n; ++i) {
            require(o[i] != nullptr && m[i] != nullptr && l[i] != nullptr, "combine partial pointers must not be null");
            host[i] = o[i];
            host[64 + i] = m[i];
            host[128 + i] = l[i];
        }
        // Pageable source: the runtime stages the bytes before the call returns, so `host` may go out of scope.
        cuda_check(cudaMemcpyAsync(g->combine_ptrs.ptr, host.data(), host.size() * sizeof(void*),
                                   cudaMemcpyHostToDevice, ctx->stream),
                   "cudaMemcpyAsync");
        CombineParams p{};
        auto* base = static_cast<const float* const*>(g->combine_ptrs.ptr);
        p.o = base;
        p.m = base + 64;
        p.l = base + 128;
        p.n = n;
        p.num_rows = num_tokens * g->cfg.num_q_heads;
        p.head_dim = g->cfg.head_dim;
        p.dtype = g->cfg.dtype;
        p.out = out;
        if (flags != nullptr) {
            g->status_word.ensure(ctx, sizeof(uint32_t), true);
            p.flags = flags;
            p.flag_value = flag_value;
            p.max_polls = max_polls == 0 ? 2000000u : max_polls;  // ~100 ns per poll: a fraction of a second by default
            p.status = static_cast<uint32_t*>(g->status_word.ptr);
            g->sync_words.ensure(ctx, kSyncWordCount * sizeof(uint32_t), true);
            p.sync_words = static_cast<uint32_t*>(g->sync_words.ptr);
        }
        LaunchScope scope(ctx, PSI_KERNEL_CLASS_COMBINE);
        cuda_check(launch_combine(p, ctx->stream), "combine launch");
    });
}

int32_t psi_gqa_block_partial(psi_gqa* g, const void* q, const void* local_k, const void* local_v, uint32_t num_tokens,
                              uint32_t block_size, const uint32_t* slot_indices, float* o, float* m, float* l) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(q != nullptr && local_k != nullptr && local_v != nullptr, "q, local_k and local_v must not be null");
        require(o != nullptr && m != nullptr && l != nullptr, "partial outputs must not be null");
        require(block_size > 0 && block_size <= 256, "GQA block SDPA block size must be in 1..=256");
        require(num_tokens > 0, "GQA block SDPA requires tokens");
        require(num_tokens % block_size == 0, "GQA block SDPA tokens must contain complete request blocks");
        g->ctx->bind();
        BlockPartialParams p{};
        p.q = q;
        p.local_k = local_k;
        p.local_v = local_v;
        p.slot_indices = slot_indices;
        p.o = o;
        p.m = m;
        p.l = l;
        p.num_tokens = num_tokens;
        p.block_size = block_size;
        p.num_q_heads = g->cfg.num_q_heads;
        p.num_kv_heads = g->cfg.num_kv_heads;
        p.head_dim = g->cfg.head_dim;
        p.dtype = g->cfg.dtype;
        p.scale = g->cfg.scale;
        g->ctx->launches += 1;
        cuda_check(launch_block_partial(p, g->ctx->stream), "block partial launch");
    });
}

int32_t psi_gqa_combine(psi_gqa* g, const float* const* o, const float* const* m, const float* const* l, uint32_t n,
                        uint32_t num_tokens, void* out) {
    return combine_impl(g, o, m, l, n, num_tokens, out, nullptr, 0, 0);
}

int32_t psi_gqa_combine_wait(psi_gqa* g, const float* const* o, const float* const* m, const float* const* l,
                             uint32_t n, uint32_t num_tokens, void* out, const uint32_t* flags, uint32_t flag_value,
                             uint32_t max_polls) {
    if (flags == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return combine_impl(g, o, m, l, n, num_tokens, out, flags, flag_value, max_polls);
}

int32_t psi_gqa_signal(psi_gqa* g, uint32_t* flag, uint32_t value) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(flag != nullptr, "flag must not be null");
        g->ctx->bind();
        g->ctx->launches += 1;
        cuda_check(launch_signal(flag, value, g->ctx->stream), "signal launch");
    });
}

int32_t psi_gqa_attend_exchange(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k,
                                const void* v, const void* q, const psi_kv_exchange* exchange, void* out) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(exchange != nullptr, "exchange must not be null");
        const psi_kv_exchange& e = *exchange;
        require(e.world >= 1 && e.world <= 64 && e.rank < e.world && e.owner < e.world,
                "exchange rank, owner and world are out of range");
        require(e.step >= 1, "exchange steps count from 1");
        require(e.slots != nullptr && e.flags != nullptr && e.consumed != nullptr, "exchange buffers must not be null");
        require((k == nullptr) == (v == nullptr), "k and v come together or not at all");
        const bool is_owner = e.rank == e.owner;
        require(!is_owner || out != nullptr, "the owner of the exchange needs an output buffer");
        psi_ctx* ctx = g->ctx;
        require(!ctx->capturing, "the exchange carries a step counter and stays outside captured graphs");
        ctx->bind();
        AttendParams p = attend_params(g, pages, table, layer, q);
        const uint64_t rows = uint64_t(g->shape.num_tokens) * g->cfg.num_q_heads;
        const uint64_t floats = rows * (uint64_t(g->cfg.head_dim) + 2);
        require(e.slot_floats >= floats && e.slot_floats % 4 == 0,
                "exchange slot_floats must hold T * Hq * (D + 2) floats and be a multiple of 4");
        require((reinterpret_cast<uintptr_t>(e.slots) & 15u) == 0, "exchange slots must be 16-byte aligned");
        g->status_word.ensure(ctx, sizeof(uint32_t), true);
        g->sync_words.ensure(ctx, kSyncWordCount * sizeof(uint32_t), true);

        float* parity_base = e.slots + uint64_t(e.step & 1u) * e.world * e.slot_floats;
        float* slot = parity_base + uint64_t(e.rank) * e.slot_floats;
        ExchangeParams x{};
        x.flag = e.flags + e.rank;
        x.consumed = e.consumed;
        x.sync_words = static_cast<uint32_t*>(g->sync_words.ptr);
        x.recv = is_owner ? parity_base : nullptr;
        x.flags = is_owner ? e.flags : nullptr;
        x.consumed_local = is_owner ? e.consumed : nullptr;
        x.slot_stride = e.slot_floats;
        x.world = e.world;
        x.step = e.step;
        x.max_polls = e.max_polls == 0 ? 2000000u : e.max_polls;
        x.num_rows = static_cast<uint32_t>(rows);
        p.status = static_cast<uint32_t*>(g->status_word.ptr);

        require(g->plan.num_ctas() + g->chunk.num_ctas() > 0,
                "the rank's slice of the KV range is empty: a rank without keys has nothing to publish and must be left "
                "out of the exchange group");
        const bool fused = g->kernel == PSI_KERNEL_MMA && g->chunk.num_ctas() == 0 && !g->replay_reserved;
        if (fused) {
            if (k != nullptr) {
                require((reinterpret_cast<uintptr_t>(k) & 15u) == 0 && (reinterpret_cast<uintptr_t>(v) & 15u) == 0,
                        "k and v must be 16-byte aligned");
                p.new_k = k;
                p.new_v = v;
            }
            p.ext_o = slot;
            p.ext_m = slot + rows * g->cfg.head_dim;
            p.ext_l = p.ext_m + rows;
            p.out = out;
            p.xchg = x;
            run_attend(g, p);
            return;
        }
        // Three launches: the ordinary attention into local scratch, the push with the flag, the owner's wait and merge.
        if (k != nullptr) run_append(g, pages, table, layer, k, v);
        g->xchg_local.ensure(ctx, e.slot_floats * sizeof(float), false);
        float* local = static_cast<float*>(g->xchg_local.ptr);
        p.ext_o = local;
        p.ext_m = local + rows * g->cfg.head_dim;
        p.ext_l = p.ext_m + rows;
        run_attend(g, p);
        {
            LaunchScope scope(ctx, PSI_KERNEL_CLASS_COMBINE);
            cuda_check(launch_exchange_push(x, local, slot, (floats + 3) / 4 * 4, p.status, ctx->stream), "exchange push launch");
        }
        if (is_owner) {
            LaunchScope scope(ctx, PSI_KERNEL_CLASS_COMBINE);
            cuda_check(launch_exchange_merge(x, out, g->cfg.dtype, g->cfg.head_dim, p.status,
                                             static_cast<uint32_t>(ctx->sm_count), ctx->stream),
                       "exchange merge launch");
        }
    });
}

}  // extern "C"
