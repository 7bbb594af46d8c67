// C ABI: one decode step from host buffers (plan, transfers, append, attention, result) in one call.
#include "api_internal.hpp"

using namespace psi;

extern "C" {

int32_t psi_gqa_decode_step_host(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const void* k_host,
                                 const void* v_host, const void* q_host, void* out_host) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(k_host != nullptr && v_host != nullptr && q_host != nullptr && out_host != nullptr,
                "host buffers must not be null");
        require(g->prepared, "GQA batch metadata must be updated before recording");
        psi_ctx* ctx = g->ctx;
        ctx->bind();
        const uint64_t esz = dtype_bytes(g->cfg.dtype);
        const uint64_t kv_cap = uint64_t(g->cfg.max_tokens) * g->cfg.num_kv_heads * g->cfg.head_dim * esz;
        const uint64_t q_cap = uint64_t(g->cfg.max_tokens) * g->cfg.num_q_heads * g->cfg.head_dim * esz;
        const uint64_t kv_bytes = uint64_t(g->shape.num_tokens) * g->cfg.num_kv_heads * g->cfg.head_dim * esz;
        const uint64_t q_bytes = uint64_t(g->shape.num_tokens) * g->cfg.num_q_heads * g->cfg.head_dim * esz;
        g->step_k.ensure(ctx, kv_cap, false);
        g->step_v.ensure(ctx, kv_cap, false);
        g->step_q.ensure(ctx, q_cap, false);
        // Pinned, device-mapped host buffers: one launch pulls q/k/v over the host link into device staging (small
        // steps: every work item waits for its query rows, which come sooner from HBM than from the host), and the
        // attention launch stores `out` straight into the host buffer.  Two launches and one wait, no copy engine
        // round trips.
        if (g->kernel == PSI_KERNEL_MMA && kv_bytes % 16 == 0 && q_bytes % 16 == 0) {
            void* dk = mapped_device_pointer(k_host);
            void* dv = mapped_device_pointer(v_host);
            void* dq = mapped_device_pointer(q_host);
            void* dout = mapped_device_pointer(out_host);
            if (dk != nullptr && dv != nullptr && dq != nullptr && dout != nullptr) {
                // the size rule of psi_gqa_step_host: large steps without long query runs are read in place
                const bool direct = q_bytes + 2 * kv_bytes >= kDirectHostBytes && !g->replay_reserved &&
                                    g->chunk.num_ctas() == 0;
                if (!direct) {
                    const void* const src[kPullBuffers] = {dq, dk, dv, nullptr};
                    void* const dst[kPullBuffers] = {g->step_q.ptr, g->step_k.ptr, g->step_v.ptr, nullptr};
                    const uint64_t bytes[kPullBuffers] = {q_bytes, kv_bytes, kv_bytes, 0};
                    ctx->launches += 1;
                    cuda_check(launch_host_pull(src, dst, bytes, ctx->stream), "host pull launch");
                }
                AttendParams p = attend_params(g, pages, table, layer, direct ? dq : g->step_q.ptr);
                p.out = dout;
                p.new_k = direct ? dk : g->step_k.ptr;
                p.new_v = direct ? dv : g->step_v.ptr;
                run_attend(g, p);
                cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
                return;
            }
        }
        run_staged_host_step(g, pages, table, layer, k_host, v_host, q_host, out_host, kv_bytes, q_bytes, q_cap);
    });
}

int32_t psi_gqa_step_host(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const uint32_t* req_slots,
                          const uint32_t* token_indices, const uint32_t* cu_tokens, uint32_t num_reqs, const void* k_host,
                          const void* v_host, const void* q_host, void* out_host) {
    if (g == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(g->ctx, [&] {
        require(k_host != nullptr && v_host != nullptr && q_host != nullptr && out_host != nullptr,
                "host buffers must not be null");
        require(req_slots != nullptr && token_indices != nullptr && cu_tokens != nullptr, "metadata inputs must not be null");
        require(num_reqs > 0, "GQA batch metadata requires tokens");
        psi_ctx* ctx = g->ctx;
        require(!ctx->capturing, "psi_gqa_step_host waits for its result and stays outside captured graphs");
        ctx->bind();
        const uint32_t num_tokens = cu_tokens[num_reqs];
        require(num_tokens > 0, "GQA batch metadata requires tokens");
        require(num_tokens <= g->cfg.max_tokens, "GQA batch exceeds the metadata token capacity");
        const uint64_t esz = dtype_bytes(g->cfg.dtype);
        const uint64_t kv_cap = uint64_t(g->cfg.max_tokens) * g->cfg.num_kv_heads * g->cfg.head_dim * esz;
        const uint64_t q_cap = uint64_t(g->cfg.max_tokens) * g->cfg.num_q_heads * g->cfg.head_dim * esz;
        const uint64_t kv_bytes = uint64_t(num_tokens) * g->cfg.num_kv_heads * g->cfg.head_dim * esz;
        const uint64_t q_bytes = uint64_t(num_tokens) * g->cfg.num_q_heads * g->cfg.head_dim * esz;
        g->step_k.ensure(ctx, kv_cap, false);
        g->step_v.ensure(ctx, kv_cap, false);
        g->step_q.ensure(ctx, q_cap, false);
        void *dk = nullptr, *dv = nullptr, *dq = nullptr, *dout = nullptr;
        bool in_place = g->kernel == PSI_KERNEL_MMA && kv_bytes % 16 == 0 && q_bytes % 16 == 0;
        if (in_place) {
            dk = mapped_device_pointer(k_host);
            dv = mapped_device_pointer(v_host);
            dq = mapped_device_pointer(q_host);
            dout = mapped_device_pointer(out_host);
            in_place = dk != nullptr && dv != nullptr && dq != nullptr && dout != nullptr;
        }
        if (!in_place) {  // pageable buffers or the generic kernel: the two calls this one stands for
            prepare_impl(g, req_slots, token_indices, cu_tokens, num_reqs, PSI_CAPACITY_EXACT, 0, nullptr, false, nullptr);
            run_staged_host_step(g, pages, table, layer, k_host, v_host, q_host, out_host, kv_bytes, q_bytes, q_cap);
            return;
        }
        // Small steps pull q/k/v into device staging.  From
        // kDirectHostBytes on, that pull would sit in front of the attention for longer than the attention loses by
        // fetching each item's query rows and the step's K/V rows over the host link itself, so the launch reads the
        // host buffers in place and the transfer hides under the K/V stream (256 verify tokens of 24/4 heads, 5.2 MB:
        // 853 -> 778 us per step; 32 decode tokens, 0.33 MB: no difference).  Long query runs keep the staged path:
        // their kernel takes q and the appended rows through device memory.
        bool direct = q_bytes + 2 * kv_bytes >= kDirectHostBytes && !g->replay_reserved;
        if (direct && g->chunk_supported) {
            for (uint32_t r = 0; r < num_reqs && direct; ++r) {
                const uint32_t tiles = (cu_tokens[r + 1] - cu_tokens[r] + g->geo.tokens_per_tile - 1) / g->geo.tokens_per_tile;
                if (tiles >= kChunkMinTiles) direct = false;
            }
        }
        // The step is planned first; then ONE launch pulls the packed plan from its pinned staging buffer together with
        // q/k/v (or the plan alone when q/k/v are read in place), and the attention launch stores `out` straight into
        // the host buffer.
        uint64_t words = 0;
        prepare_impl(g, req_slots, token_indices, cu_tokens, num_reqs, PSI_CAPACITY_EXACT, 0, nullptr, true, &words);
        const uint64_t padded_words = (words + 3) / 4 * 4;
        void* staging_dev = nullptr;
        const bool plan_mapped = padded_words <= g->staging_words &&
                                 cudaHostGetDevicePointer(&staging_dev, g->staging, 0) == cudaSuccess &&
                                 staging_dev != nullptr && (reinterpret_cast<uintptr_t>(staging_dev) & 15u) == 0;
        if (!plan_mapped) {
            (void)cudaGetLastError();
            cuda_check(cudaMemcpyAsync(g->block.ptr, g->staging, words * sizeof(uint32_t), cudaMemcpyHostToDevice,
                                       ctx->stream), "cudaMemcpyAsync");
        }
        if (plan_mapped || !direct) {
            const void* const src[kPullBuffers] = {direct ? nullptr : dq, direct ? nullptr : dk, direct ? nullptr : dv,
                                                   plan_mapped ? staging_dev : nullptr};
            void* const dst[kPullBuffers] = {g->step_q.ptr, g->step_k.ptr, g->step_v.ptr, g->block.ptr};
            const uint64_t bytes[kPullBuffers] = {direct ? 0 : q_bytes, direct ? 0 : kv_bytes, direct ? 0 : kv_bytes,
                                                  plan_mapped ? padded_words * sizeof(uint32_t) : 0};
            ctx->launches += 1;
            cuda_check(launch_host_pull(src, dst, bytes, ctx->stream), "host pull launch");
        }
        cuda_check(cudaEventRecord(g->upload_done, ctx->stream), "cudaEventRecord");
        AttendParams p = attend_params(g, pages, table, layer, direct ? dq : g->step_q.ptr);
        p.out = dout;
        p.new_k = direct ? dk : g->step_k.ptr;
        p.new_v = direct ? dv : g->step_v.ptr;
        run_attend(g, p);
        cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
    });
}

}  // extern "C"
