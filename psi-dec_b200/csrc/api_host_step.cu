// C ABI: one decode step from host buffers (plan, transfers, append, attention, result) in one call.
#include "api_internal.hpp"

using namespace psi;

namespace {

// A large step with long query runs from pinned host buffers, cut into groups of consecutive requests.  Group i's
// q/k/v travel on one copy stream while group i-1 is planned and launched on the context's stream and group i-2's
// output travels back on a second copy stream, so the step takes about as long as the slowest of the three (on these
// boxes the inbound transfer) instead of their sum.  Every group is a step of its own for the kernels: its own plan,
// token offsets relative to its first token.
void run_pipelined_host_step(psi_gqa* g, psi_pages* pages, psi_table* table, uint32_t layer, const uint32_t* req_slots,
                             const uint32_t* token_indices, const uint32_t* cu_tokens, uint32_t num_reqs,
                             const void* k_host, const void* v_host, const void* q_host, void* out_host) {
    psi_ctx* ctx = g->ctx;
    const uint64_t esz = dtype_bytes(g->cfg.dtype);
    const uint64_t kv_row = uint64_t(g->cfg.num_kv_heads) * g->cfg.head_dim * esz;
    const uint64_t q_row = uint64_t(g->cfg.num_q_heads) * g->cfg.head_dim * esz;
    const uint32_t num_tokens = cu_tokens[num_reqs];
    const uint64_t in_bytes = uint64_t(num_tokens) * (q_row + 2 * kv_row);
    const uint32_t groups = static_cast<uint32_t>(
        std::min<uint64_t>(std::min<uint64_t>(kPipelineMaxGroups, num_reqs), std::max<uint64_t>(2, in_bytes / kPipelineGroupBytes)));
    // group boundaries (request indices): equal shares of the step's tokens, i.e. of its transfer bytes
    std::vector<uint32_t> first_req(groups + 1, num_reqs);
    first_req[0] = 0;
    for (uint32_t i = 1, r = 0; i < groups; ++i) {
        const uint64_t target = uint64_t(num_tokens) * i / groups;
        while (r < num_reqs && cu_tokens[r] < target) ++r;
        first_req[i] = std::max(r, first_req[i - 1]);
    }

    if (g->pipe_h2d == nullptr) cuda_check(cudaStreamCreateWithFlags(&g->pipe_h2d, cudaStreamNonBlocking), "cudaStreamCreate");
    if (g->pipe_d2h == nullptr) cuda_check(cudaStreamCreateWithFlags(&g->pipe_d2h, cudaStreamNonBlocking), "cudaStreamCreate");
    while (g->pipe_events.size() < 2 * kPipelineMaxGroups + 1) {
        cudaEvent_t e = nullptr;
        cuda_check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
        g->pipe_events.push_back(e);
    }
    g->step_out.ensure(ctx, uint64_t(g->cfg.max_tokens) * q_row, false);
    // the copy streams start behind whatever the context's stream still holds (an earlier step that reads the staging)
    cudaEvent_t entry = g->pipe_events[2 * kPipelineMaxGroups];
    cuda_check(cudaEventRecord(entry, ctx->stream), "cudaEventRecord");
    cuda_check(cudaStreamWaitEvent(g->pipe_h2d, entry, 0), "cudaStreamWaitEvent");
    cuda_check(cudaStreamWaitEvent(g->pipe_d2h, entry, 0), "cudaStreamWaitEvent");

    // Whatever happens below, no copy that names the caller's buffers is left in flight when the call returns.
    struct Drain {
        psi_gqa* g;
        ~Drain() {
            (void)cudaStreamSynchronize(g->pipe_h2d);
            (void)cudaStreamSynchronize(g->ctx->stream);
            (void)cudaStreamSynchronize(g->pipe_d2h);
        }
    } drain{g};
    auto at = [](const void* base, uint64_t offset) { return static_cast<const unsigned char*>(base) + offset; };
    auto at_mut = [](void* base, uint64_t offset) { return static_cast<unsigned char*>(base) + offset; };
    for (uint32_t i = 0; i < groups; ++i) {  // all inbound copies are queued first: the copy engine never waits for the host
        const uint32_t tok0 = cu_tokens[first_req[i]], ntok = cu_tokens[first_req[i + 1]] - tok0;
        if (ntok == 0) continue;
        cuda_check(cudaMemcpyAsync(at_mut(g->step_q.ptr, tok0 * q_row), at(q_host, tok0 * q_row), ntok * q_row,
                                   cudaMemcpyHostToDevice, g->pipe_h2d), "H2D q");
        cuda_check(cudaMemcpyAsync(at_mut(g->step_k.ptr, tok0 * kv_row), at(k_host, tok0 * kv_row), ntok * kv_row,
                                   cudaMemcpyHostToDevice, g->pipe_h2d), "H2D k");
        cuda_check(cudaMemcpyAsync(at_mut(g->step_v.ptr, tok0 * kv_row), at(v_host, tok0 * kv_row), ntok * kv_row,
                                   cudaMemcpyHostToDevice, g->pipe_h2d), "H2D v");
        cuda_check(cudaEventRecord(g->pipe_events[i], g->pipe_h2d), "cudaEventRecord");
    }
    std::vector<uint32_t> group_cu;
    for (uint32_t i = 0; i < groups; ++i) {
        const uint32_t r0 = first_req[i], r1 = first_req[i + 1];
        const uint32_t tok0 = cu_tokens[r0], ntok = cu_tokens[r1] - tok0;
        if (ntok == 0) continue;
        group_cu.assign(r1 - r0 + 1, 0);
        for (uint32_t r = r0; r <= r1; ++r) group_cu[r - r0] = cu_tokens[r] - tok0;
        prepare_impl(g, req_slots + r0, token_indices + r0, group_cu.data(), r1 - r0, PSI_CAPACITY_EXACT, 0, nullptr,
                     false, nullptr, /*plan_only=*/true);
        cuda_check(cudaStreamWaitEvent(ctx->stream, g->pipe_events[i], 0), "cudaStreamWaitEvent");
        AttendParams p = attend_params(g, pages, table, layer, at_mut(g->step_q.ptr, tok0 * q_row));
        p.out = at_mut(g->step_out.ptr, tok0 * q_row);
        p.new_k = at_mut(g->step_k.ptr, tok0 * kv_row);
        p.new_v = at_mut(g->step_v.ptr, tok0 * kv_row);
        run_attend(g, p);
        cudaEvent_t done = g->pipe_events[kPipelineMaxGroups + i];
        cuda_check(cudaEventRecord(done, ctx->stream), "cudaEventRecord");
        cuda_check(cudaStreamWaitEvent(g->pipe_d2h, done, 0), "cudaStreamWaitEvent");
        cuda_check(cudaMemcpyAsync(at_mut(out_host, tok0 * q_row), at(g->step_out.ptr, tok0 * q_row), ntok * q_row,
                                   cudaMemcpyDeviceToHost, g->pipe_d2h), "D2H out");
    }
    cuda_check(cudaStreamSynchronize(g->pipe_d2h), "cudaStreamSynchronize");
    cuda_check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
    g->prepared = false;  // the last plan covers the last group only
}

}  // namespace

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
        if (!direct && q_bytes + 2 * kv_bytes >= kPipelineHostBytes && num_reqs >= 2 && !g->replay_reserved &&
            g->cfg.plan_mode == PSI_PLAN_BALANCED) {
            run_pipelined_host_step(g, pages, table, layer, req_slots, token_indices, cu_tokens, num_reqs, k_host, v_host,
                                    q_host, out_host);
            return;
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
