// C++17 host-side mirror of the reference's component types over the C ABI of psi_cuda.h.
//
// The reference's boundary for this path is a set of Rust types (paths relative to the reference project root):
//   crates/inference-executor-metal/src/model/page_arena.rs                      PageArena
//   crates/inference-executor-metal/src/attn/gqa/request_page_table.rs           GQARequestPageTable
//   crates/inference-executor-core/src/attn/gqa/core.rs                          GQAPageTableLayout, GQAReplayShape
//   crates/inference-runtime-core/src/memory/u32_id_allocator.rs                 U32IDAllocator
//   crates/inference-executor-core/src/replay.rs                                 ReplayBucketPolicy
//   crates/inference-backend-metal/src/components/gqa_split_kv.rs                GQASplitKV, GQASplitKVVariant
//   crates/inference-executor-metal/src/attn/gqa/{backend,batch_metadata}.rs     GQA, GQAMetadataBuffers
// The classes below carry the same names, methods and argument meaning, own their handles (move-only, released in the
// destructor), and turn a failed call into psi::Error, whose what() is the library's message: for a violated contract
// that is the text of the reference's own assertion.  Everything is inline; link against libpsi_cuda.so.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "psi_cuda.h"

namespace psi {

using GQAPageTableLayout = psi_page_table_layout;
using GQAReplayShape = psi_replay_shape;
using GQASplitKVVariant = psi_split_kv_variant;
using GQAConfig = psi_gqa_config;
using NormRopeConfig = psi_norm_rope_config;

// A call that did not return PSI_OK.  The reference panics where this is thrown for PSI_ERR_INVALID_ARGUMENT.
class Error : public std::runtime_error {
public:
    Error(int32_t status, const std::string& message) : std::runtime_error(message), status_(status) {}
    int32_t status() const noexcept { return status_; }

private:
    int32_t status_;
};

namespace detail {

inline void check(int32_t status, psi_ctx* ctx = nullptr) {
    if (status == PSI_OK) return;
    char message[1024] = "";
    if (ctx != nullptr) (void)psi_ctx_last_error(ctx, message, sizeof message);
    if (message[0] == '\0') (void)psi_last_error(message, sizeof message);
    throw Error(status, message);
}

// Owner of one opaque handle: move-only, destroyed once.
template <typename T, int32_t (*Destroy)(T*)>
class Handle {
public:
    Handle() = default;
    explicit Handle(T* raw) : raw_(raw) {}
    Handle(Handle&& other) noexcept : raw_(std::exchange(other.raw_, nullptr)) {}
    Handle& operator=(Handle&& other) noexcept {
        if (this != &other) {
            reset();
            raw_ = std::exchange(other.raw_, nullptr);
        }
        return *this;
    }
    Handle(const Handle&) = delete;
    Handle& operator=(const Handle&) = delete;
    ~Handle() { reset(); }
    void reset() noexcept {
        if (raw_ != nullptr) (void)Destroy(std::exchange(raw_, nullptr));
    }
    T* get() const noexcept { return raw_; }

private:
    T* raw_ = nullptr;
};

}  // namespace detail

class ReplayProgram;

// Device + Stream of the reference (crates/inference-backend-metal/src/metal/device.rs, stream/mod.rs): one device,
// one stream, used from one host thread at a time.
class Context {
public:
    explicit Context(int32_t device = 0) {
        psi_ctx* raw = nullptr;
        detail::check(psi_ctx_create(device, &raw));
        handle_ = Owner(raw);
    }
    // On a stream the caller owns (a cudaStream_t).
    Context(int32_t device, void* cuda_stream) {
        psi_ctx* raw = nullptr;
        detail::check(psi_ctx_create_on_stream(device, cuda_stream, &raw));
        handle_ = Owner(raw);
    }
    psi_ctx* handle() const noexcept { return handle_.get(); }
    // ExecutionSubmission::wait
    void wait() { detail::check(psi_ctx_sync(handle()), handle()); }
    void* stream() const {
        void* out = nullptr;
        detail::check(psi_ctx_stream(handle(), &out), handle());
        return out;
    }
    int32_t sm_count() const {
        int32_t out = 0;
        detail::check(psi_ctx_sm_count(handle(), &out), handle());
        return out;
    }
    uint64_t launch_count() const {
        uint64_t out = 0;
        detail::check(psi_ctx_launch_count(handle(), &out), handle());
        return out;
    }
    // Stream::create_replay_program: the launches between the two calls become one replayable program.
    void capture_begin() { detail::check(psi_ctx_capture_begin(handle()), handle()); }
    inline ReplayProgram capture_end();

private:
    using Owner = detail::Handle<psi_ctx, psi_ctx_destroy>;
    Owner handle_;
};

// A captured launch sequence (one per bucket capacity and buffer set), replayed after each step's GQA::prepare.
class ReplayProgram {
public:
    ReplayProgram(psi_ctx* ctx, psi_graph* raw) : ctx_(ctx), handle_(raw) {}
    void launch() { detail::check(psi_graph_launch(handle_.get()), ctx_); }
    uint64_t kernel_count() const {
        uint64_t out = 0;
        detail::check(psi_graph_kernel_count(handle_.get(), &out), ctx_);
        return out;
    }

private:
    psi_ctx* ctx_;
    detail::Handle<psi_graph, psi_graph_destroy> handle_;
};

inline ReplayProgram Context::capture_end() {
    psi_graph* raw = nullptr;
    detail::check(psi_ctx_capture_end(handle(), &raw), handle());
    return ReplayProgram(handle(), raw);
}

// PageArena: num_pages x page_bytes of zero-filled device memory, or a view over memory the caller owns.
class PageArena {
public:
    PageArena(Context& ctx, uint64_t num_pages, uint32_t page_bytes) : ctx_(ctx.handle()) {
        psi_pages* raw = nullptr;
        detail::check(psi_pages_create(ctx_, num_pages, page_bytes, &raw), ctx_);
        handle_ = Owner(raw);
    }
    static PageArena wrap(Context& ctx, void* device_ptr, uint64_t num_pages, uint32_t page_bytes) {
        psi_pages* raw = nullptr;
        detail::check(psi_pages_wrap(ctx.handle(), device_ptr, num_pages, page_bytes, &raw), ctx.handle());
        return PageArena(ctx.handle(), raw);
    }
    psi_pages* handle() const noexcept { return handle_.get(); }
    void* buffer() const {
        void* out = nullptr;
        detail::check(psi_pages_device_ptr(handle(), &out), ctx_);
        return out;
    }
    void release_resources() { detail::check(psi_pages_release(handle()), ctx_); }
    void allocate_resources() { detail::check(psi_pages_allocate(handle()), ctx_); }
    void export_range(uint64_t page_begin, uint64_t page_end, void* host_out) const {
        detail::check(psi_pages_export_range(handle(), page_begin, page_end, host_out), ctx_);
    }
    void import_range(uint64_t page_begin, uint64_t page_end, const void* host_in) {
        detail::check(psi_pages_import_range(handle(), page_begin, page_end, host_in), ctx_);
    }

private:
    using Owner = detail::Handle<psi_pages, psi_pages_destroy>;
    PageArena(psi_ctx* ctx, psi_pages* raw) : ctx_(ctx), handle_(raw) {}
    psi_ctx* ctx_;
    Owner handle_;
};

// GQARequestPageTable: u32 [req_slot][layer][block][page id in block], zero-initialised.
class GQARequestPageTable {
public:
    GQARequestPageTable(Context& ctx, const GQAPageTableLayout& layout) : ctx_(ctx.handle()), layout_(layout) {
        psi_table* raw = nullptr;
        detail::check(psi_table_create(ctx_, &layout, &raw), ctx_);
        handle_ = Owner(raw);
    }
    psi_table* handle() const noexcept { return handle_.get(); }
    const GQAPageTableLayout& layout() const noexcept { return layout_; }
    void write_page_ids(uint32_t req_slot, uint32_t layer, uint32_t block, const std::vector<uint32_t>& page_ids) {
        detail::check(psi_table_write(handle(), req_slot, layer, block, page_ids.data(),
                                      static_cast<uint32_t>(page_ids.size())), ctx_);
    }
    std::vector<uint32_t> read_page_ids(uint32_t req_slot, uint32_t layer, uint32_t block) const {
        std::vector<uint32_t> out(layout_.num_page_ids_per_block);
        detail::check(psi_table_read(handle(), req_slot, layer, block, out.data(), static_cast<uint32_t>(out.size())), ctx_);
        return out;
    }
    void reset_req_slots(const std::vector<uint32_t>& req_slots) {
        detail::check(psi_table_reset_slots(handle(), req_slots.data(), static_cast<uint32_t>(req_slots.size())), ctx_);
    }
    void* page_ids_buffer() const {
        void* out = nullptr;
        detail::check(psi_table_device_ptr(handle(), &out), ctx_);
        return out;
    }
    // Every page ID written from now on must be below num_cache_pages (the check the reference makes where IDs enter
    // the table: crates/inference-executor-metal/src/model/qwen/v3_x/state/gqa.rs:97-102).
    void set_page_bound(uint64_t num_cache_pages) { detail::check(psi_table_set_page_bound(handle(), num_cache_pages), ctx_); }
    // A whole (slot, layer) row at once: num_blocks * num_page_ids_per_block entries.
    void write_row(uint32_t req_slot, uint32_t layer, const std::vector<uint32_t>& ids) {
        detail::check(psi_table_write_row(handle(), req_slot, layer, ids.data(), static_cast<uint32_t>(ids.size())), ctx_);
    }

private:
    using Owner = detail::Handle<psi_table, psi_table_destroy>;
    psi_ctx* ctx_;
    GQAPageTableLayout layout_;
    Owner handle_;
};

// U32IDAllocator: IDs freed earlier are handed out first, then never-used ones in ascending order.
class U32IDAllocator {
public:
    explicit U32IDAllocator(uint64_t capacity) {
        psi_id_allocator* raw = nullptr;
        detail::check(psi_id_allocator_create(capacity, &raw));
        handle_ = Owner(raw);
    }
    std::vector<uint32_t> alloc_many(uint64_t count) {
        std::vector<uint32_t> out(count);
        detail::check(psi_id_allocator_alloc_many(handle_.get(), count, out.data()));
        return out;
    }
    void free_many(const std::vector<uint32_t>& ids) {
        detail::check(psi_id_allocator_free_many(handle_.get(), ids.data(), ids.size()));
    }
    std::vector<uint64_t> allocated_ids_bitmap() const {
        uint64_t n = 0;
        detail::check(psi_id_allocator_bitmap(handle_.get(), nullptr, 0, &n));
        std::vector<uint64_t> out(n);
        detail::check(psi_id_allocator_bitmap(handle_.get(), out.data(), n, &n));
        return out;
    }
    uint64_t free_count() const {
        uint64_t out = 0;
        detail::check(psi_id_allocator_free_count(handle_.get(), &out));
        return out;
    }

private:
    using Owner = detail::Handle<psi_id_allocator, psi_id_allocator_destroy>;
    Owner handle_;
};

// ReplayBucketPolicy::with_topology_boundaries: host only.
class ReplayBucketPolicy {
public:
    ReplayBucketPolicy(uint32_t max_capacity, std::vector<uint32_t> topology_boundaries = {})
        : max_capacity_(max_capacity), boundaries_(std::move(topology_boundaries)) {
        (void)buckets();  // the constructor's checks
    }
    std::vector<uint32_t> buckets() const {
        uint64_t n = 0;
        std::vector<uint32_t> out(64);
        detail::check(psi_replay_bucket_policy(max_capacity_, boundaries_.data(), static_cast<uint32_t>(boundaries_.size()),
                                               out.data(), out.size(), &n));
        out.resize(n);
        return out;
    }
    uint32_t capacity(uint32_t active) const {
        uint32_t out = 0;
        detail::check(psi_replay_bucket_capacity(max_capacity_, boundaries_.data(), static_cast<uint32_t>(boundaries_.size()),
                                                 active, &out));
        return out;
    }

private:
    uint32_t max_capacity_;
    std::vector<uint32_t> boundaries_;
};

// GQASplitKV::new / new_dspark_history + select: host only.
class GQASplitKV {
public:
    GQASplitKV(uint32_t io_dtype, uint32_t page_bytes, uint32_t num_q_heads, uint32_t num_kv_heads, uint32_t head_dim,
               bool dspark_history = false)
        : io_dtype_(io_dtype), page_bytes_(page_bytes), num_q_heads_(num_q_heads), num_kv_heads_(num_kv_heads),
          head_dim_(head_dim), dspark_history_(dspark_history ? 1u : 0u) {}
    GQASplitKVVariant select(uint32_t num_tokens, uint32_t num_q_token_tiles, uint32_t* max_q_tokens_per_partial = nullptr) const {
        GQASplitKVVariant out{};
        detail::check(psi_split_kv_select(io_dtype_, page_bytes_, num_q_heads_, num_kv_heads_, head_dim_, dspark_history_,
                                          num_tokens, num_q_token_tiles, &out, max_q_tokens_per_partial));
        return out;
    }

private:
    uint32_t io_dtype_, page_bytes_, num_q_heads_, num_kv_heads_, head_dim_, dspark_history_;
};

// GQA + GQAMetadataBuffers + GQAScratch: the component that plans a step and records its launches.
class GQA {
public:
    GQA(Context& ctx, const GQAConfig& config) : ctx_(ctx.handle()), config_(config) {
        psi_gqa* raw = nullptr;
        detail::check(psi_gqa_create(ctx_, &config, &raw), ctx_);
        handle_ = Owner(raw);
    }
    psi_gqa* handle() const noexcept { return handle_.get(); }
    const GQAConfig& config() const noexcept { return config_; }

    void set_token_topology_boundaries(const std::vector<uint32_t>& boundaries) {
        detail::check(psi_gqa_set_token_topology_boundaries(handle(), boundaries.data(), static_cast<uint32_t>(boundaries.size())), ctx_);
    }
    // GQA::prepare / prepare_bucketed / prepare_bucketed_with_token_capacity (GQAMetadataBuffers::update*).
    GQAReplayShape prepare(const std::vector<uint32_t>& req_slots, const std::vector<uint32_t>& token_indices,
                           const std::vector<uint32_t>& cu_tokens) {
        return prepare_with(req_slots, token_indices, cu_tokens, PSI_CAPACITY_EXACT, 0);
    }
    GQAReplayShape prepare_bucketed(const std::vector<uint32_t>& req_slots, const std::vector<uint32_t>& token_indices,
                                    const std::vector<uint32_t>& cu_tokens) {
        return prepare_with(req_slots, token_indices, cu_tokens, PSI_CAPACITY_BUCKETED, 0);
    }
    GQAReplayShape prepare_bucketed_with_token_capacity(const std::vector<uint32_t>& req_slots,
                                                        const std::vector<uint32_t>& token_indices,
                                                        const std::vector<uint32_t>& cu_tokens, uint32_t num_total_tokens) {
        return prepare_with(req_slots, token_indices, cu_tokens, PSI_CAPACITY_CALLER_TOKENS, num_total_tokens);
    }
    GQASplitKVVariant split_kv_variant() const {
        GQASplitKVVariant out{};
        detail::check(psi_gqa_split_kv_variant(handle(), &out), ctx_);
        return out;
    }
    // GQAMetadataBuffers::req_slots() ... cu_kv_splits(): `which` is a psi_metadata_array.
    std::vector<uint32_t> metadata(uint32_t which, uint64_t offset, uint64_t count) const {
        std::vector<uint32_t> out(count);
        detail::check(psi_gqa_metadata_read(handle(), which, offset, out.data(), count), ctx_);
        return out;
    }
    // Fix every offset, scratch size and launch grid for max_tokens, so that a ReplayProgram stays valid.
    void reserve_replay() { detail::check(psi_gqa_reserve_replay(handle()), ctx_); }

    // GQAKVPageWrite::invoke_bucketed: k, v are device [num_total_tokens][Hkv][D].
    void kv_page_write(PageArena& pages, GQARequestPageTable& table, uint32_t layer, const void* k, const void* v) {
        detail::check(psi_gqa_kv_append(handle(), pages.handle(), table.handle(), layer, k, v), ctx_);
    }
    // SplitKV map + reduce over the paged cache: q, out are device [num_total_tokens][Hq][D].
    void attend(PageArena& pages, GQARequestPageTable& table, uint32_t layer, const void* q, void* out) {
        detail::check(psi_gqa_attend(handle(), pages.handle(), table.handle(), layer, q, out), ctx_);
    }
    // GQA::record's kv_page_write -> barrier -> SplitKV map -> reduce as one launch.
    void record(PageArena& pages, GQARequestPageTable& table, uint32_t layer, const void* k, const void* v, const void* q,
                void* out) {
        detail::check(psi_gqa_append_attend(handle(), pages.handle(), table.handle(), layer, k, v, q, out), ctx_);
    }
    // The same with the activation gate of backend.rs:613-624 in the epilogue (attention only; append separately).
    void attend_gated(PageArena& pages, GQARequestPageTable& table, uint32_t layer, const void* q, const void* gates,
                      void* out) {
        detail::check(psi_gqa_attend_gated(handle(), pages.handle(), table.handle(), layer, q, gates, out), ctx_);
    }
    // One prepared step through host buffers (blocking), and update + step in one call.
    void decode_step_host(PageArena& pages, GQARequestPageTable& table, uint32_t layer, const void* k_host,
                          const void* v_host, const void* q_host, void* out_host) {
        detail::check(psi_gqa_decode_step_host(handle(), pages.handle(), table.handle(), layer, k_host, v_host, q_host, out_host), ctx_);
    }
    void step_host(PageArena& pages, GQARequestPageTable& table, uint32_t layer, const std::vector<uint32_t>& req_slots,
                   const std::vector<uint32_t>& token_indices, const std::vector<uint32_t>& cu_tokens, const void* k_host,
                   const void* v_host, const void* q_host, void* out_host) {
        require_batch(req_slots, token_indices, cu_tokens);
        detail::check(psi_gqa_step_host(handle(), pages.handle(), table.handle(), layer, req_slots.data(), token_indices.data(),
                                        cu_tokens.data(), static_cast<uint32_t>(req_slots.size()), k_host, v_host, q_host,
                                        out_host), ctx_);
    }
    // Waits for the stream, then returns and clears what a bounded device-side wait or bounds check recorded (0: nothing).
    int32_t device_status() {
        int32_t out = 0;
        detail::check(psi_gqa_device_status(handle(), &out), ctx_);
        return out;
    }

private:
    using Owner = detail::Handle<psi_gqa, psi_gqa_destroy>;
    static void require_batch(const std::vector<uint32_t>& req_slots, const std::vector<uint32_t>& token_indices,
                              const std::vector<uint32_t>& cu_tokens) {
        if (req_slots.size() != token_indices.size() || cu_tokens.size() != req_slots.size() + 1) {
            throw Error(PSI_ERR_INVALID_ARGUMENT, "req_slots, token_indices and cu_tokens lengths disagree");
        }
    }
    GQAReplayShape prepare_with(const std::vector<uint32_t>& req_slots, const std::vector<uint32_t>& token_indices,
                                const std::vector<uint32_t>& cu_tokens, uint32_t capacity_mode, uint32_t caller_tokens) {
        require_batch(req_slots, token_indices, cu_tokens);
        GQAReplayShape shape{};
        detail::check(psi_gqa_prepare(handle(), req_slots.data(), token_indices.data(), cu_tokens.data(),
                                      static_cast<uint32_t>(req_slots.size()), capacity_mode, caller_tokens, &shape), ctx_);
        return shape;
    }
    psi_ctx* ctx_;
    GQAConfig config_;
    Owner handle_;
};

}  // namespace psi
