/*
 * psi_cuda.h - C ABI of the B200 (sm_100a) backend for psi-dec's paged GQA decode path.
 *
 * The reference has no FFI for this path: its boundary is the set of Rust component types of
 * crates/inference-backend-metal (GQAKVPageWrite, GQASplitKVSingleQ/TiledQ kernels, GQASplitKV selector) and the
 * executor-side owners in crates/inference-executor-metal (GQARequestPageTable, PageArena, GQAMetadataBuffers,
 * GQA::record).  A Rust crate `inference-backend-cuda` binds the functions below with `extern "C"` declarations and
 * re-creates those component types on top of them; every entry point names the reference interface it stands in for
 * (paths relative to the reference project root).
 *
 * Conventions
 *   - every function returns a psi_status (0 = PSI_OK); nothing throws or aborts across the boundary.  The reference
 *     panics on violated invariants; here the same checks run on the host before any launch and come back as
 *     PSI_ERR_INVALID_ARGUMENT, with the message available from psi_ctx_last_error / psi_last_error.
 *   - a psi_ctx is bound to one device and one stream and is used from one host thread at a time (the reference
 *     executor is one thread with one in-flight submission per stream).  Calls enqueue work on the context's stream
 *     and return; only psi_ctx_sync, the *_read / *_export functions, psi_gqa_decode_step_host and psi_gqa_step_host block.
 *   - device data layouts are the reference's, row-major, innermost last:
 *       q, out        dtype [T][Hq][D]
 *       k, v (append) dtype [T][Hkv][D]
 *       pages         dtype [num_pages][2 (K,V)][Hkv][tokens_per_page][D]
 *       page table    u32   [num_req_slots][num_gqa_layers][num_blocks][num_page_ids_per_block]
 *   - there is no CPU fallback: every compute entry point needs a CUDA device.
 */
#ifndef PSI_CUDA_H
#define PSI_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define PSI_API __attribute__((visibility("default")))
#else
#define PSI_API
#endif

typedef struct psi_ctx psi_ctx;
typedef struct psi_pages psi_pages;
typedef struct psi_table psi_table;
typedef struct psi_gqa psi_gqa;
typedef struct psi_id_allocator psi_id_allocator;

typedef enum psi_status {
    PSI_OK = 0,
    PSI_ERR_INVALID_ARGUMENT = 1,   /* a contract the reference asserts (shape, index domain, capacity) */
    PSI_ERR_RESOURCE_EXHAUSTED = 2, /* "not enough ID", out of device memory */
    PSI_ERR_INTERNAL = 3,
    PSI_ERR_TIMEOUT = 4, /* a bounded device-side wait gave up */
    PSI_ERR_CUDA = 5,    /* a CUDA runtime call failed; the message holds the CUDA error string */
    PSI_ERR_PAGE_ID = 6  /* checked build of the library only (libpsi_cuda_checked.so): a kernel met a page ID or
                            table index out of bounds; that access was skipped (reads go to page 0 instead) and the
                            launch's results are not valid; from psi_gqa_device_status */
} psi_status;

/* Storage dtype of q/k/v/out and of the page arena.  F32 and BF16 are the reference's dtypes
 * (crates/inference-backend-metal/src/components/gqa_split_kv_single_q.rs:73); F16 is an extension with the same
 * semantics. */
typedef enum psi_dtype { PSI_DTYPE_F32 = 0, PSI_DTYPE_BF16 = 1, PSI_DTYPE_F16 = 2 } psi_dtype;

/* crates/inference-executor-core/src/attn/gqa/core.rs:145-159 (GQAPageTableLayout) */
typedef struct psi_page_table_layout {
    uint32_t num_req_slots;
    uint32_t num_gqa_layers;
    uint32_t num_blocks;
    uint32_t num_page_ids_per_block;
} psi_page_table_layout;

/* crates/inference-executor-core/src/attn/gqa/core.rs:93-143 (GQAReplayShape) */
typedef struct psi_replay_shape {
    uint32_t num_tokens;
    uint32_t num_total_tokens;
    uint32_t num_q_token_tiles;
    uint32_t num_total_q_token_tiles;
    uint32_t num_sdpa_map_task_templates;
    uint32_t num_total_sdpa_map_task_templates;
    uint32_t reduce_sdpa_partial_outputs; /* bool */
} psi_replay_shape;

/* crates/inference-backend-metal/src/components/gqa_split_kv.rs:8-19 (GQASplitKVVariant) */
typedef struct psi_split_kv_variant {
    uint32_t tiled_q;            /* 0 = SingleQ, 1 = TiledQ */
    uint32_t q_token_tile_size;  /* TiledQ only, else 0 */
    uint32_t kv_token_tile_size;
    uint32_t num_threads_per_threadblock; /* SingleQ only, else 0 */
    uint32_t q_head_tile_size;
} psi_split_kv_variant;

/* How psi_gqa_prepare cuts the step into device work. */
typedef enum psi_plan_mode {
    /* Equal KV bytes per resident CTA: the flattened (q tile, KV head) work list is cut into one contiguous share per
     * CTA slot of the device, in whole 16-token KV tiles. */
    PSI_PLAN_BALANCED = 0,
    /* The reference's planner and variant selector (batch_metadata.rs:352-523, gqa_split_kv.rs:127-157): one CTA per
     * (KV split, KV head), split count capped by max_tokens. */
    PSI_PLAN_REFERENCE = 1
} psi_plan_mode;

typedef enum psi_kernel_mode {
    PSI_KERNEL_AUTO = 0,    /* tensor-core kernel when the profile allows, else the generic kernel */
    PSI_KERNEL_GENERIC = 1, /* CUDA-core kernels: any dtype, head_dim <= 256, any tokens_per_page (staged in shared
                               memory when head_dim is a multiple of four) */
    PSI_KERNEL_MMA = 2,     /* bf16/f16 mma kernel: head_dim in {64,128,256}, tokens_per_page a power of two >= 8 */
    PSI_KERNEL_MMA_SYNC = 3, /* as PSI_KERNEL_MMA, but long query runs stay on the mma.sync chunk kernel instead of
                                the tcgen05 / TMEM kernel (kept for A/B measurement) */
    PSI_KERNEL_MMA_TMA = 4   /* as PSI_KERNEL_MMA, but the decode kernel brings whole K/V tiles from their pages as
                                TMA boxes (cp.async.bulk.tensor, one instruction per tile and warp) instead of 16-byte
                                cp.async copies.  Kept for A/B measurement: it measured 1-5 % slower at head_dim 128
                                and 256 and 22 % slower at head_dim 64, so it is not what PSI_KERNEL_AUTO picks. */
} psi_kernel_mode;

/* Replay capacity policy of psi_gqa_prepare (batch_metadata.rs:60-69, GQAReplayCapacity). */
typedef enum psi_capacity_mode {
    PSI_CAPACITY_EXACT = 0,
    PSI_CAPACITY_BUCKETED = 1,
    PSI_CAPACITY_CALLER_TOKENS = 2
} psi_capacity_mode;

/* RMSNormRopeConfig + RopeScaling (crates/inference-backend-metal/src/components/rms_norm_rope.rs:42-165). */
typedef struct psi_norm_rope_config {
    uint32_t rope_dim; /* rotated leading dims of each head (even, <= head_dim) */
    float eps;
    float rope_theta;
    uint32_t yarn_enabled; /* 0 = RopeScaling::Default */
    float yarn_factor;
    float yarn_attention_factor;
    float yarn_beta_fast;
    float yarn_beta_slow;
    uint32_t yarn_original_max_position_embeddings;
    uint32_t yarn_truncate;
} psi_norm_rope_config;

/* GQA::new + GQAMetalConfig + GQAScratch sizing (crates/inference-executor-metal/src/attn/gqa/backend.rs:253-282,
 * scratch.rs:49-92). */
typedef struct psi_gqa_config {
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    float scale; /* softmax scale, applied as given (never assumed 1/sqrt(D)) */
    uint32_t page_bytes;
    uint32_t dtype; /* psi_dtype */
    psi_page_table_layout layout;
    uint32_t max_tokens;  /* flat query-token capacity of one step */
    uint32_t plan_mode;   /* psi_plan_mode */
    uint32_t kernel_mode; /* psi_kernel_mode */
    uint32_t max_ctas;    /* 0 = one CTA slot per SM x resident CTAs; otherwise caps the balanced plan's CTA count */
} psi_gqa_config;

/* ---- context ---------------------------------------------------------------------------------------------------- */

/* Device::system_default() + Stream::new (crates/inference-backend-metal/src/metal/device.rs, stream/mod.rs).
 * psi_ctx_create makes its own non-blocking stream; psi_ctx_create_on_stream borrows the caller's cudaStream_t. */
PSI_API int32_t psi_ctx_create(int32_t device, psi_ctx** out);
PSI_API int32_t psi_ctx_create_on_stream(int32_t device, void* cuda_stream, psi_ctx** out);
PSI_API int32_t psi_ctx_destroy(psi_ctx* ctx);
/* ExecutionSubmission::wait (crates/inference-executor-core/src/backend/runtime.rs:8-17) */
PSI_API int32_t psi_ctx_sync(psi_ctx* ctx);
PSI_API int32_t psi_ctx_stream(psi_ctx* ctx, void** out_cuda_stream);
PSI_API int32_t psi_ctx_sm_count(psi_ctx* ctx, int32_t* out);
/* Copies the context's last error message (NUL-terminated, truncated to n) into buf. */
PSI_API int32_t psi_ctx_last_error(psi_ctx* ctx, char* buf, size_t n);
/* Last error of the calling thread for calls that have no context yet (creation failures). */
PSI_API int32_t psi_last_error(char* buf, size_t n);

/* Measurement aid with no counterpart in the reference: streams `bytes` (>= 16, rounded down to 16) of a scratch
 * buffer through read-only 16-byte loads `iterations` times after one warm-up pass and returns the best pass in GB/s:
 * the ceiling of a kernel that only reads HBM, to stand beside the read+write copy bandwidth. */
PSI_API int32_t psi_ctx_read_bandwidth(psi_ctx* ctx, uint64_t bytes, uint32_t iterations, double* out_gbs);

/* ---- page arena (crates/inference-executor-metal/src/model/page_arena.rs:6-46) ------------------------------------ */

/* PageArena::new: num_pages x page_bytes of device memory, zero-filled. */
PSI_API int32_t psi_pages_create(psi_ctx* ctx, uint64_t num_pages, uint32_t page_bytes, psi_pages** out);
/* The same view over caller-owned device memory (not freed by psi_pages_destroy, not zeroed). */
PSI_API int32_t psi_pages_wrap(psi_ctx* ctx, void* device_ptr, uint64_t num_pages, uint32_t page_bytes,
                               psi_pages** out);
PSI_API int32_t psi_pages_destroy(psi_pages* pages);
/* PageArena::buffer */
PSI_API int32_t psi_pages_device_ptr(psi_pages* pages, void** out);
/* PageArena::release_resources / allocate_resources (hibernation); allocate zero-fills again. */
PSI_API int32_t psi_pages_release(psi_pages* pages);
PSI_API int32_t psi_pages_allocate(psi_pages* pages);
/* Selected page-ID range [page_begin, page_end) to / from host memory (page_arena/file_io.rs; blocking). */
PSI_API int32_t psi_pages_export_range(psi_pages* pages, uint64_t page_begin, uint64_t page_end, void* host_out);
PSI_API int32_t psi_pages_import_range(psi_pages* pages, uint64_t page_begin, uint64_t page_end, const void* host_in);

/* ---- hibernation snapshots (crates/inference-executor-metal/src/model/state_snapshot.rs:40-881) --------------------
 * A snapshot is a directory: one raw payload file per buffer ("page-arena", "main-gqa-request-page-table", ...) and a
 * "manifest" (magic "PSISTATE", version 3, the hibernation plan, the sorted file list with payload lengths), written
 * into a temporary sibling directory and published by rename.  StateSnapshotWriter::{new, write_full_buffer,
 * write_selected_buffer, write_metadata, commit} and StateSnapshotReader::{open, read_full_buffer,
 * read_selected_buffer, read_metadata, finish} keep their validation rules and messages.  With a selected plan the
 * page arena is written / read by the plan's page-ID ranges (entry = one page) and a page table by its request-slot
 * ranges (entry = one slot row), as PageArena and GQARequestPageTable do in
 * crates/inference-executor-metal/src/attn/gqa/request_page_table/file_io.rs:14-60.  All calls block. */
typedef struct psi_snapshot_writer psi_snapshot_writer;
typedef struct psi_snapshot_reader psi_snapshot_reader;
typedef struct psi_u32_range {
    uint32_t begin, end; /* [begin, end) */
} psi_u32_range;
typedef struct psi_hibernation_plan { /* ExecutorHibernationPlan: All (selected = 0) or Selected */
    uint32_t selected;
    const psi_u32_range* request_slot_ranges;
    uint64_t num_request_slot_ranges;
    const psi_u32_range* page_id_ranges;
    uint64_t num_page_id_ranges;
} psi_hibernation_plan;
typedef enum psi_snapshot_file { /* StateSnapshotFile, in manifest order */
    PSI_SNAPSHOT_PAGE_ARENA = 0,
    PSI_SNAPSHOT_MAIN_GQA_REQUEST_PAGE_TABLE = 1,
    PSI_SNAPSHOT_MAIN_GDN_REQUEST_STATE_TABLE = 2, /* the one metadata (not buffer) file */
    PSI_SNAPSHOT_MAIN_GDN_RECURRENT_STATE = 3,
    PSI_SNAPSHOT_MAIN_GDN_CONV_STATE = 4,
    PSI_SNAPSHOT_MTP_GQA_REQUEST_PAGE_TABLE = 5,
    PSI_SNAPSHOT_DSPARK_GQA_REQUEST_PAGE_TABLE = 6
} psi_snapshot_file;
PSI_API int32_t psi_snapshot_writer_create(const char* destination, const uint32_t* expected_files, uint64_t num_files,
                                           const psi_hibernation_plan* plan, psi_snapshot_writer** out);
/* Whole arena / table under the All plan, the plan's page-ID / request-slot ranges under a Selected plan. */
PSI_API int32_t psi_snapshot_write_pages(psi_snapshot_writer* writer, uint32_t file, psi_pages* pages);
PSI_API int32_t psi_snapshot_write_table(psi_snapshot_writer* writer, uint32_t file, psi_table* table);
/* A caller-held host buffer: whole (entry_ranges == NULL) or the given entry ranges of entry_bytes each. */
PSI_API int32_t psi_snapshot_write_host_buffer(psi_snapshot_writer* writer, uint32_t file, const void* host, uint64_t bytes,
                                               const psi_u32_range* entry_ranges, uint64_t num_ranges, uint64_t entry_bytes);
PSI_API int32_t psi_snapshot_write_metadata(psi_snapshot_writer* writer, uint32_t file, const void* bytes, uint64_t n);
PSI_API int32_t psi_snapshot_writer_commit(psi_snapshot_writer* writer);
/* Also abandons an uncommitted snapshot (its temporary directory is removed). */
PSI_API int32_t psi_snapshot_writer_destroy(psi_snapshot_writer* writer);
PSI_API int32_t psi_snapshot_reader_open(const char* path, const uint32_t* expected_files, uint64_t num_files,
                                         const psi_hibernation_plan* plan, psi_snapshot_reader** out);
PSI_API int32_t psi_snapshot_read_pages(psi_snapshot_reader* reader, uint32_t file, psi_pages* pages);
PSI_API int32_t psi_snapshot_read_table(psi_snapshot_reader* reader, uint32_t file, psi_table* table);
PSI_API int32_t psi_snapshot_read_host_buffer(psi_snapshot_reader* reader, uint32_t file, void* host, uint64_t bytes,
                                              const psi_u32_range* entry_ranges, uint64_t num_ranges, uint64_t entry_bytes);
/* Copies the metadata payload into out (capacity cap) and stores its length in *out_n. */
PSI_API int32_t psi_snapshot_read_metadata(psi_snapshot_reader* reader, uint32_t file, void* out, uint64_t cap, uint64_t* out_n);
PSI_API int32_t psi_snapshot_reader_finish(psi_snapshot_reader* reader);
PSI_API int32_t psi_snapshot_reader_destroy(psi_snapshot_reader* reader);

/* ---- request page table (crates/inference-executor-metal/src/attn/gqa/request_page_table.rs:13-122) --------------- */

/* GQARequestPageTable::new: zero-initialised u32 table on the device with a host mirror. */
PSI_API int32_t psi_table_create(psi_ctx* ctx, const psi_page_table_layout* layout, psi_table** out);
PSI_API int32_t psi_table_destroy(psi_table* table);
/* write_page_ids: n must equal num_page_ids_per_block. */
PSI_API int32_t psi_table_write(psi_table* table, uint32_t req_slot, uint32_t layer, uint32_t block,
                                const uint32_t* page_ids, uint32_t n);
/* Declares the number of pages of the arena this table indexes (0 = no bound, the initial state).  From then on
 * psi_table_write, psi_table_write_row and psi_snapshot_read_table refuse page IDs at or beyond it with the message of
 * the reference's check at the point where IDs enter the table (crates/inference-executor-metal/src/state/gqa.rs:97-102),
 * before anything reaches the device.  Independently of this, in the checked build of the library every kernel
 * compares the IDs it reads with the page count of the psi_pages it was given (PSI_ERR_PAGE_ID through
 * psi_gqa_device_status). */
PSI_API int32_t psi_table_set_page_bound(psi_table* table, uint64_t num_cache_pages);

/* Qwen3xGQAState::write_page_ids (crates/inference-executor-metal/src/model/qwen/v3_x/state/gqa.rs:88-106): one block
 * of every layer, n == num_gqa_layers * num_page_ids_per_block, every id < num_cache_pages. */
PSI_API int32_t psi_table_write_all_layers(psi_table* table, uint32_t req_slot, uint32_t block,
                                           const uint32_t* page_ids, uint32_t n, uint64_t num_cache_pages);
/* read_page_ids (blocking; reads the device copy). */
PSI_API int32_t psi_table_read(psi_table* table, uint32_t req_slot, uint32_t layer, uint32_t block, uint32_t* out,
                               uint32_t n);
/* reset_req_slots: zero every row of the listed slots. */
PSI_API int32_t psi_table_reset_slots(psi_table* table, const uint32_t* req_slots, uint32_t n);
/* page_ids_buffer */
PSI_API int32_t psi_table_device_ptr(psi_table* table, void** out);
/* Bulk load of whole (slot, layer) rows from host memory: ids holds num_blocks*num_page_ids_per_block entries. */
PSI_API int32_t psi_table_write_row(psi_table* table, uint32_t req_slot, uint32_t layer, const uint32_t* ids,
                                    uint32_t n);

/* ---- host-side policy (no device work) ----------------------------------------------------------------------------- */

/* ReplayBucketPolicy::with_topology_boundaries / buckets (crates/inference-executor-core/src/replay.rs:25-55):
 * writes the bucket list into out (capacity out_cap) and its length into out_n. */
PSI_API int32_t psi_replay_bucket_policy(uint32_t max_capacity, const uint32_t* topology_boundaries,
                                         uint32_t num_boundaries, uint32_t* out, uint64_t out_cap, uint64_t* out_n);
/* ReplayBucketPolicy::capacity (replay.rs:57-62) */
PSI_API int32_t psi_replay_bucket_capacity(uint32_t max_capacity, const uint32_t* topology_boundaries,
                                           uint32_t num_boundaries, uint32_t active, uint32_t* out);
/* GQASplitKV::new / new_dspark_history + select (crates/inference-backend-metal/src/components/gqa_split_kv.rs:85-157).
 * out_max_q_tokens_per_partial may be NULL. */
PSI_API int32_t psi_split_kv_select(uint32_t io_dtype, uint32_t page_bytes, uint32_t num_q_heads,
                                    uint32_t num_kv_heads, uint32_t head_dim, uint32_t dspark_history,
                                    uint32_t num_tokens, uint32_t num_q_token_tiles, psi_split_kv_variant* out,
                                    uint32_t* out_max_q_tokens_per_partial);

/* GQAMetadataBuffers::update / update_bucketed / update_bucketed_with_token_capacity on caller-provided host arrays
 * (crates/inference-executor-metal/src/attn/gqa/batch_metadata.rs:128-317): the metadata half of psi_gqa_prepare
 * without a device.  The five buffers are capacity-sized (max_tokens, max_tokens, 2*max_tokens, 3*max_tokens,
 * max_tokens+1 u32) and only the prefixes the reference writes change. */
PSI_API int32_t psi_metadata_update_host(uint32_t max_tokens, const uint32_t* req_slots, const uint32_t* token_indices,
                                         const uint32_t* cu_tokens, uint32_t num_reqs,
                                         const psi_split_kv_variant* variant, uint32_t capacity_mode,
                                         const uint32_t* token_topology_boundaries, uint32_t num_boundaries,
                                         uint32_t caller_num_total_tokens, uint32_t* buf_req_slots,
                                         uint32_t* buf_flat_token_indices, uint32_t* buf_q_token_tiles,
                                         uint32_t* buf_kv_splits, uint32_t* buf_cu_kv_splits,
                                         psi_replay_shape* out_shape);
/* The balanced device work plan of a batch, computed on the host (what psi_gqa_prepare uploads in
 * PSI_PLAN_BALANCED).  out_items receives 6 u32 per item {q tile, head selection, kv_begin, kv_end, partial slot or
 * 0xFFFFFFFF, flat token begin of the tile}; out_cta_item_begin receives num_ctas+1 entries; out_counts receives
 * {items, ctas, partial slots, reduce units, q tiles, total 16-token KV tiles (saturated)}.  item_start_cost is the
 * number of KV tiles one additional item is charged when the shares are balanced.  No reference counterpart:
 * the reference's planner is psi_metadata_update_host. */
PSI_API int32_t psi_plan_preview(uint32_t num_q_heads, uint32_t num_kv_heads, const uint32_t* token_indices,
                                 const uint32_t* cu_tokens, uint32_t num_reqs, uint32_t max_ctas,
                                 uint32_t min_kv_tiles_per_cta, uint32_t item_start_cost, uint32_t* out_items,
                                 uint64_t items_cap, uint32_t* out_cta_item_begin, uint64_t cta_cap,
                                 uint32_t* out_counts);

/* The work plan of the long-query (chunk) kernels for a batch in which EVERY request carries a long run, computed on
 * the host.  equal_shares selects the plan for working sets that stay in L2 (contiguous shares of equal size) instead
 * of stream order.  out_items receives 10 u32 per item {request, kv head, flat token begin, tokens, kv_begin, kv_end,
 * partial slot or 0xFFFFFFFF, pieces of its unit, first slot of the unit, first arrival counter of the unit};
 * out_cta_item_begin num_ctas+1 entries; out_counts {items, ctas, partial slots, arrival counters, total 16-token KV
 * tiles (saturated)}.  No reference counterpart. */
PSI_API int32_t psi_chunk_plan_preview(uint32_t num_q_heads, uint32_t num_kv_heads, const uint32_t* token_indices,
                                       const uint32_t* cu_tokens, uint32_t num_reqs, uint32_t max_ctas,
                                       uint32_t equal_shares, uint32_t* out_items, uint64_t items_cap,
                                       uint32_t* out_cta_item_begin, uint64_t cta_cap, uint32_t* out_counts);

/* U32IDAllocator (crates/inference-runtime-core/src/memory/u32_id_allocator.rs:69-172): freed IDs first, in the order
 * they were freed, then fresh IDs from a counter.  Runtime core keeps its own allocator; this one drives synthetic
 * admit/finish traces with the same observable behaviour. */
PSI_API int32_t psi_id_allocator_create(uint64_t capacity, psi_id_allocator** out);
PSI_API int32_t psi_id_allocator_destroy(psi_id_allocator* a);
PSI_API int32_t psi_id_allocator_alloc_many(psi_id_allocator* a, uint64_t count, uint32_t* out_ids);
PSI_API int32_t psi_id_allocator_free_many(psi_id_allocator* a, const uint32_t* ids, uint64_t count);
PSI_API int32_t psi_id_allocator_bitmap(psi_id_allocator* a, uint64_t* out_words, uint64_t cap, uint64_t* out_n);
PSI_API int32_t psi_id_allocator_free_count(psi_id_allocator* a, uint64_t* out);

/* ---- the GQA component (crates/inference-executor-metal/src/attn/gqa/backend.rs:253-657) -------------------------- */

/* GQA::new + GQAMetadataBuffers::new + GQA::new_scratch: fixes the profile, allocates the device metadata block and
 * the partial-output scratch. */
PSI_API int32_t psi_gqa_create(psi_ctx* ctx, const psi_gqa_config* config, psi_gqa** out);
PSI_API int32_t psi_gqa_destroy(psi_gqa* gqa);
/* GQAReplayBucketPolicy::new's token topology boundaries (batch_metadata.rs:20-27); default none. */
PSI_API int32_t psi_gqa_set_token_topology_boundaries(psi_gqa* gqa, const uint32_t* boundaries, uint32_t n);

/* GQA::prepare / prepare_bucketed / prepare_bucketed_with_token_capacity -> GQAMetadataBuffers::update*
 * (backend.rs:283-356, batch_metadata.rs:128-317).  Host arrays: req_slots[num_reqs], token_indices[num_reqs]
 * (request-absolute position of each request's first query token), cu_tokens[num_reqs+1].  Builds the per-token
 * metadata, selects the SplitKV variant, plans the KV splits, and uploads everything in one copy on the stream. */
PSI_API int32_t psi_gqa_prepare(psi_gqa* gqa, const uint32_t* req_slots, const uint32_t* token_indices,
                                const uint32_t* cu_tokens, uint32_t num_reqs, uint32_t capacity_mode,
                                uint32_t caller_num_total_tokens, psi_replay_shape* out_shape);
/* The variant the last prepare selected (GQAMetadataBuffers::split_kv_variant). */
PSI_API int32_t psi_gqa_split_kv_variant(psi_gqa* gqa, psi_split_kv_variant* out);

typedef enum psi_metadata_array {
    PSI_MD_REQ_SLOTS = 0,          /* [max_tokens] */
    PSI_MD_FLAT_TOKEN_INDICES = 1, /* [max_tokens] */
    PSI_MD_Q_TOKEN_TILES = 2,      /* [max_tokens][2] */
    PSI_MD_KV_SPLITS = 3,          /* [max_tokens][3] */
    PSI_MD_CU_KV_SPLITS = 4        /* [max_tokens+1] */
} psi_metadata_array;
/* Read / overwrite the reference-format metadata arrays (GQAMetadataBuffers::req_slots() ... cu_kv_splits(),
 * Buffer::read_typed / write_typed).  Offsets and counts are in u32 elements. */
PSI_API int32_t psi_gqa_metadata_read(psi_gqa* gqa, uint32_t which, uint64_t offset, uint32_t* out, uint64_t n);
PSI_API int32_t psi_gqa_metadata_write(psi_gqa* gqa, uint32_t which, uint64_t offset, const uint32_t* in, uint64_t n);

/* Plan statistics of the last prepare: out[0]=CTAs launched by the map kernel, out[1]=work items, out[2]=partial
 * slots, out[3]=reduce units, out[4]=exec q tiles, out[5]=kernel (1 generic, 2 mma), out[6]=total 16-token KV tiles,
 * out[7]=rows per q tile, out[8]=CTAs of the long-query (chunk) kernel, out[9]=its work items, out[10]=launches of
 * the tcgen05 chunk kernel since the object was created, out[11]=launches of the mma.sync chunk kernel (the fallback
 * when PSI_KERNEL_MMA_SYNC asks for it or the page arena cannot be described to the TMA unit). */
PSI_API int32_t psi_gqa_plan_stats(psi_gqa* gqa, uint32_t* out, uint32_t n);

/* KV append: GQAKVPageWrite::invoke_bucketed (crates/inference-backend-metal/src/components/gqa_kv_page_write.rs:
 * 125-177; shader metal/gqa_kv_page_write.metal:6-53).  k, v: device [num_total_tokens][Hkv][D]; rows at or beyond
 * the prepared num_tokens are not read and their pages not touched.  Bit copy. */
PSI_API int32_t psi_gqa_kv_append(psi_gqa* gqa, psi_pages* pages, psi_table* table, uint32_t layer, const void* k,
                                  const void* v);

/* Attention over the paged cache: SplitKV map + reduce (gqa_split_kv_single_q.rs:293-383, gqa_split_kv_tiled_q.rs:
 * 246-327; shaders metal/gqa_split_kv_single_q_{map,reduce}.metal, metal/gqa_split_kv_tiled_q.metal).  q, out: device
 * [num_total_tokens][Hq][D]; query token i of a request sees keys [0, token_index+i]; output rows at or beyond the
 * prepared num_tokens are left untouched.  Enqueue after psi_gqa_kv_append of the same step (stream order is the
 * reference's barrier) so that a token attends to itself. */
PSI_API int32_t psi_gqa_attend(psi_gqa* gqa, psi_pages* pages, psi_table* table, uint32_t layer, const void* q,
                               void* out);

/* The two stages above as one launch: the attention kernel itself writes this step's K/V rows into their pages and
 * reads them from k / v instead of from the pages, so the step has no kernel boundary between append and attend
 * (GQA::record's kv_page_write -> barrier -> SplitKV map -> reduce, crates/inference-executor-metal/src/attn/gqa/
 * backend.rs:493-612, in one submission).  Same results as psi_gqa_kv_append followed by psi_gqa_attend.  k, v must
 * be 16-byte aligned. */
PSI_API int32_t psi_gqa_append_attend(psi_gqa* gqa, psi_pages* pages, psi_table* table, uint32_t layer, const void* k,
                                      const void* v, const void* q, void* out);

/* ---- neighbours of the path that the reference records around it ---------------------------------------------------- */

/* RopeScaling::kernel_parameters (rms_norm_rope.rs:167-230), host only: rope_dim/2 inverse frequencies, the attention
 * factor, and Yarn's correction range (0, 0 without Yarn; either pointer may be NULL). */
PSI_API int32_t psi_rope_parameters(const psi_norm_rope_config* config, float* out_inverse_frequencies,
                                    float* out_attention_factor, float* out_correction_low,
                                    float* out_correction_high);
/* Fixes the q / k RMSNorm + RoPE profile of the component: the bf16 norm weights (host arrays of head_dim values,
 * RMSNormRopeBuffers::norm_weight) and the rope parameters are uploaded once. */
PSI_API int32_t psi_gqa_set_norm_rope(psi_gqa* gqa, const psi_norm_rope_config* config,
                                      const uint16_t* q_norm_weight_bf16, const uint16_t* k_norm_weight_bf16);
/* The three stages GQA::record puts before the attention (backend.rs:465-513: q norm/rope, k norm/rope,
 * kv_page_write; shaders metal/rms_norm_rope.metal, metal/gqa_kv_page_write.metal) as ONE launch: q_out receives the
 * normalised, rotated queries, the normalised, rotated keys go straight into their pages (no k scratch), the values
 * are copied into theirs.  q_in/q_out [T][Hq][D], k_in/v_in [T][Hkv][D], device, positions = the prepared batch. */
PSI_API int32_t psi_gqa_norm_rope_append(psi_gqa* gqa, psi_pages* pages, psi_table* table, uint32_t layer,
                                         const void* q_in, const void* k_in, const void* v_in, void* q_out);
/* psi_gqa_norm_rope_append reading q, k and v (and the gates) where the fused projection left them, which also
 * removes the de-interleave stage GQA::record puts in front of them (backend.rs:449-464; GQAQGKVSplitKernel,
 * crates/inference-backend-metal/src/components/gqa_qgkv_split.rs:152-200 with metal/gqa_qgkv_split.metal:14-42, and
 * the ungated GQAQKVSplitKernel of ungated_backend.rs:218-227, gqa_qkv_split.rs with metal/gqa_qkv_split.metal:13-36).  projection: device
 * [T][width] in the I/O dtype; gated = 1: width = 2*Hq*D + 2*Hkv*D, per token Hq pairs (q[D] | gate[D]), then Hkv k
 * rows, then Hkv v rows; gated = 0: width = Hq*D + 2*Hkv*D, q rows, k rows, v rows.  q_out [T][Hq][D] receives the
 * normalised, rotated queries; gates_out [T][Hq][D] (gated only, else may be NULL) a bit copy of the gate rows, ready
 * for psi_gqa_attend_gated.  T * width beyond the u32 range is refused with the reference's message. */
PSI_API int32_t psi_gqa_projection_norm_rope_append(psi_gqa* gqa, psi_pages* pages, psi_table* table, uint32_t layer,
                                                    const void* projection, uint32_t gated, void* q_out,
                                                    void* gates_out);
/* psi_gqa_attend with the stage the reference records after it fused into the epilogue: out = attention *
 * sigmoid(gates) (backend.rs:613-624, metal/gqa_activation_gate.metal).  gates: device [T][Hq][D] in the I/O dtype. */
PSI_API int32_t psi_gqa_attend_gated(psi_gqa* gqa, psi_pages* pages, psi_table* table, uint32_t layer, const void* q,
                                     const void* gates, void* out);

/* The same map + reduce, stopping before normalisation to the output dtype: f32 o [T][Hq][D] (normalised within the
 * local KV), m [T][Hq] (natural-log running max of scale*q.k), l [T][Hq] (sum of exp(logit - m)).  This is the
 * reference's partial-output ABI (gqa_split_kv_single_q_map.metal:231-252) lifted to one partial per device, for KV
 * ranges that are split across devices.  o/m/l may point into a peer device's memory when peer access is enabled. */
PSI_API int32_t psi_gqa_attend_partial(psi_gqa* gqa, psi_pages* pages, psi_table* table, uint32_t layer,
                                       const void* q, float* o, float* m, float* l);

/* Dense bidirectional attention of every query token against the tokens of its own block of block_size tokens
 * (GQABlockSDPAKernel::invoke, crates/inference-backend-metal/src/components/gqa_block_attention.rs:129-271; shader
 * metal/gqa_block_sdpa.metal:5-77), written in the same partial ABI as psi_gqa_attend_partial so that
 * psi_gqa_combine merges it with the paged history of the same tokens (the DSpark composite).  q [T][Hq][D],
 * local_k / local_v [T][Hkv][D]: device, component dtype, unpaged; num_tokens must be a whole number of blocks
 * (block_size <= 256).  slot_indices: NULL (token t writes partial slot t) or device [T] slot numbers
 * (block_sdpa_map_task_template_indices); o [slots][Hq][D], m and l [slots][Hq], device f32. */
PSI_API int32_t psi_gqa_block_partial(psi_gqa* gqa, const void* q, const void* local_k, const void* local_v,
                                      uint32_t num_tokens, uint32_t block_size, const uint32_t* slot_indices, float* o,
                                      float* m, float* l);

/* Merge n partials per (token, head) exactly like the reference reduce (gqa_split_kv_single_q_reduce.metal:27-48):
 * M = max m_i, w_i = exp(m_i - M) * l_i (0 when m_i is not finite), out = sum w_i o_i / sum w_i (0 when the sum is 0).
 * o/m/l are host arrays of n device pointers; out is device [num_tokens][Hq][D] in the component's dtype. */
PSI_API int32_t psi_gqa_combine(psi_gqa* gqa, const float* const* o, const float* const* m, const float* const* l,
                                uint32_t n, uint32_t num_tokens, void* out);

/* KV ranges split across devices, exchange without a library collective: a producer runs psi_gqa_attend_partial with
 * o/m/l pointing into the owner's receive buffers (peer memory) and then psi_gqa_signal, which release-stores `value`
 * to `flag` (in the owner's memory) once everything enqueued before it is visible system-wide.  The owner runs
 * psi_gqa_combine_wait: the merge of psi_gqa_combine, preceded by a BOUNDED wait until each of the n flags (device
 * array in the owner's own memory) has reached flag_value.  If a producer never publishes, the wait gives up after
 * max_polls polls (0 = default, roughly a fraction of a second), writes nothing to `out` (the launch reaches one
 * verdict for all of its CTAs), and records PSI_ERR_TIMEOUT, which psi_gqa_device_status returns (and clears) after
 * waiting for the stream; the context stays usable.  Flag values should increase from step to step (a step counter),
 * so flags never need resetting.  This form has ONE receive buffer per producer and nothing in it holds a producer
 * back: the caller must not let any producer start step s + 1 before the owner's psi_gqa_combine_wait of step s has
 * finished (otherwise the merge can read a mix of two steps); psi_gqa_attend_exchange below carries that ordering in
 * its own protocol and is the form to use.  No reference counterpart: the
 * reference has no multi-device path (crates/inference-runtime-core/src/network/mod.rs is empty). */
PSI_API int32_t psi_gqa_signal(psi_gqa* gqa, uint32_t* flag, uint32_t value);
PSI_API int32_t psi_gqa_combine_wait(psi_gqa* gqa, const float* const* o, const float* const* m, const float* const* l,
                                     uint32_t n, uint32_t num_tokens, void* out, const uint32_t* flags,
                                     uint32_t flag_value, uint32_t max_polls);

/* The same exchange as ONE launch per rank.  A group of `world` devices each holds one page-aligned slice of every
 * sequence's KV range; the owner holds a receive area (memory every rank can store to: peer-mapped or symmetric
 * memory) of 2 x world slots, one pair per rank, each slot `slot_floats` f32 laid out as o [T][Hq][D] | m [T][Hq] |
 * l [T][Hq], followed wherever the caller likes by `world` u32 arrival flags and one u32 "consumed" word, all zero
 * before the first step.  Every rank calls psi_gqa_attend_exchange once per step with the same `step` = 1, 2, 3, ...:
 *   - the attention launch writes the rank's partial straight into slot [step & 1][rank] (plain peer stores; no bulk
 *     or tensor copies touch peer memory), and the CTA that finishes the launch last release-stores `step` into
 *     flags[rank];
 *   - on the owner the same launch then waits, with a bound, until every flag has reached `step` and merges the
 *     partials into `out` with the reference's reduce algebra (gqa_split_kv_single_q_reduce.metal:27-48), after which
 *     it release-stores `step` into the consumed word;
 *   - slots alternate with the step's parity and a rank stores step s only once the consumed word has reached
 *     s - 2 (bounded wait), so ranks may run ahead of the owner without overwriting a partial it has not merged.
 * Every wait gives up after max_polls polls of about 100 ns (0 = default, a fraction of a second): the launch then
 * writes no output at all (one verdict per launch), records PSI_ERR_TIMEOUT for psi_gqa_device_status, and the context
 * stays usable.  `k`/`v` (nullable, both or neither) are this step's K/V rows for the rank that holds the end of the
 * range; they are appended by the same launch.  `out` is needed on the owner only.  Profiles without the tensor-core
 * decode kernel (f32, odd page sizes) and steps with long query runs run the same protocol as three launches
 * (attention into local scratch, push + flag, wait + merge).  On the owner, all of the launch's CTAs must be able to
 * be resident together (they are: the launch never has more CTAs than the device has SMs), because the merging CTAs
 * wait for the launch's own flag.  No reference counterpart: the reference splits a KV range only within one device
 * (docs/executor_gqa.md:104-109,556-587). */
typedef struct psi_kv_exchange {
    uint32_t rank;
    uint32_t world;        /* 1..64 */
    uint32_t owner;        /* rank whose memory holds slots, flags and consumed, and which produces `out` */
    uint32_t step;         /* >= 1, the same on every rank, +1 per call */
    float* slots;          /* the owner's receive area as addressed from THIS device: f32 [2][world][slot_floats] */
    uint64_t slot_floats;  /* >= T * Hq * (D + 2), a multiple of 4 */
    uint32_t* flags;       /* u32 [world] in the owner's memory, as addressed from this device */
    uint32_t* consumed;    /* u32 [1] in the owner's memory, as addressed from this device */
    uint32_t max_polls;    /* 0 = default */
} psi_kv_exchange;
PSI_API int32_t psi_gqa_attend_exchange(psi_gqa* gqa, psi_pages* pages, psi_table* table, uint32_t layer, const void* k,
                                        const void* v, const void* q, const psi_kv_exchange* exchange, void* out);
PSI_API int32_t psi_gqa_device_status(psi_gqa* gqa, int32_t* out);

/* One whole decode step through host memory: k, v [T][Hkv][D] and q [T][Hq][D] come from host buffers, out [T][Hq][D]
 * lands in a host buffer, and the call waits for it.  T is the prepared num_tokens.  With pinned (page-locked,
 * device-mapped) buffers the attention launch reads and writes them in place over the host link; with pageable
 * buffers the inputs are staged through device copies first. */
PSI_API int32_t psi_gqa_decode_step_host(psi_gqa* gqa, psi_pages* pages, psi_table* table, uint32_t layer,
                                         const void* k_host, const void* v_host, const void* q_host, void* out_host);

/* psi_gqa_prepare (exact capacity) and psi_gqa_decode_step_host in one call, for a host loop that hands over a step's
 * metadata and buffers together (the executor's update-then-submit pair of
 * crates/inference-executor-metal/src/attn/gqa/batch_metadata.rs:128-317 and backend.rs:493-612): with pinned buffers
 * one launch pulls the packed plan and q/k/v over the host link (no copy-engine transfer) and the attention launch
 * stores out straight into the host buffer; from 1 MiB of q + k + v on (and no long query runs in the step) the attention launch reads the pinned
 * buffers in place, so that the transfer runs under the K/V stream instead of in front of it.  Same result as the two
 * calls.  A step with long query runs and 64 MiB or more of q + k + v in pinned buffers (balanced plan mode, no replay
 * reservation) runs as up to eight groups of consecutive requests instead: group i's inputs travel on a copy stream
 * while group i-1 is planned and launched and group i-2's output travels back on a second copy stream, so the step
 * takes about as long as the slowest of transfer in, compute and transfer out rather than their sum.  Every group gets a
 * plan of its own (its KV splits differ from the whole step's: results agree within the tolerance of any other split),
 * and the component is left unprepared afterwards (its metadata would describe the last group only). */
PSI_API int32_t psi_gqa_step_host(psi_gqa* gqa, psi_pages* pages, psi_table* table, uint32_t layer,
                                  const uint32_t* req_slots, const uint32_t* token_indices, const uint32_t* cu_tokens,
                                  uint32_t num_reqs, const void* k_host, const void* v_host, const void* q_host,
                                  void* out_host);

/* Page gather: tokens [tok_begin, tok_end) of one request slot and layer into contiguous device K and V
 * [n][Hkv][D].  The reference fuses this address walk into its map kernels
 * (metal/gqa_split_kv_single_q_map.metal:96-111,195-209); standalone it is the inverse of the append. */
PSI_API int32_t psi_page_gather(psi_gqa* gqa, psi_pages* pages, psi_table* table, uint32_t req_slot, uint32_t layer,
                                uint32_t tok_begin, uint32_t tok_end, void* k_out, void* v_out);

/* Attention for callers that must not allocate device memory (no counterpart in the reference, whose Metal buffers
 * are all created up front).  A server that gave all remaining HBM to its KV arena, a host runtime that owns every
 * device allocation through its own pool, or a decode loop that cannot take the device-wide stall of an allocation
 * can still run the split-KV attention of psi_gqa_attend through this call: the plan, the arrival counters and the
 * partial outputs live in one fixed device array of PSI_STATIC_SCRATCH_BYTES that each GPU loading the library holds
 * until exit, and the call makes no cudaMalloc, cudaFree or other allocating CUDA call.
 *
 * Takes no psi_ctx / psi_gqa: `device` and `cuda_stream` name where to run, `config` the profile (plan_mode is
 * ignored, the balanced plan is used; max_ctas may lower the CTA count further), `pages` the device arena,
 * `page_table` the device table in the layout of config->layout, and the host arrays req_slots / token_indices /
 * cu_tokens the batch exactly as for psi_gqa_prepare.  q and out are device [T][Hq][D].  The work is enqueued on the
 * stream and the call returns; results equal psi_gqa_attend's.
 *
 * Limits: head_dim <= PSI_STATIC_MAX_HEAD_DIM, at most PSI_STATIC_MAX_CTAS CTAs (so less of a large GPU is used than
 * by psi_gqa_attend) and PSI_STATIC_MAX_ITEMS work items - roughly (query tiles x KV heads) + PSI_STATIC_MAX_CTAS; a
 * step beyond them returns PSI_ERR_INVALID_ARGUMENT with the reason in `error` and enqueues nothing.
 * The first call on a device resolves the scratch address (cudaGetSymbolAddress); make that call outside any stream
 * capture.  Every call uploads its plan from host memory that is gone when the call returns, so a call on a stream
 * that is being captured is refused (PSI_ERR_INVALID_ARGUMENT, nothing enqueued).  The caller's current device is
 * the same after the call as before it.  All calls on a device share the one scratch, which keeps the previous call's contents: each call
 * rewrites its plan and clears the arrival counters itself, and two calls whose work overlaps on the GPU (different
 * streams, or different host threads) race on it - serialise them on one stream.  `error` (may be NULL) receives a
 * NUL-terminated message on failure. */
#define PSI_STATIC_MAX_HEAD_DIM 256
#define PSI_STATIC_MAX_CTAS 64
#define PSI_STATIC_MAX_ITEMS 512
#define PSI_STATIC_SCRATCH_BYTES 2148608
PSI_API int32_t psi_gqa_attend_static(int32_t device, void* cuda_stream, const psi_gqa_config* config,
                                      const void* pages, const uint32_t* page_table, const uint32_t* req_slots,
                                      const uint32_t* token_indices, const uint32_t* cu_tokens, uint32_t num_reqs,
                                      uint32_t layer, const void* q, void* out, char* error, size_t error_len);

/* Number of kernels this library has launched on the context since creation (for launch accounting). */
PSI_API int32_t psi_ctx_launch_count(psi_ctx* ctx, uint64_t* out);

/* Per-kernel device timing for measurement harnesses (the reference offers no GPU timestamps; its benches time whole
 * submissions).  While enabled, every launch of the library on this context is bracketed by CUDA events on the
 * context's stream.  psi_ctx_kernel_timing waits for the stream, then returns the summed duration and the launch
 * count of one kernel class since timing was last enabled or reset. */
typedef enum psi_kernel_class {
    PSI_KERNEL_CLASS_APPEND = 0,
    PSI_KERNEL_CLASS_ATTEND_MAP = 1,
    PSI_KERNEL_CLASS_ATTEND_REDUCE = 2,
    PSI_KERNEL_CLASS_COMBINE = 3,
    PSI_KERNEL_CLASS_GATHER = 4,
    PSI_KERNEL_CLASS_ATTEND_CHUNK = 5,
    PSI_KERNEL_CLASS_NORM_ROPE_APPEND = 6
} psi_kernel_class;
PSI_API int32_t psi_ctx_enable_kernel_timing(psi_ctx* ctx, int32_t enable);
PSI_API int32_t psi_ctx_kernel_timing(psi_ctx* ctx, uint32_t kernel_class, float* out_total_ms, uint64_t* out_launches);

/* ---- replayed launch sequences (Stream::create_replay_program / submit_replay_with_arguments,
 * crates/inference-backend-metal/src/metal/stream; ReplayU32::Parameter -> the device scalar block) ----------------
 * The reference records a layer's kernels once per replay bucket into an indirect command buffer whose scalar
 * arguments live in a parameter buffer rewritten per submission.  Here: psi_gqa_reserve_replay fixes, for the
 * component's max_tokens, every array offset of the per-step device block, every scratch buffer and every launch
 * grid (launches then always run append, map, chunk and reduce kernels at their capacity grids and take their active
 * counts from the device block; a fused step becomes append + attend); psi_ctx_capture_begin / _end capture whatever the library launches
 * on the context's stream in between (any number of layers; psi_gqa_prepare stays outside) into a CUDA graph;
 * psi_graph_launch replays it after each step's psi_gqa_prepare.  One graph per (bucket capacity, buffer set), as
 * the reference keeps one recorded program per bucket.  A step beyond the reserved capacity, or a buffer that would
 * have to grow during capture, is refused with PSI_ERR_INVALID_ARGUMENT. */
typedef struct psi_graph psi_graph;
PSI_API int32_t psi_gqa_reserve_replay(psi_gqa* gqa);
PSI_API int32_t psi_ctx_capture_begin(psi_ctx* ctx);
PSI_API int32_t psi_ctx_capture_end(psi_ctx* ctx, psi_graph** out);
PSI_API int32_t psi_graph_launch(psi_graph* graph);
PSI_API int32_t psi_graph_kernel_count(psi_graph* graph, uint64_t* out);
PSI_API int32_t psi_graph_destroy(psi_graph* graph);

#ifdef __cplusplus
}
#endif
#endif /* PSI_CUDA_H */
