// C ABI: page arena, request page table and page-ID allocator.
#include "api_internal.hpp"

using namespace psi;

extern "C" {

static void pages_allocate(psi_pages* pages) {
    require(pages->ptr == nullptr, "page arena state is already loaded");
    const uint64_t bytes = pages->num_pages * pages->page_bytes;
    cudaError_t err = cudaMalloc(&pages->ptr, bytes);
    if (err == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        pages->ptr = nullptr;
        throw ExhaustedError("out of device memory for the page arena");
    }
    cuda_check(err, "cudaMalloc");
    cuda_check(cudaMemsetAsync(pages->ptr, 0, bytes, pages->ctx->stream), "cudaMemsetAsync");
}

int32_t psi_pages_create(psi_ctx* ctx, uint64_t num_pages, uint32_t page_bytes, psi_pages** out) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        require(out != nullptr, "out must not be null");
        *out = nullptr;
        require(num_pages > 0, "page arena requires pages");
        require(page_bytes > 0, "page arena requires nonzero page size");
        require(num_pages <= (uint64_t(1) << 62) / page_bytes, "page arena byte length must fit usize");
        ctx->bind();
        auto pages = std::make_unique<psi_pages>();
        pages->ctx = ctx;
        pages->owned = true;
        pages->num_pages = num_pages;
        pages->page_bytes = page_bytes;
        pages_allocate(pages.get());
        *out = pages.release();
    });
}

int32_t psi_pages_wrap(psi_ctx* ctx, void* device_ptr, uint64_t num_pages, uint32_t page_bytes, psi_pages** out) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        require(out != nullptr && device_ptr != nullptr, "out and device_ptr must not be null");
        require(num_pages > 0 && page_bytes > 0, "page arena requires pages of nonzero size");
        auto pages = std::make_unique<psi_pages>();
        pages->ctx = ctx;
        pages->ptr = device_ptr;
        pages->owned = false;
        pages->num_pages = num_pages;
        pages->page_bytes = page_bytes;
        *out = pages.release();
    });
}

int32_t psi_pages_destroy(psi_pages* pages) {
    if (pages == nullptr) return PSI_OK;
    int32_t status = guarded(pages->ctx, [&] {
        pages->ctx->bind();
        if (pages->owned && pages->ptr != nullptr) {
            (void)cudaStreamSynchronize(pages->ctx->stream);
            cuda_check(cudaFree(pages->ptr), "cudaFree");
        }
    });
    delete pages;
    return status;
}

int32_t psi_pages_device_ptr(psi_pages* pages, void** out) {
    if (pages == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(pages->ctx, [&] {
        require(pages->ptr != nullptr, "page arena state must be loaded before execution");
        *out = pages->ptr;
    });
}

int32_t psi_pages_release(psi_pages* pages) {
    if (pages == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(pages->ctx, [&] {
        require(pages->owned, "a wrapped page arena does not own its memory");
        require(pages->ptr != nullptr, "page arena state is not loaded");
        pages->ctx->bind();
        cuda_check(cudaStreamSynchronize(pages->ctx->stream), "cudaStreamSynchronize");
        cuda_check(cudaFree(pages->ptr), "cudaFree");
        pages->ptr = nullptr;
    });
}

int32_t psi_pages_allocate(psi_pages* pages) {
    if (pages == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(pages->ctx, [&] {
        require(pages->owned, "a wrapped page arena does not own its memory");
        pages->ctx->bind();
        pages_allocate(pages);
    });
}

static int32_t pages_copy_range(psi_pages* pages, uint64_t begin, uint64_t end, void* host, bool to_host) {
    if (pages == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(pages->ctx, [&] {
        require(host != nullptr, "host buffer must not be null");
        require(pages->ptr != nullptr, "page arena state must be loaded before execution");
        require(begin <= end && end <= pages->num_pages, "page-ID range outside the page arena");
        pages->ctx->bind();
        auto* dev = static_cast<unsigned char*>(pages->ptr) + begin * pages->page_bytes;
        const uint64_t bytes = (end - begin) * pages->page_bytes;
        if (bytes == 0) return;
        if (to_host) {
            cuda_check(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, pages->ctx->stream), "cudaMemcpyAsync");
        } else {
            cuda_check(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, pages->ctx->stream), "cudaMemcpyAsync");
        }
        cuda_check(cudaStreamSynchronize(pages->ctx->stream), "cudaStreamSynchronize");
    });
}

int32_t psi_pages_export_range(psi_pages* pages, uint64_t page_begin, uint64_t page_end, void* host_out) {
    return pages_copy_range(pages, page_begin, page_end, host_out, true);
}

int32_t psi_pages_import_range(psi_pages* pages, uint64_t page_begin, uint64_t page_end, const void* host_in) {
    return pages_copy_range(pages, page_begin, page_end, const_cast<void*>(host_in), false);
}

int32_t psi_table_create(psi_ctx* ctx, const psi_page_table_layout* layout, psi_table** out) {
    if (ctx == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        require(out != nullptr && layout != nullptr, "out and layout must not be null");
        *out = nullptr;
        validate_layout(*layout);
        ctx->bind();
        auto table = std::make_unique<psi_table>();
        table->ctx = ctx;
        table->layout = *layout;
        const uint64_t words = uint64_t(layout->num_req_slots) * layout->num_gqa_layers * table->row_words();
        table->host.assign(words, 0);
        cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&table->dev), words * sizeof(uint32_t));
        if (err == cudaErrorMemoryAllocation) {
            (void)cudaGetLastError();
            throw ExhaustedError("out of device memory for the page table");
        }
        cuda_check(err, "cudaMalloc");
        cuda_check(cudaMemsetAsync(table->dev, 0, words * sizeof(uint32_t), ctx->stream), "cudaMemsetAsync");
        *out = table.release();
    });
}

int32_t psi_table_destroy(psi_table* table) {
    if (table == nullptr) return PSI_OK;
    int32_t status = guarded(table->ctx, [&] {
        table->ctx->bind();
        (void)cudaStreamSynchronize(table->ctx->stream);
        if (table->dev != nullptr) cuda_check(cudaFree(table->dev), "cudaFree");
    });
    delete table;
    return status;
}

static void table_check(const psi_table* t, uint32_t slot, uint32_t layer, uint32_t block) {
    require(slot < t->layout.num_req_slots, "GQA request page table req_slot out of range");
    require(layer < t->layout.num_gqa_layers, "GQA request page table layer out of range");
    require(block < t->layout.num_blocks, "GQA request page table block out of range");
}

static void table_upload(psi_table* t, uint64_t start, uint64_t count) {
    if (count == 0) return;
    cuda_check(cudaMemcpyAsync(t->dev + start, t->host.data() + start, count * sizeof(uint32_t),
                               cudaMemcpyHostToDevice, t->ctx->stream),
               "cudaMemcpyAsync");
}

int32_t psi_table_write(psi_table* table, uint32_t req_slot, uint32_t layer, uint32_t block, const uint32_t* page_ids,
                        uint32_t n) {
    if (table == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table->ctx, [&] {
        require(page_ids != nullptr, "page_ids must not be null");
        table_check(table, req_slot, layer, block);
        require(n == table->layout.num_page_ids_per_block,
                "GQA page-id count must match one request/GQA-layer/block entry");
        table->check_ids(page_ids, n);
        table->ctx->bind();
        const uint64_t start = table->start_index(req_slot, layer, block);
        std::copy(page_ids, page_ids + n, table->host.begin() + start);
        table_upload(table, start, n);
    });
}

int32_t psi_table_set_page_bound(psi_table* table, uint64_t num_cache_pages) {
    if (table == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table->ctx, [&] {
        require(num_cache_pages <= (uint64_t(1) << 32), "GQA page IDs are u32");
        // IDs stored before the bound was declared are held to it as well (zero rows are page 0, always inside)
        if (num_cache_pages != 0) {
            for (uint32_t id : table->host) {
                require(id < num_cache_pages, "the page table already holds a page ID outside the declared bound");
            }
        }
        table->page_bound = num_cache_pages;
    });
}

int32_t psi_table_write_all_layers(psi_table* table, uint32_t req_slot, uint32_t block, const uint32_t* page_ids,
                                   uint32_t n, uint64_t num_cache_pages) {
    if (table == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table->ctx, [&] {
        require(page_ids != nullptr, "page_ids must not be null");
        table_check(table, req_slot, 0, block);
        const uint32_t per_layer = table->layout.num_page_ids_per_block;
        require(uint64_t(n) == uint64_t(table->layout.num_gqa_layers) * per_layer,
                "GQA cache block must contain all layer page IDs");
        for (uint32_t i = 0; i < n; ++i) {
            require(page_ids[i] < num_cache_pages, "runtime supplied a GQA page ID outside the cache-page buffer");
        }
        table->ctx->bind();
        for (uint32_t layer = 0; layer < table->layout.num_gqa_layers; ++layer) {
            const uint64_t start = table->start_index(req_slot, layer, block);
            std::copy(page_ids + uint64_t(layer) * per_layer, page_ids + uint64_t(layer + 1) * per_layer,
                      table->host.begin() + start);
            table_upload(table, start, per_layer);
        }
    });
}

int32_t psi_table_write_row(psi_table* table, uint32_t req_slot, uint32_t layer, const uint32_t* ids, uint32_t n) {
    if (table == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table->ctx, [&] {
        require(ids != nullptr, "ids must not be null");
        table_check(table, req_slot, layer, 0);
        require(n <= table->row_words(), "page-id count exceeds one request/GQA-layer row");
        table->check_ids(ids, n);
        table->ctx->bind();
        const uint64_t start = table->start_index(req_slot, layer, 0);
        std::copy(ids, ids + n, table->host.begin() + start);
        table_upload(table, start, n);
    });
}

int32_t psi_table_read(psi_table* table, uint32_t req_slot, uint32_t layer, uint32_t block, uint32_t* out, uint32_t n) {
    if (table == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table->ctx, [&] {
        require(out != nullptr, "out must not be null");
        table_check(table, req_slot, layer, block);
        require(n == table->layout.num_page_ids_per_block,
                "GQA page-id count must match one request/GQA-layer/block entry");
        table->ctx->bind();
        const uint64_t start = table->start_index(req_slot, layer, block);
        cuda_check(cudaMemcpyAsync(out, table->dev + start, n * sizeof(uint32_t), cudaMemcpyDeviceToHost,
                                   table->ctx->stream),
                   "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize(table->ctx->stream), "cudaStreamSynchronize");
    });
}

int32_t psi_table_reset_slots(psi_table* table, const uint32_t* req_slots, uint32_t n) {
    if (table == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table->ctx, [&] {
        require(req_slots != nullptr || n == 0, "req_slots must not be null");
        for (uint32_t i = 0; i < n; ++i) require(req_slots[i] < table->layout.num_req_slots,
                                                 "GQA request page table req_slot out of range");
        table->ctx->bind();
        const uint64_t per_req = table->layout.num_gqa_layers * table->row_words();
        for (uint32_t i = 0; i < n; ++i) {
            const uint64_t start = table->start_index(req_slots[i], 0, 0);
            std::fill(table->host.begin() + start, table->host.begin() + start + per_req, 0u);
            cuda_check(cudaMemsetAsync(table->dev + start, 0, per_req * sizeof(uint32_t), table->ctx->stream),
                       "cudaMemsetAsync");
        }
    });
}

int32_t psi_table_device_ptr(psi_table* table, void** out) {
    if (table == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    *out = table->dev;
    return PSI_OK;
}

int32_t psi_id_allocator_create(uint64_t capacity, psi_id_allocator** out) {
    return guarded(nullptr, [&] {
        require(out != nullptr, "out must not be null");
        *out = new psi_id_allocator(capacity);
    });
}

int32_t psi_id_allocator_destroy(psi_id_allocator* a) {
    delete a;
    return PSI_OK;
}

int32_t psi_id_allocator_alloc_many(psi_id_allocator* a, uint64_t count, uint32_t* out_ids) {
    if (a == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        require(out_ids != nullptr || count == 0, "out_ids must not be null");
        a->impl.alloc_many(count, out_ids);
    });
}

int32_t psi_id_allocator_free_many(psi_id_allocator* a, const uint32_t* ids, uint64_t count) {
    if (a == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        require(ids != nullptr || count == 0, "ids must not be null");
        a->impl.free_many(ids, count);
    });
}

int32_t psi_id_allocator_bitmap(psi_id_allocator* a, uint64_t* out_words, uint64_t cap, uint64_t* out_n) {
    if (a == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        const auto& words = a->impl.bitmap();
        if (out_n != nullptr) *out_n = words.size();
        for (uint64_t i = 0; i < words.size() && i < cap && out_words != nullptr; ++i) out_words[i] = words[i];
    });
}

int32_t psi_id_allocator_free_count(psi_id_allocator* a, uint64_t* out) {
    if (a == nullptr || out == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    *out = a->impl.free_count();
    return PSI_OK;
}

}  // extern "C"
