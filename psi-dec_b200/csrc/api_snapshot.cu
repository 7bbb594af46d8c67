// C ABI: hibernation snapshots of the arena and the page tables.
#include "api_internal.hpp"

using namespace psi;

extern "C" {

static SnapshotPlan snapshot_plan(const psi_hibernation_plan* plan) {
    require(plan != nullptr, "plan must not be null");
    SnapshotPlan out;
    out.selected = plan->selected != 0;
    if (out.selected) {
        require(plan->num_request_slot_ranges == 0 || plan->request_slot_ranges != nullptr, "request slot ranges must not be null");
        require(plan->num_page_id_ranges == 0 || plan->page_id_ranges != nullptr, "page ID ranges must not be null");
        for (uint64_t i = 0; i < plan->num_request_slot_ranges; ++i)
            out.request_slot_ranges.emplace_back(plan->request_slot_ranges[i].begin, plan->request_slot_ranges[i].end);
        for (uint64_t i = 0; i < plan->num_page_id_ranges; ++i)
            out.page_id_ranges.emplace_back(plan->page_id_ranges[i].begin, plan->page_id_ranges[i].end);
    }
    return out;
}

static std::vector<U32Range> snapshot_ranges(const psi_u32_range* ranges, uint64_t n) {
    std::vector<U32Range> out;
    for (uint64_t i = 0; i < n; ++i) out.emplace_back(ranges[i].begin, ranges[i].end);
    return out;
}

static SnapshotBuffer pages_buffer(psi_pages* pages) {
    require(pages != nullptr, "pages must not be null");
    require(pages->ptr != nullptr, "page arena resources are released");
    pages->ctx->bind();
    cuda_check(cudaStreamSynchronize(pages->ctx->stream), "cudaStreamSynchronize");
    return SnapshotBuffer{pages->ptr, pages->num_pages * pages->page_bytes, true};
}

static uint64_t table_slot_bytes(const psi_table* table) {
    return uint64_t(table->layout.num_gqa_layers) * table->row_words() * sizeof(uint32_t);
}

int32_t psi_snapshot_writer_create(const char* destination, const uint32_t* expected_files, uint64_t num_files,
                                   const psi_hibernation_plan* plan, psi_snapshot_writer** out) {
    return guarded(nullptr, [&] {
        require(out != nullptr && destination != nullptr, "out and destination must not be null");
        *out = nullptr;
        require(num_files == 0 || expected_files != nullptr, "expected files must not be null");
        const std::vector<uint32_t> files(expected_files, expected_files + num_files);
        *out = new psi_snapshot_writer(destination, files, snapshot_plan(plan));
    });
}

int32_t psi_snapshot_write_pages(psi_snapshot_writer* writer, uint32_t file, psi_pages* pages) {
    if (writer == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(pages != nullptr ? pages->ctx : nullptr, [&] {
        const SnapshotBuffer buffer = pages_buffer(pages);
        if (writer->impl.plan().selected) {
            writer->impl.write_selected_buffer(file, buffer, writer->impl.plan().page_id_ranges, pages->page_bytes);
        } else {
            writer->impl.write_full_buffer(file, buffer);
        }
    });
}

int32_t psi_snapshot_write_table(psi_snapshot_writer* writer, uint32_t file, psi_table* table) {
    if (writer == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table != nullptr ? table->ctx : nullptr, [&] {
        require(table != nullptr, "table must not be null");
        // the host mirror holds exactly what the device table holds: every write goes through both
        const SnapshotBuffer buffer{table->host.data(), table->host.size() * sizeof(uint32_t), false};
        if (writer->impl.plan().selected) {
            writer->impl.write_selected_buffer(file, buffer, writer->impl.plan().request_slot_ranges, table_slot_bytes(table));
        } else {
            writer->impl.write_full_buffer(file, buffer);
        }
    });
}

int32_t psi_snapshot_write_host_buffer(psi_snapshot_writer* writer, uint32_t file, const void* host, uint64_t bytes,
                                       const psi_u32_range* entry_ranges, uint64_t num_ranges, uint64_t entry_bytes) {
    if (writer == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        require(host != nullptr || bytes == 0, "host buffer must not be null");
        const SnapshotBuffer buffer{const_cast<void*>(host), bytes, false};
        if (entry_ranges == nullptr && num_ranges == 0 && entry_bytes == 0) {
            writer->impl.write_full_buffer(file, buffer);
        } else {
            writer->impl.write_selected_buffer(file, buffer, snapshot_ranges(entry_ranges, num_ranges), entry_bytes);
        }
    });
}

int32_t psi_snapshot_write_metadata(psi_snapshot_writer* writer, uint32_t file, const void* bytes, uint64_t n) {
    if (writer == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        require(bytes != nullptr || n == 0, "metadata must not be null");
        writer->impl.write_metadata(file, bytes, n);
    });
}

int32_t psi_snapshot_writer_commit(psi_snapshot_writer* writer) {
    if (writer == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] { writer->impl.commit(); });
}

int32_t psi_snapshot_writer_destroy(psi_snapshot_writer* writer) {
    return guarded(nullptr, [&] { delete writer; });
}

int32_t psi_snapshot_reader_open(const char* path, const uint32_t* expected_files, uint64_t num_files,
                                 const psi_hibernation_plan* plan, psi_snapshot_reader** out) {
    return guarded(nullptr, [&] {
        require(out != nullptr && path != nullptr, "out and path must not be null");
        *out = nullptr;
        require(num_files == 0 || expected_files != nullptr, "expected files must not be null");
        const std::vector<uint32_t> files(expected_files, expected_files + num_files);
        *out = new psi_snapshot_reader(path, files, snapshot_plan(plan));
    });
}

int32_t psi_snapshot_read_pages(psi_snapshot_reader* reader, uint32_t file, psi_pages* pages) {
    if (reader == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(pages != nullptr ? pages->ctx : nullptr, [&] {
        const SnapshotBuffer buffer = pages_buffer(pages);
        if (reader->impl.plan().selected) {
            reader->impl.read_selected_buffer(file, buffer, reader->impl.plan().page_id_ranges, pages->page_bytes);
        } else {
            reader->impl.read_full_buffer(file, buffer);
        }
    });
}

int32_t psi_snapshot_read_table(psi_snapshot_reader* reader, uint32_t file, psi_table* table) {
    if (reader == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(table != nullptr ? table->ctx : nullptr, [&] {
        require(table != nullptr, "table must not be null");
        table->ctx->bind();
        const SnapshotBuffer buffer{table->host.data(), table->host.size() * sizeof(uint32_t), false};
        const uint64_t slot_bytes = table_slot_bytes(table);
        std::vector<U32Range> slots;
        // With a bound declared the mirror is kept aside: a snapshot taken against a larger arena must not bring IDs
        // beyond the bound, and a refused load leaves mirror and device table as they were.
        std::vector<uint32_t> before;
        if (table->page_bound != 0) before = table->host;
        try {
            if (reader->impl.plan().selected) {
                slots = reader->impl.plan().request_slot_ranges;
                reader->impl.read_selected_buffer(file, buffer, slots, slot_bytes);
            } else {
                slots.emplace_back(0u, table->layout.num_req_slots);
                reader->impl.read_full_buffer(file, buffer);
            }
            for (const auto& range : slots) {
                const uint64_t words = slot_bytes / sizeof(uint32_t);
                table->check_ids(table->host.data() + uint64_t(range.first) * words,
                                 uint64_t(range.second - range.first) * words);
            }
        } catch (...) {
            if (table->page_bound != 0) table->host = before;
            throw;
        }
        // the restored rows of the mirror go to the device table
        cuda_check(cudaStreamSynchronize(table->ctx->stream), "cudaStreamSynchronize");
        for (const auto& range : slots) {
            const uint64_t offset = uint64_t(range.first) * slot_bytes, n = uint64_t(range.second - range.first) * slot_bytes;
            cuda_check(cudaMemcpy(reinterpret_cast<unsigned char*>(table->dev) + offset,
                                  reinterpret_cast<const unsigned char*>(table->host.data()) + offset, n, cudaMemcpyHostToDevice),
                       "cudaMemcpy");
        }
    });
}

int32_t psi_snapshot_read_host_buffer(psi_snapshot_reader* reader, uint32_t file, void* host, uint64_t bytes,
                                      const psi_u32_range* entry_ranges, uint64_t num_ranges, uint64_t entry_bytes) {
    if (reader == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        require(host != nullptr || bytes == 0, "host buffer must not be null");
        const SnapshotBuffer buffer{host, bytes, false};
        if (entry_ranges == nullptr && num_ranges == 0 && entry_bytes == 0) {
            reader->impl.read_full_buffer(file, buffer);
        } else {
            reader->impl.read_selected_buffer(file, buffer, snapshot_ranges(entry_ranges, num_ranges), entry_bytes);
        }
    });
}

int32_t psi_snapshot_read_metadata(psi_snapshot_reader* reader, uint32_t file, void* out, uint64_t cap, uint64_t* out_n) {
    if (reader == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] {
        require(out_n != nullptr, "out_n must not be null");
        const std::vector<uint8_t> bytes = reader->impl.read_metadata(file);
        *out_n = bytes.size();
        require(out != nullptr && cap >= bytes.size(), "metadata output capacity too small");
        std::memcpy(out, bytes.data(), bytes.size());
    });
}

int32_t psi_snapshot_reader_finish(psi_snapshot_reader* reader) {
    if (reader == nullptr) return PSI_ERR_INVALID_ARGUMENT;
    return guarded(nullptr, [&] { reader->impl.finish(); });
}

int32_t psi_snapshot_reader_destroy(psi_snapshot_reader* reader) {
    return guarded(nullptr, [&] { delete reader; });
}

}  // extern "C"
