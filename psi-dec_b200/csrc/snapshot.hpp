// Hibernation snapshots of the page arena and the request page tables: a directory with one raw payload file per
// buffer and a `manifest`, published by renaming a temporary directory.
//
// Follows crates/inference-executor-metal/src/model/state_snapshot.rs:40-881 (format "PSISTATE" version 3, file names,
// manifest fields, validation rules and messages) and the selected-entry I/O of
// crates/inference-executor-metal/src/attn/gqa/request_page_table/file_io.rs:14-60.  The manifest bytes follow the
// documented layout of the `wincode` 0.6.1 configuration the reference uses (fixed-width native-endian integers, u32
// sequence lengths, u8 enum tags); the reference holds no byte-level vector of a manifest, so that encoding is
// restated, not pinned.
#pragma once

#include <cstdint>
#include <string>
#include <utility>
#include <vector>

namespace psi {

// StateSnapshotFile (state_snapshot.rs:50-59); the discriminant is the manifest tag and the sort key.
enum SnapshotFile : uint8_t {
    kSnapshotPageArena = 0,
    kSnapshotMainGqaRequestPageTable = 1,
    kSnapshotMainGdnRequestStateTable = 2,
    kSnapshotMainGdnRecurrentState = 3,
    kSnapshotMainGdnConvState = 4,
    kSnapshotMtpGqaRequestPageTable = 5,
    kSnapshotDsparkGqaRequestPageTable = 6,
    kSnapshotFileCount = 7
};
enum SnapshotFileKind : uint8_t { kSnapshotBuffer = 0, kSnapshotMetadata = 1 };

const char* snapshot_file_name(uint32_t file);
SnapshotFileKind snapshot_file_kind(uint32_t file);

using U32Range = std::pair<uint32_t, uint32_t>;  // [first, second)

// ExecutorHibernationPlan: everything, or the listed request slots and page ids.
struct SnapshotPlan {
    bool selected = false;
    std::vector<U32Range> request_slot_ranges;
    std::vector<U32Range> page_id_ranges;
    bool operator==(const SnapshotPlan& o) const {
        return selected == o.selected && request_slot_ranges == o.request_slot_ranges && page_id_ranges == o.page_id_ranges;
    }
};

struct SnapshotManifestEntry {
    uint8_t file;
    uint8_t kind;
    uint64_t payload_bytes;
};

struct SnapshotManifest {
    uint8_t magic[8];
    uint32_t version;
    SnapshotPlan plan;
    std::vector<SnapshotManifestEntry> files;
};

// nonempty, sorted, disjoint and nonadjacent (state_snapshot.rs:774-776)
bool are_canonical_ranges(const std::vector<U32Range>& ranges);
std::vector<uint8_t> encode_manifest(const SnapshotManifest& manifest);
SnapshotManifest decode_manifest(const std::vector<uint8_t>& bytes);  // throws on short or trailing bytes
void validate_manifest(const SnapshotManifest& manifest);

// A buffer the snapshot reads from or writes into: host memory, or device memory copied through a staging buffer.
struct SnapshotBuffer {
    void* ptr = nullptr;
    uint64_t bytes = 0;
    bool on_device = false;
};

class SnapshotWriter {
public:
    SnapshotWriter(const std::string& destination, const std::vector<uint32_t>& expected_files, const SnapshotPlan& plan);
    ~SnapshotWriter();  // removes the temporary directory unless the snapshot was published
    SnapshotWriter(const SnapshotWriter&) = delete;
    SnapshotWriter& operator=(const SnapshotWriter&) = delete;

    const SnapshotPlan& plan() const { return plan_; }
    void write_full_buffer(uint32_t file, const SnapshotBuffer& buffer);
    void write_selected_buffer(uint32_t file, const SnapshotBuffer& buffer, const std::vector<U32Range>& entry_ranges,
                               uint64_t entry_bytes);
    void write_metadata(uint32_t file, const void* bytes, uint64_t n);
    void commit();

private:
    void write_buffer_ranges(uint32_t file, const SnapshotBuffer& buffer, const std::vector<std::pair<uint64_t, uint64_t>>& ranges);
    void assert_file_is_new(uint32_t file) const;

    std::string destination_, temp_path_;
    SnapshotPlan plan_;
    std::vector<uint32_t> expected_files_;
    std::vector<std::pair<SnapshotManifestEntry, int>> files_;  // entry, open descriptor
    bool published_ = false;
};

class SnapshotReader {
public:
    SnapshotReader(const std::string& path, const std::vector<uint32_t>& expected_files, const SnapshotPlan& plan);
    const SnapshotPlan& plan() const { return plan_; }
    void read_full_buffer(uint32_t file, const SnapshotBuffer& buffer);
    void read_selected_buffer(uint32_t file, const SnapshotBuffer& buffer, const std::vector<U32Range>& entry_ranges,
                              uint64_t entry_bytes);
    std::vector<uint8_t> read_metadata(uint32_t file);
    void finish() const;

private:
    void read_buffer_ranges(uint32_t file, const SnapshotBuffer& buffer, const std::vector<std::pair<uint64_t, uint64_t>>& ranges);
    size_t file_index(uint32_t file, SnapshotFileKind expected_kind) const;

    std::string path_;
    SnapshotPlan plan_;
    std::vector<SnapshotManifestEntry> files_;
    std::vector<bool> consumed_;
};

}  // namespace psi
