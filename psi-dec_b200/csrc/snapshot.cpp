// Hibernation snapshot directories: see snapshot.hpp for the format and the reference files it follows.
#include "snapshot.hpp"

#include <cuda_runtime.h>
#include <dirent.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstring>
#include <set>

#include "host_logic.hpp"

namespace psi {

namespace {

constexpr uint8_t kMagic[8] = {'P', 'S', 'I', 'S', 'T', 'A', 'T', 'E'};
constexpr uint32_t kVersion = 3;
constexpr const char* kManifestName = "manifest";
constexpr uint64_t kStagingBytes = 16ull << 20;

std::atomic<uint64_t> g_next_temp_id{0};

[[noreturn]] void fail(const std::string& message) { throw ContractError(message); }

std::string os_error() { return std::strerror(errno); }

std::string parent_of(const std::string& path) {
    const size_t slash = path.find_last_of('/');
    if (slash == std::string::npos) return ".";
    return slash == 0 ? "/" : path.substr(0, slash);
}

std::string name_of(const std::string& path) {
    const size_t slash = path.find_last_of('/');
    return slash == std::string::npos ? path : path.substr(slash + 1);
}

void make_directories(const std::string& path) {
    if (path.empty() || path == "/" || path == ".") return;
    struct stat st;
    if (stat(path.c_str(), &st) == 0) return;
    make_directories(parent_of(path));
    if (mkdir(path.c_str(), 0777) != 0 && errno != EEXIST)
        fail("unable to create model state snapshot parent directory \"" + path + "\": " + os_error());
}

void sync_directory(const std::string& path, const char* what) {
    const int fd = open(path.c_str(), O_RDONLY | O_DIRECTORY);
    if (fd < 0) fail(std::string("unable to sync ") + what + " \"" + path + "\": " + os_error());
    const int rc = fsync(fd);
    close(fd);
    if (rc != 0) fail(std::string("unable to sync ") + what + " \"" + path + "\": " + os_error());
}

void remove_tree(const std::string& path) {
    DIR* dir = opendir(path.c_str());
    if (dir != nullptr) {
        while (dirent* e = readdir(dir)) {
            const std::string name = e->d_name;
            if (name == "." || name == "..") continue;
            unlink((path + "/" + name).c_str());
        }
        closedir(dir);
    }
    rmdir(path.c_str());
}

void write_all(int fd, const void* data, uint64_t n, const std::string& what) {
    const char* p = static_cast<const char*>(data);
    while (n > 0) {
        const ssize_t done = write(fd, p, n);
        if (done < 0) {
            if (errno == EINTR) continue;
            fail("unable to write " + what + ": " + os_error());
        }
        p += done;
        n -= static_cast<uint64_t>(done);
    }
}

void read_all(int fd, void* data, uint64_t n, const std::string& what) {
    char* p = static_cast<char*>(data);
    while (n > 0) {
        const ssize_t done = read(fd, p, n);
        if (done < 0) {
            if (errno == EINTR) continue;
            fail("unable to read " + what + ": " + os_error());
        }
        if (done == 0) fail("unable to read " + what + ": unexpected end of file");
        p += done;
        n -= static_cast<uint64_t>(done);
    }
}

// Pinned staging for device buffers; falls back to pageable memory when pinning fails.
struct Staging {
    void* ptr = nullptr;
    bool pinned = false;
    Staging() {
        if (cudaMallocHost(&ptr, kStagingBytes) == cudaSuccess) {
            pinned = true;
        } else {
            (void)cudaGetLastError();
            ptr = ::operator new(kStagingBytes);
        }
    }
    ~Staging() {
        if (pinned) {
            cudaFreeHost(ptr);
        } else {
            ::operator delete(ptr);
        }
    }
};

void cuda_ok(cudaError_t err, const char* what) {
    if (err != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
}

void buffer_to_file(const SnapshotBuffer& buffer, uint64_t offset, int fd, uint64_t n, const std::string& what) {
    const char* base = static_cast<const char*>(buffer.ptr) + offset;
    if (!buffer.on_device) {
        write_all(fd, base, n, what);
        return;
    }
    Staging staging;
    for (uint64_t done = 0; done < n;) {
        const uint64_t chunk = std::min(kStagingBytes, n - done);
        cuda_ok(cudaMemcpy(staging.ptr, base + done, chunk, cudaMemcpyDeviceToHost), "snapshot device-to-host copy");
        write_all(fd, staging.ptr, chunk, what);
        done += chunk;
    }
}

void file_to_buffer(int fd, const SnapshotBuffer& buffer, uint64_t offset, uint64_t n, const std::string& what) {
    char* base = static_cast<char*>(buffer.ptr) + offset;
    if (!buffer.on_device) {
        read_all(fd, base, n, what);
        return;
    }
    Staging staging;
    for (uint64_t done = 0; done < n;) {
        const uint64_t chunk = std::min(kStagingBytes, n - done);
        read_all(fd, staging.ptr, chunk, what);
        cuda_ok(cudaMemcpy(base + done, staging.ptr, chunk, cudaMemcpyHostToDevice), "snapshot host-to-device copy");
        done += chunk;
    }
}

std::set<uint32_t> validate_expected_file_set(const std::vector<uint32_t>& expected_files) {
    std::set<uint32_t> expected(expected_files.begin(), expected_files.end());
    for (uint32_t file : expected_files) require(file < kSnapshotFileCount, "unknown model state snapshot file");
    if (expected.size() != expected_files.size()) fail("model state snapshot expected file set contains duplicates");
    if (expected.empty()) fail("model state snapshot expected file set must not be empty");
    return expected;
}

std::string debug_name(uint32_t file) {
    static const char* names[kSnapshotFileCount] = {"PageArena", "MainGQARequestPageTable", "MainGDNRequestStateTable",
                                                    "MainGDNRecurrentState", "MainGDNConvState", "MTPGQARequestPageTable",
                                                    "DSparkGQARequestPageTable"};
    return file < kSnapshotFileCount ? names[file] : "?";
}

void validate_expected_files(const std::vector<SnapshotManifestEntry>& actual, const std::vector<uint32_t>& expected_files) {
    const std::set<uint32_t> expected = validate_expected_file_set(expected_files);
    std::set<uint32_t> present;
    for (const auto& entry : actual) present.insert(entry.file);
    for (uint32_t file : expected)
        if (present.count(file) == 0) fail("model state snapshot file is missing: file=" + debug_name(file));
    for (uint32_t file : present)
        if (expected.count(file) == 0) fail("model state snapshot contains an unexpected file: file=" + debug_name(file));
}

void validate_plan(const SnapshotPlan& plan) {
    if (!plan.selected) return;
    if (!are_canonical_ranges(plan.request_slot_ranges))
        fail("model state snapshot request slot ranges must be nonempty, sorted, disjoint, and nonadjacent");
    if (!are_canonical_ranges(plan.page_id_ranges))
        fail("model state snapshot page ID ranges must be nonempty, sorted, disjoint, and nonadjacent");
}

void validate_snapshot_directory(const std::string& path, const std::vector<SnapshotManifestEntry>& files) {
    std::set<std::string> expected_names;
    for (const auto& entry : files) expected_names.insert(snapshot_file_name(entry.file));
    expected_names.insert(kManifestName);
    DIR* dir = opendir(path.c_str());
    if (dir == nullptr) fail("unable to enumerate model state snapshot \"" + path + "\": " + os_error());
    std::string problem;
    while (dirent* e = readdir(dir)) {
        const std::string name = e->d_name;
        if (name == "." || name == "..") continue;
        if (expected_names.erase(name) == 0) {
            problem = "model state snapshot contains an unexpected file: \"" + name + "\"";
            break;
        }
        struct stat st;
        if (lstat((path + "/" + name).c_str(), &st) != 0 || !S_ISREG(st.st_mode)) {
            problem = "model state snapshot entry must be a regular file: \"" + name + "\"";
            break;
        }
    }
    closedir(dir);
    if (!problem.empty()) fail(problem);
    if (!expected_names.empty()) fail("model state snapshot file is missing: \"" + *expected_names.begin() + "\"");
    for (const auto& entry : files) {
        struct stat st;
        const std::string file_path = path + "/" + snapshot_file_name(entry.file);
        if (stat(file_path.c_str(), &st) != 0) fail("unable to inspect model state snapshot entry \"" + file_path + "\": " + os_error());
        if (static_cast<uint64_t>(st.st_size) != entry.payload_bytes)
            fail("model state snapshot file length mismatch: file=" + debug_name(entry.file) + " expected=" +
                 std::to_string(entry.payload_bytes) + " actual=" + std::to_string(st.st_size));
    }
}

std::vector<std::pair<uint64_t, uint64_t>> selected_buffer_ranges(const SnapshotBuffer& buffer, const std::vector<U32Range>& entry_ranges,
                                                                  uint64_t entry_bytes) {
    require(entry_bytes > 0, "model state snapshot buffer entry size must be positive");
    require(entry_ranges.empty() || are_canonical_ranges(entry_ranges),
            "model state snapshot buffer entry ranges must be nonempty, sorted, disjoint, and nonadjacent");
    std::vector<std::pair<uint64_t, uint64_t>> out;
    for (const auto& range : entry_ranges) {
        const uint64_t start = static_cast<uint64_t>(range.first) * entry_bytes;
        const uint64_t end = static_cast<uint64_t>(range.second) * entry_bytes;
        if (end > buffer.bytes) fail("model state snapshot buffer entry range is out of bounds");
        out.emplace_back(start, end);
    }
    return out;
}

// ---- manifest encoding: fixed-width native-endian integers, u32 sequence lengths, u8 enum tags ------------------------
struct Encoder {
    std::vector<uint8_t> bytes;
    void raw(const void* p, size_t n) {
        const uint8_t* b = static_cast<const uint8_t*>(p);
        bytes.insert(bytes.end(), b, b + n);
    }
    void u8(uint8_t v) { bytes.push_back(v); }
    void u32(uint32_t v) { raw(&v, 4); }
    void u64(uint64_t v) { raw(&v, 8); }
    void ranges(const std::vector<U32Range>& r) {
        u32(static_cast<uint32_t>(r.size()));
        for (const auto& x : r) {
            u32(x.first);
            u32(x.second);
        }
    }
};

struct Decoder {
    const std::vector<uint8_t>& bytes;
    size_t at = 0;
    void raw(void* p, size_t n) {
        if (bytes.size() - at < n) fail("unable to decode model state manifest: unexpected end of input");
        std::memcpy(p, bytes.data() + at, n);
        at += n;
    }
    uint8_t u8() {
        uint8_t v;
        raw(&v, 1);
        return v;
    }
    uint32_t u32() {
        uint32_t v;
        raw(&v, 4);
        return v;
    }
    uint64_t u64() {
        uint64_t v;
        raw(&v, 8);
        return v;
    }
    std::vector<U32Range> ranges() {
        const uint32_t n = u32();
        if ((bytes.size() - at) / 8 < n) fail("unable to decode model state manifest: unexpected end of input");
        std::vector<U32Range> out(n);
        for (auto& x : out) {
            x.first = u32();
            x.second = u32();
        }
        return out;
    }
};

}  // namespace

const char* snapshot_file_name(uint32_t file) {
    static const char* names[kSnapshotFileCount] = {"page-arena", "main-gqa-request-page-table", "main-gdn-request-state-table",
                                                    "main-gdn-recurrent-state", "main-gdn-conv-state",
                                                    "mtp-gqa-request-page-table", "dspark-gqa-request-page-table"};
    require(file < kSnapshotFileCount, "unknown model state snapshot file");
    return names[file];
}

SnapshotFileKind snapshot_file_kind(uint32_t file) {
    return file == kSnapshotMainGdnRequestStateTable ? kSnapshotMetadata : kSnapshotBuffer;
}

bool are_canonical_ranges(const std::vector<U32Range>& ranges) {
    for (const auto& r : ranges)
        if (r.first >= r.second) return false;
    for (size_t i = 1; i < ranges.size(); ++i)
        if (ranges[i - 1].second >= ranges[i].first) return false;
    return true;
}

std::vector<uint8_t> encode_manifest(const SnapshotManifest& manifest) {
    Encoder e;
    e.raw(manifest.magic, 8);
    e.u32(manifest.version);
    e.u8(manifest.plan.selected ? 1 : 0);
    if (manifest.plan.selected) {
        e.ranges(manifest.plan.request_slot_ranges);
        e.ranges(manifest.plan.page_id_ranges);
    }
    e.u32(static_cast<uint32_t>(manifest.files.size()));
    for (const auto& entry : manifest.files) {
        e.u8(entry.file);
        e.u8(entry.kind);
        e.u64(entry.payload_bytes);
    }
    return e.bytes;
}

SnapshotManifest decode_manifest(const std::vector<uint8_t>& bytes) {
    Decoder d{bytes};
    SnapshotManifest m{};
    d.raw(m.magic, 8);
    m.version = d.u32();
    const uint8_t plan_tag = d.u8();
    if (plan_tag > 1) fail("unable to decode model state manifest: invalid plan tag");
    m.plan.selected = plan_tag == 1;
    if (m.plan.selected) {
        m.plan.request_slot_ranges = d.ranges();
        m.plan.page_id_ranges = d.ranges();
    }
    const uint32_t n = d.u32();
    if ((bytes.size() - d.at) / 10 < n) fail("unable to decode model state manifest: unexpected end of input");
    m.files.resize(n);
    for (auto& entry : m.files) {
        entry.file = d.u8();
        entry.kind = d.u8();
        if (entry.file >= kSnapshotFileCount || entry.kind > 1) fail("unable to decode model state manifest: invalid file tag");
        entry.payload_bytes = d.u64();
    }
    if (d.at != bytes.size())
        fail("model state manifest contains trailing bytes: file_bytes=" + std::to_string(bytes.size()) +
             " consumed=" + std::to_string(d.at));
    return m;
}

void validate_manifest(const SnapshotManifest& manifest) {
    if (std::memcmp(manifest.magic, kMagic, 8) != 0) fail("model state snapshot magic mismatch");
    if (manifest.version != kVersion)
        fail("model state snapshot version mismatch: expected=" + std::to_string(kVersion) +
             " actual=" + std::to_string(manifest.version));
    validate_plan(manifest.plan);
    if (manifest.files.empty()) fail("model state snapshot must contain at least one file");
    for (size_t i = 1; i < manifest.files.size(); ++i)
        if (manifest.files[i - 1].file >= manifest.files[i].file) fail("model state snapshot files must be unique and sorted");
    for (const auto& entry : manifest.files) {
        if (entry.kind == kSnapshotMetadata && entry.payload_bytes == 0)
            fail("model state snapshot metadata files must not be empty");
        if (entry.kind != snapshot_file_kind(entry.file)) fail("model state snapshot file kind does not match its semantic file");
    }
}

// ---- writer -----------------------------------------------------------------------------------------------------------
SnapshotWriter::SnapshotWriter(const std::string& destination, const std::vector<uint32_t>& expected_files, const SnapshotPlan& plan)
    : destination_(destination), plan_(plan), expected_files_(expected_files) {
    validate_plan(plan);
    validate_expected_file_set(expected_files);
    require(!destination.empty() && !name_of(destination).empty(), "model state snapshot path has no file name");
    const std::string parent = parent_of(destination);
    make_directories(parent);
    struct stat st;
    if (lstat(destination.c_str(), &st) == 0) fail("model state snapshot destination already exists: \"" + destination + "\"");
    if (errno != ENOENT) fail("unable to inspect model state snapshot destination \"" + destination + "\": " + os_error());
    temp_path_ = parent + "/." + name_of(destination) + ".tmp-" + std::to_string(getpid()) + "-" +
                 std::to_string(g_next_temp_id.fetch_add(1));
    if (mkdir(temp_path_.c_str(), 0777) != 0)
        fail("unable to create temporary model state snapshot directory \"" + temp_path_ + "\": " + os_error());
}

SnapshotWriter::~SnapshotWriter() {
    for (auto& f : files_)
        if (f.second >= 0) close(f.second);
    if (!published_) remove_tree(temp_path_);
}

void SnapshotWriter::assert_file_is_new(uint32_t file) const {
    for (const auto& f : files_)
        if (f.first.file == file) fail("model state snapshot file was written twice: file=" + debug_name(file));
}

void SnapshotWriter::write_full_buffer(uint32_t file, const SnapshotBuffer& buffer) {
    if (buffer.bytes == 0) fail("model state snapshot buffer must not be empty: file=" + debug_name(file));
    write_buffer_ranges(file, buffer, {{0, buffer.bytes}});
}

void SnapshotWriter::write_selected_buffer(uint32_t file, const SnapshotBuffer& buffer, const std::vector<U32Range>& entry_ranges,
                                           uint64_t entry_bytes) {
    write_buffer_ranges(file, buffer, selected_buffer_ranges(buffer, entry_ranges, entry_bytes));
}

void SnapshotWriter::write_buffer_ranges(uint32_t file, const SnapshotBuffer& buffer,
                                         const std::vector<std::pair<uint64_t, uint64_t>>& ranges) {
    require(file < kSnapshotFileCount, "unknown model state snapshot file");
    if (snapshot_file_kind(file) != kSnapshotBuffer)
        fail("model state snapshot file does not contain a buffer: file=" + debug_name(file));
    assert_file_is_new(file);
    const std::string path = temp_path_ + "/" + snapshot_file_name(file);
    const int fd = open(path.c_str(), O_WRONLY | O_CREAT | O_EXCL, 0666);
    if (fd < 0) fail("unable to create model state buffer file " + debug_name(file) + " at \"" + path + "\": " + os_error());
    files_.push_back({SnapshotManifestEntry{static_cast<uint8_t>(file), kSnapshotBuffer, 0}, fd});
    uint64_t payload = 0;
    for (const auto& range : ranges) {
        buffer_to_file(buffer, range.first, fd, range.second - range.first, "model state buffer file " + debug_name(file));
        payload += range.second - range.first;
    }
    files_.back().first.payload_bytes = payload;
}

void SnapshotWriter::write_metadata(uint32_t file, const void* bytes, uint64_t n) {
    require(file < kSnapshotFileCount, "unknown model state snapshot file");
    if (snapshot_file_kind(file) != kSnapshotMetadata)
        fail("model state snapshot file does not contain metadata: file=" + debug_name(file));
    assert_file_is_new(file);
    if (n == 0) fail("model state snapshot metadata must not be empty: file=" + debug_name(file));
    const std::string path = temp_path_ + "/" + snapshot_file_name(file);
    const int fd = open(path.c_str(), O_WRONLY | O_CREAT | O_EXCL, 0666);
    if (fd < 0) fail("unable to create model state metadata file " + debug_name(file) + " at \"" + path + "\": " + os_error());
    files_.push_back({SnapshotManifestEntry{static_cast<uint8_t>(file), kSnapshotMetadata, n}, fd});
    write_all(fd, bytes, n, "model state metadata file " + debug_name(file));
}

void SnapshotWriter::commit() {
    std::sort(files_.begin(), files_.end(), [](const auto& a, const auto& b) { return a.first.file < b.first.file; });
    std::vector<SnapshotManifestEntry> entries;
    for (const auto& f : files_) entries.push_back(f.first);
    validate_expected_files(entries, expected_files_);
    for (auto& f : files_) {
        if (fsync(f.second) != 0) fail("unable to sync model state file " + debug_name(f.first.file) + ": " + os_error());
        close(f.second);
        f.second = -1;
    }
    SnapshotManifest manifest{};
    std::memcpy(manifest.magic, kMagic, 8);
    manifest.version = kVersion;
    manifest.plan = plan_;
    manifest.files = entries;
    const std::vector<uint8_t> bytes = encode_manifest(manifest);
    const std::string manifest_path = temp_path_ + "/" + kManifestName;
    const int fd = open(manifest_path.c_str(), O_WRONLY | O_CREAT | O_EXCL, 0666);
    if (fd < 0) fail("unable to create model state manifest \"" + manifest_path + "\": " + os_error());
    try {
        write_all(fd, bytes.data(), bytes.size(), "model state manifest");
        if (fsync(fd) != 0) fail("unable to sync model state manifest \"" + manifest_path + "\": " + os_error());
    } catch (...) {
        close(fd);
        throw;
    }
    close(fd);
    files_.clear();
    sync_directory(temp_path_, "temporary model state snapshot directory");
    if (rename(temp_path_.c_str(), destination_.c_str()) != 0)
        fail("unable to publish model state snapshot directory \"" + temp_path_ + "\" as \"" + destination_ + "\": " + os_error());
    published_ = true;
    sync_directory(parent_of(destination_), "model state snapshot parent directory");
}

// ---- reader -----------------------------------------------------------------------------------------------------------
SnapshotReader::SnapshotReader(const std::string& path, const std::vector<uint32_t>& expected_files, const SnapshotPlan& plan)
    : path_(path), plan_(plan) {
    validate_plan(plan);
    validate_expected_file_set(expected_files);
    struct stat st;
    if (lstat(path.c_str(), &st) != 0) fail("unable to inspect model state snapshot \"" + path + "\": " + os_error());
    if (!S_ISDIR(st.st_mode)) fail("model state snapshot must be a directory: \"" + path + "\"");
    const std::string manifest_path = path + "/" + kManifestName;
    const int fd = open(manifest_path.c_str(), O_RDONLY);
    if (fd < 0) fail("unable to open model state manifest \"" + manifest_path + "\": " + os_error());
    std::vector<uint8_t> bytes;
    if (fstat(fd, &st) == 0) bytes.resize(static_cast<size_t>(st.st_size));
    try {
        read_all(fd, bytes.data(), bytes.size(), "model state manifest");
    } catch (...) {
        close(fd);
        throw;
    }
    close(fd);
    const SnapshotManifest manifest = decode_manifest(bytes);
    validate_manifest(manifest);
    if (!(manifest.plan == plan)) fail("model state snapshot hibernation plan does not match the requested plan");
    validate_expected_files(manifest.files, expected_files);
    validate_snapshot_directory(path, manifest.files);
    files_ = manifest.files;
    consumed_.assign(files_.size(), false);
}

size_t SnapshotReader::file_index(uint32_t file, SnapshotFileKind expected_kind) const {
    size_t index = files_.size();
    for (size_t i = 0; i < files_.size(); ++i)
        if (files_[i].file == file) index = i;
    if (index == files_.size()) fail("model state snapshot file is missing: file=" + debug_name(file));
    if (consumed_[index]) fail("model state snapshot file was read twice: file=" + debug_name(file));
    if (files_[index].kind != expected_kind) fail("model state snapshot file kind mismatch: file=" + debug_name(file));
    return index;
}

void SnapshotReader::read_full_buffer(uint32_t file, const SnapshotBuffer& buffer) {
    read_buffer_ranges(file, buffer, {{0, buffer.bytes}});
}

void SnapshotReader::read_selected_buffer(uint32_t file, const SnapshotBuffer& buffer, const std::vector<U32Range>& entry_ranges,
                                          uint64_t entry_bytes) {
    read_buffer_ranges(file, buffer, selected_buffer_ranges(buffer, entry_ranges, entry_bytes));
}

void SnapshotReader::read_buffer_ranges(uint32_t file, const SnapshotBuffer& buffer,
                                        const std::vector<std::pair<uint64_t, uint64_t>>& ranges) {
    const size_t index = file_index(file, kSnapshotBuffer);
    uint64_t expected = 0;
    for (const auto& range : ranges) expected += range.second - range.first;
    if (files_[index].payload_bytes != expected)
        fail("model state snapshot file length mismatch: file=" + debug_name(file) + " expected=" + std::to_string(expected) +
             " actual=" + std::to_string(files_[index].payload_bytes));
    if (!ranges.empty()) {
        const std::string path = path_ + "/" + snapshot_file_name(file);
        const int fd = open(path.c_str(), O_RDONLY);
        if (fd < 0) fail("unable to open model state buffer file " + debug_name(file) + " at \"" + path + "\": " + os_error());
        try {
            for (const auto& range : ranges)
                file_to_buffer(fd, buffer, range.first, range.second - range.first, "model state buffer file " + debug_name(file));
        } catch (...) {
            close(fd);
            throw;
        }
        close(fd);
    }
    consumed_[index] = true;
}

std::vector<uint8_t> SnapshotReader::read_metadata(uint32_t file) {
    const size_t index = file_index(file, kSnapshotMetadata);
    std::vector<uint8_t> bytes(static_cast<size_t>(files_[index].payload_bytes));
    const std::string path = path_ + "/" + snapshot_file_name(file);
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) fail("unable to open model state metadata file " + debug_name(file) + " at \"" + path + "\": " + os_error());
    try {
        read_all(fd, bytes.data(), bytes.size(), "model state metadata file " + debug_name(file));
    } catch (...) {
        close(fd);
        throw;
    }
    close(fd);
    consumed_[index] = true;
    return bytes;
}

void SnapshotReader::finish() const {
    for (size_t i = 0; i < files_.size(); ++i)
        if (!consumed_[i]) fail("model state snapshot file was not read: file=" + debug_name(files_[i].file));
}

}  // namespace psi
