// A C++17 caller of include/psi_cuda.hpp: the reference's component types as a compiled host sees them.
//
//   host_mirror_check host            the host-only types against the vectors of the reference's own tests
//                                     (ReplayBucketPolicy: crates/inference-executor-core/src/replay.rs:94-180;
//                                     GQASplitKV: crates/inference-backend-metal/src/components/gqa_split_kv.rs:177-231;
//                                     U32IDAllocator: crates/inference-runtime-core/src/memory/u32_id_allocator.rs:179-217)
//                                     and the messages their contracts fail with; no GPU needed
//   host_mirror_check step <out.bin>  the CPU-scale configuration end to end on device 0 through PageArena,
//                                     GQARequestPageTable and GQA (prepare, then record: append + attention as one
//                                     launch), written as q | k | v | arena after the step | out for the caller to check;
//                                     then the same step again through kv_page_write + attend, which must reproduce
//                                     the arena bit for bit and the output within one f16 step
//
// Inputs come from the 32-bit LCG of the reference's parity fixtures
// (crates/inference-backend-metal/src/components/gqa_split_kv_single_q_test.rs:432-440), truncated to f16.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

#include "psi_cuda.hpp"

namespace {

int failures = 0;

void expect(bool ok, const char* what) {
    if (!ok) {
        std::fprintf(stderr, "FAILED: %s\n", what);
        ++failures;
    }
}
#define EXPECT(cond) expect((cond), #cond)

// The call must throw psi::Error whose message contains `text`.
void expect_error(const std::function<void()>& call, const char* text) {
    try {
        call();
    } catch (const psi::Error& e) {
        if (std::string(e.what()).find(text) == std::string::npos) {
            std::fprintf(stderr, "FAILED: message \"%s\" lacks \"%s\"\n", e.what(), text);
            ++failures;
        }
        return;
    }
    std::fprintf(stderr, "FAILED: no error, expected \"%s\"\n", text);
    ++failures;
}

using U32s = std::vector<uint32_t>;

int run_host() {
    // ReplayBucketPolicy (replay.rs:94-180)
    const U32s base = {1, 2, 4, 6, 8, 12, 16, 20, 24, 32, 40, 48, 56, 64};
    EXPECT(psi::ReplayBucketPolicy(64).buckets() == base);
    U32s wide = base;
    for (uint32_t b : {80u, 96u, 112u, 128u}) wide.push_back(b);
    EXPECT(psi::ReplayBucketPolicy(128).buckets() == wide);
    EXPECT((psi::ReplayBucketPolicy(6).buckets() == U32s{1, 2, 4, 6}));
    EXPECT(psi::ReplayBucketPolicy(70).buckets().back() == 70);
    const psi::ReplayBucketPolicy p64(64);
    const uint32_t active[] = {1, 3, 5, 9, 25, 64}, padded[] = {1, 4, 6, 12, 32, 64};
    for (int i = 0; i < 6; ++i) EXPECT(p64.capacity(active[i]) == padded[i]);
    const psi::ReplayBucketPolicy topo(64, {5, 6, 10, 12, 18});
    const uint32_t t_active[] = {5, 9, 10, 11, 17, 18}, t_padded[] = {5, 9, 11, 11, 17, 20};
    for (int i = 0; i < 6; ++i) EXPECT(topo.capacity(t_active[i]) == t_padded[i]);
    EXPECT((psi::ReplayBucketPolicy(8, {6}).buckets() == U32s{1, 2, 4, 5, 6, 8}));
    expect_error([] { (void)psi::ReplayBucketPolicy(6).capacity(7); }, "replay active work exceeds capacity");
    expect_error([] { (void)psi::ReplayBucketPolicy(6).capacity(0); }, "replay bucket requires active work");

    // GQASplitKV (gqa_split_kv.rs:177-231): bf16, two KV heads
    auto selector = [](uint32_t head_dim, uint32_t group, uint32_t tokens_per_page, bool dspark = false) {
        const uint32_t hkv = 2;
        return psi::GQASplitKV(PSI_DTYPE_BF16, 2 * hkv * head_dim * tokens_per_page * 2, hkv * group, hkv, head_dim, dspark);
    };
    auto same = [](const psi::GQASplitKVVariant& v, uint32_t tiled, uint32_t q_tile, uint32_t kv_tile, uint32_t threads,
                   uint32_t head_tile) {
        return v.tiled_q == tiled && v.q_token_tile_size == q_tile && v.kv_token_tile_size == kv_tile &&
               v.num_threads_per_threadblock == threads && v.q_head_tile_size == head_tile;
    };
    uint32_t per_partial = 0;
    EXPECT(same(selector(256, 6, 16).select(4, 4, &per_partial), 0, 0, 256, 256, 6));
    EXPECT(per_partial == 8);
    EXPECT(same(selector(256, 6, 16).select(8, 4), 1, 8, 16, 0, 3));
    EXPECT(same(selector(256, 6, 16).select(16, 4), 1, 8, 16, 0, 6));
    EXPECT(same(selector(256, 6, 8).select(16, 4), 1, 8, 16, 0, 6));
    EXPECT(same(selector(128, 8, 8).select(8, 4), 1, 8, 16, 0, 8));
    EXPECT(selector(256, 8, 4).select(16, 4).tiled_q == 0);
    EXPECT(selector(128, 8, 8, true).select(16, 4).tiled_q == 0);

    // U32IDAllocator (u32_id_allocator.rs:69-126, 179-217): freed IDs first, then fresh ones in ascending order
    psi::U32IDAllocator ids(130);
    const U32s first = ids.alloc_many(66);
    const uint64_t full = ~uint64_t(0);
    EXPECT((ids.allocated_ids_bitmap() == std::vector<uint64_t>{full, 0b11, 0}));
    ids.free_many({1, 63, 64, 65});
    EXPECT((ids.allocated_ids_bitmap() == std::vector<uint64_t>{full & ~(uint64_t(0b10) | (uint64_t(1) << 63)), 0, 0}));
    EXPECT(ids.free_count() == 130 - 62);
    U32s again = ids.alloc_many(4);
    std::sort(again.begin(), again.end());
    EXPECT((again == U32s{1, 63, 64, 65}));  // the freed IDs come back before any fresh one
    EXPECT((ids.allocated_ids_bitmap() == std::vector<uint64_t>{full, 0b11, 0}));
    ids.free_many(first);
    EXPECT((ids.allocated_ids_bitmap() == std::vector<uint64_t>{0, 0, 0}));
    expect_error([] { (void)psi::U32IDAllocator(3).alloc_many(4); }, "not enough ID");

    std::printf(failures == 0 ? "host ok\n" : "host FAILED\n");
    return failures == 0 ? 0 : 1;
}

uint32_t lcg_state = 0x4C8F17D2u;

float lcg_next() {
    lcg_state = lcg_state * 1664525u + 1013904223u;
    return static_cast<float>(lcg_state >> 8) / 16777216.0f * 2.0f - 1.0f;
}

uint16_t to_half(float f) {  // round toward zero; enough for values in (-1, 1)
    uint32_t x;
    std::memcpy(&x, &f, sizeof x);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const int32_t exponent = static_cast<int32_t>((x >> 23) & 0xFFu) - 127 + 15;
    if (exponent <= 0) return static_cast<uint16_t>(sign);
    if (exponent >= 31) return static_cast<uint16_t>(sign | 0x7BFFu);
    return static_cast<uint16_t>(sign | (static_cast<uint32_t>(exponent) << 10) | ((x & 0x7FFFFFu) >> 13));
}

float from_half(uint16_t h) {
    const uint32_t sign = (h & 0x8000u) << 16, exponent = (h >> 10) & 0x1Fu, mantissa = h & 0x3FFu;
    if (exponent == 0) return (sign ? -1.0f : 1.0f) * std::ldexp(static_cast<float>(mantissa), -24);
    const uint32_t bits = sign | ((exponent + 112u) << 23) | (mantissa << 13);
    float f;
    std::memcpy(&f, &bits, sizeof f);
    return f;
}

// A device buffer for the step's q / k / v / out.
struct DeviceBytes {
    void* ptr = nullptr;
    explicit DeviceBytes(size_t bytes) {
        if (cudaMalloc(&ptr, bytes) != cudaSuccess) throw psi::Error(PSI_ERR_CUDA, "cudaMalloc failed");
    }
    ~DeviceBytes() { (void)cudaFree(ptr); }
    DeviceBytes(const DeviceBytes&) = delete;
    DeviceBytes& operator=(const DeviceBytes&) = delete;
};

int run_step(const char* out_path) {
    constexpr uint32_t HQ = 4, HKV = 1, D = 128, P = 16, PAGES = 64, CONTEXT = 256;
    constexpr uint32_t page_bytes = 2u * HKV * P * D * 2u;
    constexpr size_t page_elems = page_bytes / 2u;
    psi::Context ctx(0);
    psi::PageArena pages(ctx, PAGES, page_bytes);
    const psi::GQAPageTableLayout layout{1, 1, PAGES, 1};
    psi::GQARequestPageTable table(ctx, layout);
    table.set_page_bound(PAGES);

    std::vector<uint16_t> arena(PAGES * page_elems), q(HQ * D), k(HKV * D), v(HKV * D), out(HQ * D), out2(HQ * D);
    for (auto& x : arena) x = to_half(lcg_next());
    for (auto& x : q) x = to_half(lcg_next());
    for (auto& x : k) x = to_half(lcg_next());
    for (auto& x : v) x = to_half(lcg_next());
    pages.import_range(0, PAGES, arena.data());
    U32s ids(PAGES);
    for (uint32_t i = 0; i < PAGES; ++i) ids[i] = (i * 37u + 11u) % PAGES;
    table.write_row(0, 0, ids);
    expect_error([&] { table.write_page_ids(0, 0, 0, {PAGES}); },
                 "runtime supplied a GQA page ID outside the cache-page buffer");
    EXPECT(table.read_page_ids(0, 0, 5) == U32s{ids[5]});

    psi::GQAConfig config{};
    config.num_q_heads = HQ;
    config.num_kv_heads = HKV;
    config.head_dim = D;
    config.scale = 0.08838834764831845f;  // 1 / sqrt(128)
    config.page_bytes = page_bytes;
    config.dtype = PSI_DTYPE_F16;
    config.layout = layout;
    config.max_tokens = 1;
    config.plan_mode = PSI_PLAN_BALANCED;
    config.kernel_mode = PSI_KERNEL_AUTO;
    psi::GQA gqa(ctx, config);
    expect_error([&] { (void)gqa.prepare({0}, {CONTEXT}, {0, 2}); }, "GQA batch exceeds the metadata token capacity");
    expect_error([&] { (void)gqa.prepare({0, 1}, {CONTEXT}, {0, 1}); }, "lengths disagree");

    DeviceBytes dq(q.size() * 2), dk(k.size() * 2), dv(v.size() * 2), dout(out.size() * 2);
    cudaMemcpy(dq.ptr, q.data(), q.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dk.ptr, k.data(), k.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dv.ptr, v.data(), v.size() * 2, cudaMemcpyHostToDevice);
    expect_error([&] { gqa.attend(pages, table, 0, dq.ptr, dout.ptr); }, "GQA batch metadata must be updated before recording");

    const psi::GQAReplayShape shape = gqa.prepare({0}, {CONTEXT}, {0, 1});
    EXPECT(shape.num_tokens == 1 && shape.num_total_tokens == 1);
    const uint64_t launches_before = ctx.launch_count();
    gqa.record(pages, table, 0, dk.ptr, dv.ptr, dq.ptr, dout.ptr);
    EXPECT(ctx.launch_count() == launches_before + 1);  // append + attention as ONE launch
    ctx.wait();
    EXPECT(gqa.device_status() == 0);
    cudaMemcpy(out.data(), dout.ptr, out.size() * 2, cudaMemcpyDeviceToHost);
    std::vector<uint16_t> arena_after(arena.size());
    pages.export_range(0, PAGES, arena_after.data());

    // the reference's recorded order, as two launches, on a second arena with the same contents
    psi::PageArena pages2(ctx, PAGES, page_bytes);
    pages2.import_range(0, PAGES, arena.data());
    gqa.kv_page_write(pages2, table, 0, dk.ptr, dv.ptr);
    gqa.attend(pages2, table, 0, dq.ptr, dout.ptr);
    ctx.wait();
    cudaMemcpy(out2.data(), dout.ptr, out2.size() * 2, cudaMemcpyDeviceToHost);
    std::vector<uint16_t> arena2(arena.size());
    pages2.export_range(0, PAGES, arena2.data());
    EXPECT(arena2 == arena_after);
    float worst = 0.0f;
    for (size_t i = 0; i < out.size(); ++i) worst = std::fmax(worst, std::fabs(from_half(out[i]) - from_half(out2[i])));
    EXPECT(worst <= 1e-3f);

    if (FILE* f = std::fopen(out_path, "wb")) {
        std::fwrite(q.data(), 2, q.size(), f);
        std::fwrite(k.data(), 2, k.size(), f);
        std::fwrite(v.data(), 2, v.size(), f);
        std::fwrite(arena_after.data(), 2, arena_after.size(), f);
        std::fwrite(out.data(), 2, out.size(), f);
        std::fclose(f);
    } else {
        return 1;
    }
    std::printf(failures == 0 ? "step ok\n" : "step FAILED\n");
    return failures == 0 ? 0 : 1;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc >= 2 && std::strcmp(argv[1], "host") == 0) return run_host();
        if (argc >= 3 && std::strcmp(argv[1], "step") == 0) return run_step(argv[2]);
    } catch (const psi::Error& e) {
        std::fprintf(stderr, "psi::Error %d: %s\n", e.status(), e.what());
        return 1;
    }
    std::fprintf(stderr, "usage: host_mirror_check host | host_mirror_check step <out.bin>\n");
    return 2;
}
