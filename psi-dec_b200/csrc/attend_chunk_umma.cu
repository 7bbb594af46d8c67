// Multi-query attention for long query runs on the 5th-generation tensor cores (tcgen05 / TMEM).
//
// Same work items as attend_chunk.cu (a super-tile of up to eight 16-row query tiles of one request and KV head: 128
// rows = one native UMMA M tile), different engine: the 128 query rows sit in shared memory once, K and V tiles of 64
// tokens are staged with 16-byte cp.async into 128-byte-swizzled operand layouts, one elected thread issues
//   S[128x64]  = Q[128xD] . K^T      (tcgen05.mma, both operands K-major from shared memory, accumulator in TMEM)
//   O[128xD]  += P[128x64] . V       (P from shared memory, V as an MN-major operand, accumulator in TMEM)
// and the 128 threads own one accumulator row each: they read their S row from TMEM (tcgen05.ld), apply the causal
// limit and the online softmax without any cross-thread traffic, write P back as an MMA operand, and rescale their O
// row in TMEM only when a running max moved.  Completion of the MMAs is tracked with mbarriers (tcgen05.commit); every
// wait is bounded and reports PSI_ERR_TIMEOUT through the status word instead of hanging.  The epilogue (direct
// output, per-tile partial slots, last-arriver merge) matches attend_chunk.cu.
//
// Arithmetic replaced: crates/inference-backend-metal/src/components/metal/gqa_split_kv_tiled_q.metal:49-378.
#include <type_traits>

#include "mma_common.cuh"

namespace psi {

namespace {

constexpr uint32_t kUmmaThreads = 128;
constexpr uint32_t kUmmaM = 128;   // query rows per CTA = TMEM lanes
constexpr uint32_t kUmmaN = 64;    // KV tokens per tile
constexpr uint32_t kMaxPolls = 200000;

__device__ __forceinline__ uint32_t smem_u32(const void* ptr) { return static_cast<uint32_t>(__cvta_generic_to_shared(ptr)); }

// Shared-memory matrix descriptor of a 128-byte-swizzled operand: start address, leading / stride byte offsets in
// 16-byte units, descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>((leading_bytes >> 4) & 0x3FFFu) << 16) |
           (static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor of kind::f16: f32 accumulator, A/B element format (0 = f16, 1 = bf16), B major (0 = K,
// 1 = MN), N >> 3 and M >> 4.
template <typename T>
__device__ __forceinline__ uint32_t umma_idesc(uint32_t n, bool b_mn_major) {
    const uint32_t format = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
    return (1u << 4) | (format << 7) | (format << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((n >> 3) << 17) |
           ((kUmmaM >> 4) << 24);
}

__device__ __forceinline__ void umma_issue(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Bounded wait on one phase of an mbarrier; false when the bound ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kMaxPolls; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// 32 consecutive f32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_load32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_store32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}

__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// Byte offset of the 16-byte chunk `chunk` (8 elements) of row `row` in a stack of [blocks][rows][64 elements] tiles
// with the 128-byte swizzle the descriptors above announce (chunk index XOR row % 8 inside each 128-byte row).
__device__ __forceinline__ uint32_t operand_offset(uint32_t rows, uint32_t row, uint32_t chunk) {
    return (chunk >> 3) * rows * 128 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

template <typename T, int D>
__global__ void __launch_bounds__(kUmmaThreads, 1) attend_chunk_umma_kernel(AttendParams p) {
    constexpr uint32_t kChunks = D / 8;                       // 16-byte chunks per row of Q / K / V
    constexpr uint32_t kQBytes = D * 2 * kUmmaM;              // [D/64][128][64]
    constexpr uint32_t kTileBytes = D * 2 * kUmmaN;           // one K or V tile: [D/64][64][64]
    constexpr uint32_t kStageBytes = 2 * kTileBytes;          // K then V
    constexpr uint32_t kPOffset = kQBytes + 2 * kStageBytes;  // P: [1][128][64]
    constexpr uint32_t kTmemColumns = 512;
    constexpr uint32_t kColS = 0, kColO = kUmmaN;

    const uint32_t cta = blockIdx.x;
    if (cta >= p.scalars[kScalarNumChunkCtas]) return;

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_s, bar_o;
    __shared__ uint32_t tmem_base_s, abort_s, last_s[kWarps];

    const uint32_t tid = threadIdx.x, warp = tid >> 5;
    // the swizzled operand layouts repeat every 1024 bytes: place them on that boundary whatever the toolchain did
    const uint32_t smem_pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
    unsigned char* smem = smem_raw + smem_pad;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_s_addr = smem_u32(&bar_s), bar_o_addr = smem_u32(&bar_o);

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                     "r"(kTmemColumns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_s_addr), "r"(1u) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_o_addr), "r"(1u) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        abort_s = 0;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    const uint32_t lane_base = (warp * 32u) << 16;            // this warp's TMEM lanes
    const uint32_t tmem_s = tmem + kColS, tmem_o = tmem + kColO;
    uint32_t phase_s = 0, phase_o = 0;

    const uint32_t idesc_qk = umma_idesc<T>(kUmmaN, false);
    const uint32_t idesc_pv = umma_idesc<T>(D, true);

    const uint32_t page_mask = p.geo.tokens_per_page - 1;
    const uint32_t page_shift = 31 - __clz(p.geo.tokens_per_page);
    const unsigned char* pages = static_cast<const unsigned char*>(p.geo.pages);
    const uint64_t page_bytes = p.geo.page_elems * 2;
    const uint64_t v_region_bytes = v_region_offset(p.geo) * 2;
    const bool fused = p.new_k != nullptr;

    // A wait that ran out flags the launch and lets every later wait fall through: results are then garbage, the
    // status word says so, and the kernel still frees its TMEM and returns.
    auto wait = [&](uint32_t bar, uint32_t parity) {
        if (*reinterpret_cast<volatile uint32_t*>(&abort_s)) return;
        if (!mbar_wait(bar, parity)) {
            abort_s = 1;
            if (p.status != nullptr) atomicExch(p.status, static_cast<uint32_t>(PSI_ERR_TIMEOUT));
        }
    };

    const uint32_t item_begin = p.cta_item_begin[cta], item_end = p.cta_item_begin[cta + 1];
    for (uint32_t index = item_begin; index < item_end; ++index) {
        const ItemView v = view_item(p, index);
        __syncthreads();  // the previous item is done with shared memory

        // row of this thread: 16-row tile w, row rr inside it -> (token, head) of the super-tile
        const uint32_t w = tid >> 4, rr = tid & 15;
        const uint32_t token_off = w * p.tokens_per_tile + rr / v.num_heads;
        const bool row_valid = rr < p.tokens_per_tile * v.num_heads && token_off < v.num_tokens;
        const uint32_t limit = row_valid ? min(v.kv_end, v.first_pos + token_off + 1) : v.kv_end;
        const uint32_t min_limit = min(v.kv_end, v.first_pos + 1);
        const uint64_t out_row =
            static_cast<uint64_t>(v.flat_begin + (row_valid ? token_off : 0)) * p.num_q_heads + v.head0 + rr % v.num_heads;
        const uint32_t paged_end = fused ? min(v.kv_end, v.new_begin) : v.kv_end;
        const uint32_t* row_ids = table_row(p.geo, v.req_slot);
        const uint64_t head_bytes = static_cast<uint64_t>(v.kv_head) * p.geo.tokens_per_page * (D * 2);
        const uint32_t first_tile = v.kv_begin / kUmmaN;
        const uint32_t num_tiles = (v.kv_end + kUmmaN - 1) / kUmmaN - first_tile;

        // K and V tile i -> stage i % 2, 16 bytes per cp.async, rows = tokens, swizzled operand layout
        auto issue = [&](uint32_t i) {
            const uint32_t stage = smem_base + kQBytes + (i & 1) * kStageBytes;
            const uint32_t token0 = (first_tile + i) * kUmmaN;
            for (uint32_t c = tid; c < kUmmaN * kChunks; c += kUmmaThreads) {
                const uint32_t row = c / kChunks, chunk = c % kChunks;
                const uint32_t token = token0 + row;
                const unsigned char* k_src = pages;
                const unsigned char* v_src = pages;
                uint32_t bytes = 16u;
                if (token >= v.kv_end) {
                    bytes = 0u;  // beyond the item: zero-fill
                } else if (token >= paged_end) {
                    const uint64_t fresh = (static_cast<uint64_t>(v.flat_req_begin + (token - v.new_begin)) * p.geo.num_kv_heads +
                                            v.kv_head) * (D * 2) + chunk * 16;
                    k_src = static_cast<const unsigned char*>(p.new_k) + fresh;
                    v_src = static_cast<const unsigned char*>(p.new_v) + fresh;
                } else {
                    k_src = pages + static_cast<uint64_t>(row_ids[token >> page_shift]) * page_bytes + head_bytes +
                            (token & page_mask) * (D * 2) + chunk * 16;
                    v_src = k_src + v_region_bytes;
                }
                const uint32_t dst = stage + operand_offset(kUmmaN, row, chunk);
                cp_async_16(dst, k_src, bytes);
                cp_async_16(dst + kTileBytes, v_src, bytes);
            }
        };

        if (num_tiles > 0) issue(0);
        cp_async_commit();

        // query rows (zero for rows the super-tile does not have), and in the fused step this item's K/V page writes
        for (uint32_t c = tid; c < kUmmaM * kChunks; c += kUmmaThreads) {
            const uint32_t row = c / kChunks, chunk = c % kChunks;
            const uint32_t rw = row >> 4, rrr = row & 15;
            const uint32_t tok = rw * p.tokens_per_tile + rrr / v.num_heads;
            uint4 value = make_uint4(0, 0, 0, 0);
            if (rrr < p.tokens_per_tile * v.num_heads && tok < v.num_tokens) {
                const uint64_t grow = static_cast<uint64_t>(v.flat_begin + tok) * p.num_q_heads + v.head0 + rrr % v.num_heads;
                value = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.q) + grow * D + chunk * 8);
            }
            *reinterpret_cast<uint4*>(smem + operand_offset(kUmmaM, row, chunk)) = value;
        }
        if (fused && v.writes_kv) {
            for (uint32_t i = tid; i < v.num_tokens * 2 * kChunks; i += kUmmaThreads) {
                const uint32_t c = i % kChunks, which = (i / kChunks) & 1, j = i / (2 * kChunks);
                const uint32_t pos = v.first_pos + j;
                if (pos >= v.kv_begin && pos < v.kv_end) {
                    const unsigned char* fresh = static_cast<const unsigned char*>(which ? p.new_v : p.new_k);
                    const uint4 value = *reinterpret_cast<const uint4*>(
                        fresh + (static_cast<uint64_t>(v.flat_begin + j) * p.geo.num_kv_heads + v.kv_head) * (D * 2) + c * 16);
                    unsigned char* dst = const_cast<unsigned char*>(pages) +
                                         static_cast<uint64_t>(row_ids[pos >> page_shift]) * page_bytes + head_bytes +
                                         (which ? v_region_bytes : 0) + (pos & page_mask) * (D * 2) + c * 16;
                    *reinterpret_cast<uint4*>(dst) = value;
                }
            }
        }

        float row_max = -INFINITY, row_sum = 0.0f;
        for (uint32_t i = 0; i < num_tiles; ++i) {
            if (i + 1 < num_tiles) issue(i + 1);  // its stage was released when P V of tile i-1 completed
            cp_async_commit();
            cp_async_wait<1>();                   // tile i (and, for i == 0, the query rows) have landed
            fence_async_smem();
            tc_fence_before();
            __syncthreads();
            tc_fence_after();
            const uint32_t stage = smem_base + kQBytes + (i & 1) * kStageBytes;
            const uint32_t token0 = (first_tile + i) * kUmmaN;

            // ---- S = Q K^T --------------------------------------------------------------------------------------------
            if (tid == 0) {
#pragma unroll
                for (uint32_t ks = 0; ks < D / 16; ++ks) {
                    const uint64_t a = umma_desc(smem_base + (ks >> 2) * (kUmmaM * 128) + (ks & 3) * 32, 16, 1024);
                    const uint64_t b = umma_desc(stage + (ks >> 2) * (kUmmaN * 128) + (ks & 3) * 32, 16, 1024);
                    umma_issue(tmem_s, a, b, idesc_qk, ks > 0);
                }
                umma_commit(bar_s_addr);
            }
            __syncwarp();
            wait(bar_s_addr, phase_s);
            phase_s ^= 1;
            tc_fence_after();

            // ---- this thread's row: scale, visibility, online softmax ------------------------------------------------------
            float s[kUmmaN];
            {
                float part[32];
                tmem_load32(tmem_s + lane_base, part);
#pragma unroll
                for (int c = 0; c < 32; ++c) s[c] = part[c] * p.scale_log2;
                tmem_load32(tmem_s + lane_base + 32, part);
#pragma unroll
                for (int c = 0; c < 32; ++c) s[32 + c] = part[c] * p.scale_log2;
            }
            if (token0 < v.kv_begin || token0 + kUmmaN > min_limit) {
#pragma unroll
                for (int c = 0; c < int(kUmmaN); ++c) {
                    const uint32_t token = token0 + c;
                    if (token >= limit || token < v.kv_begin) s[c] = -INFINITY;
                }
            }
            float tile_max = s[0];
#pragma unroll
            for (int c = 1; c < int(kUmmaN); ++c) tile_max = fmaxf(tile_max, s[c]);
            const float new_max = fmaxf(row_max, tile_max);
            const bool moved = new_max > row_max;
            if (i > 0 && __any_sync(0xFFFFFFFFu, moved)) {
                // rescale this warp's O rows in TMEM (P V of the previous tile has completed: waited below)
                const float corr = new_max == -INFINITY ? 1.0f : exp2f(row_max - new_max);
                row_sum *= corr;
#pragma unroll 1
                for (uint32_t c = 0; c < uint32_t(D); c += 32) {
                    float o[32];
                    tmem_load32(tmem_o + lane_base + c, o);
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] *= corr;
                    tmem_store32(tmem_o + lane_base + c, o);
                }
                tmem_store_wait();
            }
            row_max = new_max;
            const float base = row_max == -INFINITY ? 0.0f : row_max;
            float tile_sum = 0.0f;
#pragma unroll
            for (int c8 = 0; c8 < int(kUmmaN) / 8; ++c8) {
                float e[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    e[k] = exp2f(s[c8 * 8 + k] - base);
                    tile_sum += e[k];
                }
                const uint4 packed = make_uint4(Mma<T>::pack(e[0], e[1]), Mma<T>::pack(e[2], e[3]), Mma<T>::pack(e[4], e[5]),
                                                Mma<T>::pack(e[6], e[7]));
                *reinterpret_cast<uint4*>(smem + kPOffset + operand_offset(kUmmaM, tid, c8)) = packed;
            }
            row_sum += tile_sum;
            fence_async_smem();
            tc_fence_before();
            __syncthreads();
            tc_fence_after();

            // ---- O += P V ------------------------------------------------------------------------------------------------
            if (tid == 0) {
#pragma unroll
                for (uint32_t ks = 0; ks < kUmmaN / 16; ++ks) {
                    const uint64_t a = umma_desc(smem_base + kPOffset + ks * 32, 16, 1024);
                    const uint64_t b = umma_desc(stage + kTileBytes + ks * 2048, kUmmaN * 128, 1024);
                    umma_issue(tmem_o, a, b, idesc_pv, (i > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit(bar_o_addr);
            }
            __syncwarp();
            wait(bar_o_addr, phase_o);  // O, P and this tile's stage are free again
            phase_o ^= 1;
            tc_fence_after();
        }
        cp_async_wait<0>();

        // ---- epilogue: every thread finishes its own row ---------------------------------------------------------------
        const float inv = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;
        const bool is_partial = v.partial_slot != kU32Max;
        const uint64_t prow = is_partial ? static_cast<uint64_t>(v.partial_slot + w) * kMaxRows + rr : 0;
#pragma unroll 1
        for (uint32_t c = 0; c < uint32_t(D); c += 32) {
            float o[32];
            if (num_tiles > 0) {
                tmem_load32(tmem_o + lane_base + c, o);
            } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) o[e] = 0.0f;
            }
            if (!row_valid) continue;  // after the warp-collective load
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
                const float4 value = make_float4(o[e] * inv, o[e + 1] * inv, o[e + 2] * inv, o[e + 3] * inv);
                if (is_partial) {
                    *reinterpret_cast<float4*>(p.partial_o + prow * D + c + e) = value;
                } else if (p.ext_o != nullptr) {
                    *reinterpret_cast<float4*>(p.ext_o + out_row * D + c + e) = value;
                } else {
                    store_out4<T>(p, out_row * D + c + e, value);
                }
            }
        }
        if (row_valid) {
            if (is_partial) {
                p.partial_m[prow] = row_max;
                p.partial_l[prow] = row_sum;
            } else if (p.ext_o != nullptr) {
                p.ext_m[out_row] = row_max * kLn2;
                p.ext_l[out_row] = row_sum;
            }
        }
        tc_fence_before();

        // ---- units shared with other CTAs: whoever delivers a tile's last partial merges it ---------------------------
        if (is_partial) {
            __threadfence();
            __syncthreads();
            if (tid < kWarps) {
                const bool has_rows = tid * p.tokens_per_tile < v.num_tokens;
                last_s[tid] = has_rows && atomicAdd(p.unit_counters + v.reduce_unit + tid, 1u) == v.unit_num_items - 1;
            }
            __syncthreads();
            for (uint32_t tile = 0; tile < uint32_t(kWarps); ++tile) {
                if (!last_s[tile]) continue;
                __threadfence();
                const uint32_t tile_tokens = min(p.tokens_per_tile, v.num_tokens - tile * p.tokens_per_tile);
                const uint32_t tile_rows = tile_tokens * v.num_heads;
                for (uint32_t i = tid; i < tile_rows * (D / 4); i += kUmmaThreads) {
                    const uint32_t r = i / (D / 4), c4 = i % (D / 4);
                    float global_max = -INFINITY;
#pragma unroll 4
                    for (uint32_t s_i = 0; s_i < v.unit_num_items; ++s_i) {
                        const uint64_t row = static_cast<uint64_t>(v.unit_first_slot + s_i * kWarps + tile) * kMaxRows + r;
                        global_max = fmaxf(global_max, __ldcg(p.partial_m + row));
                    }
                    float sum = 0.0f;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                    for (uint32_t s_i = 0; s_i < v.unit_num_items; ++s_i) {
                        const uint64_t row = static_cast<uint64_t>(v.unit_first_slot + s_i * kWarps + tile) * kMaxRows + r;
                        const float pm = __ldcg(p.partial_m + row);
                        const float weight = pm == -INFINITY ? 0.0f : exp2f(pm - global_max) * __ldcg(p.partial_l + row);
                        const float4 part = __ldcg(reinterpret_cast<const float4*>(p.partial_o + row * D + 4 * c4));
                        sum += weight;
                        acc.x += weight * part.x;
                        acc.y += weight * part.y;
                        acc.z += weight * part.z;
                        acc.w += weight * part.w;
                    }
                    const float scale = sum > 0.0f ? 1.0f / sum : 0.0f;
                    acc.x *= scale;
                    acc.y *= scale;
                    acc.z *= scale;
                    acc.w *= scale;
                    const uint64_t row = static_cast<uint64_t>(v.flat_begin + tile * p.tokens_per_tile + r / v.num_heads) * p.num_q_heads +
                                         v.head0 + r % v.num_heads;
                    if (p.ext_o != nullptr) {
                        *reinterpret_cast<float4*>(p.ext_o + row * D + 4 * c4) = acc;
                        if (c4 == 0) {
                            p.ext_m[row] = global_max * kLn2;
                            p.ext_l[row] = sum;
                        }
                    } else {
                        store_out4<T>(p, row * D + 4 * c4, acc);
                    }
                }
                if (tid == 0) p.unit_counters[v.reduce_unit + tile] = 0;  // ready for the next launch
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns) : "memory");
    }
}

template <typename T, int D>
cudaError_t launch_one(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    constexpr uint32_t kSmem = D * 2 * kUmmaM + 2 * (2 * D * 2 * kUmmaN) + kUmmaM * 128 + 1024;
    auto kernel = attend_chunk_umma_kernel<T, D>;
    static int configured_device = -1;
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return err;
    if (configured_device != device) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmem));
        if (err != cudaSuccess) return err;
        configured_device = device;
    }
    kernel<<<num_ctas, kUmmaThreads, kSmem, stream>>>(p);
    return cudaGetLastError();
}

template <typename T>
cudaError_t launch_for_dim(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    switch (p.geo.head_dim) {
        case 128: return launch_one<T, 128>(p, num_ctas, stream);
        case 256: return launch_one<T, 256>(p, num_ctas, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

cudaError_t launch_attend_chunk_umma(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    if (num_ctas == 0) return cudaSuccess;
    return p.dtype == PSI_DTYPE_BF16 ? launch_for_dim<__nv_bfloat16>(p, num_ctas, stream)
                                     : launch_for_dim<__half>(p, num_ctas, stream);
}

}  // namespace psi
