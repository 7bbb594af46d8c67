// Multi-query attention over the paged cache for long query runs (chunked prefill, wide speculative verify).
//
// Where a request brings many query tokens, the decode kernel would stream the request's whole KV history once per
// 16-row query tile.  Here one CTA takes up to eight consecutive query tiles of one request and KV head - one tile
// (16 rows = tokens x group heads) per warp, 128 rows per CTA - and streams the KV range ONCE through a CTA-wide ring
// of shared-memory stages (16-byte cp.async, all threads copying, one barrier per 16-token tile); every warp scores
// the same K tile against its own rows with its own causal limit (keys beyond a token's position do not count, a
// warp skips tiles that lie entirely beyond its last token) and accumulates its own O.  No merge between warps: each
// warp normalises and writes its rows, or one partial slot when the KV range of its (tile, KV head) unit is shared
// with other CTAs; the warp that delivers a unit's last partial merges them (arrival counter, no waiting).
//
// This is the arithmetic of crates/inference-backend-metal/src/components/metal/gqa_split_kv_tiled_q.metal:49-319
// (Q tokens x Q-head tile per threadblock, K/V tiles staged in threadgroup memory, in-kernel causal mask) with the
// reduce of :324-378 folded in.
#include "launch_util.hpp"
#include "mma_common.cuh"

namespace psi {

namespace {

template <int D, int NSTAGE>
struct ChunkSmem {
    static constexpr uint32_t kRowBytes = D * 2;
    static constexpr uint32_t kTileBytes = kTile * kRowBytes;      // one K or V tile, or one warp's Q tile
    static constexpr uint32_t kStageBytes = 2 * kTileBytes;        // K then V
    static constexpr uint32_t kQBytes = kWarps * kTileBytes;
    static constexpr uint32_t kRingOffset = kQBytes;
    static constexpr uint32_t kTotal = kRingOffset + NSTAGE * kStageBytes;
};

template <typename T, int D, int NSTAGE>
__global__ void __launch_bounds__(kThreads, 1) attend_chunk_kernel(AttendParams p) {
    using L = ChunkSmem<D, NSTAGE>;
    constexpr uint32_t kChunks = D / 8;                               // 16-byte chunks per row
    constexpr uint32_t kCopiesPerTile = kTile * kChunks / kThreads;   // per thread, per K or V tile
    static_assert(kTile * kChunks % kThreads == 0, "a tile is copied by whole passes of the CTA");
    constexpr uint32_t kRowsPerPass = kThreads / kChunks;

    const uint32_t cta = blockIdx.x;
    if (cta >= p.scalars[kScalarNumChunkCtas]) return;

    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const uint32_t q_tile = smem_base + warp * L::kTileBytes;
    const uint32_t ring_base = smem_base + L::kRingOffset;
    const FragmentLanes frag(lane, L::kRowBytes);

    const uint32_t page_mask = p.geo.tokens_per_page - 1;  // tokens_per_page is a power of two
    const uint32_t page_shift = 31 - __clz(p.geo.tokens_per_page);
    const unsigned char* pages = static_cast<const unsigned char*>(p.geo.pages);
    const uint64_t page_bytes = p.geo.page_elems * 2;
    const uint64_t v_region_bytes = v_region_offset(p.geo) * 2;
    const bool fused = p.new_k != nullptr;

    // copy roles: this thread moves chunk copy_chunk of rows copy_row + pass * kRowsPerPass
    const uint32_t copy_row = tid / kChunks, copy_chunk = tid % kChunks;

    const uint32_t item_begin = p.cta_item_begin[cta], item_end = p.cta_item_begin[cta + 1];
    for (uint32_t index = item_begin; index < item_end; ++index) {
        const ItemView v = view_item(p, index);
        __syncthreads();  // the previous item is done with the ring

        const uint32_t tokens_per_warp = p.tokens_per_tile;  // query tokens the plan packs into one 16-row tile
        const uint32_t token_off = min(v.num_tokens, warp * tokens_per_warp);
        const uint32_t my_tokens = min(tokens_per_warp, v.num_tokens - token_off);
        const uint32_t my_rows = my_tokens * v.num_heads;
        const uint32_t my_first_pos = v.first_pos + token_off;
        // keys my rows may see: row r -> [0, my_first_pos + r / heads]; nothing at or beyond my_end counts for me
        const uint32_t my_end = min(v.kv_end, my_first_pos + my_tokens);
        const uint32_t my_min_limit = min(v.kv_end, my_first_pos + 1);
        const uint32_t limit0 = frag.quad_row < my_rows ? min(v.kv_end, my_first_pos + frag.quad_row / v.num_heads + 1) : v.kv_end;
        const uint32_t limit1 =
            frag.quad_row + 8 < my_rows ? min(v.kv_end, my_first_pos + (frag.quad_row + 8) / v.num_heads + 1) : v.kv_end;
        const uint32_t paged_end = fused ? min(v.kv_end, v.new_begin) : v.kv_end;

        const uint32_t first_tile = v.kv_begin / kTile;
        const uint32_t num_tiles = (v.kv_end + kTile - 1) / kTile - first_tile;
        const uint32_t* row_ids = table_row(p.geo, v.req_slot);
        const uint64_t head_bytes = static_cast<uint64_t>(v.kv_head) * p.geo.tokens_per_page * L::kRowBytes;

        // Page id of this thread's row in pass `pass` of local tile i.
        auto lookup = [&](uint32_t i, uint32_t (&ids)[kCopiesPerTile]) {
#pragma unroll
            for (uint32_t pass = 0; pass < kCopiesPerTile; ++pass) {
                const uint32_t token = (first_tile + i) * kTile + pass * kRowsPerPass + copy_row;
                ids[pass] = token < paged_end ? page_id_or_zero(p.geo, row_ids, token >> page_shift) : 0u;
            }
        };
        auto issue = [&](uint32_t i, const uint32_t (&ids)[kCopiesPerTile]) {
            const uint32_t stage = ring_base + (i % NSTAGE) * L::kStageBytes;
#pragma unroll
            for (uint32_t pass = 0; pass < kCopiesPerTile; ++pass) {
                const uint32_t row = pass * kRowsPerPass + copy_row;
                const uint32_t token = (first_tile + i) * kTile + row;
                const unsigned char* k_src = pages;
                const unsigned char* v_src = pages;
                uint32_t bytes = 16u;
                if (token >= v.kv_end) {
                    bytes = 0u;  // beyond the item: zero-fill
                } else if (token >= paged_end) {
                    const uint64_t fresh = (static_cast<uint64_t>(v.flat_req_begin + (token - v.new_begin)) * p.geo.num_kv_heads +
                                            v.kv_head) * L::kRowBytes + copy_chunk * 16;
                    k_src = static_cast<const unsigned char*>(p.new_k) + fresh;
                    v_src = static_cast<const unsigned char*>(p.new_v) + fresh;
                } else {
                    k_src = pages + static_cast<uint64_t>(ids[pass]) * page_bytes + head_bytes +
                            (token & page_mask) * L::kRowBytes + copy_chunk * 16;
                    v_src = k_src + v_region_bytes;
                }
                const uint32_t dst = stage + swizzled(row, copy_chunk, L::kRowBytes);
                cp_async_16(dst, k_src, bytes);
                cp_async_16(dst + L::kTileBytes, v_src, bytes);
            }
        };

        uint32_t ids[kCopiesPerTile];
#pragma unroll
        for (uint32_t i = 0; i < NSTAGE - 1; ++i) {
            if (i < num_tiles) {
                lookup(i, ids);
                issue(i, ids);
            }
            cp_async_commit();
        }
        if (NSTAGE - 1 < num_tiles) lookup(NSTAGE - 1, ids);

        // ---- with the first tiles in flight: this warp's query rows (zero beyond its own), and in the fused step the
        // item's share of the step's K/V rows into their pages ------------------------------------------------------------
        for (uint32_t i = lane; i < kTile * kChunks; i += 32) {
            const uint32_t r = i / kChunks, c = i % kChunks;
            uint4 value = make_uint4(0, 0, 0, 0);
            if (r < my_rows) {
                const uint64_t row = static_cast<uint64_t>(v.flat_begin + token_off + r / v.num_heads) * p.num_q_heads +
                                     v.head0 + r % v.num_heads;
                value = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.q) + row * D + c * 8);
            }
            *reinterpret_cast<uint4*>(smem + warp * L::kTileBytes + swizzled(r, c, L::kRowBytes)) = value;
        }
        if (fused && v.writes_kv) {
            for (uint32_t i = tid; i < v.num_tokens * 2 * kChunks; i += kThreads) {
                const uint32_t c = i % kChunks, which = (i / kChunks) & 1, j = i / (2 * kChunks);
                const uint32_t pos = v.first_pos + j;
                uint32_t write_id = 0;
                if (pos >= v.kv_begin && pos < v.kv_end && checked_page_id(p.geo, row_ids, pos >> page_shift, write_id)) {
                    const unsigned char* fresh = static_cast<const unsigned char*>(which ? p.new_v : p.new_k);
                    const uint4 value = *reinterpret_cast<const uint4*>(
                        fresh + (static_cast<uint64_t>(v.flat_begin + j) * p.geo.num_kv_heads + v.kv_head) * L::kRowBytes + c * 16);
                    unsigned char* dst = const_cast<unsigned char*>(pages) +
                                         static_cast<uint64_t>(write_id) * page_bytes + head_bytes +
                                         (which ? v_region_bytes : 0) + (pos & page_mask) * L::kRowBytes + c * 16;
                    *reinterpret_cast<uint4*>(dst) = value;
                }
            }
        }
        __syncwarp();

        RowState<D> st;
        st.clear();
        uint32_t pa[4];
        for (uint32_t i = 0; i < num_tiles; ++i) {
            cp_async_wait<NSTAGE - 2>();
            __syncthreads();  // tile i has landed for every thread; everyone is done with the stage tile i-1 used
            const uint32_t ahead = i + NSTAGE - 1;
            if (ahead < num_tiles) issue(ahead, ids);
            cp_async_commit();
            if (ahead + 1 < num_tiles) lookup(ahead + 1, ids);

            const uint32_t token0 = (first_tile + i) * kTile;
            if (token0 < my_end) {  // else: the tile lies beyond this warp's last token (or the warp has no rows)
                const uint32_t stage = ring_base + (i % NSTAGE) * L::kStageBytes;
                const bool masked = token0 < v.kv_begin || token0 + kTile > my_min_limit;
                TileMath<T, D>::scores(frag, q_tile, stage, p.scale_log2, masked, token0, limit0, limit1, v.kv_begin, st, pa);
                TileMath<T, D>::values(frag, stage + L::kTileBytes, pa, st);
            }
        }
        cp_async_wait<0>();

        // ---- each warp finishes its own rows -------------------------------------------------------------------------------
        if (my_rows == 0) continue;  // warp-uniform; the loop-top barrier keeps the CTA together
        st.l0 += __shfl_xor_sync(0xFFFFFFFFu, st.l0, 1);
        st.l0 += __shfl_xor_sync(0xFFFFFFFFu, st.l0, 2);
        st.l1 += __shfl_xor_sync(0xFFFFFFFFu, st.l1, 1);
        st.l1 += __shfl_xor_sync(0xFFFFFFFFu, st.l1, 2);
        const float inv0 = st.l0 > 0.0f ? 1.0f / st.l0 : 0.0f, inv1 = st.l1 > 0.0f ? 1.0f / st.l1 : 0.0f;
        const uint32_t r0 = frag.quad_row, r1 = frag.quad_row + 8;
        const bool is_partial = v.partial_slot != kU32Max;
        auto out_row = [&](uint32_t r) {
            return static_cast<uint64_t>(v.flat_begin + token_off + r / v.num_heads) * p.num_q_heads + v.head0 + r % v.num_heads;
        };
        if (is_partial) {
            const uint64_t base = static_cast<uint64_t>(v.partial_slot + warp) * kMaxRows;
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                const uint32_t col = 8 * j + 2 * frag.quad_col;
                if (r0 < my_rows) *reinterpret_cast<float2*>(p.partial_o + (base + r0) * D + col) = make_float2(st.o[j][0] * inv0, st.o[j][1] * inv0);
                if (r1 < my_rows) *reinterpret_cast<float2*>(p.partial_o + (base + r1) * D + col) = make_float2(st.o[j][2] * inv1, st.o[j][3] * inv1);
            }
            if (frag.quad_col == 0) {
                if (r0 < my_rows) {
                    p.partial_m[base + r0] = st.m0;
                    p.partial_l[base + r0] = st.l0;
                }
                if (r1 < my_rows) {
                    p.partial_m[base + r1] = st.m1;
                    p.partial_l[base + r1] = st.l1;
                }
            }
            // the warp that delivers the last partial of its (tile, KV head) unit merges the unit
            __threadfence();
            __syncwarp();
            uint32_t arrival = 0;
            if (lane == 0) arrival = atomicAdd(p.unit_counters + v.reduce_unit + warp, 1u);
            arrival = __shfl_sync(0xFFFFFFFFu, arrival, 0);
            if (arrival == v.unit_num_items - 1) {
                __threadfence();
                for (uint32_t i = lane; i < my_rows * (D / 4); i += 32) {
                    const uint32_t r = i / (D / 4), c4 = i % (D / 4);
                    float global_max = -INFINITY;
#pragma unroll 4
                    for (uint32_t s_i = 0; s_i < v.unit_num_items; ++s_i) {
                        const uint64_t prow = static_cast<uint64_t>(v.unit_first_slot + s_i * kWarps + warp) * kMaxRows + r;
                        global_max = fmaxf(global_max, __ldcg(p.partial_m + prow));
                    }
                    float sum = 0.0f;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                    for (uint32_t s_i = 0; s_i < v.unit_num_items; ++s_i) {
                        const uint64_t prow = static_cast<uint64_t>(v.unit_first_slot + s_i * kWarps + warp) * kMaxRows + r;
                        const float pm = __ldcg(p.partial_m + prow);
                        const float weight = pm == -INFINITY ? 0.0f : exp2f(pm - global_max) * __ldcg(p.partial_l + prow);
                        const float4 part = __ldcg(reinterpret_cast<const float4*>(p.partial_o + prow * D + 4 * c4));
                        sum += weight;
                        acc.x += weight * part.x;
                        acc.y += weight * part.y;
                        acc.z += weight * part.z;
                        acc.w += weight * part.w;
                    }
                    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
                    acc.x *= inv;
                    acc.y *= inv;
                    acc.z *= inv;
                    acc.w *= inv;
                    const uint64_t row = out_row(r);
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
                if (lane == 0) p.unit_counters[v.reduce_unit + warp] = 0;  // ready for the next launch
            }
        } else if (p.ext_o != nullptr) {
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                const uint32_t col = 8 * j + 2 * frag.quad_col;
                if (r0 < my_rows) *reinterpret_cast<float2*>(p.ext_o + out_row(r0) * D + col) = make_float2(st.o[j][0] * inv0, st.o[j][1] * inv0);
                if (r1 < my_rows) *reinterpret_cast<float2*>(p.ext_o + out_row(r1) * D + col) = make_float2(st.o[j][2] * inv1, st.o[j][3] * inv1);
            }
            if (frag.quad_col == 0) {
                if (r0 < my_rows) {
                    p.ext_m[out_row(r0)] = st.m0 * kLn2;
                    p.ext_l[out_row(r0)] = st.l0;
                }
                if (r1 < my_rows) {
                    p.ext_m[out_row(r1)] = st.m1 * kLn2;
                    p.ext_l[out_row(r1)] = st.l1;
                }
            }
        } else {
            const uint64_t row0 = r0 < my_rows ? out_row(r0) : 0, row1 = r1 < my_rows ? out_row(r1) : 0;
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                const uint32_t col = 8 * j + 2 * frag.quad_col;
                if (r0 < my_rows) store_out2<T>(p, row0 * D + col, st.o[j][0] * inv0, st.o[j][1] * inv0);
                if (r1 < my_rows) store_out2<T>(p, row1 * D + col, st.o[j][2] * inv1, st.o[j][3] * inv1);
            }
        }
    }
}

template <int D>
constexpr int chunk_stages() {
    return D == 256 ? 4 : 6;
}

template <typename T, int D>
cudaError_t launch_one(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    constexpr int NSTAGE = chunk_stages<D>();
    using L = ChunkSmem<D, NSTAGE>;
    auto kernel = attend_chunk_kernel<T, D, NSTAGE>;
    static std::atomic<uint64_t> configured{0};  // per instantiation, one bit per device
    cudaError_t err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), static_cast<int>(L::kTotal), configured);
    if (err != cudaSuccess) return err;
    kernel<<<num_ctas, kThreads, L::kTotal, stream>>>(p);
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

bool attend_chunk_supported(uint32_t dtype, uint32_t head_dim, uint32_t tokens_per_page) {
    return attend_mma_supported(dtype, head_dim, tokens_per_page) && (head_dim == 128 || head_dim == 256);
}

cudaError_t launch_attend_chunk(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    if (num_ctas == 0) return cudaSuccess;
    return p.dtype == PSI_DTYPE_BF16 ? launch_for_dim<__nv_bfloat16>(p, num_ctas, stream)
                                     : launch_for_dim<__half>(p, num_ctas, stream);
}

}  // namespace psi
