// Split-KV flash-decode map kernel on CUDA cores with staged K/V: what the tensor-core decode kernel does not take
// (f32, page sizes that are no power of two, head dims that are no multiple of 64) at a useful fraction of the HBM
// rate.  Same work items, partial slots and reduce pass as attend_generic_kernel; head_dim must be a multiple of four.
//
// One CTA of eight warps walks its items.  An item's KV range is cut into tiles of 32 tokens.  While a tile is being
// worked on, every thread already holds its share of the next tile's K and V rows in registers (16- or 8-byte global
// loads, issued before the arithmetic of the current tile and consumed after it), so the loads of tile i + 1 overlap
// the arithmetic of tile i without a second shared-memory stage.  Per tile:
//   scores   lane = token, warp w = query rows w and w + 8: S[r][t] = q[r] . K[t] over float4 pieces from shared memory
//            (K rows padded by four floats, so the 32 lanes' float4 reads fall into distinct banks; q is a broadcast);
//   softmax  online, in the log2 domain, per row inside the owning warp (quad-free: a row's 32 scores sit in one warp);
//   values   thread = (row, float4 column): O[r][c] += sum_t P[r][t] V[t][c], V read along the row (conflict-free).
// f32 accumulation throughout; the arithmetic this replaces is the reference's SingleQ map shader
// (crates/inference-backend-metal/src/components/metal/gqa_split_kv_single_q_map.metal:85-252) with the per-row causal
// limit of metal/gqa_split_kv_tiled_q.metal:233-244.
#include <atomic>

#include "device_common.cuh"
#include "launch_util.hpp"

namespace psi {

namespace {

constexpr int kStagedThreads = 256;
constexpr uint32_t kStagedWarps = kStagedThreads / 32;
constexpr uint32_t kStagedTile = 32;    // KV tokens per tile: one per lane in the score phase
constexpr uint32_t kStagedChunks = 16;  // 4-element pieces one thread moves per tile at head_dim 256
constexpr uint32_t kStagedOutputs = 4;  // (row, float4 column) outputs per thread at 16 rows x head_dim 256

// Four consecutive elements of the I/O dtype as they travel through registers.
template <typename T>
struct Piece {
    using Raw = uint2;
    static __device__ __forceinline__ float4 widen(uint2 raw);
};
template <>
struct Piece<float> {
    using Raw = float4;
    static __device__ __forceinline__ float4 widen(float4 raw) { return raw; }
};
template <>
__device__ __forceinline__ float4 Piece<__nv_bfloat16>::widen(uint2 raw) {
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
template <>
__device__ __forceinline__ float4 Piece<__half>::widen(uint2 raw) {
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, offset));
    return v;
}

// Shared memory in floats: q [16][D] | `stages` x (K tile [32][D + 4] | V tile [32][D]) | P [16][32] | per-row words.
__host__ __device__ constexpr uint32_t staged_tile_floats(uint32_t head_dim) {
    return kStagedTile * (head_dim + 4) + kStagedTile * head_dim;
}
__host__ __device__ constexpr uint32_t staged_smem_floats(uint32_t head_dim, uint32_t stages) {
    return kMaxRows * head_dim + stages * staged_tile_floats(head_dim) + kMaxRows * kStagedTile + 4 * kMaxRows +
           4 * kStagedTile;
}

__device__ __forceinline__ void staged_cp_async_16(float* dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))),
                 "l"(src), "r"(src_bytes)
                 : "memory");
}

// Two CTAs per SM for the 16-bit types (one's loads under the other's arithmetic: 452 against 578 us on the layer-decode
// batch); f32 holds twice the registers per piece and measured slower that way (spills), so it keeps one.
template <typename T>
__global__ void __launch_bounds__(kStagedThreads, sizeof(T) == 4 ? 1 : 2) attend_staged_kernel(AttendParams p) {
    using Raw = typename Piece<T>::Raw;
    // f32 needs no conversion on the way in: its tiles go straight from the pages into one of two shared-memory
    // stages by 16-byte cp.async (zero-filled beyond the item's range), the next tile's copies in flight under the
    // current tile's arithmetic, and nothing is held in registers.
    constexpr bool kAsync = sizeof(T) == 4;
    constexpr uint32_t kStages = kAsync ? 2 : 1;
    const uint32_t cta = blockIdx.x;
    if (cta >= p.scalars[kScalarNumCtas]) return;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t D = p.geo.head_dim, C4 = D / 4, k_stride = D + 4;

    extern __shared__ __align__(16) float staged_smem[];
    float* q_s = staged_smem;
    float* tiles_s = q_s + kMaxRows * D;  // stage s: K tile at s * staged_tile_floats(D), its V tile behind it
    float* p_s = tiles_s + kStages * staged_tile_floats(D);
    float* corr_s = p_s + kMaxRows * kStagedTile;
    float* m_s = corr_s + kMaxRows;
    float* l_s = m_s + kMaxRows;
    uint32_t* limit_s = reinterpret_cast<uint32_t*>(l_s + kMaxRows);
    // Element offset of the K row of every token of the tile that is being fetched, two buffers by tile parity: warp 0
    // writes tile i + 1's while slower warps may still read tile i's.
    unsigned long long* row_s = reinterpret_cast<unsigned long long*>(limit_s + kMaxRows);

    // This thread's pieces of a tile: piece j is number tid + 256 * j of the tile's 32 tokens x (K row | V row) x C4
    // pieces, walked without divisions.
    const uint32_t pieces_per_token = 2 * C4;
    const uint32_t step_token = kStagedThreads / pieces_per_token, step_piece = kStagedThreads % pieces_per_token;
    const uint32_t first_token = tid / pieces_per_token, first_piece = tid % pieces_per_token;
    const uint32_t tile_pieces = kStagedTile * pieces_per_token;
    const uint64_t v_off = v_region_offset(p.geo);
    const T* arena = static_cast<const T*>(p.geo.pages);

    for (uint32_t index = p.cta_item_begin[cta]; index < p.cta_item_begin[cta + 1]; ++index) {
        const ItemView v = view_item(p, index);
        const uint32_t rows = v.rows;
        const uint32_t* row_ids = table_row(p.geo, v.req_slot);
        __syncthreads();  // the previous item is done with q_s, limit_s and the tiles
        for (uint32_t i = tid; i < rows * D; i += kStagedThreads) {
            const uint32_t r = i / D, d = i % D;
            q_s[r * D + d] = load_as_float(p.q, item_row_index(p, v, r) * D + d, p.dtype);
        }
        if (tid < kMaxRows) limit_s[tid] = tid < rows ? item_row_limit(v, tid) : 0u;

        // this thread's outputs: (row, float4 column) number tid + 256 * j of rows x C4
        uint32_t out_row[kStagedOutputs], out_col[kStagedOutputs];
        float4 acc[kStagedOutputs];
#pragma unroll
        for (uint32_t j = 0; j < kStagedOutputs; ++j) {
            const uint32_t o = tid + kStagedThreads * j;
            out_row[j] = o < rows * C4 ? o / C4 : kU32Max;
            out_col[j] = o % C4;
            acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        // running statistics of rows warp and warp + 8 (the same in every lane of the warp)
        float run_m[2] = {-INFINITY, -INFINITY}, run_l[2] = {0.f, 0.f};

        const uint32_t num_tiles = (v.kv_end - v.kv_begin + kStagedTile - 1) / kStagedTile;
        Raw held[kStagedChunks];
        // Fetches tile `tile` into `held`; row_s holds that tile's row offsets.  The
        // fetch of tile 0 and the row offsets of tile 1 are not separated by a barrier, hence the two buffers.
        auto fetch = [&](uint32_t tile) {
            const unsigned long long* rows_of_tile = row_s + (tile & 1u) * kStagedTile;
            uint32_t token = first_token, piece = first_piece;
#pragma unroll
            for (uint32_t j = 0; j < kStagedChunks; ++j) {
                // Unconditional within the tile (tokens beyond the item's range read a valid row and are zeroed when
                // the piece goes to shared memory): a load that feeds a select would have to be waited for at once.
                if (tid + kStagedThreads * j < tile_pieces) {
                    const bool is_v = piece >= C4;
                    const uint64_t elem = rows_of_tile[token] + (is_v ? v_off : 0) + 4 * (piece - (is_v ? C4 : 0));
                    held[j] = *reinterpret_cast<const Raw*>(arena + elem);
                }
                token += step_token;
                piece += step_piece;
                if (piece >= pieces_per_token) {
                    piece -= pieces_per_token;
                    token += 1;
                }
            }
        };
        auto row_offsets_of = [&](uint32_t tile) {
            if (tid < kStagedTile) {
                const uint32_t pos = v.kv_begin + tile * kStagedTile + tid;
                const uint32_t at = min(pos, v.kv_end - 1);  // beyond the range: the last row again (valid memory)
                const uint32_t page_id = page_id_or_zero(p.geo, row_ids, at / p.geo.tokens_per_page);
                row_s[(tile & 1u) * kStagedTile + tid] = kv_row_offset(p.geo, page_id, v.kv_head, at % p.geo.tokens_per_page);
            }
        };
        // f32: the copies of tile `tile` into its stage (one commit group per tile and thread)
        auto copy_async = [&](uint32_t tile) {
            const unsigned long long* rows_of_tile = row_s + (tile & 1u) * kStagedTile;
            const uint32_t in_range = v.kv_end - (v.kv_begin + tile * kStagedTile);
            float* k_dst = tiles_s + (tile & 1u) * staged_tile_floats(D);
            float* v_dst = k_dst + kStagedTile * k_stride;
            uint32_t token = first_token, piece = first_piece;
#pragma unroll
            for (uint32_t j = 0; j < kStagedChunks; ++j) {
                if (tid + kStagedThreads * j < tile_pieces) {
                    const bool is_v = piece >= C4;
                    const uint64_t elem = rows_of_tile[token] + (is_v ? v_off : 0) + 4 * (piece - (is_v ? C4 : 0));
                    float* dst = is_v ? v_dst + token * D + 4 * (piece - C4) : k_dst + token * k_stride + 4 * piece;
                    staged_cp_async_16(dst, arena + elem, token < in_range ? 16u : 0u);
                }
                token += step_token;
                piece += step_piece;
                if (piece >= pieces_per_token) {
                    piece -= pieces_per_token;
                    token += 1;
                }
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        };
        if (num_tiles > 0) row_offsets_of(0);
        __syncthreads();  // q_s, limit_s and the first tile's page ids are in place
        if (num_tiles > 0) {
            if constexpr (kAsync) copy_async(0); else fetch(0);
        }

        for (uint32_t tile = 0; tile < num_tiles; ++tile) {
            float* k_s = tiles_s + (kAsync ? (tile & 1u) * staged_tile_floats(D) : 0u);
            float* v_s = k_s + kStagedTile * k_stride;
            // ---- 16-bit types: the held tile goes to shared memory as f32 -----------------------------------------------
            if constexpr (!kAsync) {
                const uint32_t in_range = v.kv_end - (v.kv_begin + tile * kStagedTile);  // tokens of this tile inside the item
                uint32_t token = first_token, piece = first_piece;
#pragma unroll
                for (uint32_t j = 0; j < kStagedChunks; ++j) {
                    if (tid + kStagedThreads * j < tile_pieces) {
                        const bool is_v = piece >= C4;
                        float* dst = is_v ? v_s + token * D + 4 * (piece - C4) : k_s + token * k_stride + 4 * piece;
                        const float4 value = Piece<T>::widen(held[j]);
                        *reinterpret_cast<float4*>(dst) = token < in_range ? value : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    token += step_token;
                    piece += step_piece;
                    if (piece >= pieces_per_token) {
                        piece -= pieces_per_token;
                        token += 1;
                    }
                }
            }
            if (tile + 1 < num_tiles) row_offsets_of(tile + 1);
            if constexpr (kAsync) asm volatile("cp.async.wait_group 0;\n" ::: "memory");  // this thread's copies of the tile
            __syncthreads();
            if (tile + 1 < num_tiles) {  // in flight during the arithmetic below
                if constexpr (kAsync) copy_async(tile + 1); else fetch(tile + 1);
            }

            // ---- scores and online softmax: lane = token, this warp's rows ----------------------------------------------
            const uint32_t pos = v.kv_begin + tile * kStagedTile + lane;
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h) {
                const uint32_t r = warp + h * kStagedWarps;
                if (r >= rows) continue;
                const float4* k_row = reinterpret_cast<const float4*>(k_s + lane * k_stride);
                const float4* q_row = reinterpret_cast<const float4*>(q_s + r * D);
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);  // four independent chains
#pragma unroll 4
                for (uint32_t c = 0; c < C4; ++c) {
                    const float4 a = q_row[c], b = k_row[c];
                    sum.x += a.x * b.x;
                    sum.y += a.y * b.y;
                    sum.z += a.z * b.z;
                    sum.w += a.w * b.w;
                }
                const float dot = (sum.x + sum.y) + (sum.z + sum.w);
                const bool visible = pos < limit_s[r];  // limit_s is clipped to the item's kv_end
                const float x = visible ? dot * p.scale_log2 : -INFINITY;
                const float m_new = fmaxf(run_m[h], warp_max(x));
                const float corr = m_new == -INFINITY ? 1.0f : exp2f(run_m[h] - m_new);  // run_m = -inf -> 0
                const float w = visible ? exp2f(x - m_new) : 0.0f;
                run_l[h] = run_l[h] * corr + warp_sum(w);
                run_m[h] = m_new;
                p_s[r * kStagedTile + lane] = w;
                if (lane == 0) corr_s[r] = corr;
            }
            __syncthreads();

            // ---- values: this thread's (row, float4 column) outputs ------------------------------------------------------
#pragma unroll
            for (uint32_t j = 0; j < kStagedOutputs; ++j) {
                if (out_row[j] == kU32Max) continue;
                const float corr = corr_s[out_row[j]];
                float4 a = acc[j];
                a.x *= corr;
                a.y *= corr;
                a.z *= corr;
                a.w *= corr;
                const float* weights = p_s + out_row[j] * kStagedTile;
                const float4* column = reinterpret_cast<const float4*>(v_s) + out_col[j];
#pragma unroll 8
                for (uint32_t t = 0; t < kStagedTile; ++t) {
                    const float w = weights[t];
                    const float4 value = column[t * C4];
                    a.x += w * value.x;
                    a.y += w * value.y;
                    a.z += w * value.z;
                    a.w += w * value.w;
                }
                acc[j] = a;
            }
            __syncthreads();  // the tile, the weights and the corrections may be overwritten
        }

        // ---- the item's result: final output, one partial slot, or an external partial ----------------------------------
#pragma unroll
        for (uint32_t h = 0; h < 2; ++h) {
            const uint32_t r = warp + h * kStagedWarps;
            if (r < rows && lane == 0) {
                m_s[r] = run_m[h];
                l_s[r] = run_l[h];
            }
        }
        __syncthreads();
#pragma unroll
        for (uint32_t j = 0; j < kStagedOutputs; ++j) {
            if (out_row[j] == kU32Max) continue;
            const uint32_t r = out_row[j], d = 4 * out_col[j];
            const float l = l_s[r];
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            const float4 value = make_float4(acc[j].x * inv, acc[j].y * inv, acc[j].z * inv, acc[j].w * inv);
            const uint64_t row = item_row_index(p, v, r);
            if (v.partial_slot != kU32Max) {
                const uint64_t prow = static_cast<uint64_t>(v.partial_slot) * kMaxRows + r;
                *reinterpret_cast<float4*>(p.partial_o + prow * D + d) = value;
                if (d == 0) {
                    p.partial_m[prow] = m_s[r];
                    p.partial_l[prow] = l;
                }
            } else if (p.ext_o != nullptr) {
                *reinterpret_cast<float4*>(p.ext_o + row * D + d) = value;
                if (d == 0) {
                    p.ext_m[row] = m_s[r] * kLn2;
                    p.ext_l[row] = l;
                }
            } else {
                const uint64_t at = row * D + d;
                store_from_float(p.out, at, p.dtype, value.x * gate_factor(p, at));
                store_from_float(p.out, at + 1, p.dtype, value.y * gate_factor(p, at + 1));
                store_from_float(p.out, at + 2, p.dtype, value.z * gate_factor(p, at + 2));
                store_from_float(p.out, at + 3, p.dtype, value.w * gate_factor(p, at + 3));
            }
        }
    }
}

template <typename T>
cudaError_t launch_staged(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    auto kernel = attend_staged_kernel<T>;
    constexpr uint32_t stages = sizeof(T) == 4 ? 2 : 1;
    const int bytes = static_cast<int>(staged_smem_floats(p.geo.head_dim, stages) * sizeof(float));
    static std::atomic<uint64_t> configured{0};
    // the largest head_dim sets the limit once; smaller ones fit under it
    cudaError_t err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel),
                                          static_cast<int>(staged_smem_floats(256, stages) * sizeof(float)), configured);
    if (err != cudaSuccess) return err;
    kernel<<<num_ctas, kStagedThreads, bytes, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

uint32_t attend_staged_ctas_per_sm(uint32_t dtype) { return dtype == PSI_DTYPE_F32 ? 1u : 2u; }

// head_dim a multiple of four up to 256, and arena, q and partial buffers on 16-byte boundaries.
bool attend_staged_supported(const AttendParams& p) {
    const uint32_t d = p.geo.head_dim;
    const uintptr_t elem = p.dtype == PSI_DTYPE_F32 ? 4 : 2;
    const bool aligned = (reinterpret_cast<uintptr_t>(p.geo.pages) & (4 * elem - 1)) == 0 &&
                         (reinterpret_cast<uintptr_t>(p.partial_o) & 15u) == 0 &&
                         (p.ext_o == nullptr || (reinterpret_cast<uintptr_t>(p.ext_o) & 15u) == 0);
    return d >= 4 && d <= 256 && d % 4 == 0 && aligned;
}

cudaError_t launch_attend_staged(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    if (num_ctas == 0) return cudaSuccess;
    switch (p.dtype) {
        case PSI_DTYPE_F32: return launch_staged<float>(p, num_ctas, stream);
        case PSI_DTYPE_BF16: return launch_staged<__nv_bfloat16>(p, num_ctas, stream);
        case PSI_DTYPE_F16: return launch_staged<__half>(p, num_ctas, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace psi
