// Generic split-KV flash-decode map kernel on CUDA cores, the partial reduce and the cross-device combine.
//
// launch_attend_generic hands a launch to the staged kernel of attend_staged.cu when it qualifies (head_dim a multiple
// of four, aligned buffers); the one-warp kernel below takes the rest.  It takes every profile the reference's SingleQ kernel takes (f32 / bf16, any tokens_per_page,
// head_dim up to 256) plus f16: one warp per CTA walks its work items; lanes split head_dim, every KV row is read
// once per item and scored against all rows (tokens x group heads) of the item with f32 accumulation and an online
// softmax in the log2 domain.  Semantics follow
// crates/inference-backend-metal/src/components/metal/gqa_split_kv_single_q_map.metal:85-252 (visibility through
// kv_end only) extended with the per-row causal limit of metal/gqa_split_kv_tiled_q.metal:233-244.
#include <cmath>

#include "device_common.cuh"
#include "exchange.cuh"

namespace psi {

namespace {

constexpr int kGenericThreads = 32;

template <int DPL>
__global__ void __launch_bounds__(kGenericThreads) attend_generic_kernel(AttendParams p) {
    const uint32_t cta = blockIdx.x;
    if (cta >= p.scalars[kScalarNumCtas]) return;
    const uint32_t lane = threadIdx.x;
    const uint32_t D = p.geo.head_dim;
    __shared__ float q_s[kMaxRows * 256];
    __shared__ uint32_t limit_s[kMaxRows];

    for (uint32_t index = p.cta_item_begin[cta]; index < p.cta_item_begin[cta + 1]; ++index) {
        const ItemView v = view_item(p, index);
        __syncwarp();
        for (uint32_t i = lane; i < v.rows * D; i += kGenericThreads) {
            const uint32_t r = i / D, d = i % D;
            q_s[r * D + d] = load_as_float(p.q, item_row_index(p, v, r) * D + d, p.dtype);
        }
        if (lane < v.rows) limit_s[lane] = item_row_limit(v, lane);
        __syncwarp();

        float m[kMaxRows], l[kMaxRows], o[kMaxRows][DPL];
#pragma unroll
        for (int r = 0; r < int(kMaxRows); ++r) {
            m[r] = -INFINITY;
            l[r] = 0.0f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) o[r][i] = 0.0f;
        }

        const uint32_t* row_ids = table_row(p.geo, v.req_slot);
        const uint64_t v_off = v_region_offset(p.geo);
        for (uint32_t t = v.kv_begin; t < v.kv_end; ++t) {
            const uint32_t page_id = page_id_or_zero(p.geo, row_ids, t / p.geo.tokens_per_page);
            const uint64_t base = kv_row_offset(p.geo, page_id, v.kv_head, t % p.geo.tokens_per_page);
            float kreg[DPL], vreg[DPL];
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const uint32_t d = lane + 32 * i;
                kreg[i] = d < D ? load_as_float(p.geo.pages, base + d, p.dtype) : 0.0f;
                vreg[i] = d < D ? load_as_float(p.geo.pages, base + v_off + d, p.dtype) : 0.0f;
            }
#pragma unroll
            for (int r = 0; r < int(kMaxRows); ++r) {
                if (r < int(v.rows)) {
                    float dot = 0.0f;
#pragma unroll
                    for (int i = 0; i < DPL; ++i) {
                        const uint32_t d = lane + 32 * i;
                        dot += d < D ? q_s[r * D + d] * kreg[i] : 0.0f;
                    }
                    dot = warp_sum(dot);
                    if (t < limit_s[r]) {
                        const float x = dot * p.scale_log2;
                        const float m_new = fmaxf(m[r], x);
                        const float corr = exp2f(m[r] - m_new);  // m = -inf -> 0
                        const float w = exp2f(x - m_new);
                        l[r] = l[r] * corr + w;
#pragma unroll
                        for (int i = 0; i < DPL; ++i) o[r][i] = o[r][i] * corr + w * vreg[i];
                        m[r] = m_new;
                    }
                }
            }
        }

#pragma unroll
        for (int r = 0; r < int(kMaxRows); ++r) {
            if (r < int(v.rows)) {
                const float inv = l[r] > 0.0f ? 1.0f / l[r] : 0.0f;
                const uint64_t row = item_row_index(p, v, r);
                if (v.partial_slot != kU32Max) {
                    const uint64_t prow = static_cast<uint64_t>(v.partial_slot) * kMaxRows + r;
#pragma unroll
                    for (int i = 0; i < DPL; ++i) {
                        const uint32_t d = lane + 32 * i;
                        if (d < D) p.partial_o[prow * D + d] = o[r][i] * inv;
                    }
                    if (lane == 0) {
                        p.partial_m[prow] = m[r];
                        p.partial_l[prow] = l[r];
                    }
                } else if (p.ext_o != nullptr) {
#pragma unroll
                    for (int i = 0; i < DPL; ++i) {
                        const uint32_t d = lane + 32 * i;
                        if (d < D) p.ext_o[row * D + d] = o[r][i] * inv;
                    }
                    if (lane == 0) {
                        p.ext_m[row] = m[r] * kLn2;
                        p.ext_l[row] = l[r];
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < DPL; ++i) {
                        const uint32_t d = lane + 32 * i;
                        if (d < D) store_from_float(p.out, row * D + d, p.dtype, o[r][i] * inv * gate_factor(p, row * D + d));
                    }
                }
            }
        }
    }
}

// One CTA per (unit, query row) of every (tile, head selection) unit that more than one item contributed to:
// M = max m_i, w_i = 2^(m_i - M) * l_i (0 when m_i is not finite), out = sum w_i o_i / sum w_i (0 when empty),
// crates/inference-backend-metal/src/components/metal/gqa_split_kv_single_q_reduce.metal:27-48.  The items' weights are
// worked out once per CTA (a block-wide max and sum over the items' statistics, 128 items at a time) and kept in shared
// memory; every thread then owns output columns and walks the items with independent, coalesced loads.
constexpr int kReduceThreads = 128;

__device__ __forceinline__ float reduce_warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, offset));
    return v;
}

__global__ void __launch_bounds__(kReduceThreads) attend_reduce_kernel(AttendParams p) {
    const uint32_t unit = blockIdx.x, r = blockIdx.y;
    if (unit >= p.scalars[kScalarNumReduces]) return;
    const ReduceUnit ru = p.reduces[unit];
    const ItemView v = view_item(p, ru.first_item);
    if (r >= v.rows) return;
    const uint32_t D = p.geo.head_dim, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t first_slot = v.partial_slot;  // slots of one unit are consecutive
    const uint32_t n = ru.num_items;
    __shared__ float weight_s[kReduceThreads];
    __shared__ float across_s[kReduceThreads / 32];

    // the row's maximum over all items
    float local_max = -INFINITY;
    for (uint32_t s = tid; s < n; s += kReduceThreads)
        local_max = fmaxf(local_max, p.partial_m[static_cast<uint64_t>(first_slot + s) * kMaxRows + r]);
    local_max = reduce_warp_max(local_max);
    if (lane == 0) across_s[warp] = local_max;
    __syncthreads();
    float global_max = across_s[0];
#pragma unroll
    for (int w = 1; w < kReduceThreads / 32; ++w) global_max = fmaxf(global_max, across_s[w]);
    __syncthreads();

    float acc[2] = {0.0f, 0.0f};  // columns tid and tid + 128 (head_dim <= 256)
    float weight_sum = 0.0f;      // this thread's share of the weights; summed over the CTA at the end
    for (uint32_t base = 0; base < n; base += kReduceThreads) {
        const uint32_t count = min(n - base, static_cast<uint32_t>(kReduceThreads));
        if (tid < count) {
            const uint64_t prow = static_cast<uint64_t>(first_slot + base + tid) * kMaxRows + r;
            const float pm = p.partial_m[prow];
            const float w = isfinite(pm) ? exp2f(pm - global_max) * p.partial_l[prow] : 0.0f;
            weight_s[tid] = w;
            weight_sum += w;
        }
        __syncthreads();
        const float* o_row = p.partial_o + (static_cast<uint64_t>(first_slot + base) * kMaxRows + r) * D;
#pragma unroll 4
        for (uint32_t s = 0; s < count; ++s) {
            const float w = weight_s[s];
            const float* o = o_row + static_cast<uint64_t>(s) * kMaxRows * D;
            if (tid < D) acc[0] += w * o[tid];
            if (tid + kReduceThreads < D) acc[1] += w * o[tid + kReduceThreads];
        }
        __syncthreads();
    }
    weight_sum = warp_sum(weight_sum);
    if (lane == 0) across_s[warp] = weight_sum;
    __syncthreads();
    float sum = 0.0f;
#pragma unroll
    for (int w = 0; w < kReduceThreads / 32; ++w) sum += across_s[w];

    const uint64_t row = item_row_index(p, v, r);
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) {
        const uint32_t d = tid + j * kReduceThreads;
        if (d >= D) continue;
        const float value = sum > 0.0f ? acc[j] / sum : 0.0f;
        if (p.ext_o != nullptr) {
            p.ext_o[row * D + d] = value;
            if (d == 0) {
                p.ext_m[row] = global_max * kLn2;
                p.ext_l[row] = sum;
            }
        } else {
            store_from_float(p.out, row * D + d, p.dtype, value * gate_factor(p, row * D + d));
        }
    }
}

// Dense bidirectional attention of every query token against the tokens of its own block (local, unpaged K/V), written
// as a partial in the reduce's ABI so that it can be merged with the paged history of the same tokens
// (crates/inference-backend-metal/src/components/metal/gqa_block_sdpa.metal:5-77).  One warp per (token, q head): lanes
// split head_dim for the dot products and for the output columns; the block's weights sit in shared memory.
constexpr uint32_t kBlockPartialWarps = 4;
constexpr uint32_t kBlockPartialMaxBlock = 256;

__global__ void __launch_bounds__(kBlockPartialWarps * 32) block_partial_kernel(BlockPartialParams p) {
    __shared__ float weights_s[kBlockPartialWarps][kBlockPartialMaxBlock];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint64_t pair = static_cast<uint64_t>(blockIdx.x) * kBlockPartialWarps + warp;
    if (pair >= static_cast<uint64_t>(p.num_tokens) * p.num_q_heads) return;
    const uint32_t token = static_cast<uint32_t>(pair / p.num_q_heads), head = static_cast<uint32_t>(pair % p.num_q_heads);
    const uint32_t kv_head = head / (p.num_q_heads / p.num_kv_heads);
    const uint32_t begin = token / p.block_size * p.block_size;
    const uint64_t q_row = (static_cast<uint64_t>(token) * p.num_q_heads + head) * p.head_dim;
    float* weights = weights_s[warp];

    float block_max = -INFINITY;
    for (uint32_t j = 0; j < p.block_size; ++j) {
        const uint64_t k_row = (static_cast<uint64_t>(begin + j) * p.num_kv_heads + kv_head) * p.head_dim;
        float score = 0.0f;
        for (uint32_t d = lane; d < p.head_dim; d += 32)
            score += load_as_float(p.q, q_row + d, p.dtype) * load_as_float(p.local_k, k_row + d, p.dtype);
        score = warp_sum(score) * p.scale;
        if (lane == 0) weights[j] = score;
        block_max = fmaxf(block_max, score);
    }
    __syncwarp();
    float exp_sum = 0.0f;
    for (uint32_t j = 0; j < p.block_size; ++j) {
        const float w = expf(weights[j] - block_max);
        exp_sum += w;
        __syncwarp();
        if (lane == 0) weights[j] = w;
    }
    __syncwarp();
    const uint64_t slot = p.slot_indices != nullptr ? p.slot_indices[token] : token;
    const uint64_t out_row = slot * p.num_q_heads + head;
    if (lane == 0) {
        p.m[out_row] = block_max;
        p.l[out_row] = exp_sum;
    }
    for (uint32_t d = lane; d < p.head_dim; d += 32) {
        float acc = 0.0f;
        for (uint32_t j = 0; j < p.block_size; ++j) {
            const uint64_t v_row = (static_cast<uint64_t>(begin + j) * p.num_kv_heads + kv_head) * p.head_dim;
            acc += weights[j] * load_as_float(p.local_v, v_row + d, p.dtype);
        }
        p.o[out_row * p.head_dim + d] = exp_sum > 0.0f ? acc / exp_sum : 0.0f;
    }
}

// Cross-device merge of per-device partials in the natural-log domain (same algebra as above).
__global__ void __launch_bounds__(kReduceThreads) combine_kernel(CombineParams p) {
    bool ready = true;
    if (p.flags != nullptr) {
        // Partials arrive from other devices: wait, with a bound, until every producer has published this step.  The
        // launch reaches one verdict (settle_verdict), so `out` is written completely or not at all.
        __shared__ uint32_t verdict_s;
        if (threadIdx.x < 32) {
            const uint32_t verdict = settle_verdict(p.sync_words + kSyncVerdict, p.flags, p.n, p.flag_value, p.max_polls);
            if (threadIdx.x == 0) verdict_s = verdict;
        }
        __syncthreads();
        ready = verdict_s == kVerdictReady;
        if (!ready && threadIdx.x == 0) atomicExch(p.status, static_cast<uint32_t>(PSI_ERR_TIMEOUT));
    }
    const uint64_t total = ready ? static_cast<uint64_t>(p.num_rows) * p.head_dim : 0;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kReduceThreads + threadIdx.x; i < total;
         i += static_cast<uint64_t>(gridDim.x) * kReduceThreads) {
        const uint64_t row = i / p.head_dim;
        float global_max = -INFINITY;
        for (uint32_t s = 0; s < p.n; ++s) global_max = fmaxf(global_max, __ldcg(p.m[s] + row));
        float sum = 0.0f, acc = 0.0f;
        for (uint32_t s = 0; s < p.n; ++s) {
            const float pm = __ldcg(p.m[s] + row);
            const float w = isfinite(pm) ? expf(pm - global_max) * __ldcg(p.l[s] + row) : 0.0f;
            sum += w;
            acc += w * __ldcg(p.o[s] + i);
        }
        store_from_float(p.out, i, p.dtype, sum > 0.0f ? acc / sum : 0.0f);
    }
    if (p.flags != nullptr) {
        // the CTA that leaves last clears the verdict for the next launch
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(p.sync_words + kSyncMergeArrivals, 1u) + 1 == gridDim.x) {
                p.sync_words[kSyncMergeArrivals] = 0;
                p.sync_words[kSyncVerdict] = 0;
            }
        }
    }
}

__global__ void signal_kernel(uint32_t* flag, uint32_t value) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

}  // namespace

cudaError_t launch_signal(uint32_t* flag, uint32_t value, cudaStream_t stream) {
    signal_kernel<<<1, 1, 0, stream>>>(flag, value);
    return cudaGetLastError();
}

uint32_t attend_generic_ctas_per_sm(uint32_t head_dim, uint32_t dtype) {
    return head_dim % 4 == 0 ? attend_staged_ctas_per_sm(dtype) : 8u;
}

cudaError_t launch_attend_generic(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream) {
    if (num_ctas == 0) return cudaSuccess;
    if (attend_staged_supported(p)) return launch_attend_staged(p, num_ctas, stream);
    const uint32_t dpl = (p.geo.head_dim + 31) / 32;
    if (dpl <= 1) {
        attend_generic_kernel<1><<<num_ctas, kGenericThreads, 0, stream>>>(p);
    } else if (dpl <= 2) {
        attend_generic_kernel<2><<<num_ctas, kGenericThreads, 0, stream>>>(p);
    } else if (dpl <= 4) {
        attend_generic_kernel<4><<<num_ctas, kGenericThreads, 0, stream>>>(p);
    } else if (dpl <= 8) {
        attend_generic_kernel<8><<<num_ctas, kGenericThreads, 0, stream>>>(p);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_attend_reduce(const AttendParams& p, uint32_t num_reduces, cudaStream_t stream) {
    if (num_reduces == 0) return cudaSuccess;
    attend_reduce_kernel<<<dim3(num_reduces, kMaxRows), kReduceThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_block_partial(const BlockPartialParams& p, cudaStream_t stream) {
    const uint64_t pairs = static_cast<uint64_t>(p.num_tokens) * p.num_q_heads;
    if (pairs == 0) return cudaSuccess;
    if (p.block_size == 0 || p.block_size > kBlockPartialMaxBlock) return cudaErrorInvalidValue;
    const uint64_t blocks = (pairs + kBlockPartialWarps - 1) / kBlockPartialWarps;
    block_partial_kernel<<<static_cast<uint32_t>(blocks), kBlockPartialWarps * 32, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_combine(const CombineParams& p, cudaStream_t stream) {
    const uint64_t total = static_cast<uint64_t>(p.num_rows) * p.head_dim;
    if (total == 0) return cudaSuccess;
    const uint64_t blocks = (total + kReduceThreads - 1) / kReduceThreads;
    combine_kernel<<<static_cast<unsigned>(blocks < 4096 ? blocks : 4096), kReduceThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace psi
