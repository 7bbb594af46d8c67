// The stages the reference records directly before the page write, fused with it into one launch: per-head RMSNorm
// and RoPE of q (to q_out) and of k (straight into its page), and the V rows into their pages.
//
// Reference stages: crates/inference-executor-metal/src/attn/gqa/backend.rs:465-513 (q norm/rope, k norm/rope,
// kv_page_write), shader crates/inference-backend-metal/src/components/metal/rms_norm_rope.metal:7-82 and
// metal/gqa_kv_page_write.metal:20-52.  One warp per (token, head) row; the rounding order of the shader is kept:
// T(weight) * T(x * inv_rms) in the storage dtype T, rotation in f32, one final rounding to T.
//
// The inputs are addressed through strides, so the same launch also stands for the stage before those three: the
// de-interleave of the fused projection output (metal/gqa_qgkv_split.metal:14-42 with gates,
// metal/gqa_qkv_split.metal:13-36 without).  Its q, g, k and v rows are read where the projection left them; only the
// gate rows, which the attention epilogue wants contiguous, are copied out.
#include "device_common.cuh"

namespace psi {

namespace {

template <uint32_t DTYPE>
__device__ __forceinline__ float round_to(float v) {
    if (DTYPE == PSI_DTYPE_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    if (DTYPE == PSI_DTYPE_F16) return __half2float(__float2half_rn(v));
    return v;
}

constexpr int kPrepWarps = 8;

// Bit copy of one element (V rows and gate rows pass through unchanged, NaN payloads included).
__device__ __forceinline__ void copy_element(void* dst, uint64_t dst_index, const void* src, uint64_t src_index,
                                             uint32_t dtype) {
    if (dtype == PSI_DTYPE_F32) {
        static_cast<uint32_t*>(dst)[dst_index] = static_cast<const uint32_t*>(src)[src_index];
    } else {
        static_cast<uint16_t*>(dst)[dst_index] = static_cast<const uint16_t*>(src)[src_index];
    }
}

template <uint32_t DTYPE>
__global__ void __launch_bounds__(kPrepWarps * 32) norm_rope_append_kernel(PrepParams p) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t num_active = min(p.scalars[kScalarNumActiveTokens], p.num_total_tokens);
    const uint32_t hq = p.num_q_heads, hkv = p.geo.num_kv_heads, D = p.geo.head_dim;
    const uint64_t q_rows = static_cast<uint64_t>(num_active) * hq, kv_rows = static_cast<uint64_t>(num_active) * hkv;
    const uint64_t g_rows = p.g_in != nullptr ? q_rows : 0;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * kPrepWarps + (threadIdx.x >> 5);
    if (row >= q_rows + 2 * kv_rows + g_rows) return;

    if (row >= q_rows + 2 * kv_rows) {
        // gate row: a bit copy out of the projection into the contiguous [T][Hq][D] the attention epilogue reads
        const uint64_t local = row - q_rows - 2 * kv_rows;
        const uint64_t src_base = (local / hq) * p.q_token_stride + (local % hq) * p.q_head_stride;
        for (uint32_t d = lane; d < D; d += 32) copy_element(p.g_out, local * D + d, p.g_in, src_base + d, DTYPE);
        return;
    }

    // which tensor, which (token, head)
    const bool is_q = row < q_rows, is_v = row >= q_rows + kv_rows;
    const uint64_t local = is_q ? row : (is_v ? row - q_rows - kv_rows : row - q_rows);
    const uint32_t heads = is_q ? hq : hkv;
    const uint32_t token = static_cast<uint32_t>(local / heads), head = static_cast<uint32_t>(local % heads);
    const void* src = is_q ? p.q_in : (is_v ? p.v_in : p.k_in);
    const uint64_t src_base = is_q ? token * p.q_token_stride + head * p.q_head_stride
                                   : token * p.kv_token_stride + static_cast<uint64_t>(head) * D;

    // destination: q_out row, or the row's place in its page
    void* dst = p.q_out;
    uint64_t dst_base = local * D;
    if (!is_q) {
        const uint32_t pos = p.flat_token_indices[token];
        const uint32_t page_index = pos / p.geo.tokens_per_page;
        uint32_t page_id;
        if (!checked_page_id(p.geo, table_row(p.geo, p.req_slots[token]), page_index, page_id)) return;  // write skipped
        dst = const_cast<void*>(p.geo.pages);
        dst_base = kv_row_offset(p.geo, page_id, head, pos % p.geo.tokens_per_page) + (is_v ? v_region_offset(p.geo) : 0);
    }
    if (is_v) {
        for (uint32_t d = lane; d < D; d += 32) copy_element(dst, dst_base + d, src, src_base + d, DTYPE);
        return;
    }

    float acc = 0.0f;
    for (uint32_t d = lane; d < D; d += 32) {
        const float x = load_as_float(src, src_base + d, DTYPE);
        acc += x * x;
    }
    acc = warp_sum(acc);
    const float inv_rms = 1.0f / sqrtf(acc / static_cast<float>(D) + p.eps);
    const __nv_bfloat16* weight = reinterpret_cast<const __nv_bfloat16*>(is_q ? p.q_weight : p.k_weight);
    const float position = static_cast<float>(p.flat_token_indices[token]);
    const uint32_t rope_half = p.rope_dim / 2;
    auto normed = [&](uint32_t d) {
        const float w = round_to<DTYPE>(__bfloat162float(weight[d]));
        return round_to<DTYPE>(w * round_to<DTYPE>(load_as_float(src, src_base + d, DTYPE) * inv_rms));
    };
    for (uint32_t d = lane; d < D; d += 32) {
        if (d < rope_half) {
            const uint32_t d2 = d + rope_half;
            const float x1 = normed(d), x2 = normed(d2);
            float s, c;
            sincosf(position * p.inverse_frequencies[d], &s, &c);
            store_from_float(dst, dst_base + d, DTYPE, p.attention_factor * (x1 * c - x2 * s));
            store_from_float(dst, dst_base + d2, DTYPE, p.attention_factor * (x1 * s + x2 * c));
        } else if (d >= p.rope_dim) {
            store_from_float(dst, dst_base + d, DTYPE, normed(d));
        }
    }
}

}  // namespace

cudaError_t launch_norm_rope_append(const PrepParams& p, cudaStream_t stream) {
    const uint64_t rows = static_cast<uint64_t>(p.num_total_tokens) *
                          ((p.g_in != nullptr ? 2ull : 1ull) * p.num_q_heads + 2ull * p.geo.num_kv_heads);
    if (rows == 0) return cudaSuccess;
    const unsigned blocks = static_cast<unsigned>((rows + kPrepWarps - 1) / kPrepWarps);
    switch (p.dtype) {
        case PSI_DTYPE_F32: norm_rope_append_kernel<PSI_DTYPE_F32><<<blocks, kPrepWarps * 32, 0, stream>>>(p); break;
        case PSI_DTYPE_BF16: norm_rope_append_kernel<PSI_DTYPE_BF16><<<blocks, kPrepWarps * 32, 0, stream>>>(p); break;
        default: norm_rope_append_kernel<PSI_DTYPE_F16><<<blocks, kPrepWarps * 32, 0, stream>>>(p); break;
    }
    return cudaGetLastError();
}

}  // namespace psi
