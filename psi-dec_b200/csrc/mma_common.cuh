// Building blocks shared by the tensor-core attention kernels: mma.sync / ldmatrix / cp.async wrappers, the XOR
// swizzle of shared-memory tiles, and the per-tile math (S = Q K^T with visibility mask and online softmax, O += P V)
// on one warp's 16 query rows against one 16-token KV tile.
#pragma once

#include <cmath>

#include "device_common.cuh"

namespace psi {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kTile = 16;  // KV tokens per tile == query rows of one warp

template <typename T>
struct Mma;

template <>
struct Mma<__nv_bfloat16> {
    __device__ static __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __device__ static __forceinline__ void store4(void* dst, float4 v) {
        uint2 packed = make_uint2(pack(v.x, v.y), pack(v.z, v.w));
        *reinterpret_cast<uint2*>(dst) = packed;
    }
};

template <>
struct Mma<__half> {
    __device__ static __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __device__ static __forceinline__ void store4(void* dst, float4 v) {
        uint2 packed = make_uint2(pack(v.x, v.y), pack(v.z, v.w));
        *reinterpret_cast<uint2*>(dst) = packed;
    }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// 16-byte global->shared copy; src_bytes == 0 zero-fills the destination without reading the source.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// An L2 policy for data that is read once: its lines are the first to be evicted, so that a K/V stream several times
// the size of the L2 does not push out what the launch reads again (plan, page table rows, partial outputs).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(policy));
    return policy;
}

// Policy for what the next launch reads again (the step's plan, the page table): evicted last.
__device__ __forceinline__ uint64_t l2_evict_last_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\n" : "=l"(policy));
    return policy;
}

// cp_async_16 under an L2 cache policy.
__device__ __forceinline__ void cp_async_16_hinted(uint32_t dst, const void* src, uint32_t src_bytes, uint64_t policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;\n" ::"r"(dst), "l"(src),
                 "r"(src_bytes), "l"(policy)
                 : "memory");
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }

template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold `row_bytes` bytes: the chunk index is
// XOR-ed with the low row bits so that the eight rows one ldmatrix phase reads fall into distinct banks.
__device__ __forceinline__ uint32_t swizzled(uint32_t row, uint32_t chunk, uint32_t row_bytes) {
    return row * row_bytes + ((chunk ^ (row & 7u)) << 4);
}

// Final output stores: optional gate (out = attention * sigmoid(gate)), then one rounding to the I/O dtype.
template <typename T>
__device__ __forceinline__ void store_out4(const AttendParams& p, uint64_t index, float4 v) {
    if (p.gates != nullptr) {
        const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const T*>(p.gates) + index);
        const T* g = reinterpret_cast<const T*>(&raw);
        v.x *= gate_sigmoid(static_cast<float>(g[0]));
        v.y *= gate_sigmoid(static_cast<float>(g[1]));
        v.z *= gate_sigmoid(static_cast<float>(g[2]));
        v.w *= gate_sigmoid(static_cast<float>(g[3]));
    }
    Mma<T>::store4(static_cast<T*>(p.out) + index, v);
}

// Eight consecutive outputs as one 16-byte store.
template <typename T>
__device__ __forceinline__ void store_out8(const AttendParams& p, uint64_t index, const float* v) {
    float g[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
    if (p.gates != nullptr) {
        const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.gates) + index);
        const T* gate = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) g[i] = gate_sigmoid(static_cast<float>(gate[i]));
    }
    const uint4 packed = make_uint4(Mma<T>::pack(v[0] * g[0], v[1] * g[1]), Mma<T>::pack(v[2] * g[2], v[3] * g[3]),
                                    Mma<T>::pack(v[4] * g[4], v[5] * g[5]), Mma<T>::pack(v[6] * g[6], v[7] * g[7]));
    *reinterpret_cast<uint4*>(static_cast<T*>(p.out) + index) = packed;
}

template <typename T>
__device__ __forceinline__ void store_out2(const AttendParams& p, uint64_t index, float a, float b) {
    if (p.gates != nullptr) {
        const uint32_t raw = *reinterpret_cast<const uint32_t*>(static_cast<const T*>(p.gates) + index);
        const T* g = reinterpret_cast<const T*>(&raw);
        a *= gate_sigmoid(static_cast<float>(g[0]));
        b *= gate_sigmoid(static_cast<float>(g[1]));
    }
    *reinterpret_cast<uint32_t*>(static_cast<T*>(p.out) + index) = Mma<T>::pack(a, b);
}

// Lane roles of the ldmatrix fetches, pre-folded into byte offsets (constant for a whole kernel).
struct FragmentLanes {
    uint32_t q_lane, q_x;   // A operand (query rows x k halves): address = q_tile_base + q_lane + (q_x ^ 32*ks)
    uint32_t k_lane, k_x;   // B operand of Q K^T:               address = k_tile_base + k_lane + (k_x ^ 32*ks)
    uint32_t v_lane, v_x;   // B operand of P V (transposed):    address = v_tile_base + v_lane + (v_x ^ 32*j)
    uint32_t quad_row, quad_col;
    // `atom_group_bytes` == 0: K and V tiles are rows of `row_bytes` with the chunk index XOR-ed over the whole row
    // (what the cp.async copies write).  Otherwise they are in the layout a TMA box of the page arena lands in
    // (operand_offset in tma_common.cuh): 8-row groups `atom_group_bytes` apart, each a run of 1 KiB swizzle atoms of
    // 8 rows x 128 bytes; the k-step (or output-column) term then selects the atom as well as the chunk inside it.
    // The query tile is always in the row layout.
    __device__ __forceinline__ FragmentLanes(uint32_t lane, uint32_t row_bytes, uint32_t atom_group_bytes = 0) {
        const uint32_t mat = lane >> 3, mat_row = lane & 7;
        const uint32_t q_row = mat_row + 8 * (mat & 1), k_row = mat_row + 8 * (mat >> 1), v_row = mat_row + 8 * (mat & 1);
        q_lane = q_row * row_bytes;
        q_x = ((mat >> 1) ^ (q_row & 7)) << 4;
        if (atom_group_bytes == 0) {
            k_lane = k_row * row_bytes;
            v_lane = v_row * row_bytes;
        } else {
            k_lane = (k_row >> 3) * atom_group_bytes + (k_row & 7) * 128;
            v_lane = (v_row >> 3) * atom_group_bytes + (v_row & 7) * 128;
        }
        k_x = ((mat & 1) ^ (k_row & 7)) << 4;
        v_x = ((mat >> 1) ^ (v_row & 7)) << 4;
        quad_row = lane >> 2;
        quad_col = lane & 3;
    }
};

// Running softmax state of the two accumulator rows a thread holds (quad_row and quad_row + 8) and its O fragments.
template <int D>
struct RowState {
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    float o[D / 8][4];
    __device__ __forceinline__ void clear() {
        m0 = m1 = -INFINITY;
        l0 = l1 = 0.0f;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    }
};

// kAtom: the K/V tile is in the TMA box layout (see FragmentLanes); step s of a row then lives in atom s / 4 at
// chunk pair s % 4.
template <typename T, int D, bool kAtom = false>
struct TileMath {
    static constexpr int kKSteps = D / 16;
    __device__ __forceinline__ static constexpr uint32_t step_term(uint32_t x, int s) {
        return kAtom ? static_cast<uint32_t>(s >> 2) * 1024u + (x ^ (32u * static_cast<uint32_t>(s & 3)))
                     : (x ^ (32u * static_cast<uint32_t>(s)));
    }

    // S = Q K^T for one 16-token K tile, visibility mask, online softmax update; leaves P (packed for the A operand
    // of P V) in `pa`.  Keys at or beyond a row's limit, or before `kv_begin`, do not count.
    __device__ __forceinline__ static void scores(const FragmentLanes& f, uint32_t q_tile, uint32_t k_tile,
                                                  float scale_log2, bool masked, uint32_t token0, uint32_t limit0,
                                                  uint32_t limit1, uint32_t kv_begin, RowState<D>& st,
                                                  uint32_t (&pa)[4]) {
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float s_odd[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};  // odd k-steps: a second dependency chain
#pragma unroll
        for (int ks = 0; ks < kKSteps; ++ks) {
            uint32_t a[4], b[4];
            ldmatrix_x4(a, q_tile + f.q_lane + (f.q_x ^ (32u * ks)));
            ldmatrix_x4(b, k_tile + f.k_lane + step_term(f.k_x, ks));
            if (ks & 1) {
                Mma<T>::run(s_odd[0], a, b[0], b[1]);
                Mma<T>::run(s_odd[1], a, b[2], b[3]);
            } else {
                Mma<T>::run(s[0], a, b[0], b[1]);
                Mma<T>::run(s[1], a, b[2], b[3]);
            }
        }
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[n][e] = (s[n][e] + s_odd[n][e]) * scale_log2;
        if (masked) {
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t token = token0 + 8 * n + 2 * f.quad_col + (e & 1);
                    const uint32_t limit = e < 2 ? limit0 : limit1;
                    if (token >= limit || token < kv_begin) s[n][e] = -INFINITY;
                }
        }
        float max0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        float max1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
        max0 = fmaxf(max0, __shfl_xor_sync(0xFFFFFFFFu, max0, 1));
        max0 = fmaxf(max0, __shfl_xor_sync(0xFFFFFFFFu, max0, 2));
        max1 = fmaxf(max1, __shfl_xor_sync(0xFFFFFFFFu, max1, 1));
        max1 = fmaxf(max1, __shfl_xor_sync(0xFFFFFFFFu, max1, 2));
        const float new0 = fmaxf(st.m0, max0), new1 = fmaxf(st.m1, max1);
        const bool moved = new0 > st.m0 || new1 > st.m1;
        if (__any_sync(0xFFFFFFFFu, moved)) {  // O is rescaled only when some row's running max moved
            const float corr0 = new0 == -INFINITY ? 1.0f : exp2f(st.m0 - new0);
            const float corr1 = new1 == -INFINITY ? 1.0f : exp2f(st.m1 - new1);
            st.l0 *= corr0;
            st.l1 *= corr1;
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                st.o[j][0] *= corr0;
                st.o[j][1] *= corr0;
                st.o[j][2] *= corr1;
                st.o[j][3] *= corr1;
            }
            st.m0 = new0;
            st.m1 = new1;
        }
        const float base0 = st.m0 == -INFINITY ? 0.0f : st.m0, base1 = st.m1 == -INFINITY ? 0.0f : st.m1;
        const float p00 = exp2f(s[0][0] - base0), p01 = exp2f(s[0][1] - base0);
        const float p02 = exp2f(s[0][2] - base1), p03 = exp2f(s[0][3] - base1);
        const float p10 = exp2f(s[1][0] - base0), p11 = exp2f(s[1][1] - base0);
        const float p12 = exp2f(s[1][2] - base1), p13 = exp2f(s[1][3] - base1);
        st.l0 += (p00 + p01) + (p10 + p11);  // per-thread part of the row sum; the quad is summed once at the end
        st.l1 += (p02 + p03) + (p12 + p13);
        pa[0] = Mma<T>::pack(p00, p01);
        pa[1] = Mma<T>::pack(p02, p03);
        pa[2] = Mma<T>::pack(p10, p11);
        pa[3] = Mma<T>::pack(p12, p13);
    }

    // O += P V for one 16-token V tile.
    __device__ __forceinline__ static void values(const FragmentLanes& f, uint32_t v_tile, const uint32_t (&pa)[4],
                                                  RowState<D>& st) {
#pragma unroll
        for (int j = 0; j < D / 16; ++j) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, v_tile + f.v_lane + step_term(f.v_x, j));
            Mma<T>::run(st.o[2 * j], pa, b[0], b[1]);
            Mma<T>::run(st.o[2 * j + 1], pa, b[2], b[3]);
        }
    }
};

}  // namespace psi
