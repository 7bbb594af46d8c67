// Device side of the KV-range exchange that runs inside the attention launch (see ExchangeParams in kernels.cuh).
//
// Peer memory is only ever touched with plain stores (partials, flag) and plain loads (the consumed word): no bulk or
// tensor copies and no multicast.  Every wait is bounded: when it runs out the launch records PSI_ERR_TIMEOUT in the
// status word, writes no output, and returns, so the context stays usable.
//
// The merge is the reference's reduce algebra (crates/inference-backend-metal/src/components/metal/
// gqa_split_kv_single_q_reduce.metal:27-48) over one partial per rank: M = max m_i, w_i = exp(m_i - M) * l_i (0 when
// m_i is not finite), out = sum w_i o_i / sum w_i (0 when the sum is 0).
#pragma once

#include "device_common.cuh"

namespace psi {

constexpr uint32_t kVerdictReady = 1;
constexpr uint32_t kVerdictTimeout = 2;
constexpr uint32_t kArrivalFailed = 0x10000u;  // added to the launch arrival count by a CTA that gave up

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* address) {
    uint32_t value;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
    return value;
}

__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* address) {
    uint32_t value;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
    return value;
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* address) {
    uint32_t value;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
    return value;
}

__device__ __forceinline__ void st_release_sys(uint32_t* address, uint32_t value) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}

// True once `seen` has reached `wanted` (step counters; wrap-safe).
__device__ __forceinline__ bool reached(uint32_t seen, uint32_t wanted) {
    return static_cast<int32_t>(seen - wanted) >= 0;
}

// A slot of the receive area is written again two steps later (slots alternate with the step's parity), so a rank
// may store step s only after the owner has merged step s - 2.  `early` is a value of the consumed word read at the
// start of the launch; one thread calls this before the CTA's first store into the slot.  Returns false when the
// bounded wait ran out.
__device__ __forceinline__ bool slot_is_free(const ExchangeParams& x, uint32_t early) {
    if (x.step < 3) return true;
    const uint32_t wanted = x.step - 2;
    uint32_t seen = early;
    uint32_t polls = 0;
    while (!reached(seen, wanted)) {
        if (++polls > x.max_polls) return false;
        __nanosleep(100);
        seen = ld_acquire_sys(x.consumed);
    }
    asm volatile("fence.acq_rel.sys;" ::: "memory");  // the stores below come after the owner's reads of step s - 2
    return true;
}

// One verdict per launch on whether every one of `n` flags has reached `value`: called by the first warp of a CTA.
// The first CTA to see every flag, or to run out of polls, settles the word with a compare-and-swap; every CTA
// returns what the word holds (kVerdictReady or kVerdictTimeout).  The caller zeroes the word once the launch is over.
__device__ __forceinline__ uint32_t settle_verdict(uint32_t* word, const uint32_t* flags, uint32_t n, uint32_t value,
                                                   uint32_t max_polls) {
    const uint32_t lane = threadIdx.x & 31u;
    uint32_t verdict = 0, polls = 0;
    for (;;) {
        verdict = ld_acquire_gpu(word);
        if (verdict != 0) break;
        bool all_in = true;
        for (uint32_t r = lane; r < n; r += 32) all_in = all_in && reached(ld_acquire_sys(flags + r), value);
        all_in = __all_sync(0xFFFFFFFFu, all_in);
        if (all_in || ++polls > max_polls) {
            if (lane == 0) {
                __threadfence();
                atomicCAS(word, 0u, all_in ? kVerdictReady : kVerdictTimeout);
            }
            __syncwarp();
            continue;  // the word now holds a verdict, this CTA's or an earlier one
        }
        __nanosleep(100);
    }
    if (verdict == kVerdictReady) {
        // this CTA's own acquire of every flag, so that what it reads next is what the producers published
        for (uint32_t r = lane; r < n; r += 32) (void)ld_acquire_sys(flags + r);
    }
    return verdict;
}

// End of a rank's launch, part one.  Called by every thread of every active CTA after its last store into the slot:
// the CTA that arrives last release-stores the step into the rank's flag.  `failed`: this CTA did not store (its wait
// for the slot ran out), so the flag is held back and PSI_ERR_TIMEOUT recorded.
__device__ __forceinline__ void exchange_publish(const ExchangeParams& x, uint32_t* status, uint32_t num_ctas, bool failed) {
    // The barrier orders every thread's stores into the slot before thread 0's system-wide fence (cumulative), which
    // makes them visible to the owner before the arrival counts.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t mine = failed ? (1u | kArrivalFailed) : 1u;
        const uint32_t total = atomicAdd(x.sync_words + kSyncLaunchArrivals, mine) + mine;
        if ((total & 0xFFFFu) == num_ctas) {
            x.sync_words[kSyncLaunchArrivals] = 0;  // ready for the next launch (stream order)
            if (total < kArrivalFailed) {
                __threadfence_system();
                st_release_sys(x.flag, x.step);
            } else if (status != nullptr) {
                atomicExch(status, static_cast<uint32_t>(PSI_ERR_TIMEOUT));
            }
        }
    }
}

// Part two, on the owner only: CTA c waits, with a bound, until every rank has published this step, then merges
// rows c, c + mergers, ... of the partials in the local receive area into `out`.  One verdict holds for the whole
// launch (settle_verdict), so either all rows are written or none.  The CTA that finishes last re-arms the words and
// release-stores the step into the consumed word, which frees this step's slots for the producers.
template <int kThreadsPerCta>
__device__ __forceinline__ void exchange_merge(const ExchangeParams& x, uint32_t* status, void* out, uint32_t dtype,
                                               uint32_t head_dim, uint32_t cta, uint32_t num_ctas) {
    const uint32_t tid = threadIdx.x;
    __shared__ uint32_t verdict_s;
    const uint32_t mergers = min(num_ctas, x.num_rows);
    if (cta >= mergers) return;
    if (tid < 32) {
        const uint32_t verdict = settle_verdict(x.sync_words + kSyncVerdict, x.flags, x.world, x.step, x.max_polls);
        if (tid == 0) verdict_s = verdict;
    }
    __syncthreads();
    const bool ready = verdict_s == kVerdictReady;
    if (ready) {
        const uint64_t m_offset = static_cast<uint64_t>(x.num_rows) * head_dim, l_offset = m_offset + x.num_rows;
        for (uint32_t row = cta; row < x.num_rows; row += mergers) {
            float row_max = -INFINITY;
            for (uint32_t r = 0; r < x.world; ++r) row_max = fmaxf(row_max, __ldcg(x.recv + r * x.slot_stride + m_offset + row));
            for (uint32_t col = tid; col < head_dim; col += kThreadsPerCta) {
                float sum = 0.0f, acc = 0.0f;
                for (uint32_t r = 0; r < x.world; ++r) {
                    const float* slot = x.recv + r * x.slot_stride;
                    const float pm = __ldcg(slot + m_offset + row);
                    const float w = isfinite(pm) ? expf(pm - row_max) * __ldcg(slot + l_offset + row) : 0.0f;
                    sum += w;
                    acc += w * __ldcg(slot + static_cast<uint64_t>(row) * head_dim + col);
                }
                store_from_float(out, static_cast<uint64_t>(row) * head_dim + col, dtype, sum > 0.0f ? acc / sum : 0.0f);
            }
        }
    } else if (tid == 0 && status != nullptr) {
        atomicExch(status, static_cast<uint32_t>(PSI_ERR_TIMEOUT));
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(x.sync_words + kSyncMergeArrivals, 1u) + 1 == mergers) {
            x.sync_words[kSyncMergeArrivals] = 0;
            x.sync_words[kSyncVerdict] = 0;
            if (ready) {
                __threadfence_system();
                st_release_sys(x.consumed_local, x.step);
            }
        }
    }
}

}  // namespace psi
