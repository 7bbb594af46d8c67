// KV-range exchange for profiles whose attention kernel has no fused form (the CUDA-core kernel, steps with long query
// runs): the rank's partial is computed into local scratch by the ordinary launches, then one launch pushes it into
// the rank's slot of the owner's receive area and publishes the flag, and on the owner one launch waits for every
// rank and merges.  Same protocol, same bounds and same words as the fused form (exchange.cuh).
#include "exchange.cuh"

namespace psi {

namespace {

constexpr int kExchangeThreads = 256;

__global__ void __launch_bounds__(kExchangeThreads) exchange_push_kernel(ExchangeParams x, const float* local, float* slot,
                                                                        uint64_t floats, uint32_t* status) {
    __shared__ uint32_t free_s;
    if (threadIdx.x == 0) free_s = slot_is_free(x, x.step >= 3 ? ld_relaxed_sys(x.consumed) : 0u) ? 1u : 0u;
    __syncthreads();
    if (free_s) {
        const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kExchangeThreads * 4;
        for (uint64_t i = (static_cast<uint64_t>(blockIdx.x) * kExchangeThreads + threadIdx.x) * 4; i < floats; i += stride) {
            *reinterpret_cast<float4*>(slot + i) = __ldcg(reinterpret_cast<const float4*>(local + i));
        }
    }
    exchange_publish(x, status, gridDim.x, free_s == 0);
}

__global__ void __launch_bounds__(kExchangeThreads) exchange_merge_kernel(ExchangeParams x, void* out, uint32_t dtype,
                                                                         uint32_t head_dim, uint32_t* status) {
    exchange_merge<kExchangeThreads>(x, status, out, dtype, head_dim, blockIdx.x, gridDim.x);
}

}  // namespace

cudaError_t launch_exchange_push(const ExchangeParams& x, const float* local, float* slot, uint64_t floats,
                                 uint32_t* status, cudaStream_t stream) {
    if ((floats & 3u) != 0 || (reinterpret_cast<uintptr_t>(local) & 15u) != 0 || (reinterpret_cast<uintptr_t>(slot) & 15u) != 0) {
        return cudaErrorMisalignedAddress;
    }
    const uint64_t wanted = (floats / 4 + kExchangeThreads - 1) / kExchangeThreads;
    const unsigned blocks = static_cast<unsigned>(wanted < 1 ? 1 : (wanted > 64 ? 64 : wanted));
    exchange_push_kernel<<<blocks, kExchangeThreads, 0, stream>>>(x, local, slot, floats, status);
    return cudaGetLastError();
}

cudaError_t launch_exchange_merge(const ExchangeParams& x, void* out, uint32_t dtype, uint32_t head_dim, uint32_t* status,
                                  uint32_t max_ctas, cudaStream_t stream) {
    if (x.num_rows == 0) return cudaSuccess;
    const unsigned blocks = x.num_rows < max_ctas ? x.num_rows : max_ctas;
    exchange_merge_kernel<<<blocks, kExchangeThreads, 0, stream>>>(x, out, dtype, head_dim, status);
    return cudaGetLastError();
}

}  // namespace psi
