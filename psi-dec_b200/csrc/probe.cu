// Read-only streaming probe: the practical ceiling of a kernel that only reads HBM (the attention kernels read K/V and
// write next to nothing), to stand beside the read+write copy figure the rooflines are quoted against.
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels.cuh"

namespace psi {

namespace {

constexpr int kProbeThreads = 256;
constexpr int kProbeUnroll = 8;  // 16-byte loads in flight per thread

__global__ void __launch_bounds__(kProbeThreads) read_stream_kernel(const uint4* __restrict__ src, uint64_t num_vectors,
                                                                    uint32_t* __restrict__ sink) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kProbeThreads;
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * kProbeThreads + threadIdx.x;
    uint32_t acc = 0;
    for (; i + (kProbeUnroll - 1) * stride < num_vectors; i += kProbeUnroll * stride) {
        uint4 v[kProbeUnroll];
#pragma unroll
        for (int u = 0; u < kProbeUnroll; ++u) {
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                         : "l"(src + i + u * stride));
        }
#pragma unroll
        for (int u = 0; u < kProbeUnroll; ++u) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
    }
    for (; i < num_vectors; i += stride) {
        const uint4 v = src[i];
        acc ^= v.x ^ v.y ^ v.z ^ v.w;
    }
    if (acc == 0x9E3779B9u) sink[0] = acc;  // keeps the loads; practically never taken
}

}  // namespace

cudaError_t launch_read_stream(const void* src, uint64_t bytes, uint32_t* sink, uint32_t num_ctas, cudaStream_t stream) {
    if (bytes < 16 || num_ctas == 0) return cudaErrorInvalidValue;
    read_stream_kernel<<<num_ctas, kProbeThreads, 0, stream>>>(static_cast<const uint4*>(src), bytes / 16, sink);
    return cudaGetLastError();
}

}  // namespace psi
