// Host-side launch helpers shared by the kernel files.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

namespace psi {

// Raises a kernel's dynamic shared-memory limit once per device.  The attribute belongs to the (kernel, device) pair;
// `done` is the caller's per-kernel record (one bit per device, static storage), safe for host threads that launch on
// several devices at once.  Devices beyond the 64 the mask can hold set the attribute on every launch.
inline cudaError_t ensure_dynamic_smem(const void* kernel, int bytes, std::atomic<uint64_t>& done) {
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return err;
    const uint64_t bit = device < 64 ? (1ull << device) : 0ull;
    if (bit != 0 && (done.load(std::memory_order_acquire) & bit) != 0) return cudaSuccess;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (err != cudaSuccess) return err;
    if (bit != 0) done.fetch_or(bit, std::memory_order_release);
    return cudaSuccess;
}

}  // namespace psi
