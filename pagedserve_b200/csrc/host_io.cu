// Host-side plumbing of a step: the one upload of its metadata, and host memory that kernels write directly.
//
// A decode step's result is a handful of sampled token ids. Instead of a device buffer plus a device-to-host
// copy after the step, the token feedback kernel writes them straight into page-locked host memory that is
// mapped into the device's address space; after the stream is synchronised the host reads them in place.
#include "common.cuh"

// bytes of page-locked host memory, mapped for the device: *host is the CPU address, *device the address
// kernels use.
PS_EXPORT int ps_host_alloc_mapped(long long bytes, void** host, void** device) {
    if (bytes <= 0 || !host || !device) return PS_ERR_BAD_ARGUMENT;
    void* h = nullptr;
    if (cudaHostAlloc(&h, (size_t)bytes, cudaHostAllocMapped) != cudaSuccess) return PS_ERR_LAUNCH;
    void* d = nullptr;
    if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
        cudaFreeHost(h);
        return PS_ERR_LAUNCH;
    }
    memset(h, 0, (size_t)bytes);
    *host = h;
    *device = d;
    return PS_OK;
}

PS_EXPORT int ps_host_free(void* host) {
    if (!host) return PS_OK;
    return cudaFreeHost(host) == cudaSuccess ? PS_OK : PS_ERR_LAUNCH;
}

// One asynchronous copy from page-locked host memory to the device on `stream`.
PS_EXPORT int ps_copy_h2d(void* dst, const void* src, long long bytes, void* stream) {
    if (bytes <= 0) return PS_OK;
    if (!dst || !src) return PS_ERR_BAD_ARGUMENT;
    return cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream) == cudaSuccess
               ? PS_OK
               : PS_ERR_LAUNCH;
}
