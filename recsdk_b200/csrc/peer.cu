// Peer mappings of device buffers between the processes of one box (one process per GPU).
// Thin wrappers over the CUDA IPC calls: the exporting rank names the cudaMalloc allocation
// that holds its buffer, the importing ranks map it and address it with plain loads/stores
// over NVLink.  No multicast object is created and no kernel here waits on another GPU.
#include <cuda.h>

#include <cstring>

#include "common.cuh"

using namespace recsdk;

static_assert(sizeof(cudaIpcMemHandle_t) == RECSDK_PEER_HANDLE_BYTES, "handle size");

extern "C" int recsdk_peer_export(const void* dev_ptr, unsigned char* handle_out, int64_t* offset_out)
{
    if (dev_ptr == nullptr || handle_out == nullptr || offset_out == nullptr) return RECSDK_ERR_INVALID_ARG;
    // the driver entry point is resolved through the runtime so that the library does not link libcuda
    // (it must load on machines without a driver, where only its symbols are inspected)
    typedef CUresult (*range_fn_t)(CUdeviceptr*, size_t*, CUdeviceptr);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres) != cudaSuccess || fn == nullptr ||
        qres != cudaDriverEntryPointSuccess) {
        (void)cudaGetLastError();
        return RECSDK_ERR_CUDA;
    }
    CUdeviceptr base = 0;
    size_t size = 0;
    if (reinterpret_cast<range_fn_t>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(dev_ptr)) != CUDA_SUCCESS)
        return RECSDK_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) != cudaSuccess) {
        (void)cudaGetLastError();
        return RECSDK_ERR_CUDA;
    }
    std::memcpy(handle_out, &h, sizeof(h));
    *offset_out = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(dev_ptr) - base);
    return RECSDK_OK;
}

extern "C" int recsdk_peer_import(const unsigned char* handle, int64_t offset, void** dev_ptr_out)
{
    if (handle == nullptr || dev_ptr_out == nullptr || offset < 0) return RECSDK_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void* base = nullptr;
    if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        (void)cudaGetLastError();
        return RECSDK_ERR_CUDA;
    }
    *dev_ptr_out = static_cast<char*>(base) + offset;
    return RECSDK_OK;
}

extern "C" int recsdk_peer_release(void* imported_ptr, int64_t offset)
{
    if (imported_ptr == nullptr || offset < 0) return RECSDK_ERR_INVALID_ARG;
    if (cudaIpcCloseMemHandle(static_cast<char*>(imported_ptr) - offset) != cudaSuccess) {
        (void)cudaGetLastError();
        return RECSDK_ERR_CUDA;
    }
    return RECSDK_OK;
}

extern "C" int recsdk_peer_copy(void* dst, const void* src, size_t bytes, void* stream)
{
    if (bytes == 0) return RECSDK_OK;
    if (dst == nullptr || src == nullptr) return RECSDK_ERR_INVALID_ARG;
    // either side may be a mapping returned by recsdk_peer_import: the copy engines move the bytes over NVLink
    if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        (void)cudaGetLastError();
        return RECSDK_ERR_CUDA;
    }
    return RECSDK_OK;
}
