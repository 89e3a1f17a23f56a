// Small C-ABI utilities: status block, error strings, version.
#include "common.cuh"

extern "C" int recsdk_status_clear(int64_t* dev_status, void* stream)
{
    if (!dev_status) return RECSDK_ERR_INVALID_ARG;
    cudaError_t e = cudaMemsetAsync(dev_status, 0, RECSDK_STATUS_WORDS * sizeof(int64_t), static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? RECSDK_OK : RECSDK_ERR_CUDA;
}

extern "C" const char* recsdk_error_string(int code)
{
    switch (code) {
        case RECSDK_OK: return "ok";
        case RECSDK_ERR_INVALID_ARG: return "invalid argument";
        case RECSDK_ERR_WORKSPACE: return "workspace missing or too small";
        case RECSDK_ERR_CUDA: return "CUDA launch or runtime error";
        case RECSDK_ERR_NEGATIVE_KEY: return "Invalid key value";
        case RECSDK_ERR_TABLE_FULL: return "Ids map reached maxIndex, please reallocate a larger buffer";
        case RECSDK_ERR_CACHE_TOO_SMALL: return "cacheSize_ too small";
        case RECSDK_ERR_INDEX_RANGE: return "row index out of range";
        case RECSDK_ERR_HASH_FULL: return "key table has no free entry";
        case RECSDK_ERR_TOO_LARGE: return "size beyond the supported maximum";
        case RECSDK_ERR_STATIC_SCRATCH: return "the built-in scratch array could not be located on this device";
        default: return "unknown error";
    }
}

extern "C" int recsdk_version(void) { return 100; }
