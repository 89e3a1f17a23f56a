// Sorted unique + inverse of int64 ids (radix sort of (id, position) pairs,
// adjacent-difference head flags, scan).  Same result as a CPU sort followed by
// an adjacent-diff pass: unique ascending, inverse[i] = rank of ids[i].
#include "prims.cuh"

namespace recsdk {

template <typename KeyT>
__global__ void __launch_bounds__(256) unique_load_kernel(const int64_t* __restrict__ ids, int64_t n,
                                                          KeyT* __restrict__ keys, uint32_t* __restrict__ vals)
{
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        keys[i] = static_cast<KeyT>(ids[i]);
        vals[i] = static_cast<uint32_t>(i);
    }
}

template <typename KeyT>
__global__ void __launch_bounds__(256) unique_flag_kernel(const KeyT* __restrict__ keys, int64_t n, int* __restrict__ flag)
{
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        flag[i] = (i == 0 || keys[i] != keys[i - 1]) ? 1 : 0;
}

template <typename KeyT>
__global__ void __launch_bounds__(256) unique_write_kernel(const KeyT* __restrict__ keys,
                                                           const uint32_t* __restrict__ vals,
                                                           const int* __restrict__ incl, int64_t n,
                                                           int64_t* __restrict__ unique_out,
                                                           int64_t* __restrict__ inverse_out,
                                                           int64_t* __restrict__ num_unique_out)
{
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int r = incl[i] - 1;
        if (i == 0 || keys[i] != keys[i - 1]) unique_out[r] = static_cast<int64_t>(keys[i]);
        inverse_out[vals[i]] = r;
        if (i == n - 1 && num_unique_out != nullptr) *num_unique_out = r + 1;
    }
}

struct UniqueWorkspace {
    void *keys_a, *keys_b;
    uint32_t *vals_a, *vals_b, *sort_scratch;
    int *flag, *scan_scratch;
    size_t bytes;
};

static UniqueWorkspace carve_unique(void* base, int64_t N)
{
    WorkspaceCarver c(base);
    UniqueWorkspace w;
    const size_t n = static_cast<size_t>(N > 0 ? N : 1);
    w.keys_a = c.take<uint64_t>(n);
    w.keys_b = c.take<uint64_t>(n);
    w.vals_a = c.take<uint32_t>(n);
    w.vals_b = c.take<uint32_t>(n);
    w.sort_scratch = c.take<uint32_t>(sort_scratch_u32(N));
    w.flag = c.take<int>(n);
    w.scan_scratch = c.take<int>(scan_scratch_ints(N));
    w.bytes = c.used();
    return w;
}

template <typename KeyT>
static int run_unique(const int64_t* ids, int64_t n, int key_bits, int64_t* unique_out, int64_t* inverse_out,
                      int64_t* num_unique_out, const UniqueWorkspace& ws, cudaStream_t st)
{
    KeyT* ka = static_cast<KeyT*>(ws.keys_a);
    KeyT* kb = static_cast<KeyT*>(ws.keys_b);
    const int grid = grid_for(n, 256);
    unique_load_kernel<KeyT><<<grid, 256, 0, st>>>(ids, n, ka, ws.vals_a);
    const int which = radix_sort_pairs<KeyT>(ka, ws.vals_a, kb, ws.vals_b, n, key_bits, ws.sort_scratch, st);
    const KeyT* keys = which ? kb : ka;
    const uint32_t* vals = which ? ws.vals_b : ws.vals_a;
    unique_flag_kernel<KeyT><<<grid, 256, 0, st>>>(keys, n, ws.flag);
    device_scan<true>(ws.flag, ws.flag, n, ws.scan_scratch, nullptr, st);
    unique_write_kernel<KeyT><<<grid, 256, 0, st>>>(keys, vals, ws.flag, n, unique_out, inverse_out, num_unique_out);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

}  // namespace recsdk

using namespace recsdk;

extern "C" size_t recsdk_unique_sorted_workspace_bytes(int64_t n) { return carve_unique(nullptr, n).bytes; }

extern "C" int recsdk_unique_sorted(const int64_t* ids, int64_t n, int key_bits, int64_t* unique_out,
                                    int64_t* inverse_out, int64_t* num_unique_out, void* workspace,
                                    size_t workspace_bytes, void* stream)
{
    if (n < 0 || key_bits < 1 || key_bits > 64) return RECSDK_ERR_INVALID_ARG;
    if (n >= (int64_t(1) << 31)) return RECSDK_ERR_TOO_LARGE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n == 0) {
        if (num_unique_out) cudaMemsetAsync(num_unique_out, 0, sizeof(int64_t), st);
        return RECSDK_OK;
    }
    if (!ids || !unique_out || !inverse_out) return RECSDK_ERR_INVALID_ARG;
    if (!workspace) return RECSDK_ERR_WORKSPACE;
    const UniqueWorkspace ws = carve_unique(workspace, n);
    if (ws.bytes > workspace_bytes) return RECSDK_ERR_WORKSPACE;
    if (key_bits <= 32) return run_unique<uint32_t>(ids, n, key_bits, unique_out, inverse_out, num_unique_out, ws, st);
    return run_unique<uint64_t>(ids, n, key_bits, unique_out, inverse_out, num_unique_out, ws, st);
}

// ----------------------------------------------------------------------------
// Allocation-free variant: sorted unique + inverse with built-in scratch.
//
// Some callers of this library cannot allocate device memory at the point where they
// need a dedup: code running inside a framework's allocator callback or memory-pool
// hook, a preprocessing thread that was handed device buffers but no allocator, or a
// service whose device memory is fully budgeted up front and where a late cudaMalloc
// may fail or stall the device.  For them the scratch of the sort lives in a
// file-scope __device__ array, sized for at most RECSDK_UNIQUE_STATIC_MAX_N ids; every
// GPU that loads this library holds those bytes until the process exits.
//
// The array's name is only a host-side stand-in for the symbol: its device address
// is resolved with cudaGetSymbolAddress, once per device, on the first call made with
// that device current.  That first call should therefore happen before any stream
// capture is started -- and during start-up: with lazy module loading the driver places
// this file's device image (the array included) in device memory at its first use, so
// the first call is the one call of this entry point that can make the driver allocate.  All calls on one device share the same scratch, which keeps the
// contents of the previous call: nothing in this pipeline needs it zeroed (every
// scratch word is written before it is read), but two calls whose kernels overlap on
// the GPU (different streams) race on it -- serialise them.
// ----------------------------------------------------------------------------
#include <mutex>

namespace recsdk {

constexpr int64_t kUniqueStaticMaxN = RECSDK_UNIQUE_STATIC_MAX_N;
constexpr size_t kUniqueStaticBytes = size_t(8) << 20;  // >= carve_unique(kUniqueStaticMaxN).bytes, checked at set-up

static __device__ __align__(256) unsigned char g_unique_static_scratch[kUniqueStaticBytes];

static std::mutex g_unique_static_mu;
static void* g_unique_static_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (resolved once per device).
static int unique_static_scratch(void** out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return RECSDK_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_unique_static_mu);
    if (g_unique_static_ptr[dev] == nullptr) {
        if (carve_unique(nullptr, kUniqueStaticMaxN).bytes > kUniqueStaticBytes) return RECSDK_ERR_WORKSPACE;
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_unique_static_scratch) != cudaSuccess || ptr == nullptr) {
            (void)cudaGetLastError();
            return RECSDK_ERR_STATIC_SCRATCH;
        }
        g_unique_static_ptr[dev] = ptr;
    }
    *out = g_unique_static_ptr[dev];
    return RECSDK_OK;
}

}  // namespace recsdk

extern "C" int64_t recsdk_unique_sorted_static_max_n(void) { return recsdk::kUniqueStaticMaxN; }

extern "C" int recsdk_unique_sorted_static(const int64_t* ids, int64_t n, int key_bits, int64_t* unique_out,
                                           int64_t* inverse_out, int64_t* num_unique_out, void* stream)
{
    if (n < 0 || key_bits < 1 || key_bits > 64) return RECSDK_ERR_INVALID_ARG;
    if (n > recsdk::kUniqueStaticMaxN) return RECSDK_ERR_TOO_LARGE;  // beyond the built-in scratch: use recsdk_unique_sorted
    void* scratch = nullptr;
    const int rc = recsdk::unique_static_scratch(&scratch);
    if (rc != RECSDK_OK) return rc;
    return recsdk_unique_sorted(ids, n, key_bits, unique_out, inverse_out, num_unique_out, scratch,
                                recsdk::kUniqueStaticBytes, stream);
}
