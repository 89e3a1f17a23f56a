// Shared device/host helpers for the recsdk_b200 kernels (sm_100a).
#pragma once
#ifndef RECSDK_EMULATE  // host-side SIMT emulation builds provide their own shim
#include <cuda_runtime.h>
#endif
#include <stdint.h>

#include "recsdk_b200.h"

namespace recsdk {

constexpr int kWarp = 32;
constexpr unsigned kFullMask = 0xffffffffu;

// Number of SMs of the current device (148 on a B200); grids of persistent / grid-stride kernels are sized as a
// multiple of it.  Queried once per device.
constexpr int kMaxDevices = 64;
#ifdef RECSDK_EMULATE
static inline int num_sms() { return 148; }
#else
static inline int current_device_index()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
    return dev;
}
static inline int num_sms()
{
    static int cached[kMaxDevices] = {0};
    const int dev = current_device_index();
    int n = cached[dev];
    if (n <= 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = 148;
        }
        cached[dev] = n;  // racing threads store the same value
    }
    return n;
}
// Opt-in to more than 48 KB of dynamic shared memory for `func`, once per device (the attribute is per device).
// `done` is a per-kernel-instantiation table of kMaxDevices flags.
template <typename F>
static inline bool smem_optin(F func, int bytes, bool* done)
{
    const int dev = current_device_index();
    if (done[dev]) return true;
    if (cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    done[dev] = true;
    return true;
}
#endif

#define RECSDK_CUDA_CHECK_LAUNCH()                      \
    do {                                                \
        cudaError_t e__ = cudaPeekAtLastError();        \
        if (e__ != cudaSuccess) return RECSDK_ERR_CUDA; \
    } while (0)

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

static inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

// Carves a caller-provided workspace into 256-byte aligned pieces.
struct WorkspaceCarver {
    char* base;
    size_t off = 0;
    explicit WorkspaceCarver(void* p) : base(static_cast<char*>(p)) {}
    template <typename T>
    T* take(size_t count)
    {
        T* r = reinterpret_cast<T*>(base + off);
        off += align_up(count * sizeof(T));
        return r;
    }
    size_t used() const { return off; }
};

// Host-side validation of a sample-sharded matrix description for B samples.
static inline bool sample_shards_valid(const recsdk_sample_shards& sh, int64_t B)
{
    if (sh.num_shards < 1 || sh.num_shards > RECSDK_MAX_SHARDS || sh.shard_B <= 0 || sh.row_stride <= 0 ||
        sh.col_offsets == nullptr || static_cast<int64_t>(sh.num_shards) * sh.shard_B != B)
        return false;
    for (int s = 0; s < sh.num_shards; ++s)
        if (sh.ptrs[s] == nullptr) return false;
    return true;
}

// Base address of shard s.  The table sits in the kernel's parameter space; a chain of selects over constant
// indices keeps it there (indexing it with a run-time value would make every thread copy it to local memory).
__device__ __forceinline__ float* shard_base(const recsdk_sample_shards& sh, int64_t s)
{
    float* q = sh.ptrs[0];
#pragma unroll
    for (int i = 1; i < RECSDK_MAX_SHARDS; ++i)
        if (s == i) q = sh.ptrs[i];
    return q;
}

// Grid for a grid-stride kernel over `work` items handled `per_block` at a time.
static inline int grid_for(int64_t work, int64_t per_block, int max_blocks_per_sm = 16)
{
    int64_t b = ceil_div(work, per_block);
    int64_t cap = static_cast<int64_t>(num_sms()) * max_blocks_per_sm;
    if (b < 1) b = 1;
    return static_cast<int>(b < cap ? b : cap);
}

// First error wins; detail words help the host build the message the reference
// would have raised.
__device__ __forceinline__ void set_status(int64_t* st, int code, int64_t d0 = 0, int64_t d1 = 0)
{
    if (st == nullptr) return;
    unsigned long long* p = reinterpret_cast<unsigned long long*>(st);
    if (atomicCAS(p, 0ull, static_cast<unsigned long long>(code)) == 0ull) {
        st[1] = d0;
        st[2] = d1;
    }
}

__device__ __forceinline__ unsigned lanemask_lt()
{
#ifdef RECSDK_EMULATE
    return (1u << (threadIdx.x & 31)) - 1u;
#else
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
#endif
}

// 128-bit global accesses.  Table rows are read through the normal (L2
// allocating) path: Zipf-hot rows are re-used from L2.  Streams that are
// touched once (pooled output, gradient rows) use the streaming hints.
__device__ __forceinline__ float4 ld_f4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st_f4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float4 ld_f4_stream(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void st_f4_stream(float* p, float4 v) { __stcs(reinterpret_cast<float4*>(p), v); }

// Vector-width abstraction: V4 moves float4, V1 moves float (tables whose dims
// or offsets are not multiples of 4 elements).
struct V4 {
    using T = float4;
    static constexpr int W = 4;
    __device__ static T zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ static T ld(const float* p) { return ld_f4(p); }
    __device__ static T ld_stream(const float* p) { return ld_f4_stream(p); }
    __device__ static void st(float* p, T v) { st_f4(p, v); }
    __device__ static void st_stream(float* p, T v) { st_f4_stream(p, v); }
};
struct V1 {
    using T = float;
    static constexpr int W = 1;
    __device__ static T zero() { return 0.f; }
    __device__ static T ld(const float* p) { return *p; }
    __device__ static T ld_stream(const float* p) { return __ldcs(p); }
    __device__ static void st(float* p, T v) { *p = v; }
    __device__ static void st_stream(float* p, T v) { __stcs(p, v); }
};

// Element-wise float ops with explicit round-to-nearest intrinsics: never
// contracted into FMA, so results match a CPU loop compiled with
// -ffp-contract=off bit for bit.
__device__ __forceinline__ float4 add4(float4 a, float4 b)
{
    return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}
__device__ __forceinline__ float4 mul4s(float4 a, float s)
{
    return make_float4(__fmul_rn(a.x, s), __fmul_rn(a.y, s), __fmul_rn(a.z, s), __fmul_rn(a.w, s));
}
__device__ __forceinline__ float add4(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float mul4s(float a, float s) { return __fmul_rn(a, s); }

template <typename F>
__device__ __forceinline__ float4 map4(float4 a, F f)
{
    return make_float4(f(a.x), f(a.y), f(a.z), f(a.w));
}
template <typename F>
__device__ __forceinline__ float map4(float a, F f)
{
    return f(a);
}

// Smallest power of two >= x (x >= 1), capped at 32: lanes that cooperate on one row.
static inline int group_lanes_for(int vec_per_row)
{
    int g = 1;
    while (g < vec_per_row && g < 32) g <<= 1;
    return g;
}

__host__ __device__ static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace recsdk
