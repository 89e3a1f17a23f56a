// Host-side SIMT emulation for CPU tests of the CUDA kernels' control flow and index arithmetic.
// Every CUDA thread of a block is a std::thread; warp collectives (__shfl_sync, __all_sync) are rendezvous
// points keyed by (warp, mask).  A collective that not all lanes of its mask reach, or that lanes reach with
// different operations, aborts with a message -- on a GPU that is undefined behaviour (it once showed up as an
// illegal memory access), here it is a test failure.  Only what the emulated kernels use is provided.
#pragma once
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <thread>
#include <vector>
#define RECSDK_EMULATE 1
#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __restrict__
#define __launch_bounds__(...)
#define __align__(n) alignas(n)
struct float4 { float x, y, z, w; };
struct int2 { int x, y; };
struct alignas(16) int4 { int x, y, z, w; };
static inline int4 make_int4(int a, int b, int c, int d) { return int4{a, b, c, d}; }
static inline float4 make_float4(float a, float b, float c, float d) { return float4{a, b, c, d}; }
static inline int2 make_int2(int a, int b) { return int2{a, b}; }
struct dim3e { unsigned x = 1, y = 1, z = 1; };
static thread_local dim3e threadIdx, blockIdx;
static dim3e blockDim, gridDim;
typedef int cudaError_t;
typedef void* cudaStream_t;
static inline float __fadd_rn(float a, float b) { return a + b; }
static inline float __fmul_rn(float a, float b) { return a * b; }
static inline float __fdiv_rn(float a, float b) { return a / b; }
static inline float __fsqrt_rn(float a) { return sqrtf(a); }
template <typename T> static inline T __ldcs(const T* p) { return *p; }
template <typename T> static inline T __ldg(const T* p) { return *p; }
template <typename T> static inline void __stcs(T* p, T v) { *p = v; }
static std::mutex g_atomic_mu;
static inline unsigned long long atomicCAS(unsigned long long* p, unsigned long long cmp, unsigned long long v)
{ std::lock_guard<std::mutex> l(g_atomic_mu); unsigned long long o = *p; if (o == cmp) *p = v; return o; }
static inline unsigned long long atomicAdd(unsigned long long* p, unsigned long long v)
{ std::lock_guard<std::mutex> l(g_atomic_mu); unsigned long long o = *p; *p = o + v; return o; }

// ---- collective rendezvous keyed by (warp, mask)
struct Rendezvous {
    std::mutex mu; std::condition_variable cv;
    int arrived = 0, generation = 0, departed = 0;
    unsigned long long vals[32]; int preds[32];
    unsigned long long out_vals[32]; int out_all = 0;
    int tag = 0;
};
static std::mutex g_rv_mu;
static std::map<std::pair<int, unsigned>, Rendezvous*> g_rv;
static Rendezvous* rv_for(int warp, unsigned mask)
{ std::lock_guard<std::mutex> l(g_rv_mu); auto& r = g_rv[{warp, mask}]; if (!r) r = new Rendezvous(); return r; }
// every lane in mask calls with its value; returns array snapshot
static inline void collective(unsigned mask, unsigned long long my, int pred, int tag, unsigned long long* snap, int* all_out)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (!((mask >> lane) & 1u)) { fprintf(stderr, "EMU: lane %d not in its own mask %08x\n", lane, mask); abort(); }
    Rendezvous* r = rv_for(warp, mask);
    const int n = __builtin_popcount(mask);
    std::unique_lock<std::mutex> l(r->mu);
    // wait for previous round to fully drain
    r->cv.wait(l, [&] { return r->departed == 0 || r->arrived > 0 || true; });
    const int gen = r->generation;
    if (r->arrived == 0) r->tag = tag;
    else if (r->tag != tag) { fprintf(stderr, "EMU: divergent collective (tag %d vs %d) mask %08x lane %d\n", r->tag, tag, mask, lane); abort(); }
    r->vals[lane] = my; r->preds[lane] = pred; r->arrived++;
    if (r->arrived == n) {
        int all = 1;
        for (int i = 0; i < 32; ++i) if ((mask >> i) & 1u) { r->out_vals[i] = r->vals[i]; all &= (r->preds[i] != 0); }
        r->out_all = all; r->arrived = 0; r->generation++; r->cv.notify_all();
    } else {
        if (!r->cv.wait_for(l, std::chrono::seconds(10), [&] { return r->generation != gen; })) {
            fprintf(stderr, "EMU: collective timeout: lane %d mask %08x tag %d (non-uniform control flow?)\n", lane, mask, tag); abort();
        }
    }
    memcpy(snap, r->out_vals, sizeof(r->out_vals)); *all_out = r->out_all;
}
template <typename T>
static inline T __shfl_sync(unsigned mask, T v, int src, int width = 32)
{
    static_assert(sizeof(T) <= 8, "");
    unsigned long long raw = 0; memcpy(&raw, &v, sizeof(T));
    unsigned long long snap[32]; int all;
    collective(mask, raw, 1, 1, snap, &all);
    const int lane = threadIdx.x & 31;
    const int s = (lane & ~(width - 1)) | (src & (width - 1));
    if (!((mask >> s) & 1u)) { fprintf(stderr, "EMU: shfl source lane %d not in mask %08x (lane %d src %d width %d)\n", s, mask, lane, src, width); abort(); }
    T out; memcpy(&out, &snap[s], sizeof(T)); return out;
}
static inline int __all_sync(unsigned mask, int pred)
{ unsigned long long snap[32]; int all; collective(mask, 0, pred, 2, snap, &all); return all; }
