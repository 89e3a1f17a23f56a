// Fused backward of the table-batched embedding op: gradient segment-sum over
// deduplicated rows + sparse Adagrad / Adam / SGD row update, in place.
//
// Plan (all on one stream, no host sync, no atomics on floats):
//   1. expand   : every index position p -> (key, val); key identifies the row
//                 (hash_size_cumsum[t] + idx, or inverse[p] + unique_offsets[t]),
//                 val packs (feature, sample) of the bag whose gradient row p takes.
//                 The kernel also counts the first sort pass's histogram.
//   2. sort     : stable LSD radix sort of the pairs by key (prims.cuh), per pass a
//                 scan and a scatter that counts the next pass's histogram.  Equal
//                 keys stay in ascending position order -> fixed reduction order.
//   3. runs     : head flags (computed inside the scan) -> run starts, U.
//   4. records  : one thread per unique row resolves everything the update needs
//                 (row address, first gradient row address, run, width) into a
//                 32-byte record; runs longer than C reserve chunk slots.
//   4b. partial : chunk sums of the long runs (keeps Zipf-hot rows off one warp).
//   5. update   : G lanes per unique row: record (fetched one row ahead) -> w / m1 /
//                 m2 / first gradient row in one wave of loads -> remaining gradient
//                 rows or chunk sums in order -> optimizer -> one write of w / m1 /
//                 m2.  Optionally (RECSDK_BWD_STAGED_UPDATE) the rows travel through
//                 a shared-memory ring filled by bulk asynchronous copies.
// Gradient rows may live in the sample owners' buffers on other GPUs
// (recsdk_sample_shards): the same kernels then read them over peer mappings.
// The float arithmetic uses explicit round-to-nearest intrinsics in the operand
// order of the reference kernels (ComputeAdagrad / ComputeAdam / ComputeSgd).
// Device side of the fused backward (kernels and the records they share); the host driver is tbe_backward.cu
// and the dedup exchange (exchange.cu) builds its two backward phases from the same kernels.
#pragma once
#include <limits.h>
#include <math.h>
#include <stdlib.h>

#ifdef RECSDK_EMULATE
#include "common.cuh"
#else
#include "prims.cuh"
#include "tma.cuh"
#endif

namespace recsdk {

constexpr int kChunk = 64;  // the only non-zero reduce_chunk supported
// Runs of more than kDirectMax positions are summed by the chunk-sum kernel (lanes resolve the gradient rows of a
// chunk in parallel and keep eight row loads in flight), the row-update kernel then reads one partial row per
// chunk; shorter runs are summed inside the row-update kernel.  This routing does not touch the arithmetic: a run
// of at most reduce_chunk positions is ONE chunk, and 0.0f + (its sequential sum) is that sum bit for bit (with
// reduce_chunk 0 a longer run is one chunk as a whole).  Measured on the benchmark step with thresholds 8, 16, 32
// and 64: within 2 % of each other, so the threshold is the chunk length.
constexpr int kDirectMax = kChunk;
// Slots of the partial buffer / chunk descriptors that n index positions can need.
static inline size_t chunk_slots_cap(int64_t n)
{
    const size_t m = static_cast<size_t>(n > 0 ? n : 1);
    return m / kChunk + m / (kDirectMax + 1) + 2;
}
// Chunks of a run of `len` positions that went through the chunk-sum kernel.
__host__ __device__ __forceinline__ int chunks_of_run(int len, int chunk) { return chunk > 0 ? (len + chunk - 1) / chunk : 1; }

struct BwdParams {
    const float* __restrict__ grad;
    float* __restrict__ w;
    float* __restrict__ m1;
    float* __restrict__ m2;
    const int64_t* __restrict__ wofs;
    const int32_t* __restrict__ dofs;
    const int64_t* __restrict__ cumsum;
    const int64_t* __restrict__ idx;
    const int64_t* __restrict__ offs;
    const int64_t* __restrict__ uid;
    const int64_t* __restrict__ uoff;
    const int64_t* __restrict__ uinv;
    int64_t T, B, N;
    int32_t total_D, max_D, mode, opt;
    int32_t bshift;  // val = (feature << bshift) | sample
    int32_t chunk;   // 0 or kChunk
    float lr, eps, beta1, beta2, beta2sqrt, max_grad;
    int32_t clip;
    int64_t w_numel;
    int64_t* status;
    int base_aligned;
    int64_t grad_numel;  // self-check builds only
    // plan arrays
    const uint32_t* __restrict__ vals;   // sorted
    const int* __restrict__ run_start;   // [U+1]
    const int2* __restrict__ chunk_desc;  // [chunks] {begin, end} sorted positions of each chunk
    float* __restrict__ partial;         // [chunks, max_D]
    const int64_t* __restrict__ counters;  // {U, total_chunks}
    recsdk_sample_shards sh;  // num_shards > 0: gradient rows are read from the sample owners' buffers
    int staged_update;        // use update_staged_kernel where the shape allows
    // kOptStore only (the dedup exchange's local phase): where the per-row sums go.  A record's row_off is then
    // (buffer number << kLocShardShift) | element offset inside that buffer; the buffers may be peer mappings.
    float* dst_ptrs[RECSDK_MAX_SHARDS];
    int32_t direct_max;  // runs longer than this go through the chunk-sum kernel (>= kDirectMax)
};

// Internal "optimizer" of the row-update kernels: no table is read, the summed gradient of the row is stored.
constexpr int kOptStore = 0;

// ---------------------------------------------------------------------------- 1. expand
// feature of index position p in NONE mode: last t with offsets[t*B] <= p
__device__ __forceinline__ int64_t feature_of_position(const int64_t* offs, int64_t T, int64_t B, int64_t p)
{
    int64_t lo = 0, hi = T - 1;
    while (lo < hi) {
        int64_t mid = (lo + hi + 1) >> 1;
        if (offs[mid * B] <= p) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// Features that share a table put gradient rows of different column offsets into ONE run, so the 128-bit path
// is taken only when the column offset of EVERY feature is a multiple of four floats.  Block 0 of the expand
// kernel checks that and raises counters[3] (zeroed before the plan) when one is not.
__device__ __forceinline__ void flag_unaligned_columns(const BwdParams& p, int64_t* counters_rw)
{
    if (blockIdx.x != 0) return;
    bool bad = false;
    for (int64_t t = threadIdx.x; t < p.T; t += blockDim.x) {
        const int32_t c = p.sh.num_shards > 0 ? p.sh.col_offsets[t] : p.dofs[t];
        bad = bad || ((c | (p.dofs[t + 1] - p.dofs[t])) & 3) != 0;
    }
    if (bad) atomicCAS(reinterpret_cast<unsigned long long*>(counters_rw + 3), 0ull, 1ull);
}

template <typename KeyT>
__global__ void __launch_bounds__(256) expand_pooled_kernel(BwdParams p, KeyT* __restrict__ keys,
                                                            uint32_t* __restrict__ vals, SortHistSink sink,
                                                            int64_t* __restrict__ counters_rw)
{
    flag_unaligned_columns(p, counters_rw);
    const int lane = threadIdx.x & 31;
    const int64_t num_bags = p.T * p.B;
    const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t bag0 = ((static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5) * 32; bag0 < num_bags;
         bag0 += warps_total * 32) {
        const int64_t bag = bag0 + lane;
        const int64_t start = bag < num_bags ? p.offs[bag] : INT64_MAX;  // lane l: first position of bag0+l
        const int64_t last_bag = (bag0 + 32 < num_bags) ? bag0 + 32 : num_bags;
        int64_t p0 = p.offs[bag0], p1 = p.offs[last_bag];
        if (p0 < 0 || p1 > p.N || p0 > p1) {
            // offsets that do not describe N positions (e.g. a buffer rewritten under a plan made ahead): never write
            // past the workspace
            set_status(p.status, RECSDK_ERR_INDEX_RANGE, p1, p.N);
            p0 = p0 < 0 ? 0 : (p0 > p.N ? p.N : p0);
            p1 = p1 > p.N ? p.N : (p1 < p0 ? p0 : p1);
        }
        const uint32_t f_l = bag < num_bags ? static_cast<uint32_t>(bag / p.B) : 0u;
        const uint32_t b_l = bag < num_bags ? static_cast<uint32_t>(bag - static_cast<int64_t>(f_l) * p.B) : 0u;
        for (int64_t base = p0; base < p1; base += 32) {
            const int64_t pos = base + lane;
            // largest j with start_j <= pos (bags with equal starts are empty; the last one owns pos)
            int j = 0;
#pragma unroll
            for (int step = 16; step >= 1; step >>= 1) {
                const int cand = j + step;
                const int64_t sc = __shfl_sync(kFullMask, start, cand & 31);
                if (cand < 32 && sc <= pos) j = cand;
            }
            const uint32_t f = __shfl_sync(kFullMask, f_l, j);
            const uint32_t b = __shfl_sync(kFullMask, b_l, j);
            int64_t key = 0;
            if (pos < p1) {
                key = p.uid != nullptr ? p.uinv[pos] + p.uoff[f] : p.cumsum[f] + p.idx[pos];
                keys[pos] = static_cast<KeyT>(key);
                vals[pos] = (f << p.bshift) | b;
            }
            sink.add_warp(pos < p1, static_cast<KeyT>(key), pos);
        }
    }
}

template <typename KeyT>
__global__ void __launch_bounds__(256) expand_nobag_kernel(BwdParams p, KeyT* __restrict__ keys,
                                                           uint32_t* __restrict__ vals, SortHistSink sink,
                                                           int64_t* __restrict__ counters_rw)
{
    flag_unaligned_columns(p, counters_rw);
    // warp-uniform trip count: the histogram sink is a warp-wide call
    for (int64_t pos0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + (threadIdx.x & ~31); pos0 < p.N;
         pos0 += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t pos = pos0 + (threadIdx.x & 31);
        int64_t key = 0;
        if (pos < p.N) {
            const int64_t f = feature_of_position(p.offs, p.T, p.B, pos);
            key = p.uid != nullptr ? p.uinv[pos] + p.uoff[f] : p.cumsum[f] + p.idx[pos];
            keys[pos] = static_cast<KeyT>(key);
            vals[pos] = static_cast<uint32_t>(pos);
        }
        sink.add_warp(pos < p.N, static_cast<KeyT>(key), pos);
    }
}

// ---------------------------------------------------------------------------- 3. runs
// Head flags are computed on the fly inside the scan; the scan's consumer writes
// run_start[] directly (no flag array, no run-id array).
template <typename KeyT>
struct HeadFlagIn {
    const KeyT* __restrict__ keys;
    __device__ __forceinline__ int operator()(int64_t i) const { return (i == 0 || keys[i] != keys[i - 1]) ? 1 : 0; }
};
struct RunStartOut {
    int* __restrict__ run_start;
    int64_t* __restrict__ counters;
    __device__ __forceinline__ void operator()(int64_t i, int flag, int incl, int64_t n) const
    {
        if (flag) run_start[incl - 1] = static_cast<int>(i);
        if (i == n - 1) {
            run_start[incl] = static_cast<int>(n);
            counters[0] = incl;  // U
        }
    }
};

// ---------------------------------------------------------------------------- gradient rows
// Where a gradient row lies, independent of the address of the gradient buffer (so that the plan can be made
// before the gradient exists): element offset inside its buffer in the low 56 bits, shard number above.
constexpr int kLocShardShift = 56;
__device__ __forceinline__ int64_t grad_row_loc(const BwdParams& p, uint32_t v);
__device__ __forceinline__ const float* grad_row_at(const BwdParams& p, int64_t loc)
{
    const int64_t off = loc & ((int64_t(1) << kLocShardShift) - 1);
    if (p.sh.num_shards == 0) return p.grad + off;
    return shard_base(p.sh, loc >> kLocShardShift) + off;
}

__device__ __forceinline__ float* dst_row_at(const BwdParams& p, int64_t loc)
{
    const int64_t s = loc >> kLocShardShift;
    float* q = p.dst_ptrs[0];
#pragma unroll
    for (int i = 1; i < RECSDK_MAX_SHARDS; ++i)
        if (s == i) q = p.dst_ptrs[i];
    return q + (loc & ((int64_t(1) << kLocShardShift) - 1));
}

struct GradRow {
    const float* ptr;
    float scale;  // MEAN: 1/len
};

__device__ __forceinline__ GradRow grad_row_of(const BwdParams& p, uint32_t v)
{
    GradRow g;
    g.scale = 1.0f;
    if (p.mode == RECSDK_POOL_NONE) {
        g.ptr = p.grad + static_cast<int64_t>(v) * p.max_D;
    } else {
        const uint32_t f = v >> p.bshift;
        const uint32_t b = v & ((1u << p.bshift) - 1u);
        if (p.sh.num_shards == 0) {
            g.ptr = p.grad + static_cast<int64_t>(b) * p.total_D + p.dofs[f];
        } else {
            const int64_t s = static_cast<int64_t>(b) / p.sh.shard_B;
            g.ptr = shard_base(p.sh, s) + (static_cast<int64_t>(b) - s * p.sh.shard_B) * p.sh.row_stride + p.sh.col_offsets[f];
        }
        if (p.mode == RECSDK_POOL_MEAN) {
            const int64_t bag = static_cast<int64_t>(f) * p.B + b;
            g.scale = __fdiv_rn(1.0f, static_cast<float>(p.offs[bag + 1] - p.offs[bag]));
        }
    }
    return g;
}

__device__ __forceinline__ int64_t grad_row_loc(const BwdParams& p, uint32_t v)
{
    if (p.mode == RECSDK_POOL_NONE) return static_cast<int64_t>(v) * p.max_D;
    const uint32_t f = v >> p.bshift;
    const uint32_t b = v & ((1u << p.bshift) - 1u);
    if (p.sh.num_shards == 0) return static_cast<int64_t>(b) * p.total_D + p.dofs[f];
    const int64_t s = static_cast<int64_t>(b) / p.sh.shard_B;
    return (s << kLocShardShift) |
           ((static_cast<int64_t>(b) - s * p.sh.shard_B) * p.sh.row_stride + p.sh.col_offsets[f]);
}

__device__ __forceinline__ float prep_grad(const BwdParams& p, float g, float scale)
{
    if (p.clip) g = g < -p.max_grad ? -p.max_grad : (g > p.max_grad ? p.max_grad : g);
    if (p.mode == RECSDK_POOL_MEAN) g = __fmul_rn(g, scale);
    return g;
}

// Sum of the gradient rows of sorted positions [s, e), columns (cb+lane+k*G) (in
// V::W-element vectors), in position order starting from zero.
template <typename V, int G, int K>
__device__ __forceinline__ void sum_grad_rows(const BwdParams& p, int s, int e, int cb, int lane, int nvec,
                                              typename V::T (&acc)[K])
{
    int i = s;
    for (; i + 4 <= e; i += 4) {
        GradRow g[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) g[j] = grad_row_of(p, p.vals[i + j]);
        typename V::T v[4][K];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int k = 0; k < K; ++k) {
                const int c = cb + lane + k * G;
                v[j][k] = c < nvec ? V::ld_stream(g[j].ptr + V::W * c) : V::zero();
            }
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int k = 0; k < K; ++k) {
                const float sc = g[j].scale;
                acc[k] = add4(acc[k], map4(v[j][k], [&](float x) { return prep_grad(p, x, sc); }));
            }
    }
    for (; i < e; ++i) {
        const GradRow g = grad_row_of(p, p.vals[i]);
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int c = cb + lane + k * G;
            typename V::T v = c < nvec ? V::ld_stream(g.ptr + V::W * c) : V::zero();
            const float sc = g.scale;
            acc[k] = add4(acc[k], map4(v, [&](float x) { return prep_grad(p, x, sc); }));
        }
    }
}

__device__ __forceinline__ void run_geometry(const BwdParams& p, uint32_t v0, int32_t& D, int64_t& wofs, int64_t& f)
{
    f = p.mode == RECSDK_POOL_NONE ? feature_of_position(p.offs, p.T, p.B, static_cast<int64_t>(v0))
                                   : static_cast<int64_t>(v0 >> p.bshift);
    D = p.dofs[f + 1] - p.dofs[f];
    wofs = p.wofs[f];
}

// 128-bit path for a run of feature f's table: needs every address the run touches 16-byte aligned, i.e. the
// table (wofs, D), the row pitch of the gradient, and the column offsets of ALL features (counters[3], see
// flag_unaligned_columns: a run can hold gradient rows of several features that share the table).
__device__ __forceinline__ bool vec_ok_for(const BwdParams& p, int64_t wofs, int32_t D, int64_t f)
{
    (void)f;
    if (!p.base_aligned || p.counters[3] != 0) return false;
    if (p.sh.num_shards > 0) return ((wofs | D | p.sh.row_stride | p.max_D) & 3) == 0;
    return ((wofs | D | p.total_D | p.max_D) & 3) == 0;
}

// ---------------------------------------------------------------------------- 4b. chunk sums
template <typename V, int G, int K>
__device__ __forceinline__ void partial_body(const BwdParams& p, int c, int lane)
{
    const int2 be = p.chunk_desc[c];
    const int p0 = be.x, e = be.y;
    int32_t D;
    int64_t wofs, f;
    run_geometry(p, p.vals[p0], D, wofs, f);
    const int nvec = D / V::W;
    float* out = p.partial + static_cast<int64_t>(c) * p.max_D;
    for (int cb = 0; cb < nvec; cb += G * K) {
        typename V::T acc[K];
#pragma unroll
        for (int k = 0; k < K; ++k) acc[k] = V::zero();
        sum_grad_rows<V, G, K>(p, p0, e, cb, lane, nvec, acc);
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int col = cb + lane + k * G;
            if (col < nvec) V::st(out + V::W * col, acc[k]);
        }
    }
}

template <int G>
__device__ __forceinline__ unsigned group_mask();

// Chunk sums.  One group per chunk (<= kChunk sorted positions of one long run):
// lanes resolve G gradient tags at a time to addresses in parallel, then the group
// walks them in order with several independent 128-bit loads in flight.
template <int G, int K>
__global__ void __launch_bounds__(256, 4) partial_kernel(BwdParams p)
{
    const int groups_per_block = blockDim.x / G;
    const int lane = threadIdx.x % G;
    const unsigned gmask = group_mask<G>();
    const int64_t total = p.counters[1];
    constexpr int kUnroll = 8 / K;
    for (int64_t c = static_cast<int64_t>(blockIdx.x) * groups_per_block + threadIdx.x / G; c < total;
         c += static_cast<int64_t>(gridDim.x) * groups_per_block) {
        int32_t D;
        int64_t wofs, f;
        const int2 be = p.chunk_desc[c];
        run_geometry(p, p.vals[be.x], D, wofs, f);
        if (vec_ok_for(p, wofs, D, f)) {
            const int nvec = D >> 2;
            float* out = p.partial + c * p.max_D;
            for (int cb = 0; cb < nvec; cb += G * K) {
                float4 acc[K];
#pragma unroll
                for (int k = 0; k < K; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int base = be.x; base < be.y; base += G) {
                    const int pos = base + lane;
                    GradRow g_l;
                    g_l.ptr = nullptr;
                    g_l.scale = 1.0f;
                    if (pos < be.y) g_l = grad_row_of(p, p.vals[pos]);
                    const int cnt = (be.y - base) < G ? (be.y - base) : G;
                    for (int jj0 = 0; jj0 < cnt; jj0 += kUnroll) {
                        float4 v[kUnroll][K];
                        float sc[kUnroll];
#pragma unroll
                        for (int u = 0; u < kUnroll; ++u) {
                            const int jj = jj0 + u;
                            const int src = jj < cnt ? jj : 0;
                            const float* gp = reinterpret_cast<const float*>(
                                __shfl_sync(gmask, reinterpret_cast<unsigned long long>(g_l.ptr), src, G));
                            sc[u] = __shfl_sync(gmask, g_l.scale, src, G);
#pragma unroll
                            for (int k = 0; k < K; ++k) {
                                const int col = cb + lane + k * G;
                                v[u][k] = (jj < cnt && col < nvec) ? ld_f4_stream(gp + 4 * col)
                                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < kUnroll; ++u)
                            if (jj0 + u < cnt) {
                                const float s = sc[u];
#pragma unroll
                                for (int k = 0; k < K; ++k)
                                    acc[k] = add4(acc[k], map4(v[u][k], [&](float x) { return prep_grad(p, x, s); }));
                            }
                    }
                }
#pragma unroll
                for (int k = 0; k < K; ++k) {
                    const int col = cb + lane + k * G;
                    if (col < nvec) st_f4(out + 4 * col, acc[k]);
                }
            }
        } else
            partial_body<V1, G, K>(p, static_cast<int>(c), lane);
    }
}

// ---------------------------------------------------------------------------- 5. optimizer math
// Operand order follows the reference vector kernels, one rounding per operation.
template <int OPT>
__device__ __forceinline__ void opt_update(const BwdParams& p, float g, float& w, float& m1, float& m2)
{
    if (OPT == RECSDK_OPT_ADAGRAD) {
        // ComputeAdagrad, backward_codegen_adagrad_unweighted_exact_kernel_unique.h:50-62
        const float g2 = __fmul_rn(g, g);
        const float s = __fadd_rn(m1, g2);
        const float den = __fadd_rn(__fsqrt_rn(s), p.eps);
        const float q = __fdiv_rn(p.lr, den);
        const float delta = __fmul_rn(__fmul_rn(q, g), -1.0f);
        w = __fadd_rn(w, delta);
        m1 = __fadd_rn(m1, g2);
    } else if (OPT == RECSDK_OPT_ADAM) {
        // ComputeAdam, backward_codegen_adam_unweighted_exact_kernel_unique.h:70-96
        const float omb1 = 1.0f - p.beta1, omb2 = 1.0f - p.beta2;
        const float step = __fmul_rn(-p.lr, p.beta2sqrt);
        const float nm1 = __fadd_rn(__fmul_rn(m1, p.beta1), __fmul_rn(g, omb1));
        const float nm2 = __fadd_rn(__fmul_rn(m2, p.beta2), __fmul_rn(__fmul_rn(g, g), omb2));
        const float den = __fadd_rn(__fsqrt_rn(nm2), p.eps);
        const float delta = __fmul_rn(__fdiv_rn(nm1, den), step);
        w = __fadd_rn(w, delta);
        m1 = nm1;
        m2 = nm2;
    } else {
        // ComputeSgd, backward_codegen_sgd_unweighted_exact_kernel.h:107-124
        w = __fadd_rn(w, __fmul_rn(g, -p.lr));
    }
}

template <int OPT>
__device__ __forceinline__ void opt_update_vec(const BwdParams& p, float4 g, float4& w, float4& m1, float4& m2)
{
    opt_update<OPT>(p, g.x, w.x, m1.x, m2.x);
    opt_update<OPT>(p, g.y, w.y, m1.y, m2.y);
    opt_update<OPT>(p, g.z, w.z, m1.z, m2.z);
    opt_update<OPT>(p, g.w, w.w, m1.w, m2.w);
}
template <int OPT>
__device__ __forceinline__ void opt_update_vec(const BwdParams& p, float g, float& w, float& m1, float& m2)
{
    opt_update<OPT>(p, g, w, m1, m2);
}

// ---------------------------------------------------------------------------- 4. per-run records
// Everything the row update needs to know about one unique row, resolved once by one
// thread per run (fully parallel), so that the update kernel starts its row loads after
// a single 32-byte read instead of a chain of five dependent loads.
struct __align__(16) RunMeta {
    int64_t row_off;     // element offset of the row in dev_weights; -1: out of range, skip
    int64_t g0_loc;      // location (grad_row_loc) of the run's first gradient row
    int32_t rs, len;     // sorted positions [rs, rs + len)
    int32_t D;           // row width in elements; kMetaVecBit set when the 128-bit path applies
    int32_t chunk_base;  // first slot of the run in the partial buffer (len > kChunk), else -1
};
constexpr int32_t kMetaVecBit = 1 << 30;

// A run longer than kDirectMax also reserves its chunk slots in the partial buffer -- ceil(len/reduce_chunk), or one
// for the whole run when reduce_chunk is 0 -- (atomic
// counter; slot numbers differ from launch to launch but a slot's content and the order in which
// a run's slots are summed do not) and describes each chunk as [begin, end) in sorted positions.
// counters[2] collects how many indices live in chunked runs (bandwidth accounting only).
template <typename KeyT>
__global__ void __launch_bounds__(256) run_meta_kernel(BwdParams p, const KeyT* __restrict__ keys,
                                                       int64_t* __restrict__ counters, RunMeta* __restrict__ meta,
                                                       int2* __restrict__ desc)
{
    const int64_t U = counters[0];
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; r < U;
         r += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int rs = p.run_start[r], re = p.run_start[r + 1];
        const int len = re - rs;
        const int64_t key = static_cast<int64_t>(keys[rs]);
        const uint32_t v0 = p.vals[rs];
        int32_t D;
        int64_t wofs, f;
        run_geometry(p, v0, D, wofs, f);
        const int64_t row = p.uid != nullptr ? p.uid[key] : key - p.cumsum[f];
        RunMeta m;
        m.row_off = wofs + row * D;
        if (p.w_numel > 0 && (row < 0 || m.row_off + D > p.w_numel)) {
            set_status(p.status, RECSDK_ERR_INDEX_RANGE, row, m.row_off);
            m.row_off = -1;
        }
        m.g0_loc = grad_row_loc(p, v0);
        m.rs = rs;
        m.len = len;
        m.D = D | (vec_ok_for(p, wofs, D, f) ? kMetaVecBit : 0);
        m.chunk_base = -1;
        if (len > p.direct_max) {
            const int c = chunks_of_run(len, p.chunk);
            const int step = p.chunk > 0 ? p.chunk : len;
            const int base = static_cast<int>(atomicAdd(reinterpret_cast<unsigned long long*>(counters + 1),
                                                        static_cast<unsigned long long>(c)));
            atomicAdd(reinterpret_cast<unsigned long long*>(counters + 2), static_cast<unsigned long long>(len));
            m.chunk_base = base;
            for (int k = 0; k < c; ++k) {
                const int b0 = rs + k * step;
                desc[base + k] = make_int2(b0, b0 + step < re ? b0 + step : re);
            }
        }
        meta[r] = m;
    }
}

// ---------------------------------------------------------------------------- 5b. row update
// Summed gradient of one unique row, columns (cb + lane + k*G), into `acc` (zero on entry): its chunk sums when
// the run was chunked, else its gradient rows in position order; `g0` is the already loaded first row of the
// run (first_direct).
template <typename V, int G, int K>
__device__ __forceinline__ void row_gradient(const BwdParams& p, const RunMeta& m, int cb, int lane, int nvec,
                                             bool first_direct, const typename V::T (&g0)[K], typename V::T (&acc)[K])
{
    const int rs = m.rs, re = m.rs + m.len;
    const bool chunked = m.chunk_base >= 0;
    if (chunked) {
        const int nc = chunks_of_run(m.len, p.chunk);
        int c = 0;
        for (; c + 4 <= nc; c += 4) {
            typename V::T v[4][K];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int k = 0; k < K; ++k) {
                    const int col = cb + lane + k * G;
                    v[u][k] = col < nvec ? V::ld(p.partial + static_cast<int64_t>(m.chunk_base + c + u) * p.max_D + V::W * col)
                                         : V::zero();
                }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int k = 0; k < K; ++k) acc[k] = add4(acc[k], v[u][k]);
        }
        for (; c < nc; ++c) {
#pragma unroll
            for (int k = 0; k < K; ++k) {
                const int col = cb + lane + k * G;
                if (col < nvec)
                    acc[k] = add4(acc[k], V::ld(p.partial + static_cast<int64_t>(m.chunk_base + c) * p.max_D + V::W * col));
            }
        }
    } else if (first_direct) {
#pragma unroll
        for (int k = 0; k < K; ++k) acc[k] = add4(acc[k], map4(g0[k], [&](float x) { return prep_grad(p, x, 1.0f); }));
        if (re > rs + 1) sum_grad_rows<V, G, K>(p, rs + 1, re, cb, lane, nvec, acc);
    } else {
        sum_grad_rows<V, G, K>(p, rs, re, cb, lane, nvec, acc);
    }
}

template <typename V, int G, int K, int OPT>
__device__ __forceinline__ void update_body(const BwdParams& p, const RunMeta& m, int lane, int32_t D)
{
    const int rs = m.rs, re = m.rs + m.len;
    const int nvec = D / V::W;
    const bool chunked = m.chunk_base >= 0;
    const int64_t row_off = m.row_off;
    // MEAN pooling scales every gradient row by its bag length: take the general path for all rows
    const bool first_direct = !chunked && p.mode != RECSDK_POOL_MEAN;
    const float* g0_row = grad_row_at(p, m.g0_loc);
    float* dst = OPT == kOptStore ? dst_row_at(p, row_off) : nullptr;
    for (int cb = 0; cb < nvec; cb += G * K) {
        typename V::T acc[K], w[K], m1[K], m2[K], g0[K];
        // all row loads of a short run are independent: issue them together
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int col = cb + lane + k * G;
            acc[k] = V::zero();
            w[k] = m1[k] = m2[k] = g0[k] = V::zero();
            if (col < nvec) {
                if (OPT != kOptStore) w[k] = V::ld(p.w + row_off + V::W * col);
                if (OPT == RECSDK_OPT_ADAGRAD || OPT == RECSDK_OPT_ADAM) m1[k] = V::ld(p.m1 + row_off + V::W * col);
                if (OPT == RECSDK_OPT_ADAM) m2[k] = V::ld(p.m2 + row_off + V::W * col);
                if (first_direct) g0[k] = V::ld_stream(g0_row + V::W * col);
            }
        }
        row_gradient<V, G, K>(p, m, cb, lane, nvec, first_direct, g0, acc);
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int col = cb + lane + k * G;
            if (col < nvec) {
                if (OPT == kOptStore) {
                    V::st(dst + V::W * col, acc[k]);
                    continue;
                }
                opt_update_vec<OPT>(p, acc[k], w[k], m1[k], m2[k]);
                V::st(p.w + row_off + V::W * col, w[k]);
                if (OPT == RECSDK_OPT_ADAGRAD || OPT == RECSDK_OPT_ADAM) V::st(p.m1 + row_off + V::W * col, m1[k]);
                if (OPT == RECSDK_OPT_ADAM) V::st(p.m2 + row_off + V::W * col, m2[k]);
            }
        }
    }
}

#ifndef RECSDK_EMULATE
// ---------------------------------------------------------------------------- 5c. row update, rows staged by TMA
// Same result as update_kernel<32, K, OPT>, different data movement: a warp owns a ring of kStages shared-memory
// stages and keeps the rows of its next kStages-1 unique rows in flight as bulk asynchronous copies (w, m1, m2
// and the run's first gradient row, one mbarrier per stage) while it updates the current one.  The copies hold no
// registers while they are in flight, so a block of 8 warps x 4 stages x 2 KB keeps ~50 KB of row data moving
// per block; three blocks fit an SM.  Lane s of the warp is the producer of stage s: it fetches the row record
// one iteration ahead, arms the barrier and issues the copies; all lanes consume.  Records of rows that cannot
// use 128-bit accesses are not staged and take the plain path.
constexpr int32_t kMetaStagedBit = 1 << 29;

template <int OPT>
struct StagedArrays {
    static constexpr int kState = OPT == RECSDK_OPT_ADAM ? 2 : (OPT == RECSDK_OPT_ADAGRAD ? 1 : 0);
    static constexpr int kCount = 1 + kState + 1;  // w, states, first gradient row
};

static inline size_t update_staged_smem_bytes(int warps, int stages, int arrays, int32_t max_D)
{
    return static_cast<size_t>(warps) * stages * (static_cast<size_t>(arrays) * max_D * 4 + sizeof(int4) * 2 + sizeof(uint64_t));
}

template <int OPT, int kStages>
__global__ void __launch_bounds__(256, 3) update_staged_kernel(BwdParams p, const RunMeta* __restrict__ meta)
{
    constexpr int NARR = StagedArrays<OPT>::kCount;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int W = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row_bytes_max = static_cast<size_t>(p.max_D) * 4;
    const size_t data_bytes = static_cast<size_t>(W) * kStages * NARR * row_bytes_max;
    unsigned char* data = smem_raw + static_cast<size_t>(warp) * kStages * NARR * row_bytes_max;
    int4* smeta = reinterpret_cast<int4*>(smem_raw + data_bytes) + static_cast<size_t>(warp) * kStages * 2;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + data_bytes + static_cast<size_t>(W) * kStages * 2 * sizeof(int4)) +
                     static_cast<size_t>(warp) * kStages;
    if (lane < kStages) mbar_init(&bars[lane], 1);
    mbar_fence_init();
    __syncwarp();

    const int64_t U = p.counters[0];
    const int64_t warps_total = static_cast<int64_t>(gridDim.x) * W;
    const int64_t wid = static_cast<int64_t>(blockIdx.x) * W + warp;
    const bool mean = p.mode == RECSDK_POOL_MEAN;

    // producer side, run by lane `s` alone: publish the record of the row that stage s will hold and start its copies
    auto arm = [&](int s, int4 lo, int4 hi) {
        const int64_t row_off = (static_cast<int64_t>(static_cast<uint32_t>(lo.y)) << 32) | static_cast<uint32_t>(lo.x);
        const int64_t g0_loc = (static_cast<int64_t>(static_cast<uint32_t>(lo.w)) << 32) | static_cast<uint32_t>(lo.z);
        const bool staged = row_off >= 0 && (hi.z & kMetaVecBit) != 0;
        if (staged) hi.z |= kMetaStagedBit;
        smeta[2 * s] = lo;
        smeta[2 * s + 1] = hi;
        if (!staged) return;
        const uint32_t rb = static_cast<uint32_t>(hi.z & (kMetaStagedBit - 1)) * 4u;
        const bool direct = hi.w < 0 && !mean;  // the first gradient row is used as it lies
        unsigned char* st = data + static_cast<size_t>(s) * NARR * row_bytes_max;
        mbar_expect_tx(&bars[s], (1u + StagedArrays<OPT>::kState + (direct ? 1u : 0u)) * rb);
        bulk_g2s(st, p.w + row_off, rb, &bars[s]);
        if (OPT != RECSDK_OPT_SGD) bulk_g2s(st + row_bytes_max, p.m1 + row_off, rb, &bars[s]);
        if (OPT == RECSDK_OPT_ADAM) bulk_g2s(st + 2 * row_bytes_max, p.m2 + row_off, rb, &bars[s]);
        if (direct) bulk_g2s(st + (NARR - 1) * row_bytes_max, grad_row_at(p, g0_loc), rb, &bars[s]);
    };

    // prologue: lane s fills stage s with the warp's s-th row
    if (lane < kStages) {
        const int64_t r = wid + static_cast<int64_t>(lane) * warps_total;
        if (r < U) arm(lane, __ldg(reinterpret_cast<const int4*>(meta + r)), __ldg(reinterpret_cast<const int4*>(meta + r) + 1));
    }
    __syncwarp();

    uint32_t phase = 0;  // bit s: parity the consumer waits for on stage s
    int s = 0;
    bool failed = false;
    for (int64_t r = wid; r < U; r += warps_total) {
        // the record of the row that will take this stage over, requested before the stage is consumed
        const int64_t rn = r + static_cast<int64_t>(kStages) * warps_total;
        int4 nlo = make_int4(0, 0, 0, 0), nhi = nlo;
        if (lane == s && rn < U) {
            nlo = __ldg(reinterpret_cast<const int4*>(meta + rn));
            nhi = __ldg(reinterpret_cast<const int4*>(meta + rn) + 1);
        }
        const int4 lo = smeta[2 * s], hi = smeta[2 * s + 1];
        RunMeta m;
        m.row_off = (static_cast<int64_t>(static_cast<uint32_t>(lo.y)) << 32) | static_cast<uint32_t>(lo.x);
        m.g0_loc = (static_cast<int64_t>(static_cast<uint32_t>(lo.w)) << 32) | static_cast<uint32_t>(lo.z);
        m.rs = hi.x;
        m.len = hi.y;
        m.D = hi.z;
        m.chunk_base = hi.w;
        const int32_t D = m.D & (kMetaStagedBit - 1);
        if (m.D & kMetaStagedBit) {
            const bool ok = mbar_wait_bounded(&bars[s], (phase >> s) & 1u);
            if (!__all_sync(kFullMask, ok)) {
                set_status(p.status, RECSDK_ERR_CUDA, -2, r);
                failed = true;
                break;
            }
            phase ^= 1u << s;
            const unsigned char* st = data + static_cast<size_t>(s) * NARR * row_bytes_max;
            const float4* sw = reinterpret_cast<const float4*>(st);
            const float4* sm1 = reinterpret_cast<const float4*>(st + row_bytes_max);
            const float4* sm2 = reinterpret_cast<const float4*>(st + 2 * row_bytes_max);
            const float4* sg = reinterpret_cast<const float4*>(st + (NARR - 1) * row_bytes_max);
            const int nvec = D >> 2;
            const bool first_direct = m.chunk_base < 0 && !mean;
            for (int cb = 0; cb < nvec; cb += 32) {
                const int col = cb + lane;
                const bool on = col < nvec;
                float4 acc[1], g0[1];
                acc[0] = make_float4(0.f, 0.f, 0.f, 0.f);
                g0[0] = (on && first_direct) ? sg[col] : make_float4(0.f, 0.f, 0.f, 0.f);
                float4 w = on ? sw[col] : make_float4(0.f, 0.f, 0.f, 0.f);
                float4 m1 = (on && OPT != RECSDK_OPT_SGD) ? sm1[col] : make_float4(0.f, 0.f, 0.f, 0.f);
                float4 m2 = (on && OPT == RECSDK_OPT_ADAM) ? sm2[col] : make_float4(0.f, 0.f, 0.f, 0.f);
                row_gradient<V4, 32, 1>(p, m, cb, lane, nvec, first_direct, g0, acc);
                if (on) {
                    opt_update_vec<OPT>(p, acc[0], w, m1, m2);
                    st_f4(p.w + m.row_off + 4 * col, w);
                    if (OPT != RECSDK_OPT_SGD) st_f4(p.m1 + m.row_off + 4 * col, m1);
                    if (OPT == RECSDK_OPT_ADAM) st_f4(p.m2 + m.row_off + 4 * col, m2);
                }
            }
        } else if (m.row_off >= 0) {
            update_body<V1, 32, 1, OPT>(p, m, lane, D);
        }
        __syncwarp();  // every lane is done with the stage before its producer refills it
        if (lane == s && rn < U) arm(s, nlo, nhi);
        __syncwarp();
        s = s + 1 == kStages ? 0 : s + 1;
    }
    if (failed) {
        // never expected: give the copies still in flight a bounded time to land before the block's shared
        // memory is released
        for (int q = 0; q < kStages; ++q) (void)mbar_wait_bounded(&bars[q], (phase >> q) & 1u, 1 << 12);
    }
}
#endif  // RECSDK_EMULATE

// G lanes per unique row; the row's record tells where everything is.  The record of the group's NEXT row is
// fetched before the current row is processed, so the record load is off the critical path of every row but
// the first.
template <int G, int K, int OPT>
__global__ void __launch_bounds__(256) update_kernel(BwdParams p, const RunMeta* __restrict__ meta)
{
    const int groups_per_block = blockDim.x / G;
    const int lane = threadIdx.x % G;
    const int64_t U = p.counters[0];
    const int64_t stride = static_cast<int64_t>(gridDim.x) * groups_per_block;
    int64_t r = static_cast<int64_t>(blockIdx.x) * groups_per_block + threadIdx.x / G;
    int4 lo = make_int4(0, 0, 0, 0), hi = lo;
    if (r < U) {
        lo = __ldg(reinterpret_cast<const int4*>(meta + r));
        hi = __ldg(reinterpret_cast<const int4*>(meta + r) + 1);
    }
    while (r < U) {
        const int64_t rn = r + stride;
        int4 nlo = make_int4(0, 0, 0, 0), nhi = nlo;
        if (rn < U) {
            nlo = __ldg(reinterpret_cast<const int4*>(meta + rn));
            nhi = __ldg(reinterpret_cast<const int4*>(meta + rn) + 1);
        }
        RunMeta m;
        m.row_off = (static_cast<int64_t>(static_cast<uint32_t>(lo.y)) << 32) | static_cast<uint32_t>(lo.x);
        m.g0_loc = (static_cast<int64_t>(static_cast<uint32_t>(lo.w)) << 32) | static_cast<uint32_t>(lo.z);
        m.rs = hi.x;
        m.len = hi.y;
        m.D = hi.z;
        m.chunk_base = hi.w;
        if (m.row_off >= 0) {
            const int32_t D = m.D & (kMetaVecBit - 1);
            if (m.D & kMetaVecBit)
                update_body<V4, G, K, OPT>(p, m, lane, D);
            else
                update_body<V1, G, K, OPT>(p, m, lane, D);
        }
        lo = nlo;
        hi = nhi;
        r = rn;
    }
}

template <int G>
__device__ __forceinline__ unsigned group_mask()
{
    if (G == 32) return kFullMask;
    return ((1u << G) - 1u) << ((threadIdx.x & 31) / G * G);
}

}  // namespace recsdk
