// Dedup exchange: the sharded lookup of one box, driven from the device over peer mappings.
//
// Per rank and step (recsdk_b200.h describes the protocol):
//   forward         expand (id -> linear row key) -> stable radix sort of (key, position) -> runs: distinct keys,
//                   inverse, per-run starts (kept as the backward's plan) -> route + pull: owner segments of the
//                   sorted distinct keys, count and local row numbers stored into each owner's inbox, the rows
//                   loaded straight from the owners' tables -> pooled gather over the fetched rows.
//   backward_local  per distinct row: records -> chunk sums of long runs -> sum, stored into the owner's inbox.
//   backward_owner  inbox (counts read on the device) -> compact (local row, source slot) pairs -> sort -> runs ->
//                   records -> row update; contributions of one row are added in source-rank order.
// Nothing here waits on another GPU, allocates or reads back to the host; peer memory is touched with plain
// 128-bit / 64-bit loads and stores.  The backward phases are built from the kernels of the fused backward
// (tbe_backward.cuh): same records, same chunking, same arithmetic.
#include "tbe_backward.cuh"

namespace recsdk {

template <typename P>
struct PeerTable {
    P ptrs[RECSDK_MAX_SHARDS];
};

// ptrs[r] for a run-time r without indexing the parameter space dynamically (that would spill the table to
// local memory in every thread)
template <typename P>
__device__ __forceinline__ P pick(const PeerTable<P>& t, int r)
{
    P q = t.ptrs[0];
#pragma unroll
    for (int i = 1; i < RECSDK_MAX_SHARDS; ++i)
        if (r == i) q = t.ptrs[i];
    return q;
}

struct XchgParams {
    int32_t W, me, partition, D;
    int64_t F, B, N, cap;
    const int64_t* __restrict__ part_base;
    const int64_t* __restrict__ rank_base;
    const int64_t* __restrict__ table_rows;
    int64_t* status;
    int32_t mode, bshift;
    int32_t one_hot;  // the caller states that every bag holds exactly one id (checked by the expand kernel)
};

__device__ __forceinline__ int64_t xchg_key(const XchgParams& x, int64_t f, int64_t id)
{
    if (id < 0 || (x.table_rows != nullptr && id >= x.table_rows[f])) {
        set_status(x.status, RECSDK_ERR_INDEX_RANGE, id, f);
        id = 0;
    }
    if (x.partition == RECSDK_XCHG_TABLE_WISE) return x.part_base[f] + id;
    const int64_t r = id % x.W;
    return x.part_base[r * x.F + f] + id / x.W;
}

// ---------------------------------------------------------------------------- forward 1: expand
// Position -> (linear row key, position); the (feature, sample) tag of every position is kept aside for the
// backward.  Block 0 also lays down the two small layout arrays the pooled gather over the fetched rows needs.
template <typename KeyT>
__global__ void __launch_bounds__(256) xchg_expand_pooled_kernel(XchgParams x, const int64_t* __restrict__ idx,
                                                                 const int64_t* __restrict__ offs,
                                                                 KeyT* __restrict__ keys, uint32_t* __restrict__ vals,
                                                                 uint32_t* __restrict__ tag_of_pos, SortHistSink sink,
                                                                 int64_t* __restrict__ zeros_F,
                                                                 int32_t* __restrict__ dofs)
{
    if (blockIdx.x == 0)
        for (int64_t f = threadIdx.x; f <= x.F; f += blockDim.x) {
            if (f < x.F) zeros_F[f] = 0;
            dofs[f] = static_cast<int32_t>(f * x.D);
        }
    const int lane = threadIdx.x & 31;
    const int64_t num_bags = x.F * x.B;
    const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t bag0 = ((static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5) * 32; bag0 < num_bags;
         bag0 += warps_total * 32) {
        const int64_t bag = bag0 + lane;
        const int64_t start = bag < num_bags ? offs[bag] : INT64_MAX;
        const int64_t last_bag = (bag0 + 32 < num_bags) ? bag0 + 32 : num_bags;
        const int64_t p0 = offs[bag0], p1 = offs[last_bag];
        const uint32_t f_l = bag < num_bags ? static_cast<uint32_t>(bag / x.B) : 0u;
        const uint32_t b_l = bag < num_bags ? static_cast<uint32_t>(bag - static_cast<int64_t>(f_l) * x.B) : 0u;
        if (x.one_hot && bag < num_bags && offs[bag + 1] - start != 1)
            set_status(x.status, RECSDK_ERR_INVALID_ARG, bag, offs[bag + 1] - start);  // not one id per bag
        for (int64_t base = p0; base < p1; base += 32) {
            const int64_t pos = base + lane;
            int j = 0;  // largest j with start_j <= pos (empty bags share a start; the last one owns pos)
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
                key = xchg_key(x, f, idx[pos]);
                keys[pos] = static_cast<KeyT>(key);
                vals[pos] = static_cast<uint32_t>(pos);
                if (!x.one_hot) tag_of_pos[pos] = (f << x.bshift) | b;
            }
            sink.add_warp(pos < p1, static_cast<KeyT>(key), pos);
        }
    }
}

template <typename KeyT>
__global__ void __launch_bounds__(256) xchg_expand_nobag_kernel(XchgParams x, const int64_t* __restrict__ idx,
                                                                const int64_t* __restrict__ offs,
                                                                KeyT* __restrict__ keys, uint32_t* __restrict__ vals,
                                                                SortHistSink sink, int64_t* __restrict__ zeros_F,
                                                                int32_t* __restrict__ dofs)
{
    if (blockIdx.x == 0)
        for (int64_t f = threadIdx.x; f <= x.F; f += blockDim.x) {
            if (f < x.F) zeros_F[f] = 0;
            dofs[f] = static_cast<int32_t>(f * x.D);
        }
    for (int64_t pos0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + (threadIdx.x & ~31); pos0 < x.N;
         pos0 += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t pos = pos0 + (threadIdx.x & 31);
        int64_t key = 0;
        if (pos < x.N) {
            key = xchg_key(x, feature_of_position(offs, x.F, x.B, pos), idx[pos]);
            keys[pos] = static_cast<KeyT>(key);
            vals[pos] = static_cast<uint32_t>(pos);
        }
        sink.add_warp(pos < x.N, static_cast<KeyT>(key), pos);
    }
}

// ---------------------------------------------------------------------------- forward 3: runs
// Consumer of the head-flag scan over the sorted keys: run starts, distinct keys, inverse, and the backward's tags
// in sorted order.
template <typename KeyT>
struct XchgRunOut {
    const KeyT* __restrict__ keys;
    const uint32_t* __restrict__ pos_sorted;
    const uint32_t* __restrict__ tag_of_pos;  // nullptr (NONE pooling): the tag is the position
    int* __restrict__ run_start;
    int64_t* __restrict__ uniq;
    int64_t* __restrict__ inverse;
    uint32_t* __restrict__ tags_sorted;
    int64_t* __restrict__ counters;
    int64_t one_hot_B;  // > 0: one id per bag, position p is bag (p / B, p % B); no inverse is needed
    int32_t bshift;
    __device__ __forceinline__ void operator()(int64_t i, int flag, int incl, int64_t n) const
    {
        const int u = incl - 1;
        const uint32_t pos = pos_sorted[i];
        if (flag) {
            run_start[u] = static_cast<int>(i);
            uniq[u] = static_cast<int64_t>(keys[i]);
        }
        if (one_hot_B > 0) {
            const uint32_t f = static_cast<uint32_t>(pos / one_hot_B);
            tags_sorted[i] = (f << bshift) | static_cast<uint32_t>(pos - f * one_hot_B);
        } else {
            inverse[pos] = u;
            tags_sorted[i] = tag_of_pos != nullptr ? tag_of_pos[pos] : pos;
        }
        if (i == n - 1) {
            run_start[incl] = static_cast<int>(n);
            counters[0] = incl;
        }
    }
};

// ---------------------------------------------------------------------------- forward 4: route + pull
// first u in [0, U) with uniq[u] >= bound
__device__ __forceinline__ int64_t lower_bound_i64(const int64_t* __restrict__ a, int64_t n, int64_t bound)
{
    int64_t lo = 0, hi = n;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (a[mid] < bound) lo = mid + 1; else hi = mid;
    }
    return lo;
}

__device__ __forceinline__ int owner_of(const int64_t* seg, int W, int64_t u)
{
    int r = 0;
    for (int i = 1; i < W; ++i)
        if (seg[i] <= u) r = i;
    return r;
}

// The sorted distinct keys are grouped by owner.  One warp finds the segment bounds (W+1 binary searches),
// publishes them and stores this rank's counts into the owners' inboxes.
__global__ void __launch_bounds__(32) xchg_seg_kernel(XchgParams x, const int64_t* __restrict__ uniq,
                                                      const int64_t* __restrict__ counters,
                                                      int64_t* __restrict__ seg_out, PeerTable<int64_t*> inbox_counts)
{
    __shared__ int64_t seg[RECSDK_MAX_SHARDS + 1];
    const int64_t U = counters[0];
    const int t = threadIdx.x;
    if (t <= x.W) seg[t] = t == x.W ? U : lower_bound_i64(uniq, U, x.rank_base[t]);
    __syncwarp();
    if (t <= x.W) seg_out[t] = seg[t];
    if (t < x.W) {
        int64_t cnt = seg[t + 1] - seg[t];
        if (cnt > x.cap) {
            set_status(x.status, RECSDK_ERR_TOO_LARGE, cnt, x.cap);
            cnt = x.cap;
        }
        pick(inbox_counts, t)[x.me] = cnt;
    }
}

// Where distinct row u comes from: owner, row address in the owner's table; lane 0 of the group also stores the
// local row number into the owner's inbox.
struct PullSrc {
    const float* ptr;
};
__device__ __forceinline__ PullSrc xchg_resolve(const XchgParams& x, const int64_t* seg, const int64_t* rbase,
                                                const int64_t* __restrict__ uniq, int64_t u, bool store_id,
                                                const PeerTable<const float*>& tables,
                                                const PeerTable<int64_t*>& inbox_ids)
{
    PullSrc r;
    const int o = owner_of(seg, x.W, u);
    const int64_t lrow = uniq[u] - rbase[o];
    const int64_t slot = u - seg[o];
    r.ptr = nullptr;
    if (slot < x.cap) {
        if (store_id) pick(inbox_ids, o)[static_cast<int64_t>(x.me) * x.cap + slot] = lrow;
        r.ptr = pick(tables, o) + lrow * x.D;
    }
    return r;
}

// General lookups: G lanes per distinct row copy it from the owner's table into `fetched` (the pooled gather
// then runs over `fetched`), kRows rows in flight per group.
template <int G>
__global__ void __launch_bounds__(256) xchg_pull_kernel(XchgParams x, const int64_t* __restrict__ uniq,
                                                        const int64_t* __restrict__ counters,
                                                        const int64_t* __restrict__ seg_g, float* __restrict__ fetched,
                                                        PeerTable<const float*> tables, PeerTable<int64_t*> inbox_ids)
{
    constexpr int kRows = 4;
    __shared__ int64_t seg[RECSDK_MAX_SHARDS + 1];
    __shared__ int64_t rbase[RECSDK_MAX_SHARDS + 1];
    const int64_t U = counters[0];
    if (threadIdx.x <= x.W) {
        rbase[threadIdx.x] = x.rank_base[threadIdx.x];
        seg[threadIdx.x] = seg_g[threadIdx.x];
    }
    __syncthreads();
    const int lane = threadIdx.x % G;
    const int nvec = x.D >> 2;
    const int64_t groups_total = static_cast<int64_t>(gridDim.x) * (blockDim.x / G);
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * (blockDim.x / G) + threadIdx.x / G;
    for (int64_t u0 = gid * kRows; u0 < U; u0 += groups_total * kRows) {
        const float* src[kRows];
#pragma unroll
        for (int j = 0; j < kRows; ++j)
            src[j] = u0 + j < U ? xchg_resolve(x, seg, rbase, uniq, u0 + j, lane == 0, tables, inbox_ids).ptr : nullptr;
        for (int c = lane; c < nvec; c += G) {
            float4 v[kRows];
#pragma unroll
            for (int j = 0; j < kRows; ++j) v[j] = src[j] != nullptr ? ld_f4(src[j] + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < kRows; ++j)
                if (u0 + j < U) st_f4(fetched + (u0 + j) * x.D + 4 * c, v[j]);
        }
    }
}

// One id per bag (SUM or MEAN pooling): the pooled row of a bag IS the row of its id, so each distinct row is
// loaded once from its owner and stored to every bag of its run -- no intermediate copy, no second pass over the
// rows.  Work items: the distinct rows with runs of at most kDirectMax positions (G lanes each, kRows rows in flight),
// then the chunks of the longer runs (their row is loaded once per chunk).  A bag's row is written as 0.0f + x, the
// value a sum over the bag's single row gives.
template <int G>
__global__ void __launch_bounds__(256) xchg_pull_scatter_kernel(XchgParams x, const int64_t* __restrict__ uniq,
                                                                const int64_t* __restrict__ counters,
                                                                const int64_t* __restrict__ seg_g,
                                                                const RunMeta* __restrict__ meta,
                                                                const int2* __restrict__ desc,
                                                                const int* __restrict__ chunk_row,
                                                                const uint32_t* __restrict__ tags,
                                                                float* __restrict__ out, PeerTable<const float*> tables,
                                                                PeerTable<int64_t*> inbox_ids)
{
    constexpr int kRows = 4;
    __shared__ int64_t seg[RECSDK_MAX_SHARDS + 1];
    __shared__ int64_t rbase[RECSDK_MAX_SHARDS + 1];
    const int64_t U = counters[0];
    const int64_t n_chunks = counters[1];
    if (threadIdx.x <= x.W) {
        rbase[threadIdx.x] = x.rank_base[threadIdx.x];
        seg[threadIdx.x] = seg_g[threadIdx.x];
    }
    __syncthreads();
    const int lane = threadIdx.x % G;
    const int nvec = x.D >> 2;
    const int64_t total_D = x.F * x.D;
    const uint32_t bmask = (1u << x.bshift) - 1u;
    const int64_t groups_total = static_cast<int64_t>(gridDim.x) * (blockDim.x / G);
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * (blockDim.x / G) + threadIdx.x / G;
    auto out_row = [&](uint32_t tag) { return out + static_cast<int64_t>(tag & bmask) * total_D + static_cast<int64_t>(tag >> x.bshift) * x.D; };
    for (int64_t u0 = gid * kRows; u0 < U; u0 += groups_total * kRows) {
        const float* src[kRows];
        int rs[kRows], len[kRows];
#pragma unroll
        for (int j = 0; j < kRows; ++j) {
            src[j] = nullptr;
            rs[j] = len[j] = 0;
            if (u0 + j < U) {
                src[j] = xchg_resolve(x, seg, rbase, uniq, u0 + j, lane == 0, tables, inbox_ids).ptr;
                const int4 hi = __ldg(reinterpret_cast<const int4*>(meta + u0 + j) + 1);
                rs[j] = hi.x;
                len[j] = hi.w >= 0 ? 0 : hi.y;  // chunked runs are written by the chunk items below
            }
        }
        for (int c = lane; c < nvec; c += G) {
            float4 v[kRows];
#pragma unroll
            for (int j = 0; j < kRows; ++j) v[j] = src[j] != nullptr ? ld_f4(src[j] + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < kRows; ++j) {
                const float4 r = add4(make_float4(0.f, 0.f, 0.f, 0.f), v[j]);
                for (int i = 0; i < len[j]; ++i) st_f4_stream(out_row(__ldg(tags + rs[j] + i)) + 4 * c, r);
            }
        }
    }
    for (int64_t ch = gid; ch < n_chunks; ch += groups_total) {
        const int2 be = desc[ch];
        const float* src = xchg_resolve(x, seg, rbase, uniq, chunk_row[ch], false, tables, inbox_ids).ptr;
        for (int c = lane; c < nvec; c += G) {
            const float4 r = add4(make_float4(0.f, 0.f, 0.f, 0.f), src != nullptr ? ld_f4(src + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f));
            for (int i = be.x; i < be.y; ++i) st_f4_stream(out_row(__ldg(tags + i)) + 4 * c, r);
        }
    }
}

// ---------------------------------------------------------------------------- backward (local) records
// One thread per distinct row: where its sum goes (the owner's gradient inbox, slot = position inside the owner's
// segment), its first gradient row, its run; runs longer than kDirectMax reserve chunk slots exactly as the fused
// backward's records do.
__global__ void __launch_bounds__(256) xchg_local_meta_kernel(BwdParams p, XchgParams x, const int64_t* __restrict__ seg_g,
                                                              int64_t* __restrict__ counters, RunMeta* __restrict__ meta,
                                                              int2* __restrict__ desc, int* __restrict__ chunk_row)
{
    __shared__ int64_t seg[RECSDK_MAX_SHARDS + 1];
    if (threadIdx.x <= x.W) seg[threadIdx.x] = seg_g[threadIdx.x];
    __syncthreads();
    const int64_t U = counters[0];
    const bool vec = p.base_aligned && (((x.D | p.total_D | p.max_D) & 3) == 0);
    for (int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; u < U;
         u += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int rs = p.run_start[u], re = p.run_start[u + 1];
        const int len = re - rs;
        const int r = owner_of(seg, x.W, u);
        const int64_t slot = u - seg[r];
        RunMeta m;
        m.row_off = slot < x.cap ? ((static_cast<int64_t>(r) << kLocShardShift) |
                                    ((static_cast<int64_t>(x.me) * x.cap + slot) * x.D))
                                 : -1;
        m.g0_loc = grad_row_loc(p, p.vals[rs]);
        m.rs = rs;
        m.len = len;
        m.D = x.D | (vec ? kMetaVecBit : 0);
        m.chunk_base = -1;
        if (len > p.direct_max) {
            const int c = chunks_of_run(len, kChunk);
            const int base = static_cast<int>(atomicAdd(reinterpret_cast<unsigned long long*>(counters + 1),
                                                        static_cast<unsigned long long>(c)));
            atomicAdd(reinterpret_cast<unsigned long long*>(counters + 2), static_cast<unsigned long long>(len));
            m.chunk_base = base;
            for (int k = 0; k < c; ++k) {
                const int b0 = rs + k * kChunk;
                desc[base + k] = make_int2(b0, b0 + kChunk < re ? b0 + kChunk : re);
                chunk_row[base + k] = static_cast<int>(u);
            }
        }
        meta[u] = m;
    }
}

// ---------------------------------------------------------------------------- backward (owner) expand
// The inbox holds, per source rank q, count[q] local row numbers at [q*cap, q*cap + count[q]).  Compact position
// p (source-rank major) -> (key = local row, val = inbox slot q*cap + i); the total is left in counters[4] for the
// kernels that follow.  Block 0 also writes the one-table layout arrays of the update.
template <typename KeyT>
__global__ void __launch_bounds__(256) xchg_owner_expand_kernel(XchgParams x, const int64_t* __restrict__ ids,
                                                                const int64_t* __restrict__ counts,
                                                                KeyT* __restrict__ keys, uint32_t* __restrict__ vals,
                                                                SortHistSink sink, int64_t* __restrict__ counters,
                                                                int64_t* __restrict__ lay_i64,
                                                                int32_t* __restrict__ lay_i32, int64_t local_rows)
{
    __shared__ int64_t prefix[RECSDK_MAX_SHARDS + 1];
    if (threadIdx.x == 0) {
        int64_t s = 0;
        for (int q = 0; q < x.W; ++q) {
            prefix[q] = s;
            int64_t c = counts[q];
            c = c < 0 ? 0 : (c > x.cap ? x.cap : c);
            s += c;
        }
        prefix[x.W] = s;
        if (blockIdx.x == 0) {
            counters[4] = s;
            lay_i64[0] = 0;           // weights_offsets[0]
            lay_i64[1] = 0;           // hash_size_cumsum[0]
            lay_i64[2] = local_rows;  // hash_size_cumsum[1]
            lay_i32[0] = 0;           // D_offsets
            lay_i32[1] = x.D;
        }
    }
    __syncthreads();
    const int64_t total = prefix[x.W];
    for (int64_t pos0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + (threadIdx.x & ~31); pos0 < total;
         pos0 += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t pos = pos0 + (threadIdx.x & 31);
        int64_t key = 0;
        if (pos < total) {
            const int q = owner_of(prefix, x.W, pos);
            const int64_t slot = static_cast<int64_t>(q) * x.cap + (pos - prefix[q]);
            key = ids[slot];
            keys[pos] = static_cast<KeyT>(key);
            vals[pos] = static_cast<uint32_t>(slot);
        }
        sink.add_warp(pos < total, static_cast<KeyT>(key), pos);
    }
}

// ---------------------------------------------------------------------------- workspace
struct XchgWorkspace {
    // local plan (forward -> backward_local)
    int64_t* lc;  // [8] {U, chunks, ids in chunked runs, -, ...}
    int64_t* seg;  // [MAX_SHARDS+1]
    void *keys_a, *keys_b;
    uint32_t *vals_a, *vals_b, *sort_scratch, *tag_of_pos, *tags_sorted;
    int *run_start, *scan_scratch;
    int64_t *uniq, *inverse, *zeros_F;
    int32_t* dofs;
    RunMeta* meta;
    int2* desc;
    int* chunk_row;
    float *partial, *fetched;
    // owner plan
    int64_t* oc;  // [8] {U, chunks, -, unaligned, ids received, ...}
    int64_t* lay_i64;
    int32_t* lay_i32;
    void *okeys_a, *okeys_b;
    uint32_t *ovals_a, *ovals_b, *osort_scratch;
    int *orun_start, *oscan_scratch;
    RunMeta* ometa;
    int2* odesc;
    float* opartial;
    size_t bytes;
};

static XchgWorkspace carve_xchg(void* base, int64_t max_ids, int64_t inbox_cap, int32_t world, int32_t D, int64_t F)
{
    WorkspaceCarver c(base);
    XchgWorkspace w;
    const size_t n = static_cast<size_t>(max_ids > 0 ? max_ids : 1);
    const size_t chunks = chunk_slots_cap(max_ids);
    w.lc = c.take<int64_t>(8);
    w.seg = c.take<int64_t>(RECSDK_MAX_SHARDS + 1);
    w.keys_a = c.take<uint64_t>(n);
    w.keys_b = c.take<uint64_t>(n);
    w.vals_a = c.take<uint32_t>(n);
    w.vals_b = c.take<uint32_t>(n);
    w.sort_scratch = c.take<uint32_t>(sort_scratch_u32_fused(max_ids));
    w.tag_of_pos = c.take<uint32_t>(n);
    w.tags_sorted = c.take<uint32_t>(n);
    w.run_start = c.take<int>(n + 1);
    w.scan_scratch = c.take<int>(scan_scratch_ints(max_ids));
    w.uniq = c.take<int64_t>(n);
    w.inverse = c.take<int64_t>(n);
    w.zeros_F = c.take<int64_t>(static_cast<size_t>(F > 0 ? F : 1));
    w.dofs = c.take<int32_t>(static_cast<size_t>(F + 1));
    w.meta = c.take<RunMeta>(n);
    w.desc = c.take<int2>(chunks);
    w.chunk_row = c.take<int>(chunks);
    w.partial = c.take<float>(chunks * static_cast<size_t>(D));
    w.fetched = c.take<float>(n * static_cast<size_t>(D));
    const int64_t in_cap = static_cast<int64_t>(world) * inbox_cap;
    const size_t m = static_cast<size_t>(in_cap > 0 ? in_cap : 1);
    const size_t ochunks = chunk_slots_cap(in_cap);
    w.oc = c.take<int64_t>(8);
    w.lay_i64 = c.take<int64_t>(4);
    w.lay_i32 = c.take<int32_t>(4);
    w.okeys_a = c.take<uint64_t>(m);
    w.okeys_b = c.take<uint64_t>(m);
    w.ovals_a = c.take<uint32_t>(m);
    w.ovals_b = c.take<uint32_t>(m);
    w.osort_scratch = c.take<uint32_t>(sort_scratch_u32_fused(in_cap));
    w.orun_start = c.take<int>(m + 1);
    w.oscan_scratch = c.take<int>(scan_scratch_ints(in_cap));
    w.ometa = c.take<RunMeta>(m);
    w.odesc = c.take<int2>(ochunks);
    w.opartial = c.take<float>(ochunks * static_cast<size_t>(D));
    w.bytes = c.used();
    return w;
}

static int xchg_bits_for(int64_t v)
{
    int b = 0;
    while (b < 63 && (int64_t(1) << b) <= v) ++b;
    return b < 1 ? 1 : b;
}

static int xchg_validate(const recsdk_xchg_t* x, int64_t N)
{
    if (x == nullptr) return RECSDK_ERR_INVALID_ARG;
    if (x->world < 1 || x->world > RECSDK_MAX_SHARDS || x->rank < 0 || x->rank >= x->world) return RECSDK_ERR_INVALID_ARG;
    if (x->partition != RECSDK_XCHG_TABLE_WISE && x->partition != RECSDK_XCHG_ROW_WISE) return RECSDK_ERR_INVALID_ARG;
    if (x->D <= 0 || (x->D & 3) != 0 || x->F <= 0 || x->B <= 0 || N < 0 || x->max_ids <= 0 || x->inbox_cap <= 0)
        return RECSDK_ERR_INVALID_ARG;
    if (N > x->max_ids || x->max_ids >= (int64_t(1) << 31)) return RECSDK_ERR_TOO_LARGE;
    if (static_cast<int64_t>(x->world) * x->inbox_cap >= (int64_t(1) << 31)) return RECSDK_ERR_TOO_LARGE;
    if (x->key_bits < 1 || x->key_bits > 63 || !x->part_base || !x->rank_base) return RECSDK_ERR_INVALID_ARG;
    for (int r = 0; r < x->world; ++r)
        if (!x->tables[r] || !x->inbox_ids[r] || !x->inbox_counts[r] || !x->inbox_grads[r] || !aligned16(x->tables[r]) ||
            !aligned16(x->inbox_grads[r]))
            return RECSDK_ERR_INVALID_ARG;
    if (!x->workspace || !aligned16(x->workspace)) return RECSDK_ERR_WORKSPACE;
    if (carve_xchg(nullptr, x->max_ids, x->inbox_cap, x->world, x->D, x->F).bytes > x->workspace_bytes)
        return RECSDK_ERR_WORKSPACE;
    return RECSDK_OK;
}

static XchgParams xchg_params(const recsdk_xchg_t* x, int64_t N, int32_t mode)
{
    XchgParams q{};
    q.W = x->world;
    q.me = x->rank;
    q.partition = x->partition;
    q.D = x->D;
    q.F = x->F;
    q.B = x->B;
    q.N = N;
    q.cap = x->inbox_cap;
    q.part_base = x->part_base;
    q.rank_base = x->rank_base;
    q.table_rows = x->table_rows;
    q.status = x->dev_status;
    q.mode = mode;
    q.bshift = xchg_bits_for(x->B - 1 > 0 ? x->B - 1 : 1);
    q.one_hot = (x->flags & RECSDK_XCHG_ONE_HOT) ? 1 : 0;
    return q;
}

// Parameters of the local backward phase (records, chunk sums, per-row sums).  `grad` may be NULL while only the
// records are made (forward); the gradient must then be 16-byte aligned when it arrives, which backward_local checks.
static BwdParams xchg_local_params(const recsdk_xchg_t* x, const XchgWorkspace& ws, const XchgParams& q, const float* grad,
                                   const int64_t* offsets, int64_t N, int32_t mode, int32_t clip, float max_grad)
{
    BwdParams p{};
    p.grad = grad;
    p.wofs = ws.zeros_F;  // read by the chunk-sum kernel's geometry; the sums are not table rows
    p.dofs = ws.dofs;
    p.offs = offsets;
    p.T = x->F;
    p.B = x->B;
    p.N = N;
    p.total_D = static_cast<int32_t>(x->F * x->D);
    p.max_D = x->D;
    p.mode = mode;
    p.opt = kOptStore;
    p.bshift = q.bshift;
    p.chunk = kChunk;
    p.direct_max = kDirectMax;
    p.max_grad = max_grad;
    p.clip = clip;
    p.status = x->dev_status;
    p.base_aligned = aligned16(ws.partial) ? 1 : 0;
    p.vals = ws.tags_sorted;
    p.run_start = ws.run_start;
    p.chunk_desc = ws.desc;
    p.partial = ws.partial;
    p.counters = ws.lc;
    for (int r = 0; r < RECSDK_MAX_SHARDS; ++r) p.dst_ptrs[r] = x->inbox_grads[r < x->world ? r : 0];
    return p;
}

template <typename KeyT>
static int xchg_forward_impl(const recsdk_xchg_t* x, const XchgWorkspace& ws, const int64_t* indices,
                             const int64_t* offsets, int64_t N, int32_t mode, float* out, int32_t flags, cudaStream_t st)
{
    const XchgParams q = xchg_params(x, N, mode);
    if ((flags & RECSDK_XCHG_FWD_FETCH_ONLY) == 0) {
        // the plan: touches this rank's ids and scratch only -- no table, no inbox -- so it may run before the fence
        // that makes the tables final, beside the owner phase of the previous step
        KeyT* ka = static_cast<KeyT*>(ws.keys_a);
        KeyT* kb = static_cast<KeyT*>(ws.keys_b);
        cudaMemsetAsync(ws.lc, 0, 8 * sizeof(int64_t), st);
        const RadixFusedPlan plan = radix_fused_begin(N, x->key_bits, ws.sort_scratch, st);
        if (mode == RECSDK_POOL_NONE)
            xchg_expand_nobag_kernel<KeyT><<<grid_for(N, 256), 256, 0, st>>>(q, indices, offsets, ka, ws.vals_a, plan.first,
                                                                             ws.zeros_F, ws.dofs);
        else
            xchg_expand_pooled_kernel<KeyT><<<grid_for(x->F * x->B, 8 * 32), 256, 0, st>>>(
                q, indices, offsets, ka, ws.vals_a, ws.tag_of_pos, plan.first, ws.zeros_F, ws.dofs);
        const int which = radix_sort_pairs_fused<KeyT>(plan, ka, ws.vals_a, kb, ws.vals_b, N, ws.sort_scratch, st);
        const KeyT* keys = which ? kb : ka;
        const uint32_t* pos_sorted = which ? ws.vals_b : ws.vals_a;
        device_scan_fn<true>(HeadFlagIn<KeyT>{keys},
                             XchgRunOut<KeyT>{keys, pos_sorted, mode == RECSDK_POOL_NONE ? nullptr : ws.tag_of_pos,
                                              ws.run_start, ws.uniq, ws.inverse, ws.tags_sorted, ws.lc,
                                              (q.one_hot && mode != RECSDK_POOL_NONE) ? x->B : 0, q.bshift},
                             N, ws.scan_scratch, nullptr, st);
    }
    if (flags & RECSDK_XCHG_FWD_PLAN_ONLY) {
        RECSDK_CUDA_CHECK_LAUNCH();
        return RECSDK_OK;
    }
    PeerTable<const float*> tables;
    PeerTable<int64_t*> in_ids, in_counts;
    for (int r = 0; r < RECSDK_MAX_SHARDS; ++r) {
        const int s = r < x->world ? r : 0;
        tables.ptrs[r] = x->tables[s];
        in_ids.ptrs[r] = x->inbox_ids[s];
        in_counts.ptrs[r] = x->inbox_counts[s];
    }
    xchg_seg_kernel<<<1, 32, 0, st>>>(q, ws.uniq, ws.lc, ws.seg, in_counts);
    // the records of the local backward phase depend on the batch and on the LAYOUT of the gradient only: made here,
    // they also tell the one-id-per-bag forward which runs are chunked
    const BwdParams lp = xchg_local_params(x, ws, q, nullptr, offsets, N, mode, 0, 0.f);
    // the records reserve chunk slots by counting up from zero: reset here, not only in the plan, so that a fetch
    // repeated on the same plan stays inside the slot arrays
    cudaMemsetAsync(ws.lc + 1, 0, 2 * sizeof(int64_t), st);
    xchg_local_meta_kernel<<<grid_for(N, 256), 256, 0, st>>>(lp, q, ws.seg, ws.lc, ws.meta, ws.desc, ws.chunk_row);
    const int G = group_lanes_for(x->D >> 2);
    // kRows rows per group and pass; several resident blocks per SM keep many peer loads in flight
    const int grid = grid_for(ceil_div(N, 4), 256 / G, 8);
    if (q.one_hot && mode != RECSDK_POOL_NONE) {
        switch (G) {
#define RECSDK_PULL(GG)                                                                                                  \
    case GG:                                                                                                             \
        xchg_pull_scatter_kernel<GG><<<grid, 256, 0, st>>>(q, ws.uniq, ws.lc, ws.seg, ws.meta, ws.desc, ws.chunk_row,       \
                                                           ws.tags_sorted, out, tables, in_ids);                          \
        break
            RECSDK_PULL(1);
            RECSDK_PULL(2);
            RECSDK_PULL(4);
            RECSDK_PULL(8);
            RECSDK_PULL(16);
            default: RECSDK_PULL(32);
#undef RECSDK_PULL
        }
        RECSDK_CUDA_CHECK_LAUNCH();
        return RECSDK_OK;
    }
    switch (G) {
#define RECSDK_PULL(GG) \
    case GG: xchg_pull_kernel<GG><<<grid, 256, 0, st>>>(q, ws.uniq, ws.lc, ws.seg, ws.fetched, tables, in_ids); break
        RECSDK_PULL(1);
        RECSDK_PULL(2);
        RECSDK_PULL(4);
        RECSDK_PULL(8);
        RECSDK_PULL(16);
        default: RECSDK_PULL(32);
#undef RECSDK_PULL
    }
    RECSDK_CUDA_CHECK_LAUNCH();
    // pooled gather over the fetched rows: they are the table, the inverse positions are the indices
    recsdk_tbe_forward_args fa{};
    fa.dev_weights = ws.fetched;
    fa.weights_offsets = ws.zeros_F;
    fa.D_offsets = ws.dofs;
    fa.indices = ws.inverse;
    fa.offsets = offsets;
    fa.out = out;
    fa.T = x->F;
    fa.B = x->B;
    fa.N = N;
    fa.total_D = static_cast<int32_t>(x->F * x->D);
    fa.max_D = x->D;
    fa.pooling_mode = mode;
    fa.weights_numel = 0;
    fa.dev_status = x->dev_status;
    return recsdk_tbe_forward(&fa, st);
}

#define RECSDK_XCHG_DISPATCH_GK(vec_per_row, CALL)            \
    do {                                                      \
        const int G__ = group_lanes_for(vec_per_row);         \
        switch (G__) {                                        \
            case 1: CALL(1, 1); break;                        \
            case 2: CALL(2, 1); break;                        \
            case 4: CALL(4, 1); break;                        \
            case 8: CALL(8, 1); break;                        \
            case 16: CALL(16, 1); break;                      \
            default:                                          \
                if ((vec_per_row) <= 32) { CALL(32, 1); }     \
                else if ((vec_per_row) <= 64) { CALL(32, 2); } \
                else { CALL(32, 4); }                         \
                break;                                        \
        }                                                     \
    } while (0)

template <int G, int K>
static void xchg_launch_partial(const BwdParams& p, int64_t n, cudaStream_t st)
{
    partial_kernel<G, K><<<grid_for(static_cast<int64_t>(chunk_slots_cap(n)), 256 / G, 4), 256, 0, st>>>(p);
}

template <int G, int K>
static void xchg_launch_update(const BwdParams& p, const RunMeta* meta, int64_t n, int opt, cudaStream_t st)
{
    const int grid = grid_for(n, 256 / G, 4);
    switch (opt) {
        // the store variant needs 40 registers: six resident blocks per SM keep more gradient rows in flight
        case kOptStore: update_kernel<G, K, kOptStore><<<grid_for(n, 256 / G, 6), 256, 0, st>>>(p, meta); break;
        case RECSDK_OPT_ADAGRAD: update_kernel<G, K, RECSDK_OPT_ADAGRAD><<<grid, 256, 0, st>>>(p, meta); break;
        case RECSDK_OPT_ADAM: update_kernel<G, K, RECSDK_OPT_ADAM><<<grid, 256, 0, st>>>(p, meta); break;
        default: update_kernel<G, K, RECSDK_OPT_SGD><<<grid, 256, 0, st>>>(p, meta); break;
    }
}

template <typename KeyT>
static int xchg_owner_impl(const recsdk_xchg_t* x, const XchgWorkspace& ws, BwdParams p, void* ev0, void* ev1,
                           int32_t flags, cudaStream_t st)
{
    const bool do_plan = (flags & RECSDK_XCHG_OWNER_APPLY_ONLY) == 0;
    const bool do_apply = (flags & RECSDK_XCHG_OWNER_PLAN_ONLY) == 0;
    const XchgParams q = xchg_params(x, 0, RECSDK_POOL_NONE);
    const int64_t n_cap = static_cast<int64_t>(x->world) * x->inbox_cap;
    const int key_bits = xchg_bits_for(x->local_rows);
    KeyT* ka = static_cast<KeyT*>(ws.okeys_a);
    KeyT* kb = static_cast<KeyT*>(ws.okeys_b);
    int passes, bits;
    radix_plan(key_bits, &passes, &bits);
    const int which = passes & 1;
    const KeyT* keys = which ? kb : ka;
    p.vals = which ? ws.ovals_b : ws.ovals_a;
    if (do_plan) {
        // needs the ids and counts in the inbox only (they arrive with the forwards of all ranks), not the gradient
        // sums: it can run beside this rank's local backward phase, on another stream, after a fence of its own
        cudaMemsetAsync(ws.oc, 0, 8 * sizeof(int64_t), st);
        const RadixFusedPlan plan = radix_fused_begin(n_cap, key_bits, ws.osort_scratch, st);
        xchg_owner_expand_kernel<KeyT><<<grid_for(n_cap, 256), 256, 0, st>>>(q, x->inbox_ids[x->rank],
                                                                             x->inbox_counts[x->rank], ka, ws.ovals_a,
                                                                             plan.first, ws.oc, ws.lay_i64, ws.lay_i32,
                                                                             x->local_rows);
        const int64_t* n_dev = ws.oc + 4;
        const int got = radix_sort_pairs_fused<KeyT>(plan, ka, ws.ovals_a, kb, ws.ovals_b, n_cap, ws.osort_scratch, st, n_dev);
        if (got != which) return RECSDK_ERR_CUDA;
        device_scan_fn<true>(HeadFlagIn<KeyT>{keys}, RunStartOut{ws.orun_start, ws.oc}, n_cap, ws.oscan_scratch, nullptr, st,
                             n_dev);
        run_meta_kernel<KeyT><<<grid_for(n_cap, 256), 256, 0, st>>>(p, keys, ws.oc, ws.ometa, ws.odesc);
    }
    if (!do_apply) {
        RECSDK_CUDA_CHECK_LAUNCH();
        return RECSDK_OK;
    }
    const int vec_per_row = x->D >> 2;
    if (x->world > p.direct_max) {  // a row has at most one contribution per source rank: no run is longer than `world`
#define CALL_PARTIAL(G, K) xchg_launch_partial<G, K>(p, n_cap, st)
        RECSDK_XCHG_DISPATCH_GK(vec_per_row, CALL_PARTIAL);
#undef CALL_PARTIAL
    }
    if (ev0) cudaEventRecord(static_cast<cudaEvent_t>(ev0), st);
#define CALL_UPDATE(G, K) xchg_launch_update<G, K>(p, ws.ometa, n_cap, p.opt, st)
    RECSDK_XCHG_DISPATCH_GK(vec_per_row, CALL_UPDATE);
#undef CALL_UPDATE
    if (ev1) cudaEventRecord(static_cast<cudaEvent_t>(ev1), st);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

}  // namespace recsdk

using namespace recsdk;

extern "C" size_t recsdk_xchg_workspace_bytes(int64_t max_ids, int64_t inbox_cap, int32_t world, int32_t D, int64_t F)
{
    return carve_xchg(nullptr, max_ids, inbox_cap, world, D > 0 ? D : 4, F).bytes;
}

extern "C" int recsdk_xchg_forward(const recsdk_xchg_t* x, const int64_t* indices, const int64_t* offsets, int64_t N,
                                   int32_t pooling_mode, float* out, int32_t flags, void* stream)
{
    const int rc = xchg_validate(x, N);
    if (rc != RECSDK_OK) return rc;
    if (pooling_mode < RECSDK_POOL_SUM || pooling_mode > RECSDK_POOL_NONE) return RECSDK_ERR_INVALID_ARG;
    const bool plan_only = (flags & RECSDK_XCHG_FWD_PLAN_ONLY) != 0;
    if (plan_only && (flags & RECSDK_XCHG_FWD_FETCH_ONLY)) return RECSDK_ERR_INVALID_ARG;
    if (!offsets || (!out && !plan_only) || (N > 0 && !indices)) return RECSDK_ERR_INVALID_ARG;
    if (pooling_mode != RECSDK_POOL_NONE && xchg_bits_for(x->B - 1 > 0 ? x->B - 1 : 1) + xchg_bits_for(x->F) > 32)
        return RECSDK_ERR_TOO_LARGE;
    if ((x->flags & RECSDK_XCHG_ONE_HOT) && pooling_mode != RECSDK_POOL_NONE && N != x->F * x->B)
        return RECSDK_ERR_INVALID_ARG;  // one id per bag was promised
    const XchgWorkspace ws = carve_xchg(x->workspace, x->max_ids, x->inbox_cap, x->world, x->D, x->F);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (x->key_bits <= 32) return xchg_forward_impl<uint32_t>(x, ws, indices, offsets, N, pooling_mode, out, flags, st);
    return xchg_forward_impl<uint64_t>(x, ws, indices, offsets, N, pooling_mode, out, flags, st);
}

extern "C" int recsdk_xchg_backward_local(const recsdk_xchg_t* x, const float* grad_output, const int64_t* offsets,
                                          int64_t N, int32_t pooling_mode, int32_t gradient_clipping, float max_gradient,
                                          void* stream)
{
    const int rc = xchg_validate(x, N);
    if (rc != RECSDK_OK) return rc;
    if (pooling_mode < RECSDK_POOL_SUM || pooling_mode > RECSDK_POOL_NONE) return RECSDK_ERR_INVALID_ARG;
    if (!grad_output || !offsets) return RECSDK_ERR_INVALID_ARG;
    const XchgWorkspace ws = carve_xchg(x->workspace, x->max_ids, x->inbox_cap, x->world, x->D, x->F);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!aligned16(grad_output)) return RECSDK_ERR_INVALID_ARG;  // the records made by the forward assume it
    const XchgParams q = xchg_params(x, N, pooling_mode);
    const BwdParams p = xchg_local_params(x, ws, q, grad_output, offsets, N, pooling_mode, gradient_clipping, max_gradient);
    const int vec_per_row = x->D >> 2;
#define CALL_PARTIAL(G, K) xchg_launch_partial<G, K>(p, N, st)
    RECSDK_XCHG_DISPATCH_GK(vec_per_row, CALL_PARTIAL);
#undef CALL_PARTIAL
    // The store variant is bound by the bytes a warp keeps in flight (most runs hold one position: record -> one
    // gradient row -> one store), and it is light on registers: for rows of 64 and 128 floats half as many lanes per
    // row with two vectors each put twice as many rows in flight per warp (local phase of the benchmark step 0.35 ->
    // 0.30 ms).  The optimizer variants hold w / m / v as well and lose more occupancy than they gain.
#define CALL_UPDATE(G, K) xchg_launch_update<G, K>(p, ws.meta, N, kOptStore, st)
    if (vec_per_row == 32) {
        CALL_UPDATE(16, 2);
    } else if (vec_per_row == 16) {
        CALL_UPDATE(8, 2);
    } else {
        RECSDK_XCHG_DISPATCH_GK(vec_per_row, CALL_UPDATE);
    }
#undef CALL_UPDATE
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_xchg_backward_owner(const recsdk_xchg_t* x, float* weights, float* momentum1, float* momentum2,
                                          int32_t optimizer, float learning_rate, float eps, float beta1, float beta2,
                                          int64_t iter, void* ev_update_start, void* ev_update_stop, int32_t flags,
                                          void* stream)
{
    const int rc = xchg_validate(x, 0);
    if ((flags & RECSDK_XCHG_OWNER_PLAN_ONLY) && (flags & RECSDK_XCHG_OWNER_APPLY_ONLY)) return RECSDK_ERR_INVALID_ARG;
    if (rc != RECSDK_OK) return rc;
    if (optimizer < RECSDK_OPT_ADAGRAD || optimizer > RECSDK_OPT_SGD || !weights) return RECSDK_ERR_INVALID_ARG;
    if (optimizer != RECSDK_OPT_SGD && !momentum1) return RECSDK_ERR_INVALID_ARG;
    if (optimizer == RECSDK_OPT_ADAM && !momentum2) return RECSDK_ERR_INVALID_ARG;
    if (x->local_rows <= 0) return RECSDK_ERR_INVALID_ARG;
    const XchgWorkspace ws = carve_xchg(x->workspace, x->max_ids, x->inbox_cap, x->world, x->D, x->F);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    BwdParams p{};
    p.grad = x->inbox_grads[x->rank];
    p.w = weights;
    p.m1 = momentum1;
    p.m2 = momentum2;
    p.wofs = ws.lay_i64;
    p.cumsum = ws.lay_i64 + 1;
    p.dofs = ws.lay_i32;
    p.T = 1;
    p.B = 1;
    p.N = static_cast<int64_t>(x->world) * x->inbox_cap;
    p.total_D = x->D;
    p.max_D = x->D;
    p.mode = RECSDK_POOL_NONE;
    p.opt = optimizer;
    p.chunk = kChunk;
    p.direct_max = kDirectMax;
    p.lr = learning_rate;
    p.eps = eps;
    p.beta1 = beta1;
    p.beta2 = beta2;
    p.beta2sqrt = optimizer == RECSDK_OPT_ADAM ? recsdk_adam_beta2sqrt(beta1, beta2, iter) : 0.f;
    p.w_numel = x->local_rows * x->D;
    p.status = x->dev_status;
    p.base_aligned = (aligned16(weights) && aligned16(momentum1) && aligned16(momentum2) && aligned16(p.grad) &&
                      aligned16(ws.opartial))
                         ? 1
                         : 0;
    p.run_start = ws.orun_start;
    p.chunk_desc = ws.odesc;
    p.partial = ws.opartial;
    p.counters = ws.oc;
    if (xchg_bits_for(x->local_rows) <= 32) return xchg_owner_impl<uint32_t>(x, ws, p, ev_update_start, ev_update_stop, flags, st);
    return xchg_owner_impl<uint64_t>(x, ws, p, ev_update_start, ev_update_stop, flags, st);
}

extern "C" int recsdk_xchg_counters(const recsdk_xchg_t* x, int64_t* out6, void* stream)
{
    if (x == nullptr || out6 == nullptr || x->workspace == nullptr) return RECSDK_ERR_INVALID_ARG;
    const XchgWorkspace ws = carve_xchg(x->workspace, x->max_ids, x->inbox_cap, x->world, x->D, x->F);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int64_t lc[8], oc[8];
    if (cudaMemcpyAsync(lc, ws.lc, sizeof(lc), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaMemcpyAsync(oc, ws.oc, sizeof(oc), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess) {
        (void)cudaGetLastError();
        return RECSDK_ERR_CUDA;
    }
    int64_t seg[RECSDK_MAX_SHARDS + 1];
    if (cudaMemcpyAsync(seg, ws.seg, sizeof(seg), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess) {
        (void)cudaGetLastError();
        return RECSDK_ERR_CUDA;
    }
    out6[0] = lc[0];
    out6[1] = oc[4];
    out6[2] = oc[0];
    out6[3] = lc[2];
    out6[4] = seg[x->rank + 1] - seg[x->rank];
    out6[5] = lc[1];
    return RECSDK_OK;
}
