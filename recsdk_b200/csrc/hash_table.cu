// HBM-resident dynamic key tables: IdsMapper (key -> slot), SwapManager (cache
// slot policy with clock-sweep replacement) and FeatureFilter (count admission,
// timestamp eviction).
//
// All three sit on one open-addressing scheme (linear probing, 64-bit keys >= 0,
// EMPTY = -1, TOMBSTONE = -2).  A batch is processed in phases, one kernel per
// phase, so that no thread ever waits on another:
//   lookup  -> misses insert their key (atomicCAS) and bid for it with
//   atomicMin(position) -> the lowest position of each new key is its first
//   occurrence -> exclusive scan of the first-occurrence flags = the order in
//   which a sequential loop would have met the new keys -> slots are handed out
//   as base + rank.  That reproduces the reference's first-come slot numbering
//   bit for bit while every phase is fully parallel.
// Free entries always carry value == VAL_FREE so that a bidder never races with
// an initialiser.
#include "prims.cuh"

namespace recsdk {

constexpr int64_t kEmpty = -1;
constexpr int64_t kTomb = -2;
constexpr int64_t kValFree = INT64_MAX;
constexpr int64_t kPending = int64_t(1) << 62;  // values >= kPending are position bids
constexpr int kMarkFree = 0x7fffffff;

__device__ __forceinline__ uint64_t mix64(uint64_t x)
{
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdULL;
    x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ULL;
    x ^= x >> 33;
    return x;
}

// STRIDE = int64 words per entry (2 for {key,value}, 4 for the filter).
template <int STRIDE>
__device__ __forceinline__ int64_t ht_lookup(const int64_t* __restrict__ table, int64_t cap, int64_t key)
{
    const uint64_t mask = static_cast<uint64_t>(cap) - 1;
    uint64_t e = mix64(static_cast<uint64_t>(key)) & mask;
    for (int64_t probes = 0; probes < cap; ++probes) {
        const int64_t k = table[e * STRIDE];
        if (k == key) return static_cast<int64_t>(e);
        if (k == kEmpty) return -1;
        e = (e + 1) & mask;
    }
    return -1;
}

// Warp-cooperative lookup: kProbeLanes consecutive lanes probe ONE key.  Per round they read kProbeLanes consecutive
// entries of the chain (for 16-byte entries: one 128-byte line when the chain starts on a line boundary, two
// otherwise) and vote: the first lane whose entry holds the key wins unless an EMPTY entry comes before it in probe
// order (then the key is absent).  All lanes of the group must call with the same key; every lane gets the result.
// `gmask` is the ballot mask of the group, `gl` the lane's number inside it.
constexpr int kProbeLanes = 8;
template <int STRIDE>
__device__ __forceinline__ int64_t ht_lookup_coop(const int64_t* __restrict__ table, int64_t cap, int64_t key, int gl,
                                                  unsigned gmask, int gshift)
{
    const uint64_t mask = static_cast<uint64_t>(cap) - 1;
    const uint64_t e0 = mix64(static_cast<uint64_t>(key)) & mask;
    for (int64_t probes = 0; probes < cap; probes += kProbeLanes) {
        const uint64_t e = (e0 + static_cast<uint64_t>(probes) + static_cast<uint64_t>(gl)) & mask;
        const int64_t k = table[e * STRIDE];
        const unsigned hit = (__ballot_sync(gmask, k == key) & gmask) >> gshift;
        const unsigned emp = (__ballot_sync(gmask, k == kEmpty) & gmask) >> gshift;
        const int first_hit = hit ? __ffs(hit) - 1 : kProbeLanes;
        const int first_emp = emp ? __ffs(emp) - 1 : kProbeLanes;
        if (first_hit < first_emp) return static_cast<int64_t>((e0 + static_cast<uint64_t>(probes) + first_hit) & mask);
        if (emp) return -1;
    }
    return -1;
}

// Returns the entry that holds `key` after the call (inserting it into the
// first free entry of its probe chain when absent), or -1 when no entry is free.
// Must not run concurrently with erases.
template <int STRIDE>
__device__ __forceinline__ int64_t ht_insert(int64_t* __restrict__ table, int64_t cap, int64_t key)
{
    const uint64_t mask = static_cast<uint64_t>(cap) - 1;
    uint64_t e = mix64(static_cast<uint64_t>(key)) & mask;
    for (int64_t probes = 0; probes < cap;) {
        unsigned long long* kp = reinterpret_cast<unsigned long long*>(table + e * STRIDE);
        const int64_t k = static_cast<int64_t>(*reinterpret_cast<volatile unsigned long long*>(kp));
        if (k == key) return static_cast<int64_t>(e);
        if (k == kEmpty || k == kTomb) {
            const int64_t old = static_cast<int64_t>(
                atomicCAS(kp, static_cast<unsigned long long>(k), static_cast<unsigned long long>(key)));
            if (old == k || old == key) return static_cast<int64_t>(e);
            continue;  // someone else took the entry: look at it again
        }
        e = (e + 1) & mask;
        ++probes;
    }
    return -1;
}

template <int STRIDE>
__device__ __forceinline__ int64_t ht_find_or_insert(int64_t* __restrict__ table, int64_t cap, int64_t key)
{
    const int64_t e = ht_lookup<STRIDE>(table, cap, key);
    return e >= 0 ? e : ht_insert<STRIDE>(table, cap, key);
}

__device__ __forceinline__ long long atomic_min_i64(int64_t* p, int64_t v)
{
    return atomicMin(reinterpret_cast<long long*>(p), static_cast<long long>(v));
}
__device__ __forceinline__ long long atomic_max_i64(int64_t* p, int64_t v)
{
    return atomicMax(reinterpret_cast<long long*>(p), static_cast<long long>(v));
}

#define RECSDK_GRID_STRIDE(i, n)                                                        \
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < (n); \
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)

// ---------------------------------------------------------------------------- init
static __global__ void fill_i64_kernel(int64_t* p, int64_t n, int64_t stride, int64_t v0, int64_t v1, int64_t v2, int64_t v3)
{
    RECSDK_GRID_STRIDE(i, n)
    {
        p[i * stride] = v0;
        if (stride > 1) p[i * stride + 1] = v1;
        if (stride > 2) p[i * stride + 2] = v2;
        if (stride > 3) p[i * stride + 3] = v3;
    }
}
static __global__ void fill_i32_kernel(int32_t* p, int64_t n, int32_t v)
{
    RECSDK_GRID_STRIDE(i, n) p[i] = v;
}
static __global__ void set4_kernel(int64_t* p, int64_t a, int64_t b, int64_t c, int64_t d)
{
    p[0] = a;
    p[1] = b;
    p[2] = c;
    p[3] = d;
}

static bool is_pow2(int64_t x) { return x > 0 && (x & (x - 1)) == 0; }

// ============================================================================ shared phases
// phase 1: find or claim.  kProbeLanes lanes probe one key together (ballots).  A key that the table held before
// this batch is a hit: out_slots[i] = its slot, miss[i] = 0.  Any other key is a miss: lane 0 of the group inserts
// it (or finds the entry another position of this batch has just inserted -- its value is still a bid, >= kPending)
// and bids for it with its position; ent[i] = the entry, or -1 when the table is full.
// MODE 0: mapper (negative key is an error), MODE 1: swap (-1 = not admitted -> slot 0).
template <int MODE>
static __global__ void __launch_bounds__(256) phase_find_or_claim_kernel(int64_t* __restrict__ table, int64_t cap,
                                                                         const int64_t* __restrict__ keys, int64_t n,
                                                                         int64_t* __restrict__ out_slots,
                                                                         int64_t* __restrict__ ent, int* __restrict__ miss,
                                                                         int64_t* __restrict__ slot_version,
                                                                         const int64_t* __restrict__ counters,
                                                                         int64_t* __restrict__ status)
{
    const int64_t now = MODE == 1 ? counters[1] : 0;
    const int gl = threadIdx.x & (kProbeLanes - 1);
    const int gshift = (threadIdx.x & 31) & ~(kProbeLanes - 1);
    const unsigned gmask = ((1u << kProbeLanes) - 1u) << gshift;
    const int64_t groups_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) / kProbeLanes;
    // group-uniform trip count: the ballots inside need every lane of the group
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / kProbeLanes; i < n; i += groups_total) {
        const int64_t key = keys[i];
        if (key < 0) {
            if (gl == 0) {
                out_slots[i] = 0;
                if (MODE == 0 || key != -1) set_status(status, RECSDK_ERR_NEGATIVE_KEY, key, i);
                ent[i] = -1;
                miss[i] = 0;
            }
            continue;
        }
        int64_t e = ht_lookup_coop<2>(table, cap, key, gl, gmask, gshift);
        if (gl != 0) continue;
        const int64_t held = e >= 0 ? *reinterpret_cast<const volatile int64_t*>(table + e * 2 + 1) : kValFree;
        if (held < kPending) {  // the key was there before this batch
            out_slots[i] = held;
            if (MODE == 1) slot_version[held] = now;
            ent[i] = e;
            miss[i] = 0;
            continue;
        }
        if (e < 0) e = ht_insert<2>(table, cap, key);
        if (e < 0) {
            set_status(status, RECSDK_ERR_HASH_FULL, key, i);
            out_slots[i] = 0;
        } else {
            atomic_min_i64(table + e * 2 + 1, kPending + i);
        }
        ent[i] = e;
        miss[i] = 1;
    }
}

// phase 2, as the input of a scan: 1 where position i won the bid for its key.  The scan's consumer may overwrite
// the bid of a winner with its slot while other positions are still being evaluated: a loser's comparison fails
// against the slot as it failed against the winner's bid.
struct WonBidIn {
    const int64_t* table;
    const int64_t* ent;
    const int* miss;
    __device__ __forceinline__ int operator()(int64_t i) const
    {
        return (miss[i] && ent[i] >= 0 && table[ent[i] * 2 + 1] == kPending + i) ? 1 : 0;
    }
};
// flag and exclusive rank of every position, for the kernels that need both later
struct FlagRankOut {
    int* first;
    int* rank;
    __device__ __forceinline__ void operator()(int64_t i, int item, int prefix, int64_t) const
    {
        first[i] = item;
        rank[i] = prefix;
    }
};

// last phase: every miss reads the slot its key finally got
static __global__ void __launch_bounds__(256) phase_readback_kernel(const int64_t* __restrict__ table, int64_t n,
                                                                    const int64_t* __restrict__ ent,
                                                                    const int* __restrict__ miss,
                                                                    int64_t* __restrict__ out_slots)
{
    RECSDK_GRID_STRIDE(i, n)
    {
        if (miss[i] && ent[i] >= 0) {
            const int64_t v = table[ent[i] * 2 + 1];
            out_slots[i] = v < kPending ? v : 0;
        }
    }
}

// ============================================================================ IdsMapper
struct MapperWs {
    int64_t* ent;
    int *miss, *first, *rank, *scan_scratch;
    int64_t* tmp;  // {M, U_t}
    size_t bytes;
};
static MapperWs carve_mapper(void* base, int64_t N)
{
    WorkspaceCarver c(base);
    MapperWs w;
    const size_t n = static_cast<size_t>(N > 0 ? N : 1);
    w.tmp = c.take<int64_t>(8);
    w.ent = c.take<int64_t>(n);
    w.miss = c.take<int>(n);
    w.first = c.take<int>(n);
    w.rank = c.take<int>(n);
    w.scan_scratch = c.take<int>(scan_scratch_ints(N));
    w.bytes = c.used();
    return w;
}

// slot = max_index + rank for first occurrences (ids_mapper.cpp:84-98), as the consumer of the scan over WonBidIn
struct MapperAssignOut {
    recsdk_mapper_t m;
    const int64_t* keys;
    const int64_t* ent;
    int64_t* status;
    __device__ __forceinline__ void operator()(int64_t i, int item, int prefix, int64_t) const
    {
        if (!item) return;
        const int64_t slot = m.counters[0] + prefix;
        if (slot >= m.init_max_index) {
            // the reference raises only with onlyDeviceMem; the HBM arrays of this
            // mapper hold init_max_index slots, so running past them is an error either way
            set_status(status, RECSDK_ERR_TABLE_FULL, m.init_max_index, keys[i]);
            return;
        }
        m.table[ent[i] * 2 + 1] = slot;
        m.slot_key[slot] = keys[i];
    }
};

// Last phase of the mapper: every miss reads the slot its key finally got; one thread moves max_index on by the
// number of new keys (tmp[0], the scan's total); BID: every position also bids for its slot with its position
// (first phase of the first-occurrence unique below).
template <bool BID>
static __global__ void __launch_bounds__(256) mapper_readback_kernel(recsdk_mapper_t m, int64_t n,
                                                                     const int64_t* __restrict__ ent,
                                                                     const int* __restrict__ miss,
                                                                     int64_t* __restrict__ out_slots,
                                                                     const int64_t* __restrict__ tmp)
{
    RECSDK_GRID_STRIDE(i, n)
    {
        int64_t s = 0;
        if (miss[i]) {
            if (ent[i] >= 0) {
                const int64_t v = m.table[ent[i] * 2 + 1];
                s = v < kPending ? v : 0;
            }
            out_slots[i] = s;
        } else if (BID) {
            s = out_slots[i];
        }
        if (BID && s >= 0 && s < m.init_max_index) atomicMin(m.mark + s, static_cast<int>(i));
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        // no position reads max_index in this kernel
        const int64_t v = m.counters[0] + tmp[0];
        m.counters[0] = v < m.init_max_index ? v : m.init_max_index;
    }
}

// first-occurrence unique of the slots of one segment (ids_mapper.cpp:115-174): the positions bid for their slot in
// mapper_readback_kernel<true>; position i is a first occurrence when it holds the mark of its slot
struct HoldsMarkIn {
    const int64_t* slots;
    const int32_t* mark;
    int64_t max_index;
    __device__ __forceinline__ int operator()(int64_t i) const
    {
        const int64_t s = slots[i];
        return (s >= 0 && s < max_index && mark[s] == static_cast<int>(i)) ? 1 : 0;
    }
};
static __global__ void __launch_bounds__(256) uniq_write_kernel(const int64_t* __restrict__ slots, int64_t n,
                                                                const int32_t* __restrict__ mark, int64_t max_index,
                                                                const int* __restrict__ rank,
                                                                const int64_t* __restrict__ slot_key,
                                                                int64_t* __restrict__ unique,
                                                                int64_t* __restrict__ unique_ids,
                                                                int64_t* __restrict__ inverse,
                                                                int64_t* __restrict__ unique_offset, int64_t table_id,
                                                                const int64_t* __restrict__ tmp)
{
    const int64_t base = table_id == 0 ? 0 : unique_offset[table_id];
    RECSDK_GRID_STRIDE(i, n)
    {
        const int64_t s = slots[i];
        if (s < 0 || s >= max_index) {
            inverse[i] = 0;
            continue;
        }
        const int holder = mark[s];
        if (holder == static_cast<int>(i)) {
            unique[base + rank[i]] = s;
            unique_ids[base + rank[i]] = slot_key[s];
        }
        inverse[i] = rank[holder];
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        if (table_id == 0) unique_offset[0] = 0;
        unique_offset[table_id + 1] = base + tmp[1];
    }
}
static __global__ void __launch_bounds__(256) uniq_reset_kernel(const int64_t* __restrict__ slots, int64_t n,
                                                                int32_t* __restrict__ mark, int64_t max_index)
{
    RECSDK_GRID_STRIDE(i, n)
    {
        const int64_t s = slots[i];
        if (s >= 0 && s < max_index) mark[s] = kMarkFree;
    }
}
static __global__ void empty_segment_kernel(int64_t* unique_offset, int64_t table_id)
{
    // ids_mapper.cpp:78-81
    unique_offset[table_id + 1] = unique_offset[table_id];
}

// key -> slot for ids[0..n) (find or insert, first-come numbering): find-or-claim, a scan over "won the bid" whose
// consumer numbers the new keys, read back.  `bid_marks`: the read-back also opens the first-occurrence unique.
static int mapper_map(const recsdk_mapper_t* m, const int64_t* ids, int64_t n, int64_t* hash_indices,
                      int64_t* status, const MapperWs& ws, cudaStream_t st, bool bid_marks = false)
{
    const int grid = grid_for(n, 256);
    phase_find_or_claim_kernel<0><<<grid_for(n, 256 / kProbeLanes), 256, 0, st>>>(
        m->table, m->hash_capacity, ids, n, hash_indices, ws.ent, ws.miss, nullptr, m->counters, status);
    device_scan_fn<false>(WonBidIn{m->table, ws.ent, ws.miss}, MapperAssignOut{*m, ids, ws.ent, status}, n,
                          ws.scan_scratch, ws.tmp, st);
    if (bid_marks)
        mapper_readback_kernel<true><<<grid, 256, 0, st>>>(*m, n, ws.ent, ws.miss, hash_indices, ws.tmp);
    else
        mapper_readback_kernel<false><<<grid, 256, 0, st>>>(*m, n, ws.ent, ws.miss, hash_indices, ws.tmp);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

// ============================================================================ SwapManager
struct SwapWs {
    int64_t* ent;
    int *miss, *first, *rank, *so_flag, *so_rank, *scan_scratch;
    int64_t *sweep_list, *so_key, *so_off;
    int64_t* tmp;  // {M, n_from_free, need, occupied_old, E, n_swapout}
    size_t bytes;
};
static SwapWs carve_swap(void* base, int64_t N, int64_t cache_size)
{
    WorkspaceCarver c(base);
    SwapWs w;
    const size_t n = static_cast<size_t>(N > 0 ? N : 1);
    const int64_t scan_n = cache_size > N ? cache_size : N;
    w.tmp = c.take<int64_t>(8);
    w.ent = c.take<int64_t>(n);
    w.miss = c.take<int>(n);
    w.first = c.take<int>(n);
    w.rank = c.take<int>(n);
    w.so_flag = c.take<int>(n);
    w.so_rank = c.take<int>(n);
    w.sweep_list = c.take<int64_t>(n);
    w.so_key = c.take<int64_t>(n);
    w.so_off = c.take<int64_t>(n);
    w.scan_scratch = c.take<int>(scan_scratch_ints(scan_n));
    w.bytes = c.used();
    return w;
}

// tmp[0] = M (number of new keys) is in place; decide how many come from the
// free tail and how many need the replacement sweep (swap_manager.cpp:90-100).
static __global__ void swap_plan_kernel(recsdk_swap_t s, int64_t* __restrict__ tmp)
{
    const int64_t M = tmp[0];
    const int64_t occupied = s.counters[0];
    const int64_t free_slots = s.cache_size - occupied;
    const int64_t from_free = M < free_slots ? M : free_slots;
    tmp[1] = from_free;
    tmp[2] = M - from_free;
    tmp[3] = occupied;
    tmp[4] = 0;
    tmp[5] = 0;
    s.counters[0] = occupied + from_free;
}

// Replacement sweep (swap_manager.cpp:104-118): candidate slots are visited in
// cyclic order from swap_idx; slot s can be replaced when version[s] < now-1.
// Virtual index v in [0, cache_size - mem_start) maps to the cyclic order.
__device__ __forceinline__ int64_t sweep_slot(const recsdk_swap_t& s, int64_t swap_idx, int64_t v)
{
    const int64_t x = swap_idx + v;
    return x < s.cache_size ? x : s.mem_start_offset + (x - s.cache_size);
}

static __global__ void __launch_bounds__(kScanThreads) sweep_reduce_kernel(recsdk_swap_t s, const int64_t* __restrict__ tmp,
                                                                           int* __restrict__ tile_sums)
{
    __shared__ int sm[33];
    if (tmp[2] <= 0) return;  // nothing to replace: whole kernel is a no-op
    const int64_t now = s.counters[1];
    int64_t swap_idx = s.counters[2];
    if (swap_idx >= s.cache_size) swap_idx = s.mem_start_offset;
    const int64_t span = s.cache_size - s.mem_start_offset;
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + static_cast<int64_t>(threadIdx.x) * kScanItems;
    int cnt = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
        const int64_t v = base + k;
        if (v < span) cnt += s.slot_version[sweep_slot(s, swap_idx, v)] < now - 1 ? 1 : 0;
    }
    int total;
    block_inclusive_scan(cnt, sm, &total);
    if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

static __global__ void __launch_bounds__(1024) sweep_tile_scan_kernel(int* __restrict__ tile_sums, int64_t tiles,
                                                                      int64_t* __restrict__ tmp,
                                                                      int64_t* __restrict__ status)
{
    __shared__ int sm[33];
    if (tmp[2] <= 0) return;
    int carry = 0;
    for (int64_t base = 0; base < tiles; base += blockDim.x) {
        const int64_t i = base + threadIdx.x;
        const int v = i < tiles ? tile_sums[i] : 0;
        int total;
        const int inc = block_inclusive_scan(v, sm, &total);
        if (i < tiles) tile_sums[i] = carry + inc - v;
        carry += total;
    }
    if (threadIdx.x == 0) {
        tmp[4] = carry;  // E: replaceable slots
        if (carry < tmp[2]) set_status(status, RECSDK_ERR_CACHE_TOO_SMALL, carry, tmp[2]);
    }
}

static __global__ void __launch_bounds__(kScanThreads) sweep_apply_kernel(recsdk_swap_t s, const int64_t* __restrict__ tmp,
                                                                          const int* __restrict__ tile_sums,
                                                                          int64_t* __restrict__ sweep_list, int64_t n)
{
    __shared__ int sm[33];
    const int64_t need = tmp[2];
    if (need <= 0) return;
    const int64_t now = s.counters[1];
    int64_t swap_idx = s.counters[2];
    if (swap_idx >= s.cache_size) swap_idx = s.mem_start_offset;
    const int64_t span = s.cache_size - s.mem_start_offset;
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + static_cast<int64_t>(threadIdx.x) * kScanItems;
    if (tile_sums[blockIdx.x] >= need) return;  // every candidate of this tile ranks beyond what is needed
    int f[kScanItems];
    int cnt = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
        const int64_t v = base + k;
        f[k] = (v < span && s.slot_version[sweep_slot(s, swap_idx, v)] < now - 1) ? 1 : 0;
        cnt += f[k];
    }
    int total;
    const int inc = block_inclusive_scan(cnt, sm, &total);
    int64_t run = tile_sums[blockIdx.x] + inc - cnt;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
        if (f[k]) {
            if (run < need && run < n) sweep_list[run] = sweep_slot(s, swap_idx, base + k);
            ++run;
        }
    }
}

// swap_manager.cpp:90-136 for the first occurrence of every new key
static __global__ void __launch_bounds__(256) swap_assign_kernel(recsdk_swap_t s, const int64_t* __restrict__ keys,
                                                                 int64_t n, const int64_t* __restrict__ ent,
                                                                 const int* __restrict__ first,
                                                                 const int* __restrict__ rank,
                                                                 const int64_t* __restrict__ tmp,
                                                                 const int64_t* __restrict__ sweep_list,
                                                                 int64_t* __restrict__ swapin_keys,
                                                                 int64_t* __restrict__ swapin_offs,
                                                                 int* __restrict__ so_flag, int64_t* __restrict__ so_key,
                                                                 int64_t* __restrict__ so_off)
{
    const int64_t from_free = tmp[1], occupied_old = tmp[3], E = tmp[4];
    const int64_t now = s.counters[1];
    RECSDK_GRID_STRIDE(i, n)
    {
        if (!first[i]) continue;
        const int64_t r = rank[i];
        const int64_t key = keys[i];
        int64_t slot;
        if (r < from_free) {
            slot = occupied_old + r;
        } else {
            const int64_t k = r - from_free;
            if (k >= E) continue;  // cacheSize_ too small, status already set
            slot = sweep_list[k];
            const int64_t old_key = s.slot_key[slot];
            const bool evicted_pos = s.slot_version[slot] == -2;
            if (old_key != -1) {
                const int64_t oe = ht_lookup<2>(s.table, s.hash_capacity, old_key);
                if (oe >= 0) {
                    s.table[oe * 2 + 1] = kValFree;
                    __threadfence();
                    s.table[oe * 2] = kTomb;
                }
            }
            if (!evicted_pos) {
                so_flag[k] = 1;
                so_key[k] = old_key;
                so_off[k] = slot;
            }
        }
        swapin_keys[r] = key;
        swapin_offs[r] = slot;
        s.table[ent[i] * 2 + 1] = slot;
        s.slot_key[slot] = key;
        s.slot_version[slot] = now;
    }
}

static __global__ void __launch_bounds__(256) swap_compact_out_kernel(int64_t n, const int* __restrict__ so_flag,
                                                                      const int* __restrict__ so_rank,
                                                                      const int64_t* __restrict__ so_key,
                                                                      const int64_t* __restrict__ so_off,
                                                                      int64_t* __restrict__ swapout_keys,
                                                                      int64_t* __restrict__ swapout_offs)
{
    RECSDK_GRID_STRIDE(k, n)
    {
        if (so_flag[k]) {
            swapout_keys[so_rank[k]] = so_key[k];
            swapout_offs[so_rank[k]] = so_off[k];
        }
    }
}

static __global__ void swap_finish_kernel(recsdk_swap_t s, const int64_t* __restrict__ tmp,
                                          const int64_t* __restrict__ sweep_list, int64_t* __restrict__ counts_out)
{
    const int64_t need = tmp[2] < tmp[4] ? tmp[2] : tmp[4];
    if (need > 0) s.counters[2] = sweep_list[need - 1] + 1;
    s.counters[1] += 1;  // nowVersion_++
    counts_out[0] = tmp[1] + need;
    counts_out[1] = tmp[5];
}

static __global__ void __launch_bounds__(256) swap_remove_kernel(recsdk_swap_t s, const int64_t* __restrict__ keys,
                                                                 int64_t n, const int64_t* __restrict__ n_dev)
{
    const int64_t m = n_dev != nullptr ? (*n_dev < n ? *n_dev : n) : n;
    RECSDK_GRID_STRIDE(i, m)
    {
        const int64_t key = keys[i];
        if (key < 0) continue;
        const int64_t e = ht_lookup<2>(s.table, s.hash_capacity, key);
        if (e < 0) continue;
        const int64_t slot = s.table[e * 2 + 1];
        if (slot >= 0 && slot < s.cache_size) {
            s.slot_version[slot] = -2;  // CAN_REUSE_KEY_VERSION
            s.slot_key[slot] = -1;      // INVALID_KEY
        }
        s.table[e * 2 + 1] = kValFree;
        __threadfence();
        s.table[e * 2] = kTomb;
    }
}

// ============================================================================ FeatureFilter
constexpr int64_t kTsNone = INT64_MIN;
constexpr int64_t kCountPresent = int64_t(1) << 62;

static __global__ void __launch_bounds__(256) filter_statistics_kernel(recsdk_filter_t f, const int64_t* __restrict__ keys,
                                                                       const int64_t* __restrict__ counts, int64_t n,
                                                                       int64_t* __restrict__ status)
{
    RECSDK_GRID_STRIDE(i, n)
    {
        const int64_t key = keys[i];
        if (key < 0) continue;
        int64_t c = counts != nullptr ? counts[i] : 1;
        if (c < 0) c = 0;
        const int64_t e = ht_find_or_insert<4>(f.table, f.hash_capacity, key);
        if (e < 0) {
            set_status(status, RECSDK_ERR_HASH_FULL, key, i);
            continue;
        }
        unsigned long long* cp = reinterpret_cast<unsigned long long*>(f.table + e * 4 + 1);
        atomicOr(cp, static_cast<unsigned long long>(kCountPresent));
        if (c) atomicAdd(cp, static_cast<unsigned long long>(c));
    }
}

static __global__ void __launch_bounds__(256) filter_count_filter_kernel(recsdk_filter_t f, int64_t* __restrict__ keys,
                                                                         int64_t n)
{
    RECSDK_GRID_STRIDE(i, n)
    {
        const int64_t key = keys[i];
        if (key < 0) continue;
        const int64_t e = ht_lookup<4>(f.table, f.hash_capacity, key);
        if (e < 0) continue;
        const int64_t c = f.table[e * 4 + 1];
        if ((c & kCountPresent) && static_cast<uint64_t>(c & ~kCountPresent) < static_cast<uint64_t>(f.admit_threshold))
            keys[i] = -1;
    }
}

static __global__ void __launch_bounds__(256) filter_count_of_kernel(recsdk_filter_t f, const int64_t* __restrict__ keys,
                                                                     int64_t n, int64_t* __restrict__ out)
{
    RECSDK_GRID_STRIDE(i, n)
    {
        int64_t r = -1;
        const int64_t key = keys[i];
        if (key >= 0) {
            const int64_t e = ht_lookup<4>(f.table, f.hash_capacity, key);
            if (e >= 0) {
                const int64_t c = f.table[e * 4 + 1];
                if (c & kCountPresent) r = c & ~kCountPresent;
            }
        }
        out[i] = r;
    }
}

// insert_or_assign in input order: the LAST occurrence of a key provides its timestamp
static __global__ void __launch_bounds__(256) filter_ts_bid_kernel(recsdk_filter_t f, const int64_t* __restrict__ keys,
                                                                   const int64_t* __restrict__ ts, int64_t n,
                                                                   int64_t* __restrict__ ent, int64_t* __restrict__ status)
{
    int64_t lmax = INT64_MIN;
    RECSDK_GRID_STRIDE(i, n)
    {
        const int64_t key = keys[i];
        int64_t e = -1;
        if (key >= 0) {
            e = ht_find_or_insert<4>(f.table, f.hash_capacity, key);
            if (e < 0) set_status(status, RECSDK_ERR_HASH_FULL, key, i);
            else atomic_max_i64(f.table + e * 4 + 3, i + 1);
        }
        ent[i] = e;
        lmax = ts[i] > lmax ? ts[i] : lmax;
    }
    // latestTimestamp_ = max(...): one atomic per warp
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        const int64_t other = __shfl_xor_sync(kFullMask, lmax, o);
        lmax = other > lmax ? other : lmax;
    }
    if ((threadIdx.x & 31) == 0 && lmax != INT64_MIN) atomic_max_i64(f.counters + 0, lmax);
}
static __global__ void __launch_bounds__(256) filter_ts_write_kernel(recsdk_filter_t f, const int64_t* __restrict__ ts,
                                                                     int64_t n, const int64_t* __restrict__ ent)
{
    RECSDK_GRID_STRIDE(i, n)
    {
        const int64_t e = ent[i];
        if (e >= 0 && f.table[e * 4 + 3] == i + 1) f.table[e * 4 + 2] = ts[i];
    }
}
static __global__ void __launch_bounds__(256) filter_ts_reset_kernel(recsdk_filter_t f, int64_t n,
                                                                     const int64_t* __restrict__ ent)
{
    RECSDK_GRID_STRIDE(i, n)
    {
        const int64_t e = ent[i];
        if (e >= 0) f.table[e * 4 + 3] = 0;
    }
}
// feature_filter.cpp:45-49: evict when recordTsBatchId_ > 0 && (id + 1) % interval == 0
static __global__ void filter_tick_kernel(recsdk_filter_t f, int64_t* __restrict__ tmp)
{
    const int64_t id = f.counters[1];
    int go = 0;
    if (f.evict_step_interval > 0 && id > 0 && (id + 1) % f.evict_step_interval == 0 && f.evict_threshold != 0) go = 1;
    tmp[0] = go;
    f.counters[1] = id + 1;
}
// feature_filter.cpp:52-80
static __global__ void __launch_bounds__(256) filter_evict_kernel(recsdk_filter_t f, const int64_t* __restrict__ tmp,
                                                                  int64_t* __restrict__ evict_keys, int64_t evict_cap,
                                                                  int64_t* __restrict__ status)
{
    if (tmp[0] == 0) return;
    const int64_t latest = f.counters[0];
    RECSDK_GRID_STRIDE(e, f.hash_capacity)
    {
        const int64_t key = f.table[e * 4];
        if (key < 0) continue;
        const int64_t t = f.table[e * 4 + 2];
        if (t == kTsNone) continue;
        if (latest - t > f.evict_threshold) {
            const unsigned long long pos = atomicAdd(reinterpret_cast<unsigned long long*>(f.counters + 2), 1ull);
            if (static_cast<int64_t>(pos) < evict_cap)
                evict_keys[pos] = key;
            else
                set_status(status, RECSDK_ERR_TOO_LARGE, static_cast<int64_t>(pos), evict_cap);
            f.table[e * 4 + 1] = 0;
            f.table[e * 4 + 2] = kTsNone;
            f.table[e * 4 + 3] = 0;
            __threadfence();
            f.table[e * 4] = kTomb;
        }
    }
}
static __global__ void filter_clear_evict_kernel(recsdk_filter_t f) { f.counters[2] = 0; }


// ============================================================================ load statistics and tombstone compaction
// Erased keys leave TOMBSTONE entries behind (a lookup must walk past them), and nothing in the batch phases turns
// one back into EMPTY: under steady churn -- evictions, cache replacement -- the EMPTY entries only become fewer,
// and a lookup of an absent key stops only at an EMPTY entry.  So the tables are rebuilt now and then: the live
// entries are collected into scratch, the table is cleared, the entries are inserted again.  The collect phase
// counts; when the live entries do not fit the scratch the clear and re-insert phases do nothing (they read the
// count on the device) and the status block says so.  Must not run concurrently with other work on the table.
template <int STRIDE>
static __global__ void __launch_bounds__(256) kt_stats_kernel(const int64_t* __restrict__ table, int64_t cap,
                                                              int64_t* __restrict__ stats)
{
    int64_t live = 0, tomb = 0, maxd = 0;
    const uint64_t mask = static_cast<uint64_t>(cap) - 1;
    RECSDK_GRID_STRIDE(e, cap)
    {
        const int64_t k = table[e * STRIDE];
        if (k == kTomb) ++tomb;
        if (k >= 0) {
            ++live;
            const int64_t d = static_cast<int64_t>((static_cast<uint64_t>(e) - (mix64(static_cast<uint64_t>(k)) & mask)) & mask);
            maxd = d > maxd ? d : maxd;
        }
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        live += __shfl_down_sync(kFullMask, live, o);
        tomb += __shfl_down_sync(kFullMask, tomb, o);
        const int64_t other = __shfl_down_sync(kFullMask, maxd, o);
        maxd = other > maxd ? other : maxd;
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(reinterpret_cast<unsigned long long*>(stats), static_cast<unsigned long long>(live));
        atomicAdd(reinterpret_cast<unsigned long long*>(stats + 1), static_cast<unsigned long long>(tomb));
        atomic_max_i64(stats + 2, maxd);
    }
}

template <int STRIDE>
static __global__ void __launch_bounds__(256) kt_collect_kernel(const int64_t* __restrict__ table, int64_t cap,
                                                                int64_t* __restrict__ list, int64_t max_live,
                                                                int64_t* __restrict__ counter)
{
    RECSDK_GRID_STRIDE(e, cap)
    {
        if (table[e * STRIDE] < 0) continue;
        const int64_t i = static_cast<int64_t>(atomicAdd(reinterpret_cast<unsigned long long*>(counter), 1ull));
        if (i >= max_live) continue;
#pragma unroll
        for (int w = 0; w < STRIDE; ++w) list[i * STRIDE + w] = table[e * STRIDE + w];
    }
}

template <int STRIDE>
static __global__ void __launch_bounds__(256) kt_clear_kernel(int64_t* __restrict__ table, int64_t cap, int64_t max_live,
                                                              const int64_t* __restrict__ counter, int64_t* status)
{
    if (*counter > max_live) {
        if (blockIdx.x == 0 && threadIdx.x == 0) set_status(status, RECSDK_ERR_WORKSPACE, *counter, max_live);
        return;
    }
    RECSDK_GRID_STRIDE(e, cap)
    {
        table[e * STRIDE] = kEmpty;
        if (STRIDE == 2) table[e * STRIDE + 1] = kValFree;
        if (STRIDE == 4) {
            table[e * STRIDE + 1] = 0;
            table[e * STRIDE + 2] = kTsNone;
            table[e * STRIDE + 3] = 0;
        }
    }
}

template <int STRIDE>
static __global__ void __launch_bounds__(256) kt_reinsert_kernel(int64_t* __restrict__ table, int64_t cap,
                                                                 const int64_t* __restrict__ list, int64_t max_live,
                                                                 const int64_t* __restrict__ counter, int64_t* status)
{
    const int64_t n = *counter;
    if (n > max_live) return;
    RECSDK_GRID_STRIDE(i, n)
    {
        const int64_t e = ht_insert<STRIDE>(table, cap, list[i * STRIDE]);
        if (e < 0) {
            set_status(status, RECSDK_ERR_HASH_FULL, list[i * STRIDE], i);
            continue;
        }
#pragma unroll
        for (int w = 1; w < STRIDE; ++w) table[e * STRIDE + w] = list[i * STRIDE + w];
    }
}

}  // namespace recsdk
using namespace recsdk;

extern "C" int recsdk_key_table_stats(const int64_t* table, int64_t hash_capacity, int32_t entry_words, int64_t* stats_out,
                                      void* stream)
{
    if (!table || !stats_out || !is_pow2(hash_capacity) || (entry_words != 2 && entry_words != 4)) return RECSDK_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaMemsetAsync(stats_out, 0, 4 * sizeof(int64_t), st);
    const int grid = grid_for(hash_capacity, 256, 8);
    if (entry_words == 2) kt_stats_kernel<2><<<grid, 256, 0, st>>>(table, hash_capacity, stats_out);
    else kt_stats_kernel<4><<<grid, 256, 0, st>>>(table, hash_capacity, stats_out);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" size_t recsdk_key_table_rebuild_workspace_bytes(int64_t max_live, int32_t entry_words)
{
    return align_up(8 * sizeof(int64_t)) + align_up(static_cast<size_t>(max_live > 0 ? max_live : 1) * entry_words * sizeof(int64_t));
}

extern "C" int recsdk_key_table_rebuild(int64_t* table, int64_t hash_capacity, int32_t entry_words, int64_t max_live,
                                        int64_t* dev_status, void* workspace, size_t workspace_bytes, void* stream)
{
    if (!table || !is_pow2(hash_capacity) || (entry_words != 2 && entry_words != 4) || max_live <= 0) return RECSDK_ERR_INVALID_ARG;
    if (!workspace || workspace_bytes < recsdk_key_table_rebuild_workspace_bytes(max_live, entry_words)) return RECSDK_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int64_t* counter = static_cast<int64_t*>(workspace);
    int64_t* list = reinterpret_cast<int64_t*>(static_cast<char*>(workspace) + align_up(8 * sizeof(int64_t)));
    cudaMemsetAsync(counter, 0, 8 * sizeof(int64_t), st);
    const int grid = grid_for(hash_capacity, 256, 8), grid2 = grid_for(max_live, 256, 8);
    if (entry_words == 2) {
        kt_collect_kernel<2><<<grid, 256, 0, st>>>(table, hash_capacity, list, max_live, counter);
        kt_clear_kernel<2><<<grid, 256, 0, st>>>(table, hash_capacity, max_live, counter, dev_status);
        kt_reinsert_kernel<2><<<grid2, 256, 0, st>>>(table, hash_capacity, list, max_live, counter, dev_status);
    } else {
        kt_collect_kernel<4><<<grid, 256, 0, st>>>(table, hash_capacity, list, max_live, counter);
        kt_clear_kernel<4><<<grid, 256, 0, st>>>(table, hash_capacity, max_live, counter, dev_status);
        kt_reinsert_kernel<4><<<grid2, 256, 0, st>>>(table, hash_capacity, list, max_live, counter, dev_status);
    }
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

namespace recsdk {
}  // namespace recsdk

using namespace recsdk;

// ---------------------------------------------------------------------------- C ABI: mapper
extern "C" size_t recsdk_mapper_table_bytes(int64_t hash_capacity) { return static_cast<size_t>(hash_capacity) * 16; }

extern "C" int recsdk_mapper_init(const recsdk_mapper_t* m, void* stream)
{
    if (!m || !m->table || !m->slot_key || !m->mark || !m->counters || !is_pow2(m->hash_capacity) ||
        m->init_max_index <= 0)
        return RECSDK_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    fill_i64_kernel<<<grid_for(m->hash_capacity, 256), 256, 0, st>>>(m->table, m->hash_capacity, 2, kEmpty, kValFree, 0, 0);
    fill_i64_kernel<<<grid_for(m->init_max_index, 256), 256, 0, st>>>(m->slot_key, m->init_max_index, 1, -1, 0, 0, 0);
    fill_i32_kernel<<<grid_for(m->init_max_index, 256), 256, 0, st>>>(m->mark, m->init_max_index, kMarkFree);
    set4_kernel<<<1, 1, 0, st>>>(m->counters, 0, 0, 0, 0);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" size_t recsdk_mapper_workspace_bytes(int64_t n)
{
    const size_t a = carve_mapper(nullptr, n).bytes;
    const size_t b = recsdk_unique_sorted_workspace_bytes(n);
    return a + b;
}

extern "C" int recsdk_mapper_unique_out(const recsdk_mapper_t* m, const int64_t* ids, int64_t* hash_indices,
                                        int64_t seg_start, int64_t seg_len, int64_t* unique, int64_t* unique_ids,
                                        int64_t* unique_inverse, int64_t* unique_offset, int64_t table_id,
                                        int64_t* dev_status, void* workspace, size_t workspace_bytes, void* stream)
{
    if (!m || seg_start < 0 || seg_len < 0 || table_id < 0 || !unique_offset) return RECSDK_ERR_INVALID_ARG;
    if (seg_len >= kMarkFree) return RECSDK_ERR_TOO_LARGE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (seg_len == 0) {
        empty_segment_kernel<<<1, 1, 0, st>>>(unique_offset, table_id);
        RECSDK_CUDA_CHECK_LAUNCH();
        return RECSDK_OK;
    }
    if (!ids || !hash_indices || !unique || !unique_ids || !unique_inverse) return RECSDK_ERR_INVALID_ARG;
    if (!workspace) return RECSDK_ERR_WORKSPACE;
    const MapperWs ws = carve_mapper(workspace, seg_len);
    if (ws.bytes > workspace_bytes) return RECSDK_ERR_WORKSPACE;
    const int64_t* seg_ids = ids + seg_start;
    int64_t* seg_hi = hash_indices + seg_start;
    int rc = mapper_map(m, seg_ids, seg_len, seg_hi, dev_status, ws, st, true);
    if (rc != RECSDK_OK) return rc;
    const int grid = grid_for(seg_len, 256);
    device_scan_fn<false>(HoldsMarkIn{seg_hi, m->mark, m->init_max_index}, FlagRankOut{ws.first, ws.rank}, seg_len,
                          ws.scan_scratch, ws.tmp + 1, st);
    uniq_write_kernel<<<grid, 256, 0, st>>>(seg_hi, seg_len, m->mark, m->init_max_index, ws.rank, m->slot_key, unique,
                                            unique_ids, unique_inverse + seg_start, unique_offset, table_id, ws.tmp);
    uniq_reset_kernel<<<grid, 256, 0, st>>>(seg_hi, seg_len, m->mark, m->init_max_index);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_mapper_ids2indices_unique(const recsdk_mapper_t* m, const int64_t* ids, int64_t n,
                                                int64_t* hash_indices, int64_t* unique_out, int64_t* inverse_out,
                                                int64_t* num_unique_out, int64_t* dev_status, void* workspace,
                                                size_t workspace_bytes, void* stream)
{
    if (!m || n < 0) return RECSDK_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n == 0) {
        if (num_unique_out) cudaMemsetAsync(num_unique_out, 0, sizeof(int64_t), st);
        return RECSDK_OK;
    }
    if (!ids || !hash_indices || !unique_out || !inverse_out) return RECSDK_ERR_INVALID_ARG;
    if (!workspace) return RECSDK_ERR_WORKSPACE;
    const MapperWs ws = carve_mapper(workspace, n);
    const size_t usz = recsdk_unique_sorted_workspace_bytes(n);
    if (ws.bytes + usz > workspace_bytes) return RECSDK_ERR_WORKSPACE;
    int rc = mapper_map(m, ids, n, hash_indices, dev_status, ws, st);
    if (rc != RECSDK_OK) return rc;
    int bits = 1;
    while (bits < 63 && (int64_t(1) << bits) < m->init_max_index) ++bits;
    return recsdk_unique_sorted(hash_indices, n, bits, unique_out, inverse_out, num_unique_out,
                                static_cast<char*>(workspace) + ws.bytes, usz, stream);
}

// ---------------------------------------------------------------------------- C ABI: swap manager
extern "C" int recsdk_swap_init(const recsdk_swap_t* s, void* stream)
{
    if (!s || !s->table || !s->slot_key || !s->slot_version || !s->counters || !is_pow2(s->hash_capacity) ||
        s->cache_size <= 0 || s->mem_start_offset < 0 || s->mem_start_offset > s->cache_size)
        return RECSDK_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    fill_i64_kernel<<<grid_for(s->hash_capacity, 256), 256, 0, st>>>(s->table, s->hash_capacity, 2, kEmpty, kValFree, 0, 0);
    // std::vector<KeyVersion>::resize value-initialises {key 0, version 0} (swap_manager.cpp:28)
    fill_i64_kernel<<<grid_for(s->cache_size, 256), 256, 0, st>>>(s->slot_key, s->cache_size, 1, 0, 0, 0, 0);
    fill_i64_kernel<<<grid_for(s->cache_size, 256), 256, 0, st>>>(s->slot_version, s->cache_size, 1, 0, 0, 0, 0);
    set4_kernel<<<1, 1, 0, st>>>(s->counters, s->mem_start_offset, 0, s->mem_start_offset, 0);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" size_t recsdk_swap_workspace_bytes(int64_t n, int64_t cache_size) { return carve_swap(nullptr, n, cache_size).bytes; }

extern "C" int recsdk_swap_compute(const recsdk_swap_t* s, const int64_t* keys, int64_t n, int64_t* batch_offs,
                                   int64_t* swapin_keys, int64_t* swapin_offs, int64_t* swapout_keys,
                                   int64_t* swapout_offs, int64_t* counts_out, int64_t* dev_status, void* workspace,
                                   size_t workspace_bytes, void* stream)
{
    if (!s || n < 0 || !counts_out) return RECSDK_ERR_INVALID_ARG;
    if (n >= kMarkFree || s->cache_size >= (int64_t(1) << 31)) return RECSDK_ERR_TOO_LARGE;
    if (n > 0 && (!keys || !batch_offs || !swapin_keys || !swapin_offs || !swapout_keys || !swapout_offs))
        return RECSDK_ERR_INVALID_ARG;
    if (!workspace) return RECSDK_ERR_WORKSPACE;
    const SwapWs ws = carve_swap(workspace, n, s->cache_size);
    if (ws.bytes > workspace_bytes) return RECSDK_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = grid_for(n > 0 ? n : 1, 256);
    if (n > 0) {
        phase_find_or_claim_kernel<1><<<grid_for(n, 256 / kProbeLanes), 256, 0, st>>>(
            s->table, s->hash_capacity, keys, n, batch_offs, ws.ent, ws.miss, s->slot_version, s->counters, dev_status);
    }
    device_scan_fn<false>(WonBidIn{s->table, ws.ent, ws.miss}, FlagRankOut{ws.first, ws.rank}, n, ws.scan_scratch, ws.tmp,
                          st);
    swap_plan_kernel<<<1, 1, 0, st>>>(*s, ws.tmp);
    if (n > 0) {
        const int64_t span = s->cache_size - s->mem_start_offset;
        const int64_t tiles = scan_num_tiles(span);
        sweep_reduce_kernel<<<static_cast<unsigned>(tiles), kScanThreads, 0, st>>>(*s, ws.tmp, ws.scan_scratch);
        sweep_tile_scan_kernel<<<1, 1024, 0, st>>>(ws.scan_scratch, tiles, ws.tmp, dev_status);
        sweep_apply_kernel<<<static_cast<unsigned>(tiles), kScanThreads, 0, st>>>(*s, ws.tmp, ws.scan_scratch, ws.sweep_list, n);
        cudaMemsetAsync(ws.so_flag, 0, static_cast<size_t>(n) * sizeof(int), st);
        swap_assign_kernel<<<grid, 256, 0, st>>>(*s, keys, n, ws.ent, ws.first, ws.rank, ws.tmp, ws.sweep_list,
                                                 swapin_keys, swapin_offs, ws.so_flag, ws.so_key, ws.so_off);
        device_scan<false>(ws.so_flag, ws.so_rank, n, ws.scan_scratch, ws.tmp + 5, st);
        swap_compact_out_kernel<<<grid, 256, 0, st>>>(n, ws.so_flag, ws.so_rank, ws.so_key, ws.so_off, swapout_keys,
                                                      swapout_offs);
        phase_readback_kernel<<<grid, 256, 0, st>>>(s->table, n, ws.ent, ws.miss, batch_offs);
    }
    swap_finish_kernel<<<1, 1, 0, st>>>(*s, ws.tmp, ws.sweep_list, counts_out);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_swap_remove(const recsdk_swap_t* s, const int64_t* keys, int64_t n, const int64_t* n_keys_dev,
                                  void* stream)
{
    if (!s || n < 0) return RECSDK_ERR_INVALID_ARG;
    if (n == 0) return RECSDK_OK;
    if (!keys) return RECSDK_ERR_INVALID_ARG;
    swap_remove_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(*s, keys, n, n_keys_dev);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

// ---------------------------------------------------------------------------- C ABI: feature filter
extern "C" int recsdk_filter_init(const recsdk_filter_t* f, void* stream)
{
    if (!f || !f->table || !f->counters || !is_pow2(f->hash_capacity)) return RECSDK_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    fill_i64_kernel<<<grid_for(f->hash_capacity, 256), 256, 0, st>>>(f->table, f->hash_capacity, 4, kEmpty, 0, kTsNone, 0);
    set4_kernel<<<1, 1, 0, st>>>(f->counters, 0, 0, 0, 0);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" size_t recsdk_filter_workspace_bytes(int64_t n)
{
    return align_up(8 * sizeof(int64_t)) + align_up(static_cast<size_t>(n > 0 ? n : 1) * sizeof(int64_t));
}

extern "C" int recsdk_filter_statistics(const recsdk_filter_t* f, const int64_t* keys, const int64_t* counts, int64_t n,
                                        int64_t* dev_status, void* stream)
{
    if (!f || n < 0) return RECSDK_ERR_INVALID_ARG;
    if (n == 0) return RECSDK_OK;
    if (!keys) return RECSDK_ERR_INVALID_ARG;
    filter_statistics_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(*f, keys, counts, n, dev_status);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_filter_count_filter(const recsdk_filter_t* f, int64_t* keys_inout, int64_t n, void* stream)
{
    if (!f || n < 0) return RECSDK_ERR_INVALID_ARG;
    if (n == 0 || f->admit_threshold == -1) return RECSDK_OK;  // IsAdmitEnabled, feature_filter.cpp:146-148
    if (!keys_inout) return RECSDK_ERR_INVALID_ARG;
    filter_count_filter_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(*f, keys_inout, n);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_filter_record_timestamp(const recsdk_filter_t* f, const int64_t* keys, const int64_t* ts, int64_t n,
                                              int64_t* evict_keys, int64_t evict_capacity, int64_t* dev_status,
                                              void* workspace, size_t workspace_bytes, void* stream)
{
    if (!f || n < 0) return RECSDK_ERR_INVALID_ARG;
    if (n > 0 && (!keys || !ts)) return RECSDK_ERR_INVALID_ARG;
    if (!workspace || workspace_bytes < recsdk_filter_workspace_bytes(n)) return RECSDK_ERR_WORKSPACE;
    if (f->evict_threshold != 0 && f->evict_step_interval > 0 && (!evict_keys || evict_capacity <= 0))
        return RECSDK_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    WorkspaceCarver c(workspace);
    int64_t* tmp = c.take<int64_t>(8);
    int64_t* ent = c.take<int64_t>(static_cast<size_t>(n > 0 ? n : 1));
    if (n > 0) {
        const int grid = grid_for(n, 256);
        filter_ts_bid_kernel<<<grid, 256, 0, st>>>(*f, keys, ts, n, ent, dev_status);
        filter_ts_write_kernel<<<grid, 256, 0, st>>>(*f, ts, n, ent);
        filter_ts_reset_kernel<<<grid, 256, 0, st>>>(*f, n, ent);
    }
    filter_tick_kernel<<<1, 1, 0, st>>>(*f, tmp);
    if (f->evict_threshold != 0 && f->evict_step_interval > 0)
        filter_evict_kernel<<<grid_for(f->hash_capacity, 256), 256, 0, st>>>(*f, tmp, evict_keys, evict_capacity, dev_status);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_filter_clear_evict(const recsdk_filter_t* f, void* stream)
{
    if (!f) return RECSDK_ERR_INVALID_ARG;
    filter_clear_evict_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(*f);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_filter_count_of(const recsdk_filter_t* f, const int64_t* keys, int64_t n, int64_t* count_out,
                                      void* stream)
{
    if (!f || n < 0) return RECSDK_ERR_INVALID_ARG;
    if (n == 0) return RECSDK_OK;
    if (!keys || !count_out) return RECSDK_ERR_INVALID_ARG;
    filter_count_of_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(*f, keys, n, count_out);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}
