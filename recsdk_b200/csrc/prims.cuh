// Device-wide building blocks written for this library: exclusive/inclusive
// int32 scan and a stable LSD radix sort of (key, 32-bit value) pairs.
// Both are multi-kernel, allocation-free (scratch comes from the caller) and
// use no inter-block spin waits.
#pragma once
#include "common.cuh"

namespace recsdk {

// ----------------------------------------------------------------------------
// Block-level helpers
// ----------------------------------------------------------------------------
__device__ __forceinline__ int warp_inclusive_scan(int v)
{
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(kFullMask, v, o);
        if ((threadIdx.x & 31) >= o) v += n;
    }
    return v;
}

// Inclusive scan across a block of up to 1024 threads; `smem` needs 33 ints.
// Returns the inclusive prefix of `v`; *total receives the block sum.
__device__ __forceinline__ int block_inclusive_scan(int v, int* smem, int* total)
{
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    int inc = warp_inclusive_scan(v);
    if (lane == 31) smem[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        int w = lane < nw ? smem[lane] : 0;
        int winc = warp_inclusive_scan(w);
        smem[lane] = winc - w;  // exclusive prefix of warp sums
        if (lane == 31) smem[32] = winc;
    }
    __syncthreads();
    inc += smem[wid];
    *total = smem[32];
    __syncthreads();
    return inc;
}

// ----------------------------------------------------------------------------
// Device-wide int32 scan: reduce per tile -> scan of tile sums (one block) ->
// apply.  Tile = 256 threads x 8 items.
// ----------------------------------------------------------------------------
constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;

static inline int64_t scan_num_tiles(int64_t n) { return ceil_div(n > 0 ? n : 1, kScanTile); }
// scratch ints needed by device_scan
static inline size_t scan_scratch_ints(int64_t n) { return static_cast<size_t>(scan_num_tiles(n)) + 8; }

static __global__ void __launch_bounds__(kScanThreads) scan_reduce_kernel(const int* __restrict__ in, int64_t n,
                                                                   int* __restrict__ tile_sums)
{
    __shared__ int sm[33];
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + static_cast<int64_t>(threadIdx.x) * kScanItems;
    int s = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k)
        if (base + k < n) s += in[base + k];
    int total;
    block_inclusive_scan(s, sm, &total);
    if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

// In place exclusive scan of `m` tile sums by one block; total -> *total_out (int64, optional).
static __global__ void __launch_bounds__(1024) scan_tile_sums_kernel(int* __restrict__ tile_sums, int64_t m,
                                                              int64_t* __restrict__ total_out)
{
    __shared__ int sm[33];
    int carry = 0;
    for (int64_t base = 0; base < m; base += blockDim.x) {
        int64_t i = base + threadIdx.x;
        int v = i < m ? tile_sums[i] : 0;
        int total;
        int inc = block_inclusive_scan(v, sm, &total);
        if (i < m) tile_sums[i] = carry + inc - v;
        carry += total;
    }
    if (threadIdx.x == 0 && total_out != nullptr) *total_out = carry;
}

// Up to this many tiles the apply kernels fold the scan of the tile sums into themselves (every block adds up the
// raw sums of the tiles before it -- a few KB out of L2 -- and the last block publishes the grand total): one launch
// less on the short, launch-bound scans.  Larger inputs keep the one-block scan of the sums between the two passes.
constexpr int64_t kScanFoldTiles = 1024;

// Exclusive offset of this block's tile.  `fold` == 0: tile_sums was scanned by scan_tile_sums_kernel.  Else: raw
// sums; `own_total` is this tile's sum, `sm` 33 ints of shared memory.
__device__ __forceinline__ int scan_tile_offset(const int* __restrict__ tile_sums, int fold, int own_total, int* sm,
                                                int64_t* __restrict__ total_out)
{
    if (!fold) return tile_sums[blockIdx.x];
    int part = 0;
    for (int t = threadIdx.x; t < static_cast<int>(blockIdx.x); t += blockDim.x) part += tile_sums[t];
    int before;
    block_inclusive_scan(part, sm, &before);
    if (total_out != nullptr && blockIdx.x == gridDim.x - 1 && threadIdx.x == 0)
        *total_out = static_cast<int64_t>(before) + own_total;
    return before;
}

template <bool INCLUSIVE>
__global__ void __launch_bounds__(kScanThreads) scan_apply_kernel(const int* __restrict__ in, int* __restrict__ out,
                                                                  int64_t n, const int* __restrict__ tile_sums,
                                                                  int fold, int64_t* __restrict__ total_out)
{
    __shared__ int sm[33];
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + static_cast<int64_t>(threadIdx.x) * kScanItems;
    int v[kScanItems];
    int s = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
        v[k] = (base + k < n) ? in[base + k] : 0;
        s += v[k];
    }
    int total;
    int inc = block_inclusive_scan(s, sm, &total);
    int run = scan_tile_offset(tile_sums, fold, total, sm, total_out) + inc - s;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
        if (base + k < n) out[base + k] = INCLUSIVE ? run + v[k] : run;
        run += v[k];
    }
}

// out may alias in.  scratch: scan_scratch_ints(n) ints.  total_out: device int64 or nullptr.
template <bool INCLUSIVE>
static inline void device_scan(const int* in, int* out, int64_t n, int* scratch, int64_t* total_out, cudaStream_t st)
{
    if (n <= 0) {
        if (total_out) cudaMemsetAsync(total_out, 0, sizeof(int64_t), st);
        return;
    }
    const int64_t tiles = scan_num_tiles(n);
    const int fold = tiles <= kScanFoldTiles ? 1 : 0;
    scan_reduce_kernel<<<static_cast<unsigned>(tiles), kScanThreads, 0, st>>>(in, n, scratch);
    if (!fold) scan_tile_sums_kernel<<<1, 1024, 0, st>>>(scratch, tiles, total_out);
    scan_apply_kernel<INCLUSIVE><<<static_cast<unsigned>(tiles), kScanThreads, 0, st>>>(in, out, n, scratch, fold, total_out);
}

// Functor form of the scan: the input is computed on the fly (`in(i)` -> int) and
// the result is consumed on the fly (`out(i, item, prefix, n)`), so flag arrays and
// the kernels that would write/read them disappear.
// `n_dev` (optional, device): the number of items when only the device knows it; `n` is then the capacity the
// grid was sized for and items at or past *n_dev do not exist.
__device__ __forceinline__ int64_t effective_n(int64_t n, const int64_t* __restrict__ n_dev)
{
    if (n_dev == nullptr) return n;
    const int64_t d = *n_dev;
    return d < n ? (d < 0 ? 0 : d) : n;
}

template <typename InFn>
__global__ void __launch_bounds__(kScanThreads) scan_reduce_fn_kernel(InFn in, int64_t n, int* __restrict__ tile_sums,
                                                                      const int64_t* __restrict__ n_dev)
{
    __shared__ int sm[33];
    n = effective_n(n, n_dev);
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + static_cast<int64_t>(threadIdx.x) * kScanItems;
    int s = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k)
        if (base + k < n) s += in(base + k);
    int total;
    block_inclusive_scan(s, sm, &total);
    if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

template <bool INCLUSIVE, typename InFn, typename OutFn>
__global__ void __launch_bounds__(kScanThreads) scan_apply_fn_kernel(InFn in, OutFn out, int64_t n,
                                                                     const int* __restrict__ tile_sums,
                                                                     const int64_t* __restrict__ n_dev, int fold,
                                                                     int64_t* __restrict__ total_out)
{
    __shared__ int sm[33];
    n = effective_n(n, n_dev);
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + static_cast<int64_t>(threadIdx.x) * kScanItems;
    int v[kScanItems];
    int s = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
        v[k] = (base + k < n) ? in(base + k) : 0;
        s += v[k];
    }
    int total;
    int inc = block_inclusive_scan(s, sm, &total);
    int run = scan_tile_offset(tile_sums, fold, total, sm, total_out) + inc - s;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
        if (base + k < n) out(base + k, v[k], INCLUSIVE ? run + v[k] : run, n);
        run += v[k];
    }
}

template <bool INCLUSIVE, typename InFn, typename OutFn>
static inline void device_scan_fn(InFn in, OutFn out, int64_t n, int* scratch, int64_t* total_out, cudaStream_t st,
                                  const int64_t* n_dev = nullptr)
{
    if (n <= 0) {
        if (total_out) cudaMemsetAsync(total_out, 0, sizeof(int64_t), st);
        return;
    }
    const int64_t tiles = scan_num_tiles(n);
    const int fold = tiles <= kScanFoldTiles ? 1 : 0;
    scan_reduce_fn_kernel<InFn><<<static_cast<unsigned>(tiles), kScanThreads, 0, st>>>(in, n, scratch, n_dev);
    if (!fold) scan_tile_sums_kernel<<<1, 1024, 0, st>>>(scratch, tiles, total_out);
    scan_apply_fn_kernel<INCLUSIVE, InFn, OutFn><<<static_cast<unsigned>(tiles), kScanThreads, 0, st>>>(in, out, n, scratch,
                                                                                                       n_dev, fold, total_out);
}

// ----------------------------------------------------------------------------
// Stable LSD radix sort of (key, uint32 value) pairs, 8, 9 or 10 bits per pass
// (the smallest digit that gives the fewest passes, e.g. 27-bit keys: 3 passes of
// 9 bits instead of 4 of 8; 28..30-bit keys: 3 passes of 10 bits).
// Per pass: tile histograms -> per-digit scan across tiles -> stable scatter
// (warp match-any ranking).  Tile = 256 threads x 8 items; warp w owns the
// contiguous 256 items [w*256, (w+1)*256) of the tile, taken 32 at a time, so
// the order inside a digit is the input order.
// ----------------------------------------------------------------------------
constexpr int kSortThreads = 256;
constexpr int kSortRounds = 8;
constexpr int kSortTile = kSortThreads * kSortRounds;  // 2048
constexpr int kMaxRadix = 1024;

static inline int64_t sort_num_tiles(int64_t n) { return ceil_div(n > 0 ? n : 1, kSortTile); }
// uint32 scratch needed: histogram [radix][tiles] + digit totals [radix]
static inline size_t sort_scratch_u32(int64_t n) { return static_cast<size_t>(sort_num_tiles(n)) * kMaxRadix + kMaxRadix; }
// Fused mode (see radix_sort_pairs_fused): one histogram per pass, all zeroed up front and filled by the kernel
// that PRODUCES that pass's input, so no pass reads its keys twice.
constexpr int kMaxSortPasses = 8;
static inline size_t sort_scratch_u32_fused(int64_t n)
{
    return static_cast<size_t>(sort_num_tiles(n)) * kMaxRadix * kMaxSortPasses + kMaxRadix;
}

// What the producer of a pass's input adds for the element it writes at position `pos`: one count in the
// histogram cell (digit of the key in that pass, tile of pos).
struct SortHistSink {
    uint32_t* hist;  // [radix][tiles] of the pass that will read the keys; nullptr = off
    int64_t tiles;
    int shift;
    uint32_t mask;
    // Called by ALL lanes of a warp (valid = this lane carries an element): lanes that hit the same cell --
    // the usual case for the runs of equal keys a skewed batch has -- are combined into one atomic.
    template <typename KeyT>
    __device__ __forceinline__ void add_warp(bool valid, KeyT key, int64_t pos) const
    {
        if (hist == nullptr) return;
        const unsigned lane = threadIdx.x & 31;
        const unsigned cell = valid ? static_cast<unsigned>(static_cast<int64_t>((key >> shift) & mask) * tiles + pos / kSortTile)
                                    : 0xffffffffu - lane;
        const unsigned peers = __match_any_sync(kFullMask, cell);
        if (valid && (peers & lanemask_lt()) == 0) atomicAdd(hist + cell, static_cast<uint32_t>(__popc(peers)));
    }
};

template <typename KeyT, int BITS>
__global__ void __launch_bounds__(kSortThreads) sort_hist_kernel(const KeyT* __restrict__ keys, int64_t n, int shift,
                                                                 uint32_t* __restrict__ hist, int64_t tiles)
{
    constexpr int RADIX = 1 << BITS;
    __shared__ uint32_t h[RADIX];
    for (int d = threadIdx.x; d < RADIX; d += kSortThreads) h[d] = 0;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t tile0 = static_cast<int64_t>(blockIdx.x) * kSortTile + warp * (kSortRounds * 32);
#pragma unroll
    for (int r = 0; r < kSortRounds; ++r) {
        const int64_t i = tile0 + r * 32 + lane;
        const bool valid = i < n;
        const unsigned tag = valid ? static_cast<unsigned>((keys[i] >> shift) & (RADIX - 1)) : (RADIX + lane);
        // one shared-memory atomic per distinct digit in the warp, not per item
        const unsigned peers = __match_any_sync(kFullMask, tag);
        if (valid && (peers & lanemask_lt()) == 0) atomicAdd(&h[tag], static_cast<uint32_t>(__popc(peers)));
    }
    __syncthreads();
    for (int d = threadIdx.x; d < RADIX; d += kSortThreads) hist[static_cast<int64_t>(d) * tiles + blockIdx.x] = h[d];
}

// One block per digit: exclusive scan of hist[d][0..tiles) in place, total -> totals[d].
static __global__ void __launch_bounds__(256) sort_scan_kernel(uint32_t* __restrict__ hist, int64_t tiles,
                                                        uint32_t* __restrict__ totals)
{
    __shared__ int sm[33];
    uint32_t* row = hist + static_cast<int64_t>(blockIdx.x) * tiles;
    int carry = 0;
    for (int64_t base = 0; base < tiles; base += blockDim.x) {
        int64_t i = base + threadIdx.x;
        int v = i < tiles ? static_cast<int>(row[i]) : 0;
        int total;
        int inc = block_inclusive_scan(v, sm, &total);
        if (i < tiles) row[i] = static_cast<uint32_t>(carry + inc - v);
        carry += total;
    }
    if (threadIdx.x == 0) totals[blockIdx.x] = static_cast<uint32_t>(carry);
}

template <typename KeyT, int BITS>
__global__ void __launch_bounds__(kSortThreads, 4) sort_scatter_kernel(const KeyT* __restrict__ keys_in,
                                                                    const uint32_t* __restrict__ vals_in,
                                                                    KeyT* __restrict__ keys_out,
                                                                    uint32_t* __restrict__ vals_out, int64_t n,
                                                                    int shift, const uint32_t* __restrict__ hist,
                                                                    const uint32_t* __restrict__ totals,
                                                                    int64_t tiles, SortHistSink next,
                                                                    const int64_t* __restrict__ n_dev)
{
    constexpr int RADIX = 1 << BITS;
    constexpr int PER = RADIX / kSortThreads;  // digits per thread in the block-wide steps
    n = effective_n(n, n_dev);
    if (static_cast<int64_t>(blockIdx.x) * kSortTile >= n) return;  // block-uniform: a tile past the end has no items
    __shared__ uint32_t warp_cnt[kSortThreads / 32][RADIX];
    __shared__ int sm[33];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int w = 0; w < kSortThreads / 32; ++w)
        for (int d = threadIdx.x; d < RADIX; d += kSortThreads) warp_cnt[w][d] = 0;
    __syncthreads();

    const int64_t tile0 = static_cast<int64_t>(blockIdx.x) * kSortTile + warp * (kSortRounds * 32);
    KeyT key[kSortRounds];
    uint32_t rank[kSortRounds];
    // everything the block reads from global memory is requested up front, in one wave: its keys, its values, the
    // digit totals and its own row of the scanned histogram (none of these depends on the ranking below)
    uint32_t val[kSortRounds];
#pragma unroll
    for (int r = 0; r < kSortRounds; ++r) {
        const int64_t i = tile0 + r * 32 + lane;
        key[r] = i < n ? keys_in[i] : KeyT(0);
        val[r] = i < n ? vals_in[i] : 0u;
    }
    int tot[PER];
    uint32_t mine_hist[PER];
#pragma unroll
    for (int q = 0; q < PER; ++q) {
        tot[q] = static_cast<int>(totals[threadIdx.x * PER + q]);
        mine_hist[q] = hist[static_cast<int64_t>(threadIdx.x * PER + q) * tiles + blockIdx.x];
    }
#pragma unroll
    for (int r = 0; r < kSortRounds; ++r) {
        const int64_t i = tile0 + r * 32 + lane;
        const bool valid = i < n;
        // invalid lanes get a tag no valid lane can have, so they match nobody valid
        const unsigned tag = valid ? static_cast<unsigned>((key[r] >> shift) & (RADIX - 1)) : (RADIX + lane);
        const unsigned peers = __match_any_sync(kFullMask, tag);
        const unsigned before = __popc(peers & lanemask_lt());
        uint32_t prev = 0;
        if (valid) prev = warp_cnt[warp][tag];
        __syncwarp();
        if (valid && before == 0) warp_cnt[warp][tag] = prev + __popc(peers);
        __syncwarp();
        rank[r] = prev + before;
    }
    __syncthreads();

    // digit base for this tile: exclusive scan of digit totals + this tile's prefix inside the digit;
    // thread t owns the PER consecutive digits [t*PER, t*PER+PER)
    {
        int mine = 0;
#pragma unroll
        for (int q = 0; q < PER; ++q) mine += tot[q];
        int total_all;
        const int inc = block_inclusive_scan(mine, sm, &total_all);
        uint32_t digit_base = static_cast<uint32_t>(inc - mine);
#pragma unroll
        for (int q = 0; q < PER; ++q) {
            const int d = threadIdx.x * PER + q;
            uint32_t run = digit_base + mine_hist[q];
#pragma unroll
            for (int w = 0; w < kSortThreads / 32; ++w) {
                const uint32_t c = warp_cnt[w][d];
                warp_cnt[w][d] = run;
                run += c;
            }
            digit_base += static_cast<uint32_t>(tot[q]);
        }
    }
    __syncthreads();

#pragma unroll
    for (int r = 0; r < kSortRounds; ++r) {
        const int64_t i = tile0 + r * 32 + lane;
        uint32_t pos = 0;
        if (i < n) {
            const unsigned d = static_cast<unsigned>((key[r] >> shift) & (RADIX - 1));
            pos = warp_cnt[warp][d] + rank[r];
            keys_out[pos] = key[r];
            vals_out[pos] = val[r];
        }
        next.add_warp(i < n, key[r], static_cast<int64_t>(pos));
    }
}

template <typename KeyT, int BITS>
static inline void radix_sort_pass(const KeyT* kin, const uint32_t* vin, KeyT* kout, uint32_t* vout, int64_t n, int shift,
                                   uint32_t* scratch, cudaStream_t st)
{
    constexpr int RADIX = 1 << BITS;
    const int64_t tiles = sort_num_tiles(n);
    uint32_t* hist = scratch;
    uint32_t* totals = scratch + tiles * RADIX;
    sort_hist_kernel<KeyT, BITS><<<static_cast<unsigned>(tiles), kSortThreads, 0, st>>>(kin, n, shift, hist, tiles);
    sort_scan_kernel<<<RADIX, 256, 0, st>>>(hist, tiles, totals);
    sort_scatter_kernel<KeyT, BITS><<<static_cast<unsigned>(tiles), kSortThreads, 0, st>>>(
        kin, vin, kout, vout, n, shift, hist, totals, tiles, SortHistSink{nullptr, 0, 0, 0u}, nullptr);
}

// One pass of the fused mode: the histogram of this pass already exists (its producer filled it); the scatter
// fills the histogram of the next pass (`next`) while it writes that pass's input.
template <typename KeyT, int BITS>
static inline void radix_sort_pass_fused(const KeyT* kin, const uint32_t* vin, KeyT* kout, uint32_t* vout, int64_t n,
                                         int shift, uint32_t* hist, uint32_t* totals, SortHistSink next, cudaStream_t st,
                                         const int64_t* n_dev)
{
    constexpr int RADIX = 1 << BITS;
    const int64_t tiles = sort_num_tiles(n);
    sort_scan_kernel<<<RADIX, 256, 0, st>>>(hist, tiles, totals);
    sort_scatter_kernel<KeyT, BITS><<<static_cast<unsigned>(tiles), kSortThreads, 0, st>>>(kin, vin, kout, vout, n, shift,
                                                                                          hist, totals, tiles, next, n_dev);
}

// Number of passes and bits per pass for keys of `key_bits` significant bits.
static inline void radix_plan(int key_bits, int* passes, int* bits)
{
    const int p8 = (key_bits + 7) / 8, p9 = (key_bits + 8) / 9, p10 = (key_bits + 9) / 10;
    *bits = 8;
    *passes = p8;
    if (p9 < *passes) {
        *bits = 9;
        *passes = p9;
    }
    if (p10 < *passes) {
        *bits = 10;
        *passes = p10;
    }
}

// Sorts n pairs by the key bits [0, key_bits).  Data ping-pongs between
// (keys_a, vals_a) and (keys_b, vals_b); returns 0 when the result is in the
// a-buffers, 1 when it is in the b-buffers.  n < 2^31.
template <typename KeyT>
static inline int radix_sort_pairs(KeyT* keys_a, uint32_t* vals_a, KeyT* keys_b, uint32_t* vals_b, int64_t n,
                                   int key_bits, uint32_t* scratch, cudaStream_t st)
{
    if (n <= 1 || key_bits <= 0) return 0;
    int passes, bits;
    radix_plan(key_bits, &passes, &bits);
    int cur = 0;
    for (int p = 0; p < passes; ++p) {
        KeyT* kin = cur ? keys_b : keys_a;
        uint32_t* vin = cur ? vals_b : vals_a;
        KeyT* kout = cur ? keys_a : keys_b;
        uint32_t* vout = cur ? vals_a : vals_b;
        if (bits == 10)
            radix_sort_pass<KeyT, 10>(kin, vin, kout, vout, n, p * 10, scratch, st);
        else if (bits == 9)
            radix_sort_pass<KeyT, 9>(kin, vin, kout, vout, n, p * 9, scratch, st);
        else
            radix_sort_pass<KeyT, 8>(kin, vin, kout, vout, n, p * 8, scratch, st);
        cur ^= 1;
    }
    return cur;
}

// Fused mode.  The caller (1) asks for the sink of pass 0 with radix_fused_begin -- which also zeroes all
// histograms -- (2) lets the kernel that writes keys_a call sink.add(key, position) for every element, and
// (3) calls radix_sort_pairs_fused.  Each pass is then a scan and a scatter: three launches fewer per pass
// than the plain mode and no second read of the keys.
struct RadixFusedPlan {
    int passes, bits;
    int64_t tiles;
    SortHistSink first;
};
static inline RadixFusedPlan radix_fused_begin(int64_t n, int key_bits, uint32_t* scratch, cudaStream_t st)
{
    RadixFusedPlan pl;
    radix_plan(key_bits, &pl.passes, &pl.bits);
    pl.tiles = sort_num_tiles(n);
    const size_t per_pass = static_cast<size_t>(pl.tiles) * (size_t(1) << pl.bits);
    cudaMemsetAsync(scratch, 0, per_pass * pl.passes * sizeof(uint32_t), st);
    pl.first = SortHistSink{scratch, pl.tiles, 0, (1u << pl.bits) - 1u};
    return pl;
}
template <typename KeyT>
static inline int radix_sort_pairs_fused(const RadixFusedPlan& pl, KeyT* keys_a, uint32_t* vals_a, KeyT* keys_b,
                                         uint32_t* vals_b, int64_t n, uint32_t* scratch, cudaStream_t st,
                                         const int64_t* n_dev = nullptr)
{
    // with a device-side count the passes always run (the count is unknown here), so the result's buffer depends
    // on the capacity only
    if (n <= 1 && n_dev == nullptr) return 0;
    const size_t per_pass = static_cast<size_t>(pl.tiles) * (size_t(1) << pl.bits);
    uint32_t* totals = scratch + static_cast<size_t>(pl.tiles) * kMaxRadix * kMaxSortPasses;
    int cur = 0;
    for (int p = 0; p < pl.passes; ++p) {
        KeyT* kin = cur ? keys_b : keys_a;
        uint32_t* vin = cur ? vals_b : vals_a;
        KeyT* kout = cur ? keys_a : keys_b;
        uint32_t* vout = cur ? vals_a : vals_b;
        uint32_t* hist = scratch + per_pass * p;
        SortHistSink next{nullptr, 0, 0, 0u};
        if (p + 1 < pl.passes) next = SortHistSink{scratch + per_pass * (p + 1), pl.tiles, (p + 1) * pl.bits, (1u << pl.bits) - 1u};
        if (pl.bits == 10)
            radix_sort_pass_fused<KeyT, 10>(kin, vin, kout, vout, n, p * 10, hist, totals, next, st, n_dev);
        else if (pl.bits == 9)
            radix_sort_pass_fused<KeyT, 9>(kin, vin, kout, vout, n, p * 9, hist, totals, next, st, n_dev);
        else
            radix_sort_pass_fused<KeyT, 8>(kin, vin, kout, vout, n, p * 8, hist, totals, next, st, n_dev);
        cur ^= 1;
    }
    return cur;
}

}  // namespace recsdk
