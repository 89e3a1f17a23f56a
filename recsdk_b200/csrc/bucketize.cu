// Row-hash bucketize of a jagged batch for row-wise sharding: bucket = id % world,
// output grouped by (bucket, feature, sample) in input order, plus the permute
// that undoes it; optionally a first-occurrence dedup per (bucket, feature) with
// occurrence counts.  One thread walks one bag in order, which keeps the order
// inside a (bucket, feature, sample) cell identical to the sequential CPU loop.
#include "prims.cuh"

namespace recsdk {

constexpr int kMaxWorld = 64;

#define RECSDK_GRID_STRIDE(i, n)                                                        \
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < (n); \
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)

static __global__ void __launch_bounds__(256) lengths_to_i32_kernel(const int64_t* __restrict__ lengths, int64_t L,
                                                                    int* __restrict__ out)
{
    RECSDK_GRID_STRIDE(i, L + 1) out[i] = i < L ? static_cast<int>(lengths[i]) : 0;
}

// bucketize.cpp:35-51
static __global__ void __launch_bounds__(128) bucket_count_kernel(const int* __restrict__ offs,
                                                                  const int64_t* __restrict__ indices, int64_t L, int W,
                                                                  int* __restrict__ nl)
{
    RECSDK_GRID_STRIDE(lin, L)
    {
        int cnt[kMaxWorld];
        for (int w = 0; w < W; ++w) cnt[w] = 0;
        for (int i = offs[lin]; i < offs[lin + 1]; ++i) cnt[static_cast<int>(indices[i] % W)]++;
        for (int w = 0; w < W; ++w) nl[static_cast<int64_t>(w) * L + lin] = cnt[w];
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) nl[static_cast<int64_t>(W) * L] = 0;
}

// bucketize.cpp:54-76
static __global__ void __launch_bounds__(128) bucket_fill_kernel(const int* __restrict__ offs,
                                                                 const int64_t* __restrict__ indices, int64_t L, int W,
                                                                 int64_t B, int64_t F, const int* __restrict__ noffs,
                                                                 int64_t* __restrict__ new_indices,
                                                                 int64_t* __restrict__ perm, int* __restrict__ seg_of_pos)
{
    RECSDK_GRID_STRIDE(lin, L)
    {
        int cur[kMaxWorld];
        for (int w = 0; w < W; ++w) cur[w] = noffs[static_cast<int64_t>(w) * L + lin];
        const int f = static_cast<int>(lin / B);
        for (int i = offs[lin]; i < offs[lin + 1]; ++i) {
            const int64_t id = indices[i];
            const int b = static_cast<int>(id % W);
            const int pos = cur[b]++;
            new_indices[pos] = id;
            perm[i] = pos;
            if (seg_of_pos != nullptr) seg_of_pos[pos] = b * static_cast<int>(F) + f;
        }
    }
}

static __global__ void __launch_bounds__(256) i32_to_i64_kernel(const int* __restrict__ in, int64_t n,
                                                                int64_t* __restrict__ out)
{
    RECSDK_GRID_STRIDE(i, n) out[i] = in[i];
}
static __global__ void set_i64_kernel(int64_t* p, int64_t v) { *p = v; }

// ---- dedup per (bucket, feature), bucketize.cpp:79-130 ----------------------
static __global__ void __launch_bounds__(256) dedup_load_kernel(const int64_t* __restrict__ new_indices, int64_t n,
                                                                uint64_t* __restrict__ keys, uint32_t* __restrict__ vals)
{
    RECSDK_GRID_STRIDE(i, n)
    {
        keys[i] = static_cast<uint64_t>(new_indices[i]);
        vals[i] = static_cast<uint32_t>(i);
    }
}
// Sorted by id with positions ascending inside an id; positions are
// (bucket, feature)-major, so one id's occurrences are grouped by segment.
static __global__ void __launch_bounds__(256) dedup_head_kernel(const uint64_t* __restrict__ keys,
                                                                const uint32_t* __restrict__ vals,
                                                                const int* __restrict__ seg_of_pos, int64_t n,
                                                                int* __restrict__ head, int* __restrict__ first_at_pos)
{
    RECSDK_GRID_STRIDE(j, n)
    {
        const int h = (j == 0 || keys[j] != keys[j - 1] || seg_of_pos[vals[j]] != seg_of_pos[vals[j - 1]]) ? 1 : 0;
        head[j] = h;
        first_at_pos[vals[j]] = h;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) first_at_pos[n] = 0;
}
static __global__ void __launch_bounds__(256) dedup_runs_kernel(const int* __restrict__ head, int64_t n,
                                                                int* __restrict__ rid, int* __restrict__ run_start)
{
    RECSDK_GRID_STRIDE(j, n)
    {
        const int r = rid[j] - 1;
        rid[j] = r;
        if (head[j]) run_start[r] = static_cast<int>(j);
        if (j == n - 1) run_start[r + 1] = static_cast<int>(n);
    }
}
static __global__ void __launch_bounds__(256) dedup_write_kernel(const uint64_t* __restrict__ keys,
                                                                 const uint32_t* __restrict__ vals,
                                                                 const int* __restrict__ head, const int* __restrict__ rid,
                                                                 const int* __restrict__ run_start,
                                                                 const int* __restrict__ uidx_at_pos, int64_t n,
                                                                 int64_t* __restrict__ out_indices,
                                                                 int64_t* __restrict__ counts, int* __restrict__ u_of_pos)
{
    RECSDK_GRID_STRIDE(j, n)
    {
        const int r = rid[j];
        const int hs = run_start[r];
        const int u = uidx_at_pos[vals[hs]];
        if (head[j]) {
            out_indices[u] = static_cast<int64_t>(keys[j]);
            if (counts != nullptr) counts[u] = run_start[r + 1] - hs;
        }
        u_of_pos[vals[j]] = u;
    }
}
static __global__ void __launch_bounds__(256) dedup_perm_kernel(int64_t* __restrict__ perm, int64_t n,
                                                                const int* __restrict__ u_of_pos)
{
    RECSDK_GRID_STRIDE(i, n) perm[i] = u_of_pos[perm[i]];
}
static __global__ void __launch_bounds__(256) dedup_lengths_kernel(const int* __restrict__ noffs,
                                                                   const int* __restrict__ uidx_at_pos, int64_t cells,
                                                                   int64_t* __restrict__ new_lengths)
{
    RECSDK_GRID_STRIDE(c, cells) new_lengths[c] = uidx_at_pos[noffs[c + 1]] - uidx_at_pos[noffs[c]];
}

struct BucketWs {
    int *lens, *nl, *seg, *head, *rid, *run_start, *first_at_pos, *u_of_pos, *scan_scratch;
    uint64_t *keys_a, *keys_b;
    uint32_t *vals_a, *vals_b, *sort_scratch;
    int64_t* tmp;
    size_t bytes;
};
static BucketWs carve_bucket(void* base, int64_t N, int64_t L, int64_t W)
{
    WorkspaceCarver c(base);
    BucketWs w;
    const size_t n = static_cast<size_t>(N > 0 ? N : 1);
    const size_t cells = static_cast<size_t>(L * W);
    w.tmp = c.take<int64_t>(8);
    w.lens = c.take<int>(static_cast<size_t>(L) + 1);
    w.nl = c.take<int>(cells + 1);
    w.seg = c.take<int>(n);
    w.head = c.take<int>(n);
    w.rid = c.take<int>(n);
    w.run_start = c.take<int>(n + 1);
    w.first_at_pos = c.take<int>(n + 1);
    w.u_of_pos = c.take<int>(n);
    w.keys_a = c.take<uint64_t>(n);
    w.keys_b = c.take<uint64_t>(n);
    w.vals_a = c.take<uint32_t>(n);
    w.vals_b = c.take<uint32_t>(n);
    w.sort_scratch = c.take<uint32_t>(sort_scratch_u32(N));
    const int64_t scan_n = static_cast<int64_t>(cells + 1) > N + 1 ? static_cast<int64_t>(cells + 1) : N + 1;
    w.scan_scratch = c.take<int>(scan_scratch_ints(scan_n));
    w.bytes = c.used();
    return w;
}

}  // namespace recsdk

using namespace recsdk;

extern "C" size_t recsdk_bucketize_workspace_bytes(int64_t n, int64_t lengths_size, int64_t world)
{
    return carve_bucket(nullptr, n, lengths_size, world).bytes;
}

extern "C" int recsdk_bucketize(const int64_t* lengths, int64_t lengths_size, const int64_t* indices, int64_t n,
                                int64_t num_features, int64_t world, int32_t do_unique, int32_t return_count,
                                int64_t* new_lengths, int64_t* new_indices, int64_t* unbucketize_permute,
                                int64_t* ids_counts, int64_t* num_out, void* workspace, size_t workspace_bytes,
                                void* stream)
{
    if (lengths_size <= 0 || n <= 0 || num_features <= 0 || world <= 0 || world > kMaxWorld) return RECSDK_ERR_INVALID_ARG;
    if (lengths_size % num_features != 0) return RECSDK_ERR_INVALID_ARG;
    if (!lengths || !indices || !new_lengths || !new_indices || !unbucketize_permute || !num_out) return RECSDK_ERR_INVALID_ARG;
    if (do_unique && return_count && !ids_counts) return RECSDK_ERR_INVALID_ARG;
    if (n >= (int64_t(1) << 31) || lengths_size * world >= (int64_t(1) << 31)) return RECSDK_ERR_TOO_LARGE;
    if (!workspace) return RECSDK_ERR_WORKSPACE;
    const int64_t L = lengths_size, W = world, F = num_features, B = L / F, cells = L * W;
    const BucketWs ws = carve_bucket(workspace, n, L, W);
    if (ws.bytes > workspace_bytes) return RECSDK_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    lengths_to_i32_kernel<<<grid_for(L + 1, 256), 256, 0, st>>>(lengths, L, ws.lens);
    device_scan<false>(ws.lens, ws.lens, L + 1, ws.scan_scratch, nullptr, st);  // offsets[L+1]
    bucket_count_kernel<<<grid_for(L, 128), 128, 0, st>>>(ws.lens, indices, L, static_cast<int>(W), ws.nl);
    if (!do_unique) i32_to_i64_kernel<<<grid_for(cells, 256), 256, 0, st>>>(ws.nl, cells, new_lengths);
    device_scan<false>(ws.nl, ws.nl, cells + 1, ws.scan_scratch, nullptr, st);  // new offsets[cells+1]
    bucket_fill_kernel<<<grid_for(L, 128), 128, 0, st>>>(ws.lens, indices, L, static_cast<int>(W), B, F, ws.nl,
                                                        new_indices, unbucketize_permute, do_unique ? ws.seg : nullptr);
    if (!do_unique) {
        set_i64_kernel<<<1, 1, 0, st>>>(num_out, n);
        RECSDK_CUDA_CHECK_LAUNCH();
        return RECSDK_OK;
    }
    const int grid = grid_for(n, 256);
    dedup_load_kernel<<<grid, 256, 0, st>>>(new_indices, n, ws.keys_a, ws.vals_a);
    const int which = radix_sort_pairs<uint64_t>(ws.keys_a, ws.vals_a, ws.keys_b, ws.vals_b, n, 64, ws.sort_scratch, st);
    const uint64_t* keys = which ? ws.keys_b : ws.keys_a;
    const uint32_t* vals = which ? ws.vals_b : ws.vals_a;
    dedup_head_kernel<<<grid, 256, 0, st>>>(keys, vals, ws.seg, n, ws.head, ws.first_at_pos);
    device_scan<true>(ws.head, ws.rid, n, ws.scan_scratch, nullptr, st);
    dedup_runs_kernel<<<grid, 256, 0, st>>>(ws.head, n, ws.rid, ws.run_start);
    device_scan<false>(ws.first_at_pos, ws.first_at_pos, n + 1, ws.scan_scratch, num_out, st);  // unique index at position
    dedup_write_kernel<<<grid, 256, 0, st>>>(keys, vals, ws.head, ws.rid, ws.run_start, ws.first_at_pos, n, new_indices,
                                             return_count ? ids_counts : nullptr, ws.u_of_pos);
    dedup_perm_kernel<<<grid, 256, 0, st>>>(unbucketize_permute, n, ws.u_of_pos);
    dedup_lengths_kernel<<<grid_for(cells, 256), 256, 0, st>>>(ws.nl, ws.first_at_pos, cells, new_lengths);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}
