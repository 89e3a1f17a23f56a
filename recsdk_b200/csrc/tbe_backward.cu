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
#include "tbe_backward.cuh"

#ifndef RECSDK_EMULATE
namespace recsdk {
// ---------------------------------------------------------------------------- host side
struct BwdWorkspace {
    void *keys_a, *keys_b;
    uint32_t *vals_a, *vals_b, *sort_scratch;
    int *run_start, *scan_scratch;
    RunMeta* meta;
    int2* desc;
    float* partial;
    int64_t* counters;
    size_t bytes;
};

static BwdWorkspace carve_bwd(void* base, int64_t N, int32_t max_D)
{
    WorkspaceCarver c(base);
    BwdWorkspace w;
    const size_t n = static_cast<size_t>(N > 0 ? N : 1);
    const size_t max_chunks = chunk_slots_cap(N);
    w.counters = c.take<int64_t>(8);
    w.keys_a = c.take<uint64_t>(n);
    w.keys_b = c.take<uint64_t>(n);
    w.vals_a = c.take<uint32_t>(n);
    w.vals_b = c.take<uint32_t>(n);
    w.sort_scratch = c.take<uint32_t>(sort_scratch_u32_fused(N));
    w.run_start = c.take<int>(n + 1);
    w.meta = c.take<RunMeta>(n);
    w.desc = c.take<int2>(max_chunks);
    w.scan_scratch = c.take<int>(scan_scratch_ints(N));
    w.partial = c.take<float>(max_chunks * static_cast<size_t>(max_D));
    w.bytes = c.used();
    return w;
}

static int bits_for(int64_t x)
{
    int b = 0;
    while (b < 63 && (int64_t(1) << b) <= x) ++b;
    return b < 1 ? 1 : b;
}

// Staged update: rows of 128..1024 floats with 16-byte aligned tables.  Returns false when the shape does not
// qualify (the caller then launches update_kernel).
template <int OPT, int kStages>
static bool launch_update_staged_impl(const BwdParams& p, const RunMeta* meta, int warps, cudaStream_t st)
{
    const size_t smem = update_staged_smem_bytes(warps, kStages, StagedArrays<OPT>::kCount, p.max_D);
    static bool optin_done[kMaxDevices] = {false};  // one table per instantiation
    if (!smem_optin(update_staged_kernel<OPT, kStages>, 72 * 1024, optin_done)) return false;
    update_staged_kernel<OPT, kStages><<<num_sms() * 3, warps * 32, smem, st>>>(p, meta);
    return true;
}

static bool launch_update_staged(const BwdParams& p, const RunMeta* meta, cudaStream_t st)
{
    if (!p.staged_update || !p.base_aligned || (p.max_D & 3) != 0 || p.max_D < 128 || p.max_D > 1024) return false;
    const int arrays = p.opt == RECSDK_OPT_ADAM ? 4 : (p.opt == RECSDK_OPT_ADAGRAD ? 3 : 2);
    const int stages = p.max_D <= 256 ? 4 : 2;
    int warps = 8;
    while (warps > 1 && update_staged_smem_bytes(warps, stages, arrays, p.max_D) > 72 * 1024) warps >>= 1;
    if (update_staged_smem_bytes(warps, stages, arrays, p.max_D) > 72 * 1024) return false;
#define RECSDK_STAGED(OPT) \
    (stages == 4 ? launch_update_staged_impl<OPT, 4>(p, meta, warps, st) : launch_update_staged_impl<OPT, 2>(p, meta, warps, st))
    switch (p.opt) {
        case RECSDK_OPT_ADAGRAD: return RECSDK_STAGED(RECSDK_OPT_ADAGRAD);
        case RECSDK_OPT_ADAM: return RECSDK_STAGED(RECSDK_OPT_ADAM);
        default: return RECSDK_STAGED(RECSDK_OPT_SGD);
    }
#undef RECSDK_STAGED
}

template <int G, int K>
static void launch_update(const BwdParams& p, const RunMeta* meta, int64_t N, cudaStream_t st)
{
    if (G == 32 && launch_update_staged(p, meta, st)) return;
    // blocks of 64 threads, up to 128 per SM queued (16 resident at 64 registers): small blocks retire and are replaced
    // one by one, which measured a few percent faster on the benchmark step than one resident wave of 256-thread
    // blocks striding over the rows (0.299 vs 0.315 ms); each group still walks several rows, so the record of its
    // next row is fetched ahead
    constexpr int kBlock = 64;
    const int groups_per_block = kBlock / G;
    const int grid = grid_for(N, groups_per_block, 128);
    switch (p.opt) {
        case RECSDK_OPT_ADAGRAD: update_kernel<G, K, RECSDK_OPT_ADAGRAD><<<grid, kBlock, 0, st>>>(p, meta); break;
        case RECSDK_OPT_ADAM: update_kernel<G, K, RECSDK_OPT_ADAM><<<grid, kBlock, 0, st>>>(p, meta); break;
        default: update_kernel<G, K, RECSDK_OPT_SGD><<<grid, kBlock, 0, st>>>(p, meta); break;
    }
}

template <int G, int K>
static void launch_partial(const BwdParams& p, int64_t N, cudaStream_t st)
{
    const int groups_per_block = 256 / G;
    // one resident wave (64 registers under the launch bounds: 4 blocks per SM)
    const int grid = grid_for(static_cast<int64_t>(chunk_slots_cap(N)), groups_per_block, 4);
    partial_kernel<G, K><<<grid, 256, 0, st>>>(p);
}

#define RECSDK_DISPATCH_GK(vec_per_row, CALL)                 \
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

template <typename KeyT>
static int run_backward(const recsdk_tbe_backward_args* a, BwdParams p, const BwdWorkspace& ws, int key_bits,
                        cudaStream_t st)
{
    const int64_t N = a->N;
    KeyT* ka = static_cast<KeyT*>(ws.keys_a);
    KeyT* kb = static_cast<KeyT*>(ws.keys_b);
    const bool do_plan = (a->flags & RECSDK_BWD_APPLY_ONLY) == 0;
    const bool do_apply = (a->flags & RECSDK_BWD_PLAN_ONLY) == 0;
    // where the sorted tags end up depends only on the number of passes
    int passes, bits;
    radix_plan(key_bits, &passes, &bits);
    const int which = (N > 1 ? passes : 0) & 1;
    const KeyT* keys = which ? kb : ka;
    p.vals = which ? ws.vals_b : ws.vals_a;
    p.run_start = ws.run_start;
    p.counters = ws.counters;
    p.chunk_desc = ws.desc;
    p.partial = ws.partial;
    const int vec_per_row = (a->max_D + 3) / 4;
    if (do_plan) {
        // The plan needs the indices and the LAYOUT of the gradient, not the gradient: it can run ahead, on
        // another stream, while the forward of the same batch (or the dense part) runs.
        cudaMemsetAsync(ws.counters, 0, 8 * sizeof(int64_t), st);  // {U, chunks, indices in chunked runs, unaligned columns, ...}
        // 1. expand; it also fills the histogram of the first sort pass
        const RadixFusedPlan plan = radix_fused_begin(N, key_bits, ws.sort_scratch, st);
        if (a->pooling_mode == RECSDK_POOL_NONE)
            expand_nobag_kernel<KeyT><<<grid_for(N, 256), 256, 0, st>>>(p, ka, ws.vals_a, plan.first, ws.counters);
        else
            expand_pooled_kernel<KeyT><<<grid_for(a->T * a->B, 8 * 32), 256, 0, st>>>(p, ka, ws.vals_a, plan.first,
                                                                                        ws.counters);
        // 2. sort: per pass a scan and a scatter that fills the next pass's histogram
        const int got = radix_sort_pairs_fused<KeyT>(plan, ka, ws.vals_a, kb, ws.vals_b, N, ws.sort_scratch, st);
        if (got != which) return RECSDK_ERR_CUDA;  // cannot happen: both follow radix_plan
        // 3. runs
        device_scan_fn<true>(HeadFlagIn<KeyT>{keys}, RunStartOut{ws.run_start, ws.counters}, N, ws.scan_scratch,
                             nullptr, st);
        // 4. per-run records (+ chunk descriptors of long runs)
        run_meta_kernel<KeyT><<<grid_for(N, 256), 256, 0, st>>>(p, keys, ws.counters, ws.meta, ws.desc);
    }
    if (!do_apply) {
        RECSDK_CUDA_CHECK_LAUNCH();
        return RECSDK_OK;
    }
    // 4b. chunk sums
    {
#define CALL_PARTIAL(G, K) launch_partial<G, K>(p, N, st)
        RECSDK_DISPATCH_GK(vec_per_row, CALL_PARTIAL);
#undef CALL_PARTIAL
    }
    // 5. update
    if (a->ev_update_start) cudaEventRecord(static_cast<cudaEvent_t>(a->ev_update_start), st);
#define CALL_UPDATE(G, K) launch_update<G, K>(p, ws.meta, N, st)
    RECSDK_DISPATCH_GK(vec_per_row, CALL_UPDATE);
#undef CALL_UPDATE
    if (a->ev_update_stop) cudaEventRecord(static_cast<cudaEvent_t>(a->ev_update_stop), st);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

}  // namespace recsdk

using namespace recsdk;

extern "C" float recsdk_adam_beta2sqrt(float beta1, float beta2, int64_t iter)
{
    // op_host/backward_codegen_adagrad_unweighted_exact.cpp:98-102: pow in double,
    // each intermediate stored in a float.
    const float b1 = static_cast<float>(1 - pow(static_cast<double>(beta1), static_cast<double>(iter)));
    const float b2 = static_cast<float>(1 - pow(static_cast<double>(beta2), static_cast<double>(iter)));
    return static_cast<float>(sqrt(static_cast<double>(b2)) / static_cast<double>(b1));
}

extern "C" size_t recsdk_tbe_backward_workspace_bytes(int64_t N, int32_t max_D)
{
    return carve_bwd(nullptr, N, max_D > 0 ? max_D : 1).bytes;
}

extern "C" int recsdk_tbe_backward(const recsdk_tbe_backward_args* a, void* stream)
{
    if (a == nullptr) return RECSDK_ERR_INVALID_ARG;
    if (a->T < 0 || a->B < 0 || a->N < 0 || a->max_D <= 0 || a->total_D <= 0) return RECSDK_ERR_INVALID_ARG;
    if (a->N >= (int64_t(1) << 31)) return RECSDK_ERR_TOO_LARGE;
    if (a->pooling_mode < RECSDK_POOL_SUM || a->pooling_mode > RECSDK_POOL_NONE) return RECSDK_ERR_INVALID_ARG;
    if (a->optimizer < RECSDK_OPT_ADAGRAD || a->optimizer > RECSDK_OPT_SGD) return RECSDK_ERR_INVALID_ARG;
    if (a->reduce_chunk != 0 && a->reduce_chunk != kChunk) return RECSDK_ERR_INVALID_ARG;
    if (a->T == 0 || a->B == 0 || a->N == 0) return RECSDK_OK;
    if (!a->dev_weights || !a->weights_offsets || !a->D_offsets || !a->indices || !a->offsets)
        return RECSDK_ERR_INVALID_ARG;
    const recsdk_sample_shards& sh = a->grad_shards;
    const bool plan_only = (a->flags & RECSDK_BWD_PLAN_ONLY) != 0;
    if ((a->flags & RECSDK_BWD_PLAN_ONLY) && (a->flags & RECSDK_BWD_APPLY_ONLY)) return RECSDK_ERR_INVALID_ARG;
    if (sh.num_shards == 0) {
        if (!a->grad_output && !plan_only) return RECSDK_ERR_INVALID_ARG;
    } else {
        if (!sample_shards_valid(sh, a->B) || a->pooling_mode == RECSDK_POOL_NONE) return RECSDK_ERR_INVALID_ARG;
    }
    if (a->optimizer != RECSDK_OPT_SGD && !a->momentum1) return RECSDK_ERR_INVALID_ARG;
    if (a->optimizer == RECSDK_OPT_ADAM && !a->momentum2) return RECSDK_ERR_INVALID_ARG;
    const bool have_unique = a->unique_ids != nullptr;
    if (have_unique && (!a->unique_offsets || !a->unique_inverse || a->num_unique_capacity <= 0))
        return RECSDK_ERR_INVALID_ARG;
    if (!have_unique && !a->hash_size_cumsum) return RECSDK_ERR_INVALID_ARG;
    if (!a->workspace) return RECSDK_ERR_WORKSPACE;
    const BwdWorkspace ws = carve_bwd(a->workspace, a->N, a->max_D);
    if (ws.bytes > a->workspace_bytes) return RECSDK_ERR_WORKSPACE;

    int bshift = bits_for(a->B - 1 > 0 ? a->B - 1 : 1);
    if (a->pooling_mode != RECSDK_POOL_NONE && bshift + bits_for(a->T) > 32) return RECSDK_ERR_TOO_LARGE;

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    BwdParams p{};
    p.grad = a->grad_output;
    p.w = a->dev_weights;
    p.m1 = a->momentum1;
    p.m2 = a->momentum2;
    p.wofs = a->weights_offsets;
    p.dofs = a->D_offsets;
    p.cumsum = a->hash_size_cumsum;
    p.idx = a->indices;
    p.offs = a->offsets;
    p.uid = a->unique_ids;
    p.uoff = a->unique_offsets;
    p.uinv = a->unique_inverse;
    p.T = a->T;
    p.B = a->B;
    p.N = a->N;
    p.total_D = a->total_D;
    p.max_D = a->max_D;
    p.mode = a->pooling_mode;
    p.opt = a->optimizer;
    p.bshift = bshift;
    p.chunk = a->reduce_chunk;
    p.direct_max = kDirectMax;
    p.lr = a->learning_rate;
    p.eps = a->eps;
    p.beta1 = a->beta1;
    p.beta2 = a->beta2;
    p.beta2sqrt = a->optimizer == RECSDK_OPT_ADAM ? recsdk_adam_beta2sqrt(a->beta1, a->beta2, a->iter) : 0.f;
    p.max_grad = a->max_gradient;
    p.clip = a->gradient_clipping;
    p.w_numel = a->weights_numel;
    p.grad_numel = a->pooling_mode == RECSDK_POOL_NONE ? a->N * a->max_D : a->B * static_cast<int64_t>(a->total_D);
    p.status = a->dev_status;
    bool grad_aligned = true;
    if (sh.num_shards == 0) {
        // a plan made before the gradient exists assumes a 16-byte aligned gradient; the apply call checks it
        grad_aligned = (plan_only && !a->grad_output) ? true : aligned16(a->grad_output);
        if ((a->flags & RECSDK_BWD_APPLY_ONLY) && !grad_aligned) return RECSDK_ERR_INVALID_ARG;
    } else {
        for (int s = 0; s < sh.num_shards; ++s) grad_aligned = grad_aligned && aligned16(sh.ptrs[s]);
    }
    p.sh = sh;
    p.staged_update = (a->flags & RECSDK_BWD_STAGED_UPDATE) ? 1 : 0;
    p.base_aligned = (grad_aligned && aligned16(a->dev_weights) && aligned16(a->momentum1) &&
                      aligned16(a->momentum2) && aligned16(ws.partial))
                         ? 1
                         : 0;

    int key_bits;
    if (have_unique)
        key_bits = bits_for(a->num_unique_capacity);
    else
        key_bits = (a->total_hash_size_bits > 0 && a->total_hash_size_bits <= 64) ? a->total_hash_size_bits : 64;
    if (key_bits <= 32) return run_backward<uint32_t>(a, p, ws, key_bits, st);
    return run_backward<uint64_t>(a, p, ws, key_bits, st);
}
#endif  // RECSDK_EMULATE
