// CPU build of the backward kernels (expand, per-run records, partial sums, row update) under the SIMT emulation
// of simt_emu.h.  The kernel source is the one the GPU library is built from (included, not copied); the sort and
// the scan between expand and the records -- library primitives with their own tests -- are done with std::
// algorithms here.
#include <algorithm>
#include <numeric>

#include "simt_emu.h"
namespace recsdk {
// the expand kernels count the first sort pass's histogram through this; not needed here
struct SortHistSink {
    template <typename KeyT>
    void add_warp(bool, KeyT, int64_t) const {}
};
}  // namespace recsdk
#include "../../recsdk_b200/csrc/tbe_backward.cuh"

using namespace recsdk;

template <typename F>
static void run_grid(int grid, int block, F kernel)
{
    blockDim.x = static_cast<unsigned>(block);
    gridDim.x = static_cast<unsigned>(grid);
    for (int b = 0; b < grid; ++b) {
        std::vector<std::thread> ts;
        for (int t = 0; t < block; ++t)
            ts.emplace_back([&kernel, b, t] {
                threadIdx.x = static_cast<unsigned>(t);
                blockIdx.x = static_cast<unsigned>(b);
                kernel();
            });
        for (auto& t : ts) t.join();
    }
}

template <int G, int K>
static void run_partial_update(const BwdParams& p, const RunMeta* meta, int grid, int block)
{
    run_grid(grid, block, [&] { partial_kernel<G, K>(p); });
    switch (p.opt) {
        case RECSDK_OPT_ADAGRAD: run_grid(grid, block, [&] { update_kernel<G, K, RECSDK_OPT_ADAGRAD>(p, meta); }); break;
        case RECSDK_OPT_ADAM: run_grid(grid, block, [&] { update_kernel<G, K, RECSDK_OPT_ADAM>(p, meta); }); break;
        default: run_grid(grid, block, [&] { update_kernel<G, K, RECSDK_OPT_SGD>(p, meta); }); break;
    }
}

extern "C" int emu_tbe_backward(const float* grad, float* w, float* m1, float* m2, const int64_t* wofs,
                                const int32_t* dofs, const int64_t* cumsum, const int64_t* idx, const int64_t* offs,
                                int64_t T, int64_t B, int64_t N, int32_t total_D, int32_t max_D, int32_t mode, int32_t opt,
                                int32_t chunk, float lr, float eps, float beta1, float beta2, float beta2sqrt,
                                int64_t w_numel, int64_t* status, int G, int K, int grid, int block)
{
    BwdParams p{};
    p.grad = grad; p.w = w; p.m1 = m1; p.m2 = m2; p.wofs = wofs; p.dofs = dofs; p.cumsum = cumsum;
    p.idx = idx; p.offs = offs; p.T = T; p.B = B; p.N = N; p.total_D = total_D; p.max_D = max_D;
    p.mode = mode; p.opt = opt; p.chunk = chunk; p.direct_max = kDirectMax; p.lr = lr; p.eps = eps; p.beta1 = beta1; p.beta2 = beta2;
    p.beta2sqrt = beta2sqrt; p.w_numel = w_numel; p.status = status;
    int bshift = 1;
    while ((int64_t(1) << bshift) <= (B - 1 > 0 ? B - 1 : 1)) ++bshift;
    p.bshift = bshift;
    p.base_aligned = ((reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(m1) |
                       reinterpret_cast<uintptr_t>(m2)) & 15) == 0;
    // 1. expand (emulated)
    std::vector<uint32_t> keys(N), vals(N);
    std::vector<int64_t> counters(8, 0);
    run_grid(grid, block, [&] { expand_pooled_kernel<uint32_t>(p, keys.data(), vals.data(), SortHistSink{}, counters.data()); });
    // 2.-3. stable sort by key, run starts (host)
    std::vector<int> order(N);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return keys[a] < keys[b]; });
    std::vector<uint32_t> skeys(N), svals(N);
    for (int64_t i = 0; i < N; ++i) { skeys[i] = keys[order[i]]; svals[i] = vals[order[i]]; }
    std::vector<int> run_start;
    for (int64_t i = 0; i < N; ++i)
        if (i == 0 || skeys[i] != skeys[i - 1]) run_start.push_back(static_cast<int>(i));
    const int64_t U = static_cast<int64_t>(run_start.size());
    run_start.push_back(static_cast<int>(N));
    counters[0] = U;
    const size_t max_chunks = chunk_slots_cap(N);
    std::vector<RunMeta> meta(U > 0 ? U : 1);
    std::vector<int2> desc(max_chunks);
    float* partial = static_cast<float*>(aligned_alloc(64, max_chunks * static_cast<size_t>(max_D) * sizeof(float)));
    p.vals = svals.data(); p.run_start = run_start.data(); p.counters = counters.data();
    p.chunk_desc = desc.data(); p.partial = partial;
    p.base_aligned = p.base_aligned && ((reinterpret_cast<uintptr_t>(partial) & 15) == 0);
    // 4. per-run records (emulated)
    run_grid(grid, block, [&] { run_meta_kernel<uint32_t>(p, skeys.data(), counters.data(), meta.data(), desc.data()); });
    // 4b.-5. partial sums and row update (emulated)
    int rc = 1;
#define RUN(GG, KK) if (G == GG && K == KK) { run_partial_update<GG, KK>(p, meta.data(), grid, block); rc = 0; }
    RUN(2, 1) RUN(8, 1) RUN(32, 1) RUN(32, 2)
#undef RUN
    free(partial);
    return rc;
}
