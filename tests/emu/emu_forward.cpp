// CPU build of the pooled forward kernel under the SIMT emulation of simt_emu.h: the kernel source is the one the
// GPU library is built from (included, not copied); only its <<<>>> host side is compiled out.
#include "simt_emu.h"
// the kernel file closes namespace recsdk itself in emulation builds
#include "../../recsdk_b200/csrc/tbe_forward.cu"

using namespace recsdk;

template <int G, int K>
static void run_grid(const FwdParams& p, int grid, int block)
{
    blockDim.x = static_cast<unsigned>(block);
    gridDim.x = static_cast<unsigned>(grid);
    for (int b = 0; b < grid; ++b) {  // blocks do not interact: one after the other
        std::vector<std::thread> ts;
        for (int t = 0; t < block; ++t)
            ts.emplace_back([&p, b, t] {
                threadIdx.x = static_cast<unsigned>(t);
                blockIdx.x = static_cast<unsigned>(b);
                tbe_forward_pooled_kernel<G, K>(p);
            });
        for (auto& t : ts) t.join();
    }
}

extern "C" int emu_tbe_forward_pooled(const float* w, const int64_t* wofs, const int32_t* dofs, const int64_t* idx,
                                      const int64_t* offs, float* out, int64_t T, int64_t B, int64_t N, int32_t total_D,
                                      int32_t max_D, int32_t mode, int64_t w_numel, int64_t* status, int G, int K,
                                      int grid, int block, int num_shards, float* const* shard_ptrs, int64_t shard_B,
                                      int32_t row_stride, const int32_t* col_offsets)
{
    FwdParams p{};
    p.w = w; p.wofs = wofs; p.dofs = dofs; p.idx = idx; p.offs = offs; p.out = out;
    p.T = T; p.B = B; p.N = N; p.total_D = total_D; p.max_D = max_D; p.mode = mode;
    p.w_numel = w_numel; p.status = status;
    p.base_aligned = (reinterpret_cast<uintptr_t>(w) & 15) == 0 ? 1 : 0;
    p.sh.num_shards = num_shards;
    p.sh.shard_B = shard_B;
    p.sh.row_stride = row_stride;
    p.sh.col_offsets = col_offsets;
    for (int i = 0; i < num_shards && i < RECSDK_MAX_SHARDS; ++i) p.sh.ptrs[i] = shard_ptrs[i];
#define RUN(GG, KK) if (G == GG && K == KK) { run_grid<GG, KK>(p, grid, block); return 0; }
    RUN(2, 1) RUN(4, 1) RUN(8, 1) RUN(16, 1) RUN(32, 1) RUN(32, 2)
#undef RUN
    return 1;
}
