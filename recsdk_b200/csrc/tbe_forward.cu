// Pooled embedding gather over ragged bags (forward of the table-batched
// embedding op).
//
// The op is HBM-bound, but a naive "one warp per bag" mapping is latency-bound:
// offsets -> index -> row is a chain of three dependent global loads per bag.
// Here G lanes (G*16 bytes = one row, at most a warp) own G consecutive bags:
//   * each lane fetches the metadata of ONE of the G bags (offsets, feature
//     geometry) and, 32 positions at a time, ONE index of the contiguous index
//     range those bags cover, and resolves it to a row address -- all in parallel;
//   * the group then walks the resolved rows in order, broadcasting the row
//     address with shuffles and issuing four independent 128-bit row loads per
//     lane before consuming them, so many rows are in flight per warp;
//   * rows are accumulated in index order from 0.0f and the pooled row is
//     written once with a streaming store when the walk crosses a bag boundary.
// The addition order is the order of the reference kernel (Pooling(),
// split_embedding_codegen_forward_unweighted_kernel.h:226-241) for bags that fit
// one of its blocks: bit-exact against a sequential loop.
#include "common.cuh"

namespace recsdk {

struct FwdParams {
    const float* __restrict__ w;
    const int64_t* __restrict__ wofs;
    const int32_t* __restrict__ dofs;
    const int64_t* __restrict__ idx;
    const int64_t* __restrict__ offs;
    float* __restrict__ out;
    int64_t T, B, N;
    int32_t total_D, max_D, mode;
    int64_t w_numel;
    int64_t* status;
    int base_aligned;  // dev_weights is 16-byte aligned
    recsdk_sample_shards sh;  // num_shards > 0: pooled rows go to the sample owners' buffers
};

// Where the pooled row of bag (t, b) goes.
__device__ __forceinline__ float* out_row_ptr(const FwdParams& p, int64_t t, int64_t b, int32_t d0)
{
    if (p.sh.num_shards == 0) return p.out + b * p.total_D + d0;
    const int64_t s = b / p.sh.shard_B;
    return shard_base(p.sh, s) + (b - s * p.sh.shard_B) * p.sh.row_stride + p.sh.col_offsets[t];
}

__device__ __forceinline__ bool row_ok(const FwdParams& p, int64_t idx, int64_t row_off, int32_t D)
{
    if (p.w_numel <= 0) return true;
    if (idx < 0 || row_off + D > p.w_numel) {
        set_status(p.status, RECSDK_ERR_INDEX_RANGE, idx, row_off);
        return false;
    }
    return true;
}

// Generic per-bag path (any dim / offset alignment), G lanes striding over the columns.
template <int G>
__device__ void forward_bag_scalar(const FwdParams& p, int lane, int64_t bag)
{
    const int64_t t = bag / p.B;
    const int64_t b = bag - t * p.B;
    const int64_t s = p.offs[bag], e = p.offs[bag + 1];
    const int32_t d0 = p.dofs[t];
    const int32_t D = p.dofs[t + 1] - d0;
    const int64_t wofs = p.wofs[t];
    float* out_row = out_row_ptr(p, t, b, d0);
    const float mean = __fdiv_rn(1.0f, static_cast<float>(e - s));
    for (int c = lane; c < D; c += G) {
        float acc = 0.f;
        for (int64_t i = s; i < e; ++i) {
            int64_t id = p.idx[i];
            int64_t ro = wofs + id * D;
            float v = row_ok(p, id, ro, D) ? p.w[ro + c] : 0.f;
            acc = __fadd_rn(acc, v);
        }
        if (p.mode == RECSDK_POOL_MEAN && e > s) acc = __fmul_rn(acc, mean);
        out_row[c] = acc;
    }
}

template <int G>
__device__ __forceinline__ unsigned group_mask()
{
    if (G == 32) return kFullMask;
    return ((1u << G) - 1u) << ((threadIdx.x & 31) / G * G);
}

// Independent 128-bit row loads in flight per lane (divided by K).  4, not 8: at 8 the kernel needs 96 registers
// and two blocks per SM, at 4 it needs 64 and runs four -- the pooled gather of the benchmark went from 0.30 to
// 0.22 ms.
constexpr int kFwdUnroll = 4;

template <int G, int K>
__global__ void __launch_bounds__(256) tbe_forward_pooled_kernel(FwdParams p)
{
    const int gl = threadIdx.x % G;
    const unsigned gmask = group_mask<G>();
    const int64_t num_bags = p.T * p.B;
    const int64_t groups_total = static_cast<int64_t>(gridDim.x) * blockDim.x / G;
    const int64_t gid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / G;
    const int max_nvec = p.max_D >> 2;

    for (int64_t bag0 = gid * G; bag0 < num_bags; bag0 += groups_total * G) {
        const int nb = static_cast<int>((num_bags - bag0) < G ? (num_bags - bag0) : G);
        const bool valid = gl < nb;
        const int64_t my_bag = bag0 + gl;
        const int64_t start_l = valid ? p.offs[my_bag] : INT64_MAX;
        const int64_t end_all = p.offs[bag0 + nb];
        const int64_t t_l = valid ? my_bag / p.B : 0;
        const int64_t b_l = my_bag - t_l * p.B;
        const int32_t d0_l = p.dofs[t_l];
        const int32_t D_l = p.dofs[t_l + 1] - d0_l;
        const int64_t wofs_l = p.wofs[t_l];
        const int64_t optr_l = valid ? reinterpret_cast<int64_t>(out_row_ptr(p, t_l, b_l, d0_l)) : 0;
        const bool ok_l = !valid || ((((wofs_l | D_l) & 3) == 0) && ((optr_l & 15) == 0));
        const bool all_ok = __all_sync(gmask, ok_l) != 0;  // executed by every lane of the group
        if (!(p.base_aligned && all_ok)) {
            for (int j = 0; j < nb; ++j) forward_bag_scalar<G>(p, gl, bag0 + j);
            continue;
        }
        const int64_t p0 = __shfl_sync(gmask, start_l, 0, G);

        // flush bag j: write `acc` (scaled for MEAN) or zeros
        auto flush = [&](int j, const float4 (&acc)[K], bool has_rows, int cb) {
            float* optr = reinterpret_cast<float*>(__shfl_sync(gmask, optr_l, j, G));
            const int nvec = __shfl_sync(gmask, D_l, j, G) >> 2;
            const int64_t sj = __shfl_sync(gmask, start_l, j, G);
            const int64_t nx = __shfl_sync(gmask, start_l, (j + 1) & (G - 1), G);
            const int64_t ej = (j + 1 < nb) ? nx : end_all;
            const float mean = __fdiv_rn(1.0f, static_cast<float>(ej - sj));
#pragma unroll
            for (int k = 0; k < K; ++k) {
                const int c = cb + gl + k * G;
                if (c < nvec) {
                    float4 r = has_rows ? acc[k] : make_float4(0.f, 0.f, 0.f, 0.f);
                    if (has_rows && p.mode == RECSDK_POOL_MEAN) r = mul4s(r, mean);
                    st_f4_stream(optr + 4 * c, r);
                }
            }
        };

        for (int cb = 0; cb < max_nvec; cb += G * K) {
            int cur = 0;           // bag (0..nb) whose rows are being accumulated
            bool cur_has = false;  // accumulator holds at least one row
            float4 acc[K];
#pragma unroll
            for (int k = 0; k < K; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);

            for (int64_t base = p0; base < end_all; base += G) {
                const int64_t pos = base + gl;
                const bool have = pos < end_all;
                const int64_t id = have ? p.idx[pos] : 0;
                // bag of `pos`: the largest j with start_j <= pos (empty bags share a start; the last owns it)
                int j_l = 0;
#pragma unroll
                for (int step = G >> 1; step >= 1; step >>= 1) {
                    const int cand = j_l + step;
                    const int64_t sc = __shfl_sync(gmask, start_l, cand & (G - 1), G);
                    if (cand < G && sc <= pos) j_l = cand;
                }
                const int64_t wofs_j = __shfl_sync(gmask, wofs_l, j_l, G);
                const int32_t D_j = __shfl_sync(gmask, D_l, j_l, G);
                int64_t ro_l = wofs_j + id * D_j;
                if (have && !row_ok(p, id, ro_l, D_j)) ro_l = -1;
                const int cnt = static_cast<int>((end_all - base) < G ? (end_all - base) : G);

                constexpr int kUnroll = kFwdUnroll / K;  // independent row loads in flight per lane
                for (int jj0 = 0; jj0 < cnt; jj0 += kUnroll) {
                    float4 v[kUnroll][K];
                    int bj[kUnroll];
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        const int jj = jj0 + u;
                        const int src = jj < cnt ? jj : 0;
                        const int64_t ro = __shfl_sync(gmask, ro_l, src, G);
                        bj[u] = __shfl_sync(gmask, j_l, src, G);
                        const int nvec = __shfl_sync(gmask, D_l, bj[u], G) >> 2;
#pragma unroll
                        for (int k = 0; k < K; ++k) {
                            const int c = cb + gl + k * G;
                            v[u][k] = (jj < cnt && ro >= 0 && c < nvec) ? ld_f4(p.w + ro + 4 * c)
                                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        if (jj0 + u < cnt) {
                            while (cur < bj[u]) {  // group-uniform: finished (or empty) bags
                                flush(cur, acc, cur_has, cb);
#pragma unroll
                                for (int k = 0; k < K; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                                cur_has = false;
                                ++cur;
                            }
#pragma unroll
                            for (int k = 0; k < K; ++k) acc[k] = add4(acc[k], v[u][k]);
                            cur_has = true;
                        }
                    }
                }
            }
            while (cur < nb) {
                flush(cur, acc, cur_has, cb);
#pragma unroll
                for (int k = 0; k < K; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                cur_has = false;
                ++cur;
            }
        }
    }
}

// NONE pooling (sequence embeddings): out[i, 0:D_t] = row(i), zero padded to max_D.
template <int G>
__global__ void __launch_bounds__(256) tbe_forward_nobag_kernel(FwdParams p)
{
    const int groups_per_block = blockDim.x / G;
    const int lane = threadIdx.x % G;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * groups_per_block + threadIdx.x / G; i < p.N;
         i += static_cast<int64_t>(gridDim.x) * groups_per_block) {
        // feature of position i: last t with offsets[t*B] <= i
        int64_t lo = 0, hi = p.T - 1;
        while (lo < hi) {
            int64_t mid = (lo + hi + 1) >> 1;
            if (p.offs[mid * p.B] <= i) lo = mid; else hi = mid - 1;
        }
        const int64_t t = lo;
        const int32_t D = p.dofs[t + 1] - p.dofs[t];
        const int64_t wofs = p.wofs[t];
        const int64_t id = p.idx[i];
        const int64_t ro = wofs + id * D;
        const bool ok = row_ok(p, id, ro, D);
        float* out_row = p.out + i * p.max_D;
        const bool vec_ok = aligned16(p.w) && aligned16(p.out) && (((wofs | D | p.max_D) & 3) == 0);
        if (vec_ok) {
            const int nvec = D >> 2, nvec_out = p.max_D >> 2;
            for (int c = lane; c < nvec_out; c += G) {
                float4 v = (ok && c < nvec) ? ld_f4(p.w + ro + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
                st_f4_stream(out_row + 4 * c, v);
            }
        } else {
            for (int c = lane; c < p.max_D; c += G) out_row[c] = (ok && c < D) ? p.w[ro + c] : 0.f;
        }
    }
}

#ifndef RECSDK_EMULATE  // host side: not part of host-side SIMT emulation builds (tests/emu)
template <int G, int K>
static void launch_pooled(const FwdParams& p, bool leave_room, cudaStream_t st)
{
    const int groups_per_block = 256 / G;
    // several waves of short-lived blocks rather than one resident wave: when the backward's index kernels run
    // beside this one on another stream, their blocks get SM slots as these retire (measured: 16 per SM 0.833 ms
    // per benchmark step, 8: 0.838, 2: 0.873; alone the grid size makes no difference)
    int grid = grid_for(ceil_div(p.T * p.B, G), groups_per_block, 16);
    size_t smem = 0;
    if (leave_room) {
        // unused dynamic shared memory as an occupancy limit: 60 KB per block -> three blocks per SM
        static bool optin_done[kMaxDevices] = {false};
        if (smem_optin(tbe_forward_pooled_kernel<G, K>, 60 * 1024, optin_done)) smem = 60 * 1024;
    }
    tbe_forward_pooled_kernel<G, K><<<grid, 256, smem, st>>>(p);
}

template <int G>
static void launch_nobag(const FwdParams& p, cudaStream_t st)
{
    const int groups_per_block = 256 / G;
    int grid = grid_for(p.N, groups_per_block, 8);
    tbe_forward_nobag_kernel<G><<<grid, 256, 0, st>>>(p);
}

}  // namespace recsdk

using namespace recsdk;

extern "C" int recsdk_tbe_forward(const recsdk_tbe_forward_args* a, void* stream)
{
    if (a == nullptr) return RECSDK_ERR_INVALID_ARG;
    if (a->T < 0 || a->B < 0 || a->N < 0 || a->max_D <= 0 || a->total_D <= 0) return RECSDK_ERR_INVALID_ARG;
    if (a->pooling_mode < RECSDK_POOL_SUM || a->pooling_mode > RECSDK_POOL_NONE) return RECSDK_ERR_INVALID_ARG;
    if (a->T == 0 || a->B == 0) return RECSDK_OK;
    if (!a->dev_weights || !a->weights_offsets || !a->D_offsets || !a->offsets) return RECSDK_ERR_INVALID_ARG;
    if (a->N > 0 && !a->indices) return RECSDK_ERR_INVALID_ARG;
    const recsdk_sample_shards& sh = a->out_shards;
    if (sh.num_shards == 0) {
        if (!a->out) return RECSDK_ERR_INVALID_ARG;
    } else {
        if (!sample_shards_valid(sh, a->B) || a->pooling_mode == RECSDK_POOL_NONE) return RECSDK_ERR_INVALID_ARG;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    FwdParams p{a->dev_weights, a->weights_offsets, a->D_offsets, a->indices, a->offsets, a->out, a->T, a->B, a->N,
                a->total_D, a->max_D, a->pooling_mode, a->weights_numel, a->dev_status,
                aligned16(a->dev_weights) ? 1 : 0, sh};
    const int vec_per_row = (a->max_D + 3) / 4;
    const int G = group_lanes_for(vec_per_row);
    const bool leave_room = (a->flags & RECSDK_FWD_LEAVE_ROOM) != 0;
    if (a->pooling_mode == RECSDK_POOL_NONE) {
        if (a->N == 0) return RECSDK_OK;
        switch (G) {
            case 1: launch_nobag<1>(p, st); break;
            case 2: launch_nobag<2>(p, st); break;
            case 4: launch_nobag<4>(p, st); break;
            case 8: launch_nobag<8>(p, st); break;
            case 16: launch_nobag<16>(p, st); break;
            default: launch_nobag<32>(p, st); break;
        }
    } else {
        switch (G) {
            case 1: launch_pooled<1, 1>(p, leave_room, st); break;
            case 2: launch_pooled<2, 1>(p, leave_room, st); break;
            case 4: launch_pooled<4, 1>(p, leave_room, st); break;
            case 8: launch_pooled<8, 1>(p, leave_room, st); break;
            case 16: launch_pooled<16, 1>(p, leave_room, st); break;
            default:
                if (vec_per_row <= 32) launch_pooled<32, 1>(p, leave_room, st);
                else if (vec_per_row <= 64) launch_pooled<32, 2>(p, leave_room, st);
                else launch_pooled<32, 4>(p, leave_room, st);
                break;
        }
    }
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}
#else
}  // namespace recsdk
#endif  // RECSDK_EMULATE
