// Pooled embedding gather over ragged bags (forward of the table-batched
// embedding op).  HBM-bound: G lanes cooperate on one bag, every lane moves
// 128-bit pieces of a row, rows of one bag are fetched four at a time so that
// several 128-bit loads per lane are in flight, and the pooled row is written
// once with a streaming store.  Rows are added in index order starting from
// 0.0f, which is the order of the reference kernel (Pooling(),
// split_embedding_codegen_forward_unweighted_kernel.h:226-241) for bags that
// fit one of its blocks, so the result is bit-exact against a sequential loop.
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
    int base_aligned;  // dev_weights and out are 16-byte aligned
};

__device__ __forceinline__ bool row_ok(const FwdParams& p, int64_t idx, int64_t row_off, int32_t D)
{
    if (p.w_numel <= 0) return true;
    if (idx < 0 || row_off + D > p.w_numel) {
        set_status(p.status, RECSDK_ERR_INDEX_RANGE, idx, row_off);
        return false;
    }
    return true;
}

// Scalar path for bags whose offsets/dims are not multiples of 4 elements.
template <int G>
__device__ void forward_bag_scalar(const FwdParams& p, int lane, int64_t s, int64_t e, int64_t wofs, int32_t D,
                                   float* out_row, float mean)
{
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

template <int G, int K>
__global__ void __launch_bounds__(256) tbe_forward_pooled_kernel(FwdParams p)
{
    const int groups_per_block = blockDim.x / G;
    const int lane = threadIdx.x % G;
    const int64_t num_bags = p.T * p.B;
    for (int64_t bag = static_cast<int64_t>(blockIdx.x) * groups_per_block + threadIdx.x / G; bag < num_bags;
         bag += static_cast<int64_t>(gridDim.x) * groups_per_block) {
        const int64_t t = bag / p.B;
        const int64_t b = bag - t * p.B;
        const int64_t s = p.offs[bag], e = p.offs[bag + 1];
        const int32_t d0 = p.dofs[t];
        const int32_t D = p.dofs[t + 1] - d0;
        const int64_t wofs = p.wofs[t];
        float* out_row = p.out + b * p.total_D + d0;
        const float mean = __fdiv_rn(1.0f, static_cast<float>(e - s));
        const bool vec_ok = p.base_aligned && (((wofs | D | d0 | p.total_D) & 3) == 0);
        if (!vec_ok) {
            forward_bag_scalar<G>(p, lane, s, e, wofs, D, out_row, mean);
            continue;
        }
        const int nvec = D >> 2;
        for (int cb = 0; cb < nvec; cb += G * K) {
            float4 acc[K];
#pragma unroll
            for (int k = 0; k < K; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            int64_t i = s;
            for (; i + 4 <= e; i += 4) {
                int64_t id[4];
                const float* rp[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) id[j] = p.idx[i + j];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int64_t ro = wofs + id[j] * D;
                    rp[j] = row_ok(p, id[j], ro, D) ? p.w + ro : nullptr;
                }
                float4 v[4][K];
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int k = 0; k < K; ++k) {
                        int c = cb + lane + k * G;
                        v[j][k] = (rp[j] != nullptr && c < nvec) ? ld_f4(rp[j] + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int k = 0; k < K; ++k) acc[k] = add4(acc[k], v[j][k]);
            }
            for (; i < e; ++i) {
                int64_t id = p.idx[i];
                int64_t ro = wofs + id * D;
                const float* rp = row_ok(p, id, ro, D) ? p.w + ro : nullptr;
#pragma unroll
                for (int k = 0; k < K; ++k) {
                    int c = cb + lane + k * G;
                    float4 v = (rp != nullptr && c < nvec) ? ld_f4(rp + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
                    acc[k] = add4(acc[k], v);
                }
            }
#pragma unroll
            for (int k = 0; k < K; ++k) {
                int c = cb + lane + k * G;
                if (c < nvec) {
                    float4 r = acc[k];
                    if (p.mode == RECSDK_POOL_MEAN && e > s) r = mul4s(r, mean);
                    st_f4_stream(out_row + 4 * c, r);
                }
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
        const bool vec_ok = p.base_aligned && (((wofs | D | p.max_D) & 3) == 0);
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

template <int G, int K>
static void launch_pooled(const FwdParams& p, cudaStream_t st)
{
    const int groups_per_block = 256 / G;
    int grid = grid_for(p.T * p.B, groups_per_block, 8);
    tbe_forward_pooled_kernel<G, K><<<grid, 256, 0, st>>>(p);
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
    if (!a->dev_weights || !a->weights_offsets || !a->D_offsets || !a->offsets || !a->out) return RECSDK_ERR_INVALID_ARG;
    if (a->N > 0 && !a->indices) return RECSDK_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    FwdParams p{a->dev_weights, a->weights_offsets, a->D_offsets, a->indices, a->offsets, a->out, a->T, a->B, a->N,
                a->total_D, a->max_D, a->pooling_mode, a->weights_numel, a->dev_status,
                (aligned16(a->dev_weights) && aligned16(a->out)) ? 1 : 0};
    const int vec_per_row = (a->max_D + 3) / 4;
    const int G = group_lanes_for(vec_per_row);
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
            case 1: launch_pooled<1, 1>(p, st); break;
            case 2: launch_pooled<2, 1>(p, st); break;
            case 4: launch_pooled<4, 1>(p, st); break;
            case 8: launch_pooled<8, 1>(p, st); break;
            case 16: launch_pooled<16, 1>(p, st); break;
            default:
                if (vec_per_row <= 32) launch_pooled<32, 1>(p, st);
                else if (vec_per_row <= 64) launch_pooled<32, 2>(p, st);
                else launch_pooled<32, 4>(p, st);
                break;
        }
    }
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}
