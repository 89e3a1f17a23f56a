// Row movement and per-row optimizer operators:
//   gather_rows / scatter_rows   bulk row copies by slot (cache swap-out / swap-in)
//   lookup/update by address     TF-flavour dynamic-expansion tables
//   lazy_adam, sgd               TF-flavour fused sparse optimizers
//   restore                      hash_indices from unique + inverse
//
// gather/scatter move whole rows with the bulk asynchronous copy engine (TMA,
// cp.async.bulk) through shared memory: a warp stages 8 rows per buffer, two
// buffers deep, each row fetched by its own bulk copy signalling one mbarrier,
// the contiguous side moved by a single bulk copy.  No registers or LSU slots
// are spent on the payload.  Needs 16-byte aligned rows; other shapes use the
// plain 128-bit/32-bit load path.
#include "common.cuh"
#include "tma.cuh"

namespace recsdk {

// ---------------------------------------------------------------------------- TMA row gather / scatter
constexpr int kRowsPerStage = 8;
constexpr int kStages = 2;
constexpr int kTmaWarps = 4;

// GATHER: out[i,:] = table[slots[i],:]   SCATTER: table[slots[i],:] = rows[i,:]
template <bool GATHER>
__global__ void __launch_bounds__(kTmaWarps * 32) rows_tma_kernel(float* __restrict__ table,
                                                                  const int64_t* __restrict__ slots, int64_t k,
                                                                  int32_t D, float* __restrict__ dense,
                                                                  int64_t table_rows, int64_t* __restrict__ status,
                                                                  int wait_limit)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[kTmaWarps][kStages];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row_bytes = static_cast<uint32_t>(D) * 4u;
    unsigned char* wbuf = smem_raw + static_cast<size_t>(warp) * kStages * kRowsPerStage * row_bytes;
    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&bars[warp][s], 1);
        mbar_fence_init();
    }
    __syncwarp();

    const int64_t warps_total = static_cast<int64_t>(gridDim.x) * kTmaWarps;
    const int64_t wid = static_cast<int64_t>(blockIdx.x) * kTmaWarps + warp;
    const int64_t nbatch = (k + kRowsPerStage - 1) / kRowsPerStage;
    uint32_t phase[kStages] = {0, 0};
    bool failed = false;

    // software pipeline over this warp's batches: load batch j+1 while storing batch j
    auto issue_load = [&](int64_t batch, int stage) {
        const int64_t i0 = batch * kRowsPerStage;
        const int rows = static_cast<int>((k - i0) < kRowsPerStage ? (k - i0) : kRowsPerStage);
        unsigned char* buf = wbuf + static_cast<size_t>(stage) * kRowsPerStage * row_bytes;
        if (lane == 0) mbar_expect_tx(&bars[warp][stage], rows * row_bytes);
        __syncwarp();
        if (GATHER) {
            if (lane < rows) {
                int64_t s = slots[i0 + lane];
                if (s < 0 || (table_rows > 0 && s >= table_rows)) {
                    set_status(status, RECSDK_ERR_INDEX_RANGE, s, i0 + lane);
                    s = 0;
                }
                bulk_g2s(buf + static_cast<size_t>(lane) * row_bytes, table + s * D, row_bytes, &bars[warp][stage]);
            }
        } else if (lane == 0) {
            bulk_g2s(buf, dense + i0 * D, rows * row_bytes, &bars[warp][stage]);
        }
    };
    auto issue_store = [&](int64_t batch, int stage) {
        const int64_t i0 = batch * kRowsPerStage;
        const int rows = static_cast<int>((k - i0) < kRowsPerStage ? (k - i0) : kRowsPerStage);
        unsigned char* buf = wbuf + static_cast<size_t>(stage) * kRowsPerStage * row_bytes;
        fence_async_smem();
        if (GATHER) {
            if (lane == 0) bulk_s2g(dense + i0 * D, buf, rows * row_bytes);
        } else if (lane < rows) {
            int64_t s = slots[i0 + lane];
            if (s < 0 || (table_rows > 0 && s >= table_rows))
                set_status(status, RECSDK_ERR_INDEX_RANGE, s, i0 + lane);
            else
                bulk_s2g(table + s * D, buf + static_cast<size_t>(lane) * row_bytes, row_bytes);
        }
        bulk_commit();
    };

    int64_t batch = wid;
    int stage = 0;
    if (batch < nbatch) issue_load(batch, stage);
    while (batch < nbatch) {
        const int64_t next = batch + warps_total;
        const int nstage = stage ^ 1;
        if (next < nbatch) {
            // the buffer we are about to refill was read by the store issued one iteration ago
            bulk_wait_read<0>();
            __syncwarp();
            issue_load(next, nstage);
        }
        if (!mbar_wait_bounded(&bars[warp][stage], phase[stage], wait_limit)) {
            // the wait ran out: report, stop taking work, and give the loads already issued (this stage, and the next
            // one when it was armed) a bounded time to land before the block's shared memory is released
            set_status(status, RECSDK_ERR_CUDA, -1, batch);
            failed = true;
            (void)mbar_wait_bounded(&bars[warp][stage], phase[stage]);
            if (next < nbatch) (void)mbar_wait_bounded(&bars[warp][nstage], phase[nstage]);
            break;
        }
        phase[stage] ^= 1;
        issue_store(batch, stage);
        batch = next;
        stage = nstage;
    }
    (void)failed;
    bulk_wait_all();
}

// Plain-load fallback (rows not 16-byte aligned) and the generic row copy used below.
template <bool GATHER>
__global__ void __launch_bounds__(256) rows_plain_kernel(float* __restrict__ table, const int64_t* __restrict__ slots,
                                                         int64_t k, int32_t D, float* __restrict__ dense,
                                                         int64_t table_rows, int64_t* __restrict__ status)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < k; i += warps_total) {
        const int64_t s = slots[i];
        if (s < 0 || (table_rows > 0 && s >= table_rows)) {
            set_status(status, RECSDK_ERR_INDEX_RANGE, s, i);
            continue;
        }
        float* trow = table + s * D;
        float* drow = dense + i * D;
        for (int c = lane; c < D; c += 32) {
            if (GATHER) drow[c] = trow[c]; else trow[c] = drow[c];
        }
    }
}

template <bool GATHER>
static int launch_rows(float* table, const int64_t* slots, int64_t k, int32_t D, float* dense, int64_t table_rows,
                       int64_t* status, cudaStream_t st, int wait_limit = 1 << 22)
{
    if (k == 0) return RECSDK_OK;
    const size_t row_bytes = static_cast<size_t>(D) * 4;
    const size_t smem = static_cast<size_t>(kTmaWarps) * kStages * kRowsPerStage * row_bytes;
    const bool tma_ok = (row_bytes % 16 == 0) && aligned16(table) && aligned16(dense) && smem <= 200 * 1024;
    if (tma_ok) {
        auto kern = rows_tma_kernel<GATHER>;
        if (smem > 48 * 1024) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
                return RECSDK_ERR_CUDA;
        }
        const int64_t nbatch = ceil_div(k, kRowsPerStage);
        int grid = grid_for(nbatch, kTmaWarps, 8);
        kern<<<grid, kTmaWarps * 32, smem, st>>>(table, slots, k, D, dense, table_rows, status, wait_limit);
    } else {
        rows_plain_kernel<GATHER><<<grid_for(k, 8), 256, 0, st>>>(table, slots, k, D, dense, table_rows, status);
    }
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

// ---------------------------------------------------------------------------- by address
__global__ void __launch_bounds__(256) lookup_by_address_kernel(const int64_t* __restrict__ addr, int64_t n, int32_t dim,
                                                                float* __restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < n; i += warps_total) {
        const float* src = reinterpret_cast<const float*>(static_cast<intptr_t>(addr[i]));
        float* dst = out + i * dim;
        const bool v4 = src != nullptr && (dim & 3) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
        if (v4) {
            for (int c = lane; c < (dim >> 2); c += 32) st_f4_stream(dst + 4 * c, ld_f4(src + 4 * c));
        } else {
            for (int c = lane; c < dim; c += 32) dst[c] = src != nullptr ? src[c] : 0.f;
        }
    }
}

__global__ void __launch_bounds__(256) update_by_address_kernel(const int64_t* __restrict__ addr, int64_t n, int32_t dim,
                                                                const float* __restrict__ emb, int32_t update_type)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < n; i += warps_total) {
        float* dst = reinterpret_cast<float*>(static_cast<intptr_t>(addr[i]));
        if (dst == nullptr) continue;
        const float* src = emb + i * dim;
        for (int c = lane; c < dim; c += 32) {
            if (update_type == 0) atomicAdd(dst + c, src[c]); else dst[c] = src[c];
        }
    }
}

// ---------------------------------------------------------------------------- lazy adam / sgd
// operand order of lazy_adam.cpp:170-190 (Muls, Muls, add; Muls, Mul, Muls, add; Abs, Sqrt, Adds, Muls, Div, Add)
__global__ void __launch_bounds__(256) lazy_adam_kernel(const float* __restrict__ grad, const int32_t* __restrict__ idx,
                                                        int64_t n, int32_t dim, float* __restrict__ m,
                                                        float* __restrict__ v, float* __restrict__ var, float lr,
                                                        float beta1, float beta2, float eps)
{
    const int lane = threadIdx.x & 31;
    const float omb1 = 1.0f - beta1, omb2 = 1.0f - beta2, nlr = -lr;
    const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < n; i += warps_total) {
        const int64_t r = idx[i];
        if (r < 0) continue;
        for (int c = lane; c < dim; c += 32) {
            const int64_t o = r * dim + c;
            const float g = grad[i * dim + c];
            const float nm = __fadd_rn(__fmul_rn(m[o], beta1), __fmul_rn(g, omb1));
            const float nv = fabsf(__fadd_rn(__fmul_rn(v[o], beta2), __fmul_rn(__fmul_rn(g, g), omb2)));
            const float den = __fadd_rn(__fsqrt_rn(nv), eps);
            const float upd = __fdiv_rn(__fmul_rn(nm, nlr), den);
            m[o] = nm;
            v[o] = nv;
            var[o] = __fadd_rn(upd, var[o]);
        }
    }
}

// Two phases like the reference (gather var, compute, then atomic scatter-add):
// with weight decay every occurrence of a duplicated index sees the ORIGINAL var.
__global__ void __launch_bounds__(256) sgd_compute_kernel(const float* __restrict__ grad, const int64_t* __restrict__ idx,
                                                          int64_t n, int32_t dim, const float* __restrict__ var,
                                                          float lr, float wd, int32_t use_wd, float* __restrict__ upd)
{
    const float nlr = -lr;
    const int64_t total = n * dim;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
         e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t i = e / dim;
        const int c = static_cast<int>(e - i * dim);
        const int64_t r = idx[i];
        float g = grad[e];
        if (use_wd && r >= 0) g = __fadd_rn(g, __fmul_rn(var[r * dim + c], wd));
        upd[e] = __fmul_rn(g, nlr);
    }
}

__global__ void __launch_bounds__(256) sgd_apply_kernel(const float* __restrict__ upd, const int64_t* __restrict__ idx,
                                                        int64_t n, int32_t dim, float* __restrict__ var)
{
    const int64_t total = n * dim;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
         e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t i = e / dim;
        const int c = static_cast<int>(e - i * dim);
        const int64_t r = idx[i];
        if (r >= 0) atomicAdd(var + r * dim + c, upd[e]);
    }
}

// no-weight-decay SGD needs no staging: var += g * -lr
__global__ void __launch_bounds__(256) sgd_direct_kernel(const float* __restrict__ grad, const int64_t* __restrict__ idx,
                                                         int64_t n, int32_t dim, float* __restrict__ var, float lr)
{
    const float nlr = -lr;
    const int64_t total = n * dim;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
         e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t i = e / dim;
        const int c = static_cast<int>(e - i * dim);
        const int64_t r = idx[i];
        if (r >= 0) atomicAdd(var + r * dim + c, __fmul_rn(grad[e], nlr));
    }
}

// ---------------------------------------------------------------------------- restore
__global__ void __launch_bounds__(256) restore_kernel(const int64_t* __restrict__ uidx, const int64_t* __restrict__ uinv,
                                                      const int64_t* __restrict__ uoff,
                                                      const int64_t* __restrict__ table_offs, int64_t n_tables,
                                                      int64_t n, int64_t* __restrict__ out)
{
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; r < n;
         r += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        int64_t lo = 0, hi = n_tables - 1;  // last t with table_offs[t] <= r
        while (lo < hi) {
            int64_t mid = (lo + hi + 1) >> 1;
            if (table_offs[mid] <= r) lo = mid; else hi = mid - 1;
        }
        if (r >= table_offs[n_tables]) continue;
        out[r] = uidx[uinv[r] + uoff[lo]];
    }
}

}  // namespace recsdk

using namespace recsdk;

extern "C" int recsdk_gather_rows(const float* table, const int64_t* slots, int64_t k, int32_t D, float* out,
                                  int64_t table_rows, int64_t* dev_status, void* stream)
{
    if (k < 0 || D <= 0) return RECSDK_ERR_INVALID_ARG;
    if (k > 0 && (!table || !slots || !out)) return RECSDK_ERR_INVALID_ARG;
    return launch_rows<true>(const_cast<float*>(table), slots, k, D, out, table_rows, dev_status,
                             static_cast<cudaStream_t>(stream));
}

extern "C" int recsdk_gather_rows_wait_limit(const float* table, const int64_t* slots, int64_t k, int32_t D, float* out,
                                             int64_t table_rows, int64_t* dev_status, int32_t wait_limit, void* stream)
{
    if (k < 0 || D <= 0 || wait_limit < 0) return RECSDK_ERR_INVALID_ARG;
    if (k > 0 && (!table || !slots || !out)) return RECSDK_ERR_INVALID_ARG;
    return launch_rows<true>(const_cast<float*>(table), slots, k, D, out, table_rows, dev_status,
                             static_cast<cudaStream_t>(stream), wait_limit);
}

extern "C" int recsdk_scatter_rows(float* table, const int64_t* slots, int64_t k, int32_t D, const float* rows,
                                   int64_t table_rows, int64_t* dev_status, void* stream)
{
    if (k < 0 || D <= 0) return RECSDK_ERR_INVALID_ARG;
    if (k > 0 && (!table || !slots || !rows)) return RECSDK_ERR_INVALID_ARG;
    return launch_rows<false>(table, slots, k, D, const_cast<float*>(rows), table_rows, dev_status,
                              static_cast<cudaStream_t>(stream));
}

extern "C" int recsdk_lookup_by_address(const int64_t* addresses, int64_t n, int32_t embedding_dim, float* out,
                                        void* stream)
{
    if (n < 0 || embedding_dim <= 0) return RECSDK_ERR_INVALID_ARG;
    if (n == 0) return RECSDK_OK;
    if (!addresses || !out) return RECSDK_ERR_INVALID_ARG;
    lookup_by_address_kernel<<<grid_for(n, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(addresses, n, embedding_dim, out);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_update_by_address(const int64_t* addresses, int64_t n, int32_t embedding_dim,
                                        const float* embedding, int32_t update_type, void* stream)
{
    if (n < 0 || embedding_dim <= 0) return RECSDK_ERR_INVALID_ARG;
    if (n == 0) return RECSDK_OK;
    if (!addresses || !embedding) return RECSDK_ERR_INVALID_ARG;
    update_by_address_kernel<<<grid_for(n, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(addresses, n, embedding_dim,
                                                                                         embedding, update_type);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_lazy_adam(const float* gradient, const int32_t* indices, int64_t n, int32_t dim, float* m,
                                float* v, float* var, float lr, float beta1, float beta2, float epsilon, void* stream)
{
    if (n < 0 || dim <= 0) return RECSDK_ERR_INVALID_ARG;
    if (n == 0) return RECSDK_OK;
    if (!gradient || !indices || !m || !v || !var) return RECSDK_ERR_INVALID_ARG;
    lazy_adam_kernel<<<grid_for(n, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(gradient, indices, n, dim, m, v, var,
                                                                                 lr, beta1, beta2, epsilon);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_sgd(const float* gradient, const int64_t* indices, int64_t n, int32_t dim, float* var, float lr,
                          float weight_decay, int32_t use_weight_decay, void* workspace, size_t workspace_bytes,
                          void* stream)
{
    if (n < 0 || dim <= 0) return RECSDK_ERR_INVALID_ARG;
    if (n == 0) return RECSDK_OK;
    if (!gradient || !indices || !var) return RECSDK_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!use_weight_decay) {
        sgd_direct_kernel<<<grid_for(n * dim, 256), 256, 0, st>>>(gradient, indices, n, dim, var, lr);
    } else {
        // every update is computed from the ORIGINAL var before any add lands (the reference
        // gathers all rows, computes, then scatter-adds), so the updates are staged
        const size_t need = static_cast<size_t>(n) * dim * sizeof(float);
        if (!workspace || workspace_bytes < need) return RECSDK_ERR_WORKSPACE;
        float* upd = static_cast<float*>(workspace);
        sgd_compute_kernel<<<grid_for(n * dim, 256), 256, 0, st>>>(gradient, indices, n, dim, var, lr, weight_decay, 1, upd);
        sgd_apply_kernel<<<grid_for(n * dim, 256), 256, 0, st>>>(upd, indices, n, dim, var);
    }
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_restore(const int64_t* unique_indices, const int64_t* unique_inverse,
                              const int64_t* unique_offset, const int64_t* offsets_per_table, int64_t n_tables,
                              int64_t n, int64_t* hash_indices, void* stream)
{
    if (n < 0 || n_tables < 0) return RECSDK_ERR_INVALID_ARG;
    if (n == 0 || n_tables == 0) return RECSDK_OK;
    if (!unique_indices || !unique_inverse || !unique_offset || !offsets_per_table || !hash_indices)
        return RECSDK_ERR_INVALID_ARG;
    restore_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        unique_indices, unique_inverse, unique_offset, offsets_per_table, n_tables, n, hash_indices);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}
