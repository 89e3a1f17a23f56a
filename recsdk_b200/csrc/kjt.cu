// Jagged-batch utilities that sit either side of the lookup in the input / output distribution:
// permute_2D / permute_1D sparse data, complete cumsum, jagged <-> padded dense.
// Replaces the adapters in cust_op/framework/torch_plugin/torch_library/2.6.0/{permute2d_sparse_data,
// permute1d_sparse_data,asynchronous_complete_cumsum,jagged_to_padded_dense,dense_to_jagged}/*.cpp.
// All byte movement: coalesced segment copies, 128-bit where the row width allows.
#include "common.cuh"

namespace recsdk {

constexpr int kScanTileI64 = 2048;  // 256 threads x 8

// ---------------------------------------------------------------------------- int64 scan (complete cumsum)
// block-wide inclusive scan of one value per thread (256 threads)
__device__ __forceinline__ int64_t block_scan_i64(int64_t v, int64_t* sm /*[9]*/, int64_t* total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int64_t x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int64_t y = __shfl_up_sync(kFullMask, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) sm[warp] = x;
    __syncthreads();
    if (warp == 0) {
        int64_t w = lane < 8 ? sm[lane] : 0;
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            const int64_t y = __shfl_up_sync(kFullMask, w, o);
            if (lane >= o) w += y;
        }
        if (lane < 8) sm[lane] = w;
    }
    __syncthreads();
    const int64_t before = warp > 0 ? sm[warp - 1] : 0;
    *total = sm[7];
    __syncthreads();
    return before + x;
}

// tile sums: sums[t] = sum of x over tile t
static __global__ void __launch_bounds__(256) cumsum_tile_sums_kernel(const int64_t* __restrict__ x, int64_t n,
                                                                      int64_t* __restrict__ sums)
{
    __shared__ int64_t sm[9];
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTileI64 + threadIdx.x * 8;
    int64_t s = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k)
        if (base + k < n) s += x[base + k];
    int64_t total;
    block_scan_i64(s, sm, &total);
    if (threadIdx.x == 0) sums[blockIdx.x] = total;
}

// exclusive scan of the tile sums in place (one block, any number of tiles)
static __global__ void __launch_bounds__(256) cumsum_scan_sums_kernel(int64_t* __restrict__ sums, int64_t tiles)
{
    __shared__ int64_t sm[9];
    int64_t carry = 0;
    for (int64_t b = 0; b < tiles; b += 256) {
        const int64_t i = b + threadIdx.x;
        const int64_t v = i < tiles ? sums[i] : 0;
        int64_t total;
        const int64_t inc = block_scan_i64(v, sm, &total);
        if (i < tiles) sums[i] = carry + inc - v;
        carry += total;
    }
}

// out[0] = 0, out[i + 1] = x[0] + ... + x[i]
static __global__ void __launch_bounds__(256) cumsum_apply_kernel(const int64_t* __restrict__ x, int64_t n,
                                                                  const int64_t* __restrict__ sums,
                                                                  int64_t* __restrict__ out)
{
    __shared__ int64_t sm[9];
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTileI64 + threadIdx.x * 8;
    int64_t v[8];
    int64_t s = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        v[k] = base + k < n ? x[base + k] : 0;
        s += v[k];
    }
    int64_t total;
    const int64_t inc = block_scan_i64(s, sm, &total);
    int64_t run = sums[blockIdx.x] + inc - s;
    if (blockIdx.x == 0 && threadIdx.x == 0) out[0] = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        run += v[k];
        if (base + k < n) out[base + k + 1] = run;
    }
}

static void complete_cumsum(const int64_t* x, int64_t n, int64_t* out, int64_t* tile_sums, cudaStream_t st)
{
    const int64_t tiles = ceil_div(n > 0 ? n : 1, kScanTileI64);
    cumsum_tile_sums_kernel<<<static_cast<unsigned>(tiles), 256, 0, st>>>(x, n, tile_sums);
    cumsum_scan_sums_kernel<<<1, 256, 0, st>>>(tile_sums, tiles);
    cumsum_apply_kernel<<<static_cast<unsigned>(tiles), 256, 0, st>>>(x, n, tile_sums, out);
}

// ---------------------------------------------------------------------------- permute
// row_tot[t] = sum_b lengths[t, b]  (one block per row)
static __global__ void __launch_bounds__(256) row_totals_kernel(const int64_t* __restrict__ lengths, int64_t B,
                                                                int64_t* __restrict__ row_tot)
{
    __shared__ int64_t sm[9];
    const int64_t* row = lengths + static_cast<int64_t>(blockIdx.x) * B;
    int64_t s = 0;
    for (int64_t b = threadIdx.x; b < B; b += 256) s += row[b];
    int64_t total;
    block_scan_i64(s, sm, &total);
    if (threadIdx.x == 0) row_tot[blockIdx.x] = total;
}

// out_lengths[t', :] = lengths[permute[t'], :] and out_tot[t'] = row_tot[permute[t']]
static __global__ void __launch_bounds__(256) permute_lengths_kernel(const int64_t* __restrict__ permute, int64_t T_in,
                                                                     const int64_t* __restrict__ lengths, int64_t B,
                                                                     const int64_t* __restrict__ row_tot,
                                                                     int64_t* __restrict__ out_lengths,
                                                                     int64_t* __restrict__ out_tot,
                                                                     int64_t* __restrict__ status)
{
    int64_t src = permute[blockIdx.x];
    if (src < 0 || src >= T_in) {
        if (threadIdx.x == 0) set_status(status, RECSDK_ERR_INDEX_RANGE, src, blockIdx.x);
        src = -1;
    }
    for (int64_t b = threadIdx.x; b < B; b += 256)
        out_lengths[static_cast<int64_t>(blockIdx.x) * B + b] = src >= 0 ? lengths[src * B + b] : 0;
    if (threadIdx.x == 0) out_tot[blockIdx.x] = src >= 0 ? row_tot[src] : 0;
}

// segment copy: output row t' takes input segment [in_start[permute[t']], +len).  blockIdx.y slices long rows.
template <typename V>
static __global__ void __launch_bounds__(256) permute_values_kernel(const int64_t* __restrict__ permute, int64_t T_in,
                                                                    const int64_t* __restrict__ in_start,
                                                                    const int64_t* __restrict__ out_start,
                                                                    const V* __restrict__ values,
                                                                    const float* __restrict__ weights,
                                                                    V* __restrict__ out_values,
                                                                    float* __restrict__ out_weights,
                                                                    int64_t out_capacity, int64_t* __restrict__ status)
{
    const int64_t src = permute[blockIdx.x];
    if (src < 0 || src >= T_in) return;
    const int64_t s0 = in_start[src], len = in_start[src + 1] - s0, d0 = out_start[blockIdx.x];
    if (d0 + len > out_capacity) {
        if (threadIdx.x == 0 && blockIdx.y == 0) set_status(status, RECSDK_ERR_TOO_LARGE, d0 + len, out_capacity);
        return;
    }
    for (int64_t i = static_cast<int64_t>(blockIdx.y) * 256 + threadIdx.x; i < len;
         i += static_cast<int64_t>(gridDim.y) * 256) {
        out_values[d0 + i] = values[s0 + i];
        if (weights != nullptr) out_weights[d0 + i] = weights[s0 + i];
    }
}

// ---------------------------------------------------------------------------- jagged <-> padded dense
// one group of lanes per (sample, position) row of the dense tensor
template <bool TO_DENSE>
static __global__ void __launch_bounds__(256) jagged_dense_kernel(float* __restrict__ values,
                                                                  const int64_t* __restrict__ offsets, int64_t B,
                                                                  int32_t D, int64_t L, float padding,
                                                                  float* __restrict__ dense, int vec, int lanes)
{
    // `lanes` (a power of two <= 32) threads share one row: as many as it has 128-bit words, so narrow rows do
    // not leave most of a warp idle
    const int lane = threadIdx.x & (lanes - 1);
    const int64_t rows = B * L;
    for (int64_t r = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / lanes; r < rows;
         r += static_cast<int64_t>(gridDim.x) * blockDim.x / lanes) {
        const int64_t b = r / L, l = r - b * L;
        const int64_t s = offsets[b], len = offsets[b + 1] - s;
        float* drow = dense + r * D;
        if (l < len) {
            float* vrow = values + (s + l) * D;
            if (vec) {
                for (int c = lane; c < (D >> 2); c += lanes) {
                    if (TO_DENSE) st_f4_stream(drow + 4 * c, ld_f4_stream(vrow + 4 * c));
                    else st_f4_stream(vrow + 4 * c, ld_f4_stream(drow + 4 * c));
                }
            } else {
                for (int c = lane; c < D; c += lanes) {
                    if (TO_DENSE) drow[c] = vrow[c];
                    else vrow[c] = drow[c];
                }
            }
        } else if (TO_DENSE) {
            if (vec) {
                const float4 pad = make_float4(padding, padding, padding, padding);
                for (int c = lane; c < (D >> 2); c += lanes) st_f4_stream(drow + 4 * c, pad);
            } else {
                for (int c = lane; c < D; c += lanes) drow[c] = padding;
            }
        }
    }
}

// jagged rows beyond the dense length L have no source: zero them
static __global__ void __launch_bounds__(256) jagged_tail_zero_kernel(float* __restrict__ values,
                                                                      const int64_t* __restrict__ offsets, int64_t B,
                                                                      int32_t D, int64_t L)
{
    const int lane = threadIdx.x & 31;
    for (int64_t b = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; b < B;
         b += (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5) {
        const int64_t s = offsets[b], len = offsets[b + 1] - s;
        for (int64_t l = L; l < len; ++l)
            for (int c = lane; c < D; c += 32) values[(s + l) * D + c] = 0.f;
    }
}

}  // namespace recsdk

using namespace recsdk;

static int row_lanes(int32_t D, int vec)
{
    const int words = vec ? (D >> 2) : D;
    int lanes = 1;
    while (lanes < 32 && lanes < words) lanes <<= 1;
    return lanes;
}

extern "C" size_t recsdk_complete_cumsum_workspace_bytes(int64_t n)
{
    return align_up(static_cast<size_t>(ceil_div(n > 0 ? n : 1, kScanTileI64)) * sizeof(int64_t));
}

extern "C" int recsdk_complete_cumsum(const int64_t* x, int64_t n, int64_t* out, void* workspace, size_t workspace_bytes,
                                      void* stream)
{
    if (n < 0 || out == nullptr || (n > 0 && x == nullptr)) return RECSDK_ERR_INVALID_ARG;
    if (workspace == nullptr || workspace_bytes < recsdk_complete_cumsum_workspace_bytes(n)) return RECSDK_ERR_WORKSPACE;
    complete_cumsum(x, n, out, static_cast<int64_t*>(workspace), static_cast<cudaStream_t>(stream));
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" size_t recsdk_permute_sparse_workspace_bytes(int64_t T_in, int64_t T_out)
{
    const size_t a = static_cast<size_t>(T_in > 0 ? T_in : 1), b = static_cast<size_t>(T_out > 0 ? T_out : 1);
    return align_up(a * 8) + align_up((a + 1) * 8) + align_up(b * 8) + align_up((b + 1) * 8) +
           recsdk_complete_cumsum_workspace_bytes(static_cast<int64_t>(a > b ? a : b));
}

extern "C" int recsdk_permute_2d_sparse_data(const int64_t* permute, int64_t T_out, const int64_t* lengths, int64_t T_in,
                                             int64_t B, const void* values, int32_t value_bytes, const float* weights,
                                             int64_t* out_lengths, void* out_values, float* out_weights,
                                             int64_t out_capacity, int64_t* out_total, int64_t* dev_status,
                                             void* workspace, size_t workspace_bytes, void* stream)
{
    if (T_out < 0 || T_in < 0 || B < 0 || out_capacity < 0) return RECSDK_ERR_INVALID_ARG;
    if (value_bytes != 4 && value_bytes != 8) return RECSDK_ERR_INVALID_ARG;
    if ((weights == nullptr) != (out_weights == nullptr)) return RECSDK_ERR_INVALID_ARG;
    if (T_out == 0 || B == 0) return RECSDK_OK;
    if (!permute || !lengths || !out_lengths || T_in == 0) return RECSDK_ERR_INVALID_ARG;
    if (out_capacity > 0 && (!values || !out_values)) return RECSDK_ERR_INVALID_ARG;
    if (workspace == nullptr || workspace_bytes < recsdk_permute_sparse_workspace_bytes(T_in, T_out)) return RECSDK_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    WorkspaceCarver c(workspace);
    int64_t* row_tot = c.take<int64_t>(T_in);
    int64_t* in_start = c.take<int64_t>(T_in + 1);
    int64_t* out_tot = c.take<int64_t>(T_out);
    int64_t* out_start = c.take<int64_t>(T_out + 1);
    int64_t* tiles = c.take<int64_t>(recsdk_complete_cumsum_workspace_bytes(T_in > T_out ? T_in : T_out) / 8);
    row_totals_kernel<<<static_cast<unsigned>(T_in), 256, 0, st>>>(lengths, B, row_tot);
    complete_cumsum(row_tot, T_in, in_start, tiles, st);
    permute_lengths_kernel<<<static_cast<unsigned>(T_out), 256, 0, st>>>(permute, T_in, lengths, B, row_tot, out_lengths,
                                                                        out_tot, dev_status);
    complete_cumsum(out_tot, T_out, out_start, tiles, st);
    if (out_total != nullptr)
        cudaMemcpyAsync(out_total, out_start + T_out, sizeof(int64_t), cudaMemcpyDeviceToDevice, st);
    if (out_capacity > 0) {
        const dim3 grid(static_cast<unsigned>(T_out), 32);
        if (value_bytes == 8)
            permute_values_kernel<int64_t><<<grid, 256, 0, st>>>(permute, T_in, in_start, out_start,
                                                                 static_cast<const int64_t*>(values), weights,
                                                                 static_cast<int64_t*>(out_values), out_weights, out_capacity,
                                                                 dev_status);
        else
            permute_values_kernel<int32_t><<<grid, 256, 0, st>>>(permute, T_in, in_start, out_start,
                                                                 static_cast<const int32_t*>(values), weights,
                                                                 static_cast<int32_t*>(out_values), out_weights, out_capacity,
                                                                 dev_status);
    }
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_jagged_to_padded_dense(const float* values, const int64_t* offsets, int64_t B, int32_t D,
                                             int64_t max_length, float padding_value, float* dense, void* stream)
{
    if (B < 0 || D <= 0 || max_length <= 0) return RECSDK_ERR_INVALID_ARG;
    if (B == 0) return RECSDK_OK;
    if (!offsets || !dense) return RECSDK_ERR_INVALID_ARG;
    const int vec = (aligned16(values) && aligned16(dense) && (D & 3) == 0) ? 1 : 0;
    const int lanes = row_lanes(D, vec);
    jagged_dense_kernel<true><<<grid_for(B * max_length, 256 / lanes, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        const_cast<float*>(values), offsets, B, D, max_length, padding_value, dense, vec, lanes);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}

extern "C" int recsdk_dense_to_jagged(const float* dense, const int64_t* offsets, int64_t B, int32_t D, int64_t max_length,
                                      float* values, void* stream)
{
    if (B < 0 || D <= 0 || max_length <= 0) return RECSDK_ERR_INVALID_ARG;
    if (B == 0) return RECSDK_OK;
    if (!offsets || !dense || !values) return RECSDK_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int vec = (aligned16(values) && aligned16(dense) && (D & 3) == 0) ? 1 : 0;
    const int lanes = row_lanes(D, vec);
    jagged_dense_kernel<false><<<grid_for(B * max_length, 256 / lanes, 8), 256, 0, st>>>(
        values, offsets, B, D, max_length, 0.f, const_cast<float*>(dense), vec, lanes);
    jagged_tail_zero_kernel<<<grid_for(B, 8, 8), 256, 0, st>>>(values, offsets, B, D, max_length);
    RECSDK_CUDA_CHECK_LAUNCH();
    return RECSDK_OK;
}
