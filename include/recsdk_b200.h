/*
 * recsdk_b200 -- C ABI of the B200 (sm_100a) sparse-embedding hot path.
 *
 * Every entry point is plain C: device pointers, sizes, scalars and a CUDA
 * stream (passed as void*).  No entry point allocates, frees or synchronises;
 * work is enqueued on the given stream and the call returns.  Scratch memory is
 * caller-provided: ask the matching *_workspace_bytes() function, allocate once,
 * pass it in (the same two-call shape as the reference's aclnn GetWorkspaceSize
 * + execute pair, cust_op/framework/torch_plugin/torch_library/2.6.0/common/
 * pytorch_npu_helper.hpp:512-561).
 *
 * Return value: RECSDK_OK or a RECSDK_ERR_* for errors the host can see
 * (bad arguments, workspace too small, launch failure).  Errors that only the
 * device can see (negative key, table full, cache too small, index out of
 * range) are written to a caller-provided device status block, see
 * recsdk_status_t; the host reads it when it wants to (the torch/python layer
 * does so where the reference would raise).
 *
 * All reference citations are paths inside the reference project.
 */
#ifndef RECSDK_B200_H
#define RECSDK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RECSDK_API __attribute__((visibility("default")))

/* ---- status codes (host return values and device status block) ---------- */
enum {
    RECSDK_OK = 0,
    RECSDK_ERR_INVALID_ARG = 1,     /* null pointer, negative size, unsupported mode */
    RECSDK_ERR_WORKSPACE = 2,       /* workspace smaller than *_workspace_bytes()     */
    RECSDK_ERR_CUDA = 3,            /* kernel launch / runtime error                  */
    RECSDK_ERR_NEGATIVE_KEY = 4,    /* hybrid_torchrec/src/ids_process/ids_mapper.cpp:45,83  "Invalid key value" */
    RECSDK_ERR_TABLE_FULL = 5,      /* ids_mapper.cpp:48-50,93-97 "Ids map reached maxIndex"               */
    RECSDK_ERR_CACHE_TOO_SMALL = 6, /* torchrec_embcache/csrc/embedding_cache/swap_manager.cpp:114-116      */
    RECSDK_ERR_INDEX_RANGE = 7,     /* a row index / slot / offset outside its table                        */
    RECSDK_ERR_HASH_FULL = 8,       /* open-addressing key table has no free entry left                     */
    RECSDK_ERR_TOO_LARGE = 9,       /* size beyond a stated maximum                                         */
    RECSDK_ERR_STATIC_SCRATCH = 10  /* the library's built-in scratch array could not be located on this device     */
};

/* Device status block: 4 x int64 {code, detail0, detail1, reserved}.  The first
 * error wins (atomicCAS on code).  Zero it before use (recsdk_status_clear). */
#define RECSDK_STATUS_WORDS 4
RECSDK_API int recsdk_status_clear(int64_t* dev_status, void* stream);

RECSDK_API const char* recsdk_error_string(int code);
RECSDK_API int recsdk_version(void);

/* ---- enums shared with the reference operator API ------------------------
 * cust_op/framework/torch_plugin/torch_library/2.6.0/split_embedding_codegen_forward_unweighted/
 * split_embedding_codegen_forward_unweighted.h:18-39 */
enum { RECSDK_POOL_SUM = 0, RECSDK_POOL_MEAN = 1, RECSDK_POOL_NONE = 2 };
enum { RECSDK_OPT_ADAGRAD = 1, RECSDK_OPT_ADAM = 2, RECSDK_OPT_SGD = 3 };

/* ---- sample-sharded [B,total_D] matrix (table-wise sharding on one box) -----
 * With table-wise sharding (hybrid_torchrec/hybrid_torchrec/distributed/sharding/hybrid_tw_sharding.py:43-82)
 * the table owner pools rows for the samples of EVERY rank and the reference then moves the pooled rows to
 * the sample owners with an all-to-all (torchrec PooledEmbeddingsAllToAll), and the gradients back with a
 * second one.  Here the forward kernel can store each pooled row straight into the sample owner's buffer
 * and the backward kernels can read each gradient row straight from it, over NVLink peer mappings
 * (recsdk_peer_*), so the exchange happens inside the kernels that produce / consume the data.
 *
 * num_shards == 0: off, the plain `out` / `grad_output` pointer is used.
 * num_shards == W: sample g = s*shard_B + b (0 <= b < shard_B, B == W*shard_B) is row b of ptrs[s]; a row
 * there is row_stride floats wide and feature t's columns start at col_offsets[t] (device array [T]).
 * Pooled modes only. */
#define RECSDK_MAX_SHARDS 16
typedef struct {
    int32_t num_shards;
    int32_t row_stride;
    int64_t shard_B;
    const int32_t* col_offsets;
    float* ptrs[RECSDK_MAX_SHARDS];
} recsdk_sample_shards;

/* =========================================================================
 * A6  pooled embedding gather (forward)
 * replaces aclnnSplitEmbeddingCodegenForwardUnweighted, called from
 * .../split_embedding_codegen_forward_unweighted.cpp:24-71 (kernel:
 * ascendc_op/ai_core_op/split_embedding_codegen_forward_unweighted/v220/op_kernel/
 * split_embedding_codegen_forward_unweighted_kernel.h:226-241,299-343).
 *
 * out[b, D_offsets[t]:D_offsets[t+1]] = sum (or mean) over the bag (t,b) of
 * dev_weights[weights_offsets[t] + idx*D_t : +D_t], rows added in index order
 * starting from 0.0f; empty bag -> zeros.  NONE: out[i, 0:D_t] = row(i), the
 * rest of the max_D-wide output row is zero.  `indices` is what the reference
 * calls hash_indices when those are given.  Every element of `out` is written.
 * ========================================================================= */
/* flags of recsdk_tbe_forward_args.  LEAVE_ROOM: run the pooled gather with three instead of four resident blocks
 * per SM so that kernels enqueued on other streams (the backward's plan) find SM slots beside it. */
#define RECSDK_FWD_LEAVE_ROOM 1
typedef struct {
    const float* dev_weights;       /* flat, all tables                         */
    const int64_t* weights_offsets; /* [T] element offset of each feature's table */
    const int32_t* D_offsets;       /* [T+1]                                    */
    const int64_t* indices;         /* [N]                                      */
    const int64_t* offsets;         /* [T*B+1], feature-major: offsets[t*B+b]   */
    float* out;                     /* [B,total_D]  (NONE: [N,max_D])           */
    int64_t T, B, N;
    int32_t total_D, max_D;
    int32_t pooling_mode;
    int64_t weights_numel; /* >0: rows are bounds-checked against it, violations -> status, row read as 0 */
    int64_t* dev_status;   /* optional */
    recsdk_sample_shards out_shards; /* optional (num_shards > 0): `out` is ignored */
    int32_t flags;                   /* RECSDK_FWD_* */
} recsdk_tbe_forward_args;
RECSDK_API int recsdk_tbe_forward(const recsdk_tbe_forward_args* a, void* stream);

/* =========================================================================
 * A1  sorted unique + inverse
 * replaces hybrid::UniqueParallel (hybrid_torchrec/src/ids_process/unique.cpp:55-127).
 * unique_out ascending, inverse_out[i] = rank of ids[i]; *num_unique_out (device)
 * receives U.  key_bits: number of significant low bits of the ids (<= 64;
 * pass 64 when unknown) -- the sort only walks those.  ids must be >= 0.
 * ========================================================================= */
RECSDK_API size_t recsdk_unique_sorted_workspace_bytes(int64_t n);
RECSDK_API int recsdk_unique_sorted(const int64_t* ids, int64_t n, int key_bits, int64_t* unique_out,
                                    int64_t* inverse_out, int64_t* num_unique_out, void* workspace,
                                    size_t workspace_bytes, void* stream);

/* Allocation-free variant of recsdk_unique_sorted.  It has no counterpart in the
 * reference.  It exists for callers that cannot allocate device memory where they need
 * the dedup (allocator callbacks and memory-pool hooks, preprocessing threads that own
 * device buffers but no allocator, services whose device memory is budgeted up front):
 * the sort scratch is a __device__ array built into the library, so the call performs no
 * cudaMalloc/cudaFree and takes no workspace.  Limits and rules:
 *   - n <= RECSDK_UNIQUE_STATIC_MAX_N, else RECSDK_ERR_TOO_LARGE (use recsdk_unique_sorted);
 *   - every GPU that loads the library holds the scratch (8 MiB) until the process exits;
 *   - the first call on a device resolves the array's device address
 *     (cudaGetSymbolAddress, once per device, with that device current): make that first
 *     call before starting any stream capture.  It is also a warm-up: CUDA loads a library's
 *     device image lazily, so the first use of this file's code on a device is when the
 *     driver places the image -- the 8 MiB array included -- in device memory.  Make that
 *     first call (n = 0 is enough) during start-up, where allocating is still allowed; a
 *     failure to locate the array is reported as RECSDK_ERR_STATIC_SCRATCH;
 *   - all calls on a device share the scratch and it keeps the previous call's contents
 *     (nothing needs to start at zero: every word is written before it is read); calls whose
 *     kernels overlap on the GPU race on it, so serialise them (one stream, or events).
 * Inputs and outputs are the caller's, exactly as for recsdk_unique_sorted. */
#define RECSDK_UNIQUE_STATIC_MAX_N 262144
RECSDK_API int64_t recsdk_unique_sorted_static_max_n(void);
RECSDK_API int recsdk_unique_sorted_static(const int64_t* ids, int64_t n, int key_bits, int64_t* unique_out,
                                           int64_t* inverse_out, int64_t* num_unique_out, void* stream);

/* =========================================================================
 * A7  fused backward: gradient segment-sum over deduplicated rows + sparse
 * Adagrad / Adam / SGD row update, in place.
 * replaces aclnnBackwardCodegenAdagradUnweightedExact (optim_type 1/2/3), called from
 * .../backward_codegen_{adagrad,adam,sgd}_unweighted_exact.cpp (adam: :354-412);
 * kernels ascendc_op/ai_core_op/backward_codegen_adagrad_unweighted_exact/v220/op_kernel/
 * backward_codegen_unweighted_exact_kernel_unique.h:113-268 (segment-sum),
 * backward_codegen_adagrad_unweighted_exact_kernel_unique.h:50-62 (Adagrad),
 * backward_codegen_adam_unweighted_exact_kernel_unique.h:70-96 (Adam),
 * backward_codegen_sgd_unweighted_exact_kernel.h:107-124 (SGD); Adam host
 * scalars op_host/backward_codegen_adagrad_unweighted_exact.cpp:84-111.
 *
 * With unique_ids/unique_offsets/unique_inverse (all three or none) the
 * caller's dedup is used: G[inverse[i] + unique_offsets[t]] += grad row of i,
 * row u of feature t lives at weights_offsets[t] + unique_ids[u]*D_t.
 * Without them the op dedups internally on hash_size_cumsum[t] + idx.
 *
 * Reduction order (the reference uses unordered atomics; here it is fixed):
 * the contributions of one row are taken in ascending index position;
 * reduce_chunk == 0: one sequential sum from 0.0f.  reduce_chunk == C > 0: runs
 * longer than C are split into consecutive chunks of C, each summed
 * sequentially from 0.0f, and the chunk sums are then summed sequentially from
 * 0.0f.  Both are run-to-run deterministic; C = 64 is the fast default (hot
 * rows do not serialise on one warp).
 * ========================================================================= */
/* flags of recsdk_tbe_backward_args.  STAGED_UPDATE: move the rows of the update through shared memory with bulk
 * asynchronous copies (rows of 128..1024 floats, 16-byte aligned tables; other shapes ignore the flag).  Same
 * results bit for bit; measured slightly slower than the default on the benchmark workload, so it is opt-in. */
#define RECSDK_BWD_STAGED_UPDATE 1
/* PLAN_ONLY / APPLY_ONLY split one call in two.  The plan (position -> row key, sort, runs, per-row records) reads
 * the indices and needs only the LAYOUT of the gradient (total_D / D_offsets or grad_shards), so it can be enqueued
 * on another stream while the forward of the same batch runs; grad_output may be NULL in that call.  The apply call
 * (chunk sums, row update) takes the same arguments plus the gradient and the same workspace, untouched in
 * between, and must be ordered after the plan call (an event).  Neither flag: both phases, as before. */
#define RECSDK_BWD_PLAN_ONLY 2
#define RECSDK_BWD_APPLY_ONLY 4
typedef struct {
    const float* grad_output; /* [B,total_D]  (NONE: [N,max_D]) */
    float* dev_weights;
    float* momentum1; /* Adagrad accumulator / Adam m ; NULL for SGD */
    float* momentum2; /* Adam v ; else NULL */
    const int64_t* weights_offsets;  /* [T]   */
    const int32_t* D_offsets;        /* [T+1] */
    const int64_t* hash_size_cumsum; /* [T+1] (used when unique_* are NULL) */
    const int64_t* indices;          /* [N]   */
    const int64_t* offsets;          /* [T*B+1] */
    const int64_t* unique_ids;       /* [U] or NULL */
    const int64_t* unique_offsets;   /* [T+1] or NULL */
    const int64_t* unique_inverse;   /* [N] or NULL */
    int64_t T, B, N;
    int64_t num_unique_capacity; /* numel of unique_ids (upper bound of U); 0 when NULL */
    int32_t total_D, max_D;
    int32_t pooling_mode, optimizer;
    int32_t total_hash_size_bits; /* bits needed for hash_size_cumsum[T]; 0 = derive as 64 */
    int32_t reduce_chunk;         /* 0 or 64 */
    float learning_rate, eps, beta1, beta2;
    int64_t iter; /* Adam step count t >= 1 */
    int32_t gradient_clipping;
    float max_gradient;
    int64_t weights_numel; /* >0: bounds check */
    int64_t* dev_status;   /* optional */
    void* workspace;
    size_t workspace_bytes;
    /* optional profiling hooks: cudaEvent_t handles recorded on `stream` right before and right
     * after the launch of the row-update kernel (the dominant kernel of the step); NULL = off */
    void* ev_update_start;
    void* ev_update_stop;
    recsdk_sample_shards grad_shards; /* optional (num_shards > 0): `grad_output` is ignored; read only */
    int32_t flags;                    /* RECSDK_BWD_* */
} recsdk_tbe_backward_args;
RECSDK_API size_t recsdk_tbe_backward_workspace_bytes(int64_t N, int32_t max_D);
RECSDK_API int recsdk_tbe_backward(const recsdk_tbe_backward_args* a, void* stream);

/* Adam step-size scalar exactly as the reference host computes it in float:
 * sqrt(1-beta2^t)/(1-beta1^t)  (op_host/...cpp:98-102). */
RECSDK_API float recsdk_adam_beta2sqrt(float beta1, float beta2, int64_t iter);

/* =========================================================================
 * A8  row gather / row assign by slot (swap-out / swap-in of cache rows)
 * replaces HybridSplitTableBatchedEmbeddingBagsCodegen.{gather_embs,gather_momentum,
 * scatter_update_embs,scatter_update_momentum}
 * (hybrid_torchrec/hybrid_torchrec/distributed/batched_embedding_kernel.py:297-345).
 * Rows are moved with bulk async copies (TMA) through shared memory when
 * D*4 is a multiple of 16 bytes, else with plain loads.
 * ========================================================================= */
RECSDK_API int recsdk_gather_rows(const float* table, const int64_t* slots, int64_t k, int32_t D, float* out,
                                  int64_t table_rows, int64_t* dev_status, void* stream);
RECSDK_API int recsdk_scatter_rows(float* table, const int64_t* slots, int64_t k, int32_t D, const float* rows,
                                   int64_t table_rows, int64_t* dev_status, void* stream);
/* recsdk_gather_rows with the poll limit of its mbarrier waits as an argument (the default is 2^22 polls).  For
 * failure-handling tests: with wait_limit 0 the first wait runs out at once, the kernel records RECSDK_ERR_CUDA in the
 * status block, lets the copies it already issued land (bounded) and returns; `out` is then incomplete.  The context
 * stays usable. */
RECSDK_API int recsdk_gather_rows_wait_limit(const float* table, const int64_t* slots, int64_t k, int32_t D, float* out,
                                             int64_t table_rows, int64_t* dev_status, int32_t wait_limit, void* stream);

/* =========================================================================
 * A9  TF-flavour operators (signatures of cust_op/framework/tf_plugin/src/
 * cust_embedding_by_address.cpp:19-52, lazy_adam.cpp:20-35, sgd.cpp:19-28)
 * ========================================================================= */
/* EmbeddingLookupByAddress: out[i,:] = *(float*)address[i], address 0 -> zeros
 * (ascendc_op/ai_core_op/cust_op_by_addr/v220/op_kernel/embedding_lookup_by_address.cpp:106-145).
 * Addresses are device addresses of fp32 rows. */
RECSDK_API int recsdk_lookup_by_address(const int64_t* addresses, int64_t n, int32_t embedding_dim, float* out,
                                        void* stream);
/* EmbeddingUpdateByAddress: update_type 0 -> row += embedding[i] (atomic), else row = embedding[i];
 * address 0 skipped (.../embedding_update_by_address.cpp:100-190). */
RECSDK_API int recsdk_update_by_address(const int64_t* addresses, int64_t n, int32_t embedding_dim,
                                        const float* embedding, int32_t update_type, void* stream);
/* LazyAdam: m,v,var rows at indices[i] updated with gradient[i]; lr is already bias corrected;
 * negative index skipped; indices must be unique
 * (ascendc_op/ai_core_op/fused_lazy_adam/v220/op_kernel/lazy_adam.cpp:138-207). */
RECSDK_API int recsdk_lazy_adam(const float* gradient, const int32_t* indices, int64_t n, int32_t dim, float* m,
                                float* v, float* var, float lr, float beta1, float beta2, float epsilon,
                                void* stream);
/* Sgd: var[indices[i]] += (gradient[i] (+ weight_decay*var)) * -lr, atomic add, duplicates accumulate
 * (ascendc_op/ai_core_op/fused_sgd/v220/op_kernel/sgd_kernel.h:78-190).  With weight decay the
 * updates are staged in `workspace` (n*dim*4 bytes) so that every occurrence of a duplicated
 * index sees the original var, as the reference's gather-compute-scatter does; without it
 * workspace may be NULL. */
RECSDK_API int recsdk_sgd(const float* gradient, const int64_t* indices, int64_t n, int32_t dim, float* var,
                          float lr, float weight_decay, int32_t use_weight_decay, void* workspace,
                          size_t workspace_bytes, void* stream);

/* =========================================================================
 * A10 Restore: hash_indices[r] = unique_indices[unique_inverse[r] + unique_offset[t]]
 * replaces Embcache::Restore (torchrec_embcache/csrc/ops/restore.cpp:15-51).
 * offsets_per_table [n_tables+1] is a DEVICE array here.
 * ========================================================================= */
RECSDK_API int recsdk_restore(const int64_t* unique_indices, const int64_t* unique_inverse,
                              const int64_t* unique_offset, const int64_t* offsets_per_table, int64_t n_tables,
                              int64_t n, int64_t* hash_indices, void* stream);

/* =========================================================================
 * A2  IdsMapper: key -> slot in an HBM-resident open-addressing table, slots
 * handed out in first-come (input position) order, then first-occurrence
 * unique of the slots of one table segment.
 * replaces hybrid::IdsMapper (hybrid_torchrec/src/ids_process/ids_mapper.h:30-102,
 * ids_mapper.cpp:36-61 ids2indices_unique, :63-174 ids2indices_unique_out).
 *
 * The mapper's state lives in caller-allocated device memory described by
 * recsdk_mapper_t (a plain struct the caller keeps on the host).
 * ========================================================================= */
typedef struct {
    int64_t* table;       /* [hash_capacity*2] int64 {key,value} pairs          */
    int64_t hash_capacity; /* power of two, >= 2*init_max_index recommended     */
    int64_t* slot_key;    /* [init_max_index]  slot -> key  (indice2id)         */
    int32_t* mark;        /* [init_max_index]  scratch, all 0x7fffffff between calls */
    int64_t* counters;    /* [4] device: {max_index, -, -, -}                   */
    int64_t init_max_index;
    int32_t only_device_mem; /* 1: slot >= init_max_index is RECSDK_ERR_TABLE_FULL */
} recsdk_mapper_t;
RECSDK_API size_t recsdk_mapper_table_bytes(int64_t hash_capacity);
/* initialises table / slot_key / mark / counters */
RECSDK_API int recsdk_mapper_init(const recsdk_mapper_t* m, void* stream);
RECSDK_API size_t recsdk_mapper_workspace_bytes(int64_t n);
/* ids2indices_unique_out for one table segment [seg_start, seg_start+seg_len) of
 * the batch arrays.  unique_offset is a device [T+1] array: entry table_id is
 * read as this table's base (forced to 0 for table 0), entry table_id+1 written. */
RECSDK_API int recsdk_mapper_unique_out(const recsdk_mapper_t* m, const int64_t* ids, int64_t* hash_indices,
                                        int64_t seg_start, int64_t seg_len, int64_t* unique, int64_t* unique_ids,
                                        int64_t* unique_inverse, int64_t* unique_offset, int64_t table_id,
                                        int64_t* dev_status, void* workspace, size_t workspace_bytes,
                                        void* stream);
/* ids2indices_unique: slots for all ids (written to hash_indices), then SORTED
 * unique of the slots + inverse.  Workspace: max(mapper, unique_sorted). */
RECSDK_API int recsdk_mapper_ids2indices_unique(const recsdk_mapper_t* m, const int64_t* ids, int64_t n,
                                                int64_t* hash_indices, int64_t* unique_out, int64_t* inverse_out,
                                                int64_t* num_unique_out, int64_t* dev_status, void* workspace,
                                                size_t workspace_bytes, void* stream);

/* =========================================================================
 * A4  SwapManager: slot policy of the HBM cache
 * replaces Embcache::SwapManager (torchrec_embcache/csrc/embedding_cache/swap_manager.h:28-55,
 * swap_manager.cpp:32-139 ComputeSwapInfo, :141-159 RemoveKeys).
 * ========================================================================= */
typedef struct {
    int64_t* table;        /* [hash_capacity*2] {key,value}                      */
    int64_t hash_capacity; /* power of two                                       */
    int64_t* slot_key;     /* [cache_size]  cache_[off].key                      */
    int64_t* slot_version; /* [cache_size]  cache_[off].version                  */
    int64_t* counters;     /* [4] device: {occupied, now_version, swap_idx, -}   */
    int64_t cache_size;
    int64_t mem_start_offset; /* 1 when admission is enabled, else 0            */
} recsdk_swap_t;
RECSDK_API int recsdk_swap_init(const recsdk_swap_t* s, void* stream);
RECSDK_API size_t recsdk_swap_workspace_bytes(int64_t n, int64_t cache_size);
/* keys [n] (-1 = not admitted -> slot 0).  Outputs (device): batch_offs [n];
 * swapin_keys/offs, swapout_keys/offs [n each]; counts_out [2] = {n_swapin, n_swapout}. */
RECSDK_API int recsdk_swap_compute(const recsdk_swap_t* s, const int64_t* keys, int64_t n, int64_t* batch_offs,
                                   int64_t* swapin_keys, int64_t* swapin_offs, int64_t* swapout_keys,
                                   int64_t* swapout_offs, int64_t* counts_out, int64_t* dev_status,
                                   void* workspace, size_t workspace_bytes, void* stream);
/* RemoveKeys; n_keys_dev (device int64) optional: when non-NULL only the first
 * min(n, *n_keys_dev) keys are used (lets the evict list stay on the device). */
RECSDK_API int recsdk_swap_remove(const recsdk_swap_t* s, const int64_t* keys, int64_t n,
                                  const int64_t* n_keys_dev, void* stream);

/* =========================================================================
 * A5  FeatureFilter: count-based admission and timestamp eviction
 * replaces Embcache::FeatureFilter (torchrec_embcache/csrc/feature_filter/feature_filter.h:26-60,
 * feature_filter.cpp:112-138 StatisticsKeyCount, :140-160 CountFilter,
 * :27-50 RecordTimestamp, :52-80 FeatureEvict).
 * Entries are 32 bytes: {key, count, timestamp, tag}.
 * ========================================================================= */
typedef struct {
    int64_t* table;        /* [hash_capacity*4]                                  */
    int64_t hash_capacity; /* power of two                                       */
    int64_t* counters;     /* [4] device: {latest_timestamp, record_batch_id, n_evict, -} */
    int64_t admit_threshold; /* -1: admission disabled                           */
    int64_t evict_threshold; /* 0: eviction disabled                             */
    int64_t evict_step_interval;
} recsdk_filter_t;
RECSDK_API int recsdk_filter_init(const recsdk_filter_t* f, void* stream);
RECSDK_API size_t recsdk_filter_workspace_bytes(int64_t n);
/* counts may be NULL (every occurrence counts 1). */
RECSDK_API int recsdk_filter_statistics(const recsdk_filter_t* f, const int64_t* keys, const int64_t* counts,
                                        int64_t n, int64_t* dev_status, void* stream);
/* keys_inout[i] = -1 where the key is in the count map with count < admit_threshold */
RECSDK_API int recsdk_filter_count_filter(const recsdk_filter_t* f, int64_t* keys_inout, int64_t n, void* stream);
/* insert_or_assign(key, ts) in input order (last occurrence wins), latest = max;
 * runs the evict scan when (batch_id > 0 && (batch_id+1) % interval == 0), appending
 * to evict_keys (device, capacity evict_capacity) and counters[2]. */
RECSDK_API int recsdk_filter_record_timestamp(const recsdk_filter_t* f, const int64_t* keys, const int64_t* ts,
                                              int64_t n, int64_t* evict_keys, int64_t evict_capacity,
                                              int64_t* dev_status, void* workspace, size_t workspace_bytes,
                                              void* stream);
/* resets counters[2] (evictFeatureRecord_.ClearEvictInfo) */
RECSDK_API int recsdk_filter_clear_evict(const recsdk_filter_t* f, void* stream);
/* count of one key -> *count_out (device), -1 if absent from the count map */
RECSDK_API int recsdk_filter_count_of(const recsdk_filter_t* f, const int64_t* keys, int64_t n, int64_t* count_out,
                                      void* stream);

/* =========================================================================
 * Load statistics and tombstone compaction of the open-addressing key tables above (mapper, swap manager: 2 words per
 * entry; feature filter: 4).  Erases leave TOMBSTONE entries that lookups walk past and that only a rebuild turns back
 * into EMPTY; the reference's std::unordered_map / flat_hash_map (ids_mapper.h:30-102, swap_manager.h:41-54,
 * feature_filter.h:26-60) has no such decay, so a long run rebuilds a table when live + tombstones passes ~3/4 of
 * the capacity.
 * stats_out (device, 4 words): {live entries, tombstones, longest displacement of a live entry from its home, 0}.
 * rebuild: collect the live entries into the workspace, clear, insert again (same key -> payload mapping, no
 * tombstones).  max_live bounds the scratch; when more entries are live nothing is changed and RECSDK_ERR_WORKSPACE is
 * put into the status block.  Must be ordered against every other call on the same table.
 * ========================================================================= */
RECSDK_API int recsdk_key_table_stats(const int64_t* table, int64_t hash_capacity, int32_t entry_words, int64_t* stats_out,
                                      void* stream);
RECSDK_API size_t recsdk_key_table_rebuild_workspace_bytes(int64_t max_live, int32_t entry_words);
RECSDK_API int recsdk_key_table_rebuild(int64_t* table, int64_t hash_capacity, int32_t entry_words, int64_t max_live,
                                        int64_t* dev_status, void* workspace, size_t workspace_bytes, void* stream);

/* =========================================================================
 * A3  row-hash bucketize for row-wise sharding
 * replaces hybrid::block_bucketize_sparse_features_cpu
 * (hybrid_torchrec/src/ids_process/bucketize.cpp:214-282, kernel :133-211,
 * ComputeNewLengths :35-51, FillNewIndices :54-76, Deduplicate :79-130).
 * lengths [F*B]; bucket = id % world; new_lengths [world*F*B] bucket-major;
 * new_indices grouped by (bucket, feature, sample) in input order;
 * unbucketize_permute[i] = position of input i in new_indices (or, with
 * do_unique, in the deduplicated list).  *num_out (device) = valid length of
 * new_indices / ids_counts.
 * ========================================================================= */
RECSDK_API size_t recsdk_bucketize_workspace_bytes(int64_t n, int64_t lengths_size, int64_t world);
RECSDK_API int recsdk_bucketize(const int64_t* lengths, int64_t lengths_size, const int64_t* indices, int64_t n,
                                int64_t num_features, int64_t world, int32_t do_unique, int32_t return_count,
                                int64_t* new_lengths, int64_t* new_indices, int64_t* unbucketize_permute,
                                int64_t* ids_counts, int64_t* num_out, void* workspace, size_t workspace_bytes,
                                void* stream);

/* =========================================================================
 * Jagged-batch utilities either side of the lookup (input / output distribution).
 * They replace the operators of cust_op/framework/torch_plugin/torch_library/2.6.0/:
 *   permute2d_sparse_data/permute2d_sparse_data.cpp:21-48   permute_2D_sparse_data
 *   permute1d_sparse_data/permute1d_sparse_data.cpp:57-93   permute_1D_sparse_data (the same call with B = 1)
 *   asynchronous_complete_cumsum/asynchronous_complete_cumsum.cpp:18-25
 *   jagged_to_padded_dense/jagged_to_padded_dense.cpp       jagged_to_padded_dense (+ backward = dense_to_jagged)
 *   dense_to_jagged/dense_to_jagged.cpp
 *
 * permute: out_lengths[t', :] = lengths[permute[t'], :]; the values (and weights) of output row t' are the
 * whole segment of input row permute[t'] (rows may repeat or be dropped).  values are 4- or 8-byte elements.
 * *out_total (device, optional) receives the number of output values; they must fit out_capacity
 * (else RECSDK_ERR_TOO_LARGE in the status block).  permute entries outside [0, T_in) -> RECSDK_ERR_INDEX_RANGE.
 * complete_cumsum: out[0] = 0, out[i+1] = x[0] + ... + x[i]  (out has n + 1 entries).
 * jagged_to_padded_dense: dense[b, l, :] = values[offsets[b] + l, :] for l < len_b, else padding_value.
 * dense_to_jagged: values[offsets[b] + l, :] = dense[b, l, :] for l < min(len_b, max_length), else 0.
 * ========================================================================= */
RECSDK_API size_t recsdk_complete_cumsum_workspace_bytes(int64_t n);
RECSDK_API int recsdk_complete_cumsum(const int64_t* x, int64_t n, int64_t* out, void* workspace, size_t workspace_bytes,
                                      void* stream);
RECSDK_API size_t recsdk_permute_sparse_workspace_bytes(int64_t T_in, int64_t T_out);
RECSDK_API int recsdk_permute_2d_sparse_data(const int64_t* permute, int64_t T_out, const int64_t* lengths, int64_t T_in,
                                             int64_t B, const void* values, int32_t value_bytes, const float* weights,
                                             int64_t* out_lengths, void* out_values, float* out_weights,
                                             int64_t out_capacity, int64_t* out_total, int64_t* dev_status,
                                             void* workspace, size_t workspace_bytes, void* stream);
RECSDK_API int recsdk_jagged_to_padded_dense(const float* values, const int64_t* offsets, int64_t B, int32_t D,
                                             int64_t max_length, float padding_value, float* dense, void* stream);
RECSDK_API int recsdk_dense_to_jagged(const float* dense, const int64_t* offsets, int64_t B, int32_t D, int64_t max_length,
                                      float* values, void* stream);

/* =========================================================================
 * Peer mappings for the sample-sharded buffers (one process per GPU on one box).
 * Replaces the two pooled-embedding all-to-alls of the reference's table-wise path
 * (torchrec PooledEmbeddingsAllToAll behind hybrid_torchrec/.../embeddingbag.py:550-593):
 * every rank exports the buffer that holds ITS samples' pooled rows (and the one with
 * their gradients), the other ranks map it and hand the mapped addresses to
 * recsdk_tbe_forward / recsdk_tbe_backward in a recsdk_sample_shards.
 *
 * export: handle (64 bytes, cudaIpcMemHandle_t) of the cudaMalloc allocation that
 *         contains dev_ptr, and the byte offset of dev_ptr inside it.  The memory must
 *         come from cudaMalloc (torch's default caching allocator qualifies).
 * import: maps a peer's allocation into this process (peer access enabled lazily by the
 *         driver) and returns the address that corresponds to the exported pointer.
 * release: unmaps; pass the pointer import returned and the same offset.
 * These three calls are setup-time host calls (they synchronise); plain loads and stores
 * are used on the mapped memory -- no multicast objects are created.
 * ========================================================================= */
#define RECSDK_PEER_HANDLE_BYTES 64
RECSDK_API int recsdk_peer_export(const void* dev_ptr, unsigned char* handle_out, int64_t* offset_out);
RECSDK_API int recsdk_peer_import(const unsigned char* handle, int64_t offset, void** dev_ptr_out);
RECSDK_API int recsdk_peer_release(void* imported_ptr, int64_t offset);
/* Stream-ordered copy between device buffers of which either may be a peer mapping (a pull of rows from another
 * rank's buffer, or a push into it). */
RECSDK_API int recsdk_peer_copy(void* dst, const void* src, size_t bytes, void* stream);

/* =========================================================================
 * Dedup exchange: the sharded lookup driven from the device over peer mappings.
 * Replaces, for the tables sharded over the GPUs of one box, the reference's exchange steps around the lookup:
 * the id / row / gradient all-to-alls of the table-wise and row-wise paths
 * (hybrid_torchrec/hybrid_torchrec/distributed/sharding/hybrid_tw_sharding.py:43-82, hybrid_rw_sharding.py,
 * embeddingbag.py:550-593) and the fused collectives they map to on the reference's hardware: GatherAll
 * (cust_op/ascendc_op/ai_core_op/lccl/v220/op_kernel/gather_all.h) and AllUss = all-to-all + unsorted segment sum
 * (all2all_uss.h:319-381; deterministic order all_uss_deterministic.h:102-121: contributions of one row are added
 * in source-rank order, golden cust_op/test/lccl_op_test/tf/all2all_uss.py:213-216).
 *
 * Every rank keeps ONE flat table of its rows (equal dim D) and owns the linear rows
 * [rank_base[r], rank_base[r+1]) of a global row numbering:
 *   table-wise: linear row = part_base[f] + id            (part_base [F]; tables ordered by owner)
 *   row-wise:   linear row = part_base[(id % W)*F + f] + id / W   (part_base [W*F]; bucketize.cpp:44-48)
 * One step, per rank, no host read and no allocation anywhere:
 *   forward         sort-dedup of this rank's ids on the linear row (grouped by owner) -> the distinct ids and their
 *                   count are stored into each owner's inbox (peer stores) -> the distinct rows are read straight from
 *                   the owners' tables (peer loads) -> pooled locally with the forward kernel.
 *   backward_local  per distinct row the sum of the bag gradients that used it (the forward's sort is the plan), stored
 *                   straight into the owner's gradient inbox (peer stores).
 *   -- fence: every rank's stores have landed (a stream-ordered collective on the caller's side) --
 *   backward_owner  reads the counts FROM DEVICE MEMORY, merges the lists of all source ranks (sort on the local row,
 *                   contributions of one row in source-rank order), applies the optimizer once per row.
 *   -- fence before the next forward reads the tables --
 * No kernel waits on another GPU; loads and stores on peer mappings are plain ld/st (no multicast object).
 * With world == 1 (or several logical ranks of one process whose "peer" pointers are local) the same code runs on
 * one GPU.
 * ========================================================================= */
#define RECSDK_XCHG_TABLE_WISE 0
#define RECSDK_XCHG_ROW_WISE 1
/* flags.  ONE_HOT: the caller states that every bag holds exactly one id (checked on the device: a violation is
 * RECSDK_ERR_INVALID_ARG in the status block).  With SUM / MEAN pooling the forward then loads every distinct row once
 * from its owner and stores it to all bags that use it, with no intermediate copy of the fetched rows. */
#define RECSDK_XCHG_ONE_HOT 1
typedef struct {
    int32_t world, rank;
    int32_t partition; /* RECSDK_XCHG_* */
    int32_t D;         /* row width, multiple of 4 */
    int64_t F, B;      /* features and samples of THIS rank's batch */
    int64_t max_ids;   /* capacity: the largest number of ids one step of this rank holds */
    int64_t inbox_cap; /* rows one source rank may ask of one owner per step (worst case: all its ids) */
    int32_t key_bits;  /* bits of rank_base[world] */
    int32_t flags;     /* RECSDK_XCHG_ONE_HOT */
    const int64_t* part_base;  /* device, see above */
    const int64_t* rank_base;  /* device [world+1] */
    const int64_t* table_rows; /* device [F] rows of table f (ids are checked against it), or NULL */
    int64_t local_rows;        /* rows of this rank's flat table */
    /* index r = rank r's buffer as addressed from THIS process (own buffers: plain pointers) */
    const float* tables[RECSDK_MAX_SHARDS]; /* [local_rows_r * D] weights                           */
    int64_t* inbox_ids[RECSDK_MAX_SHARDS];  /* [world * inbox_cap]  local row numbers, by source    */
    int64_t* inbox_counts[RECSDK_MAX_SHARDS]; /* [world]                                            */
    float* inbox_grads[RECSDK_MAX_SHARDS];  /* [world * inbox_cap * D] per-row gradient sums        */
    void* workspace; /* local scratch, recsdk_xchg_workspace_bytes(); holds the plan between the calls of a step */
    size_t workspace_bytes;
    int64_t* dev_status; /* optional */
} recsdk_xchg_t;
RECSDK_API size_t recsdk_xchg_workspace_bytes(int64_t max_ids, int64_t inbox_cap, int32_t world, int32_t D, int64_t F);
/* indices [N], offsets [F*B+1] feature-major, out [B, F*D] (NONE: [N, D]).  pooling_mode RECSDK_POOL_*.
 * flags 0: the whole forward.  PLAN_ONLY / FETCH_ONLY split it: the plan (sort-dedup of this rank's ids) touches only
 * the ids and this rank's scratch, so the plan of step k+1 can run on a second stream beside the owner phase of step k
 * and BEFORE the fence that makes the tables final, once this rank's recsdk_xchg_backward_local of step k is done with
 * the scratch; the fetch call (same arguments; counts and ids to the owners' inboxes, rows from the owners' tables,
 * output) follows that fence and an event wait on the plan.  `out` may be NULL in the plan call.  A caller that gives
 * the steps two workspaces in turn (x->workspace is read at every call) may make the plan of step k+1 in the other one
 * at any time after the forward of step k.  The fetch may be repeated on the plan it belongs to. */
#define RECSDK_XCHG_FWD_PLAN_ONLY 1
#define RECSDK_XCHG_FWD_FETCH_ONLY 2
RECSDK_API int recsdk_xchg_forward(const recsdk_xchg_t* x, const int64_t* indices, const int64_t* offsets, int64_t N,
                                   int32_t pooling_mode, float* out, int32_t flags, void* stream);
/* grad_output [B, F*D] (NONE: [N, D]) of the batch of the preceding recsdk_xchg_forward (same offsets). */
RECSDK_API int recsdk_xchg_backward_local(const recsdk_xchg_t* x, const float* grad_output, const int64_t* offsets,
                                          int64_t N, int32_t pooling_mode, int32_t gradient_clipping,
                                          float max_gradient, void* stream);
/* Updates this rank's table in place from its inbox.  ev_update_*: optional cudaEvent_t recorded around the row-update
 * kernel.  flags 0: the whole phase.  PLAN_ONLY / APPLY_ONLY split it: the plan (compaction of the id lists, sort, runs,
 * per-row records) reads only the ids and counts, which are complete once every rank's forward has run, so a caller
 * that fences after the forward can run it on a second stream beside recsdk_xchg_backward_local; the apply call (row
 * update) then follows the gradient fence and an event wait on the plan. */
#define RECSDK_XCHG_OWNER_PLAN_ONLY 1
#define RECSDK_XCHG_OWNER_APPLY_ONLY 2
RECSDK_API int recsdk_xchg_backward_owner(const recsdk_xchg_t* x, float* weights, float* momentum1, float* momentum2,
                                          int32_t optimizer, float learning_rate, float eps, float beta1, float beta2,
                                          int64_t iter, void* ev_update_start, void* ev_update_stop, int32_t flags,
                                          void* stream);
/* Plan counters of the most recent step, copied to host memory (6 words): [0] distinct rows this rank asked for,
 * [1] ids this rank received as an owner, [2] distinct rows it updated, [3] ids in chunked local runs, [4] how many
 * of [0] this rank owns itself (the others crossed the links), [5] chunk sums of the local phase.  Synchronises the
 * stream. */
RECSDK_API int recsdk_xchg_counters(const recsdk_xchg_t* x, int64_t* out6, void* stream);

/* =========================================================================
 * Host (DRAM) tier of the hybrid cache: key -> AoS row [w | m | v] store for the rows that are not held in the HBM
 * cache.  Replaces Embcache::EmbTable (torchrec_embcache/csrc/emb_table/emb_table.h:32-372: FindOrInsert :54-116,
 * InsertOrAssign :118-179, RemoveEmbedding, ForEachKey :300-330) and its initializers
 * (emb_table/initializer.h:36-75).  HOST pointers throughout; these calls touch no GPU.  The device side of a swap
 * is recsdk_gather_rows / recsdk_scatter_rows plus asynchronous copies of pinned staging buffers.
 *   find_or_insert    a missing key gets a new row (weights from the initializer, optimizer state zero); the rows are
 *                     copied OUT into one [n, emb_dim] block per array (optim blocks as many as optim_num)
 *   insert_or_assign  creates missing rows (no initializer) and overwrites them from the blocks
 *   export            ForEachKey: every key with its row, in the table's iteration order (unspecified, as the
 *                     reference's); keys_out == NULL only counts.  Returns the number of rows, -1 on error.
 * Thread-safe (one mutex per table).  INT64_MIN and INT64_MIN+1 are not valid keys.
 * ========================================================================= */
enum { RECSDK_HOST_INIT_LINEAR = 0, RECSDK_HOST_INIT_TRUNCATED_NORMAL = 1, RECSDK_HOST_INIT_UNIFORM = 2 };
typedef struct recsdk_host_table recsdk_host_table;
RECSDK_API recsdk_host_table* recsdk_host_table_create(int32_t emb_dim, int32_t optim_num, int32_t initializer_type,
                                                       float weight_init_min, float weight_init_max,
                                                       float weight_init_mean, float weight_init_stddev, int64_t seed,
                                                       int64_t reserve_rows);
RECSDK_API void recsdk_host_table_destroy(recsdk_host_table* t);
RECSDK_API int64_t recsdk_host_table_size(recsdk_host_table* t);
RECSDK_API int recsdk_host_table_find_or_insert(recsdk_host_table* t, const int64_t* keys, int64_t n, float* out_embs,
                                                float* out_optim1, float* out_optim2);
RECSDK_API int recsdk_host_table_insert_or_assign(recsdk_host_table* t, const int64_t* keys, int64_t n,
                                                  const float* in_embs, const float* in_optim1, const float* in_optim2);
RECSDK_API int recsdk_host_table_remove(recsdk_host_table* t, const int64_t* keys, int64_t n);
RECSDK_API int64_t recsdk_host_table_export(recsdk_host_table* t, int64_t* keys_out, float* embs_out, float* optim1_out,
                                            float* optim2_out, int64_t capacity);

#ifdef __cplusplus
}
#endif
#endif /* RECSDK_B200_H */
