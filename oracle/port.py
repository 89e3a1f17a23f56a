"""TEST INFRASTRUCTURE ONLY: numpy front end of the C oracle (``oracle.c``).

Every wrapper takes/returns numpy arrays (int64 / int32 / float32, C
contiguous) and mirrors one reference interface; see ``oracle.c`` for the
reference file:line each function follows.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "oracle.c")
LIB = os.path.join(HERE, "liboracle.so")

_lib = None

I64P = C.POINTER(C.c_int64)
I32P = C.POINTER(C.c_int32)
F32P = C.POINTER(C.c_float)


def build(force: bool = False) -> str:
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        subprocess.check_call(["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", SRC, "-o", LIB, "-lm"])
    return LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        for name in ("orc_mapper_new", "orc_swap_new", "orc_filter_new"):
            getattr(_lib, name).restype = C.c_void_p
        for name in ("orc_unique_sorted", "orc_mapper_size", "orc_mapper_ids2indices_unique", "orc_bucketize",
                     "orc_swap_occupied", "orc_filter_num_evict", "orc_filter_count_of"):
            getattr(_lib, name).restype = C.c_int64
    return _lib


def set_num_threads(n: int) -> int:
    """OpenMP threads of the C restatement from now on; returns the count in effect."""
    return int(lib().orc_set_num_threads(C.c_int(int(n))))


def _i64(a):
    a = np.ascontiguousarray(a, dtype=np.int64)
    return a


def p64(a):
    return a.ctypes.data_as(I64P) if a is not None else None


def p32(a):
    return a.ctypes.data_as(I32P) if a is not None else None


def pf(a):
    return a.ctypes.data_as(F32P) if a is not None else None


# ----------------------------------------------------------------------------- A1
def unique_sorted(ids):
    ids = _i64(ids)
    n = ids.size
    uniq = np.empty(max(n, 1), np.int64)
    inv = np.empty(max(n, 1), np.int64)
    u = lib().orc_unique_sorted(p64(ids), C.c_int64(n), p64(uniq), p64(inv))
    return uniq[:u].copy(), inv[:n].copy()


# ----------------------------------------------------------------------------- A2
class IdsMapper:
    """Restatement of ``hybrid::IdsMapper`` (same method names as the torch class)."""

    def __init__(self, init_max_index: int, only_device_mem: bool = True):
        self._h = C.c_void_p(lib().orc_mapper_new(C.c_int64(init_max_index), C.c_int(int(only_device_mem))))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_mapper_free(self._h)
            self._h = None

    def size(self) -> int:
        return lib().orc_mapper_size(self._h)

    def ids2indices_unique(self, ids):
        ids = _i64(ids)
        n = ids.size
        hi = np.empty(max(n, 1), np.int64)
        uniq = np.empty(max(n, 1), np.int64)
        inv = np.empty(max(n, 1), np.int64)
        u = lib().orc_mapper_ids2indices_unique(self._h, p64(ids), C.c_int64(n), p64(hi), p64(uniq), p64(inv))
        if u < 0:
            raise RuntimeError({1: "Invalid key value", 2: "Ids map reached maxIndex"}.get(-u, "error"))
        return hi[:n].copy(), uniq[:u].copy(), inv[:n].copy()

    def ids2indices_unique_out(self, ids, hash_indices, offset, unique, unique_ids, unique_inverse, unique_offset,
                               table_id: int):
        rc = lib().orc_mapper_unique_out(self._h, p64(ids), p64(hash_indices), p64(offset), p64(unique),
                                         p64(unique_ids), p64(unique_inverse), p64(unique_offset),
                                         C.c_int64(table_id))
        if rc != 0:
            raise RuntimeError({1: "Invalid key value", 2: "Ids map reached maxIndex"}.get(rc, "error"))


# ----------------------------------------------------------------------------- A3
def bucketize(lengths, indices, num_features: int, world: int, sequence=True, do_unique=False, return_count=False):
    lengths = _i64(lengths)
    indices = _i64(indices)
    n = indices.size
    new_lengths = np.zeros(lengths.size * world, np.int64)
    new_indices = np.empty(n, np.int64)
    perm = np.empty(n, np.int64)
    counts = np.empty(n, np.int64) if (sequence and do_unique and return_count) else None
    k = lib().orc_bucketize(p64(lengths), C.c_int64(lengths.size), p64(indices), C.c_int64(n),
                            C.c_int64(num_features), C.c_int64(world), C.c_int(int(sequence)),
                            C.c_int(int(do_unique)), C.c_int(int(return_count)), p64(new_lengths),
                            p64(new_indices), p64(perm), p64(counts))
    return new_lengths, new_indices[:k].copy(), perm, (counts[:k].copy() if counts is not None else np.empty(0, np.int64))


# ----------------------------------------------------------------------------- A4
class SwapManager:
    def __init__(self, cache_size: int, mem_start_offset: int = 0):
        self._h = C.c_void_p(lib().orc_swap_new(C.c_int64(cache_size), C.c_int64(mem_start_offset)))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_swap_free(self._h)
            self._h = None

    def compute_swap_info(self, keys):
        keys = _i64(keys)
        n = keys.size
        m = max(n, 1)
        bo, sik, sio, sok, soo = (np.empty(m, np.int64) for _ in range(5))
        nin, nout = C.c_int64(0), C.c_int64(0)
        rc = lib().orc_swap_compute(self._h, p64(keys), C.c_int64(n), p64(bo), p64(sik), p64(sio), C.byref(nin),
                                    p64(sok), p64(soo), C.byref(nout))
        if rc != 0:
            raise RuntimeError("cacheSize_ too small")
        return (sok[:nout.value].copy(), soo[:nout.value].copy(), sik[:nin.value].copy(), sio[:nin.value].copy(),
                bo[:n].copy())

    def remove_keys(self, keys):
        keys = _i64(keys)
        lib().orc_swap_remove(self._h, p64(keys), C.c_int64(keys.size))

    def occupied(self) -> int:
        return lib().orc_swap_occupied(self._h)


# ----------------------------------------------------------------------------- A5
class FeatureFilter:
    def __init__(self, admit_threshold: int = -1, evict_threshold: int = 0, evict_step_interval: int = 0):
        self._h = C.c_void_p(lib().orc_filter_new(C.c_int64(admit_threshold), C.c_uint64(evict_threshold),
                                                  C.c_uint64(evict_step_interval)))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_filter_free(self._h)
            self._h = None

    def statistics_key_count(self, keys, counts=None):
        keys = _i64(keys)
        counts = _i64(counts) if counts is not None else None
        lib().orc_filter_statistics(self._h, p64(keys), p64(counts), C.c_int64(keys.size))

    def count_filter(self, keys):
        keys = _i64(keys).copy()
        lib().orc_filter_count_filter(self._h, p64(keys), C.c_int64(keys.size))
        return keys

    def record_timestamp(self, keys, ts):
        keys = _i64(keys)
        ts = _i64(ts)
        lib().orc_filter_record_timestamp(self._h, p64(keys), p64(ts), C.c_int64(keys.size))

    def evict_keys(self):
        n = lib().orc_filter_num_evict(self._h)
        out = np.empty(max(n, 1), np.int64)
        lib().orc_filter_get_evict(self._h, p64(out))
        return out[:n].copy()

    def clear_evict(self):
        lib().orc_filter_clear_evict(self._h)

    def count_of(self, key: int) -> int:
        return lib().orc_filter_count_of(self._h, C.c_int64(key))


# ----------------------------------------------------------------------------- A6
def tbe_forward(weights, weights_offsets, D_offsets, indices, offsets, T, B, total_D, max_D, pooling_mode):
    weights = np.ascontiguousarray(weights, np.float32)
    indices = _i64(indices)
    offsets = _i64(offsets)
    wo = _i64(weights_offsets)
    do = np.ascontiguousarray(D_offsets, np.int32)
    if pooling_mode == 2:
        out = np.zeros((indices.size, max_D), np.float32)
    else:
        out = np.zeros((B, total_D), np.float32)
    lib().orc_tbe_forward(pf(weights), p64(wo), p32(do), p64(indices), p64(offsets), C.c_int64(T), C.c_int64(B),
                          C.c_int32(total_D), C.c_int32(max_D), C.c_int(pooling_mode), pf(out))
    return out


# ----------------------------------------------------------------------------- A7
def adam_beta2sqrt(beta1, beta2, it):
    out = C.c_float(0)
    lib().orc_adam_host_scalars(C.c_float(beta1), C.c_float(beta2), C.c_int64(it), C.byref(out))
    return out.value


def tbe_backward(grad_output, weights, momentum1, momentum2, weights_offsets, D_offsets, hash_size_cumsum, indices,
                 offsets, T, B, total_D, max_D, pooling_mode, optimizer, lr, eps=0.0, beta1=0.9, beta2=0.999, it=1,
                 unique_ids=None, unique_offsets=None, unique_inverse=None, gradient_clipping=False,
                 max_gradient=0.0, reduce_chunk=0):
    """In place on ``weights`` / ``momentum1`` / ``momentum2`` (float32 numpy arrays)."""
    for a in (weights, momentum1, momentum2):
        assert a is None or (a.dtype == np.float32 and a.flags.c_contiguous)
    go = np.ascontiguousarray(grad_output, np.float32)
    uid = _i64(unique_ids) if unique_ids is not None else None
    uoff = _i64(unique_offsets) if unique_ids is not None else None
    uinv = _i64(unique_inverse) if unique_ids is not None else None
    rc = lib().orc_tbe_backward(pf(go), pf(weights), pf(momentum1), pf(momentum2), p64(_i64(weights_offsets)),
                                p32(np.ascontiguousarray(D_offsets, np.int32)), p64(_i64(hash_size_cumsum)),
                                p64(_i64(indices)), p64(_i64(offsets)), p64(uid), p64(uoff), p64(uinv),
                                C.c_int64(T), C.c_int64(B), C.c_int32(total_D), C.c_int32(max_D),
                                C.c_int(pooling_mode), C.c_int(optimizer), C.c_float(lr), C.c_float(eps),
                                C.c_float(beta1), C.c_float(beta2), C.c_int64(it), C.c_int(int(gradient_clipping)),
                                C.c_float(max_gradient), C.c_int(reduce_chunk))
    assert rc == 0


# ----------------------------------------------------------------------------- A8-A10
def gather_rows(table, slots, D):
    slots = _i64(slots)
    out = np.empty((slots.size, D), np.float32)
    lib().orc_gather_rows(pf(table), p64(slots), C.c_int64(slots.size), C.c_int32(D), pf(out))
    return out


def scatter_rows(table, slots, D, rows):
    slots = _i64(slots)
    rows = np.ascontiguousarray(rows, np.float32)
    lib().orc_scatter_rows(pf(table), p64(slots), C.c_int64(slots.size), C.c_int32(D), pf(rows))


def lookup_by_address(addresses, dim):
    addresses = _i64(addresses)
    out = np.empty((addresses.size, dim), np.float32)
    lib().orc_lookup_by_address(p64(addresses), C.c_int64(addresses.size), C.c_int32(dim), pf(out))
    return out


def update_by_address(addresses, dim, rows, update_type):
    addresses = _i64(addresses)
    rows = np.ascontiguousarray(rows, np.float32)
    lib().orc_update_by_address(p64(addresses), C.c_int64(addresses.size), C.c_int32(dim), pf(rows),
                                C.c_int(update_type))


def lazy_adam(grad, indices, m, v, var, lr, beta1, beta2, eps):
    grad = np.ascontiguousarray(grad, np.float32)
    indices = np.ascontiguousarray(indices, np.int32)
    dim = grad.shape[1]
    lib().orc_lazy_adam(pf(grad), p32(indices), C.c_int64(indices.size), C.c_int32(dim), pf(m), pf(v), pf(var),
                        C.c_float(lr), C.c_float(beta1), C.c_float(beta2), C.c_float(eps))


def sgd(grad, indices, var, lr, weight_decay=None):
    grad = np.ascontiguousarray(grad, np.float32)
    indices = _i64(indices)
    dim = grad.shape[1]
    lib().orc_sgd(pf(grad), p64(indices), C.c_int64(indices.size), C.c_int32(dim), pf(var), C.c_float(lr),
                  C.c_float(weight_decay or 0.0), C.c_int(int(weight_decay is not None)))


def restore(unique_indices, unique_inverse, unique_offset, offsets_per_table):
    ui, inv, uo, opt = map(_i64, (unique_indices, unique_inverse, unique_offset, offsets_per_table))
    out = np.empty(inv.size, np.int64)
    lib().orc_restore(p64(ui), p64(inv), p64(uo), p64(opt), C.c_int64(opt.size - 1), p64(out))
    return out


# ----------------------------------------------------------------------------- jagged-batch utilities (numpy)
def asynchronous_complete_cumsum(x):
    """cust_op/framework/torch_plugin/torch_library/2.6.0/asynchronous_complete_cumsum/asynchronous_complete_cumsum.cpp:18-25"""
    x = np.asarray(x)
    return np.concatenate([[0], np.cumsum(x)]).astype(x.dtype)


def permute_2D_sparse_data(permute, lengths, values, weights=None):
    """.../permute2d_sparse_data/permute2d_sparse_data.cpp:21-48: row t' of the output is row permute[t'] of the
    input, lengths and value segments alike."""
    permute, lengths, values = np.asarray(permute), np.asarray(lengths), np.asarray(values)
    starts = np.concatenate([[0], np.cumsum(lengths.sum(axis=1))])
    segs = [np.arange(starts[t], starts[t + 1]) for t in permute]
    sel = np.concatenate(segs).astype(np.int64) if segs else np.empty(0, np.int64)
    return lengths[permute], values[sel], (np.asarray(weights)[sel] if weights is not None else None)


def permute_1D_sparse_data(permute, lengths, values, weights=None):
    """.../permute1d_sparse_data/permute1d_sparse_data.cpp:57-93"""
    out_len, v, w = permute_2D_sparse_data(permute, np.asarray(lengths).reshape(-1, 1), values, weights)
    return out_len.reshape(-1), v, w


def jagged_to_padded_dense(values, offsets, max_length, padding_value=0.0):
    """.../jagged_to_padded_dense/jagged_to_padded_dense.cpp (v1)"""
    values, offsets = np.asarray(values, np.float32), np.asarray(offsets)
    B, D = offsets.size - 1, values.shape[1]
    out = np.full((B, max_length, D), padding_value, np.float32)
    for b in range(B):
        n = min(int(offsets[b + 1] - offsets[b]), max_length)
        out[b, :n] = values[offsets[b]:offsets[b] + n]
    return out


def dense_to_jagged(dense, offsets):
    """.../dense_to_jagged/dense_to_jagged.cpp"""
    dense, offsets = np.asarray(dense, np.float32), np.asarray(offsets)
    B, L, D = dense.shape
    out = np.zeros((int(offsets[-1]), D), np.float32)
    for b in range(B):
        n = min(int(offsets[b + 1] - offsets[b]), L)
        out[offsets[b]:offsets[b] + n] = dense[b, :n]
    return out


# ----------------------------------------------------------------------------- sharded lookup with dedup exchange
class ShardedDedupOracle:
    """CPU restatement of one box's sharded lookup where each rank fetches the DISTINCT rows of its batch from
    their owners and sends back ONE summed gradient row per distinct row (the reference's row-wise flow: local
    unique, all2all of ids, gather on the owner, all2all of rows; backward: local segment-sum over the inverse,
    all2all of the sums, owner-side segment-sum and optimizer = AllUss,
    cust_op/ascendc_op/ai_core_op/lccl/v220/op_kernel/all2all_uss.h:319-381).

    The order of float additions is the two-level one of the reference's deterministic mode: a rank sums the bag
    gradients of one of its distinct rows in ascending index position (chunks of 64 for longer runs, as everywhere
    in this oracle); the owner then adds the per-rank sums of one row in SOURCE-RANK order starting from 0.0f
    (all_uss_deterministic.h:102-121; golden `expect_uss[value] += all2all[i]` over rank-major rows,
    cust_op/test/lccl_op_test/tf/all2all_uss.py:213-216) and applies the optimizer once.

    Placement: "table" = whole tables on ranks (`owner[f]`), "row" = row id on rank id % W at local row id // W
    (hybrid_torchrec/src/ids_process/bucketize.cpp:44-48).  State is kept per rank as one flat array, tables in
    (owner, table) order for "table", table after table for "row"."""

    def __init__(self, rows, dim, world, partition, owner=None, optimizer=2, lr=0.01, eps=1e-8, beta1=0.9,
                 beta2=0.999, initial_accumulator_value=0.0):
        self.rows, self.D, self.W, self.partition = [int(r) for r in rows], int(dim), int(world), partition
        self.F = len(self.rows)
        self.opt, self.hp = optimizer, (lr, eps, beta1, beta2)
        W, F = self.W, self.F
        if partition == "table":
            self.owner = [int(o) for o in owner]
            order = sorted(range(F), key=lambda f: (self.owner[f], f))
            self.base = [0] * F  # row 0 of table f inside its owner's flat table
            n_local = [0] * W
            for f in order:
                self.base[f] = n_local[self.owner[f]]
                n_local[self.owner[f]] += self.rows[f]
        else:
            self.local = [[max((self.rows[f] - r + W - 1) // W, 0) for f in range(F)] for r in range(W)]
            self.base_rf = [[sum(self.local[r][:f]) for f in range(F)] for r in range(W)]
            n_local = [sum(self.local[r]) for r in range(W)]
        self.n_local = [max(n, 1) for n in n_local]
        self.w = [np.zeros(n * self.D, np.float32) for n in self.n_local]
        self.m1 = [np.full(n * self.D, initial_accumulator_value, np.float32) for n in self.n_local]
        self.m2 = [np.zeros(n * self.D, np.float32) for n in self.n_local]
        self.it = 0

    def place(self, f, idx):
        """(owner rank, local row) of row `idx` of table f."""
        idx = _i64(idx)
        if self.partition == "table":
            return np.full(idx.shape, self.owner[f], np.int64), self.base[f] + idx
        r = idx % self.W
        return r, np.array([self.base_rf[int(rr)][f] for rr in r.reshape(-1)], np.int64).reshape(idx.shape) + idx // self.W

    def load_table(self, f, weights):
        """Distribute a whole table [rows_f, D] over the ranks' flat arrays."""
        weights = np.ascontiguousarray(weights, np.float32).reshape(self.rows[f], self.D)
        r, lrow = self.place(f, np.arange(self.rows[f]))
        for rank in range(self.W):
            sel = r == rank
            self.w[rank].reshape(-1, self.D)[lrow[sel]] = weights[sel]

    def _keys(self, indices, offsets, B):
        """Per position: (owner, local row) and the feature."""
        N = indices.size
        feat = np.searchsorted(offsets[B::B], np.arange(N), side="right") if N else np.empty(0, np.int64)
        own, lrow = np.empty(N, np.int64), np.empty(N, np.int64)
        for f in range(self.F):
            sel = feat == f
            own[sel], lrow[sel] = self.place(f, indices[sel])
        return own, lrow

    def step(self, batches, grads, B, pooling_mode=0):
        """batches[q] = (indices, offsets) of rank q's samples, grads[q] their upstream gradient.  Returns the pooled
        outputs per rank; updates the state in place."""
        W, F, D = self.W, self.F, self.D
        lr, eps, b1, b2 = self.hp
        zeros_F = np.zeros(F, np.int64)
        do = (np.arange(F + 1) * D).astype(np.int32)
        outs, sends = [], []
        for q in range(W):
            idx, offs = _i64(batches[q][0]), _i64(batches[q][1])
            N = idx.size
            own, lrow = self._keys(idx, offs, B)
            rank_span = int(max(self.n_local)) + 1
            lin = own * rank_span + lrow  # grouped by owner, ascending local row inside
            uniq, inv = np.unique(lin, return_inverse=True)
            U = uniq.size
            u_own, u_lrow = uniq // rank_span, uniq % rank_span
            fetched = np.zeros((max(U, 1), D), np.float32)
            for r in range(W):
                sel = u_own == r
                fetched[:U][sel] = self.w[r].reshape(-1, D)[u_lrow[sel]]
            # pooled locally over the fetched rows: same rows in the same order as a lookup in the whole tables
            outs.append(tbe_forward(fetched.reshape(-1), zeros_F, do, inv, offs, F, B, F * D, D, pooling_mode))
            # per distinct row: sum of its bag gradients in position order (chunks of 64); SGD with lr = -1 on zeros
            # leaves 0 + g * 1 = the sum itself
            gsum = np.zeros(max(U, 1) * D, np.float32)
            if N:
                tbe_backward(grads[q], gsum, None, None, zeros_F, do, np.array([0] * F + [U], np.int64), inv, offs, F, B,
                             F * D, D, pooling_mode, 3, -1.0, reduce_chunk=64)
            sends.append((u_own, u_lrow, gsum.reshape(-1, D)[:U]))
        self.it += 1
        for r in range(W):
            # the owner sees the lists of all source ranks, rank-major; NONE pooling with one feature per source
            # rank, all mapped to its one table: contributions of a row are summed in ascending position
            ids_in = [sends[q][1][sends[q][0] == r] for q in range(W)]
            g_in = [sends[q][2][sends[q][0] == r] for q in range(W)]
            counts = np.array([a.size for a in ids_in], np.int64)
            if counts.sum() == 0:
                continue
            idx_in = np.concatenate(ids_in)
            grad_in = np.ascontiguousarray(np.concatenate(g_in), np.float32)
            offs_in = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
            tbe_backward(grad_in, self.w[r], self.m1[r] if self.opt != 3 else None,
                         self.m2[r] if self.opt == 2 else None, np.zeros(W, np.int64),
                         (np.arange(W + 1) * D).astype(np.int32), np.array([0] * W + [self.n_local[r]], np.int64),
                         idx_in, offs_in, W, 1, W * D, D, 2, self.opt, lr, eps, b1, b2, self.it, reduce_chunk=64)
        return outs

    def table(self, f):
        """The whole table f gathered back from the ranks."""
        r, lrow = self.place(f, np.arange(self.rows[f]))
        out = np.empty((self.rows[f], self.D), np.float32)
        for rank in range(self.W):
            sel = r == rank
            out[sel] = self.w[rank].reshape(-1, self.D)[lrow[sel]]
        return out
