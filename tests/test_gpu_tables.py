"""Parity of the HBM key tables, bucketize and row operators with the golden fixtures produced by the
reference's own host code, and with the CPU oracle on larger seeded inputs.  Everything here is
integer / byte work: bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import port
from tests.golden.driver import cache_driver_steps, first_occurrence_unique, run_cache_driver, zipf_ids

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _t(a, dtype=None):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype).to(DEV)


def _np(t):
    return t.cpu().numpy()


# ----------------------------------------------------------------------------- IdsMapper (A2)
def test_ids_mapper_unique_out_matches_reference_golden(golden_dir):
    from recsdk_b200 import IdsMapper

    g = np.load(os.path.join(golden_dir, "ids_mapper.npz"))
    T = 3
    mappers = [IdsMapper(4096, True) for _ in range(T)]
    for s in range(3):
        ids = g[f"s{s}_ids"]
        offset = g[f"s{s}_offset"]
        n = ids.size
        hi, uq, uid, inv = (torch.full((max(n, 1),), -7, dtype=torch.int64, device=DEV) for _ in range(4))
        uoff = torch.zeros(T + 1, dtype=torch.int64, device=DEV)
        if s == 1:
            IdsMapper.parallel_ids2indices_unique_out(mappers, _t(ids), hi, offset, uq, uid, inv, uoff)
        else:
            for t in range(T):
                mappers[t].ids2indices_unique_out(_t(ids), hi, torch.from_numpy(offset), uq, uid, inv, uoff, t)
        U = int(uoff[-1].item())
        np.testing.assert_array_equal(_np(uoff), g[f"s{s}_unique_offset"])
        np.testing.assert_array_equal(_np(hi)[:n], g[f"s{s}_hash_indices"])
        np.testing.assert_array_equal(_np(uq)[:U], g[f"s{s}_unique"])
        np.testing.assert_array_equal(_np(uid)[:U], g[f"s{s}_unique_ids"])
        np.testing.assert_array_equal(_np(inv)[:n], g[f"s{s}_unique_inverse"])


def test_ids2indices_unique_matches_reference_golden(golden_dir):
    from recsdk_b200 import IdsMapper

    g = np.load(os.path.join(golden_dir, "ids_mapper.npz"))
    m = IdsMapper(100000, True)
    for s in range(2):
        hi, uq, inv = m.ids2indices_unique(_t(g[f"u{s}_ids"]))
        np.testing.assert_array_equal(_np(hi), g[f"u{s}_hash_indices"])
        np.testing.assert_array_equal(_np(uq), g[f"u{s}_unique"])
        np.testing.assert_array_equal(_np(inv), g[f"u{s}_inverse"])


def test_ids_mapper_large_vs_oracle():
    """131072 keys/step uniform over [0, 2^63) with 30% new keys (the dynamic-table config), 6 steps."""
    from recsdk_b200 import IdsMapper

    steps = cache_driver_steps(99, 6, 131072, 0.3, key_bits=63)
    gm, om = IdsMapper(1 << 20, True), port.IdsMapper(1 << 20, True)
    for keys in steps:
        n = keys.size
        offset = np.array([0, n], np.int64)
        ehi, euq, euid, einv = (np.empty(n, np.int64) for _ in range(4))
        euoff = np.zeros(2, np.int64)
        om.ids2indices_unique_out(keys, ehi, offset, euq, euid, einv, euoff, 0)
        hi, uq, uid, inv = (torch.empty(n, dtype=torch.int64, device=DEV) for _ in range(4))
        uoff = torch.zeros(2, dtype=torch.int64, device=DEV)
        gm.ids2indices_unique_out(_t(keys), hi, offset, uq, uid, inv, uoff, 0)
        U = int(euoff[1])
        np.testing.assert_array_equal(_np(uoff), euoff)
        np.testing.assert_array_equal(_np(hi), ehi)
        np.testing.assert_array_equal(_np(uq)[:U], euq[:U])
        np.testing.assert_array_equal(_np(uid)[:U], euid[:U])
        np.testing.assert_array_equal(_np(inv), einv)
    assert gm.size() == om.size()


def test_ids_mapper_errors():
    from recsdk_b200 import IdsMapper

    m = IdsMapper(4, True)
    with pytest.raises(RuntimeError, match="Invalid key value"):
        m.ids2indices_unique(_t(np.array([1, -5], np.int64)))
    m = IdsMapper(4, True)
    with pytest.raises(RuntimeError, match="reached maxIndex"):
        m.ids2indices_unique(_t(np.arange(10, 20, dtype=np.int64)))


# ----------------------------------------------------------------------------- cache policy (A4, A5)
class _GpuSwap:
    def __init__(self, cache, start):
        from recsdk_b200 import SwapManager

        self.s = SwapManager(cache, start)

    def compute_swap_info(self, keys):
        return tuple(_np(x) for x in self.s.ComputeSwapInfo(_t(keys)))

    def remove_keys(self, keys):
        if keys.size:
            self.s.RemoveKeys(_t(keys))


class _GpuFilter:
    def __init__(self, admit, thr, interval, capacity=1 << 16):
        from recsdk_b200 import FeatureFilter

        self.f = FeatureFilter("t", admit, thr, interval, capacity=capacity)

    def record_timestamp(self, keys, ts):
        self.f.RecordTimestamp(_t(keys), _t(ts))

    def evict_keys(self):
        return _np(self.f.GetEvictKeys())

    def clear_evict(self):
        self.f.ClearEvictInfo()

    def statistics_key_count(self, keys, counts=None):
        self.f.StatisticsKeyCount(_t(keys), _t(counts) if counts is not None else None)

    def count_filter(self, keys):
        return _np(self.f.CountFilter(_t(keys)))


def test_cache_policy_matches_reference_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "cache.npz"))
    for c in range(int(g["n_cases"][0])):
        cache, admit, evict_thr, interval, steps = (int(x) for x in g[f"c{c}_meta"])
        keys = [g[f"c{c}_s{s}_keys"] for s in range(steps)]
        admit_on = admit != -1
        swap = _GpuSwap(cache, 1 if admit_on else 0)
        filt = _GpuFilter(admit, evict_thr, interval) if (admit_on or evict_thr) else None
        rec = run_cache_driver(swap, filt, keys, interval)
        for s, r in enumerate(rec):
            for k, v in r.items():
                np.testing.assert_array_equal(v, g[f"c{c}_s{s}_{k}"], err_msg=f"case {c} step {s} {k}")


def test_cache_policy_small_capacity_vs_oracle():
    """Capacity 2^17 with 131072-key steps: the replacement sweep, version protection and reuse of evicted
    positions all run at the dynamic-table config's batch size."""
    keys = cache_driver_steps(99, 12, 131072, 0.3, key_bits=63)
    cache = 1 << 17
    gs, os_ = _GpuSwap(cache * 2, 1), port.SwapManager(cache * 2, 1)
    gf, of = _GpuFilter(2, 3, 3, capacity=1 << 21), port.FeatureFilter(2, 3, 3)
    rg = run_cache_driver(gs, gf, keys, 3)
    ro = run_cache_driver(os_, of, keys, 3)
    for s, (a, b) in enumerate(zip(rg, ro)):
        for k in b:
            np.testing.assert_array_equal(a[k], b[k], err_msg=f"step {s} {k}")
    # pure clock sweep on a cache that is too small to hold two steps
    keys = cache_driver_steps(5, 8, 4096, 0.5)
    gs, os_ = _GpuSwap(12000, 0), port.SwapManager(12000, 0)
    rg = run_cache_driver(gs, None, keys, 0)
    ro = run_cache_driver(os_, None, keys, 0)
    for s, (a, b) in enumerate(zip(rg, ro)):
        for k in b:
            np.testing.assert_array_equal(a[k], b[k], err_msg=f"step {s} {k}")
    assert any(r["swapout_keys"].size for r in ro)


def test_cache_policy_full_size_dynamic_table_config():
    """The dynamic-table config at its full size: 64 Mi cache slots, 200 steps x 131072 keys (30 % fresh keys per
    step), admit threshold 2, evict after 50 idle steps checked every 10 steps.  Every per-step output (admitted
    keys, evicted set, swap-in / swap-out lists, batch offsets) must equal the compiled reference classes'
    (SwapManager + FeatureFilter) when they are available, else the C restatement's."""
    from oracle import ref

    steps, n = 200, 131072
    keys = cache_driver_steps(99, steps, n, 0.3, key_bits=63)
    cache = 64 << 20
    try:
        if not ref.available():
            raise OSError("compiled reference classes not present")
        os_, of = ref.SwapManager(cache, 1), ref.FeatureFilter(2, 50, 10)
    except OSError:
        os_, of = port.SwapManager(cache, 1), port.FeatureFilter(2, 50, 10)
    gs, gf = _GpuSwap(cache, 1), _GpuFilter(2, 50, 10, capacity=1 << 25)
    ro = run_cache_driver(os_, of, keys, 10)
    rg = run_cache_driver(gs, gf, keys, 10)
    for s, (a, b) in enumerate(zip(rg, ro)):
        for k in b:
            np.testing.assert_array_equal(a[k], b[k], err_msg=f"step {s} {k}")
    assert sum(r["evicted"].size for r in ro) > 0 and sum(r["swapin_keys"].size for r in ro) > n


def test_cache_too_small_raises():
    from recsdk_b200 import SwapManager

    swap = SwapManager(4, 0)
    swap.ComputeSwapInfo(_t(np.array([1, 2, 3, 4], np.int64)))
    with pytest.raises(RuntimeError, match="cacheSize_ too small"):
        swap.ComputeSwapInfo(_t(np.array([5], np.int64)))


def test_admit_rule_and_counts():
    """A key absent from the count map passes; present with count < threshold is replaced by -1
    (feature_filter.cpp:140-160); counts accumulate with explicit counts."""
    from recsdk_b200 import FeatureFilter

    f = FeatureFilter("t", 3, 0, 0, capacity=1024)
    f.StatisticsKeyCount(_t([10, 11, 10, 12]))
    f.StatisticsKeyCount(_t([10, 12]), _t([1, 5]))
    np.testing.assert_array_equal(_np(f.GetCounts(_t([10, 11, 12, 13]))), [3, 1, 6, -1])
    np.testing.assert_array_equal(_np(f.CountFilter(_t([10, 11, 12, 13]))), [10, -1, 12, 13])


# ----------------------------------------------------------------------------- bucketize (A3)
def test_bucketize_matches_reference_golden(golden_dir):
    from recsdk_b200 import ops

    g = np.load(os.path.join(golden_dir, "bucketize.npz"))
    for c in range(int(g["n_cases"][0])):
        W, F, B, do_unique, ret_count = (int(x) for x in g[f"c{c}_meta"])
        nl, ni, perm, cnt, num = ops.bucketize(_t(g[f"c{c}_lengths"]), _t(g[f"c{c}_indices"]), F, W, bool(do_unique),
                                               bool(ret_count))
        k = int(num.item())
        np.testing.assert_array_equal(_np(nl), g[f"c{c}_new_lengths"], err_msg=f"case {c}")
        np.testing.assert_array_equal(_np(ni)[:k], g[f"c{c}_new_indices"], err_msg=f"case {c}")
        np.testing.assert_array_equal(_np(perm), g[f"c{c}_unbucketize_permute"], err_msg=f"case {c}")
        if ret_count:
            np.testing.assert_array_equal(_np(cnt)[:k], g[f"c{c}_ids_counts"], err_msg=f"case {c}")


@pytest.mark.parametrize("do_unique", [False, True])
def test_bucketize_large_vs_oracle(do_unique):
    """262144 one-hot ids Zipf(1.05) over 8 ranks (the row-wise sharded config's routing step) + a ragged case."""
    from recsdk_b200 import ops

    rng = np.random.default_rng(5)
    for F, B, maxlen in ((1, 262144, 1), (3, 5000, 7)):
        lengths = np.ones(F * B, np.int64) if maxlen == 1 else rng.integers(0, maxlen + 1, F * B)
        idx = zipf_ids(rng, int(lengths.sum()), 1_000_000, 1.05)
        enl, eni, eperm, ecnt = port.bucketize(lengths, idx, F, 8, True, do_unique, do_unique)
        nl, ni, perm, cnt, num = ops.bucketize(_t(lengths), _t(idx), F, 8, do_unique, do_unique)
        k = int(num.item())
        assert k == eni.size
        np.testing.assert_array_equal(_np(nl), enl)
        np.testing.assert_array_equal(_np(ni)[:k], eni)
        np.testing.assert_array_equal(_np(perm), eperm)
        if do_unique:
            np.testing.assert_array_equal(_np(cnt)[:k], ecnt)


# ----------------------------------------------------------------------------- rows (A8), TF ops (A9), restore (A10)
@pytest.mark.parametrize("D", [8, 32, 128, 6, 1024])
def test_gather_scatter_rows(D):
    from recsdk_b200 import ops

    rng = np.random.default_rng(D)
    rows = 5000
    table = rng.standard_normal((rows, D)).astype(np.float32)
    for k in (0, 1, 7, 8, 9, 1000, 4097):
        slots = rng.permutation(rows)[:k].astype(np.int64)
        out = ops.gather_rows(_t(table).view(-1), _t(slots), D)
        np.testing.assert_array_equal(_np(out), port.gather_rows(table.reshape(-1), slots, D))
        upd = rng.standard_normal((k, D)).astype(np.float32)
        dt = _t(table).view(-1)
        st = ops.new_status(DEV)
        ops.scatter_rows(dt, _t(slots), D, _t(upd), status=st)
        ops.raise_on_status(st)
        exp = table.copy().reshape(-1)
        port.scatter_rows(exp, slots, D, upd)
        np.testing.assert_array_equal(_np(dt), exp)


def test_gather_rows_bad_slot_sets_status():
    from recsdk_b200 import ops

    table = torch.zeros(10 * 8, dtype=torch.float32, device=DEV)
    st = ops.new_status(DEV)
    ops.gather_rows(table, _t([1, 99]), 8, status=st)
    with pytest.raises(RuntimeError, match="out of range"):
        ops.raise_on_status(st)


def test_lookup_update_by_address():
    """100000x8 table, 21632 addresses as in cust_op/test/aclnn_cust_op_by_addr_test; address 0 -> zeros / skipped."""
    from recsdk_b200 import ops

    rng = np.random.default_rng(3)
    rows, dim, n = 100000, 8, 21632
    table_np = rng.standard_normal((rows, dim)).astype(np.float32)
    table = _t(table_np)
    slots = rng.permutation(rows)[:n]
    addr = table.data_ptr() + slots.astype(np.int64) * dim * 4
    addr[::97] = 0
    out = ops.embedding_lookup_by_address(_t(addr), dim)
    exp = table_np[slots].copy()
    exp[::97] = 0
    np.testing.assert_array_equal(_np(out), exp)
    upd = rng.standard_normal((n, dim)).astype(np.float32)
    ops.embedding_update_by_address(_t(addr), _t(upd), 0)
    e2 = table_np.copy()
    live = addr != 0
    e2[slots[live]] = e2[slots[live]] + upd[live]
    np.testing.assert_array_equal(_np(table), e2)
    ops.embedding_update_by_address(_t(addr), _t(upd), 1)
    e2[slots[live]] = upd[live]
    np.testing.assert_array_equal(_np(table), e2)


def test_lazy_adam_bit_exact_and_reference_gate():
    """Shape of cust_op/test/aclnn_lazy_adam_test (uniform(1,2) data, beta .9/.999, lr 1e-3, eps 1e-7), scaled."""
    from recsdk_b200 import ops

    rng = np.random.default_rng(5)
    rows, dim, n = 200000, 32, 56409
    m, v, var = (rng.uniform(1, 2, (rows, dim)).astype(np.float32) for _ in range(3))
    g = rng.uniform(1, 2, (n, dim)).astype(np.float32)
    idx = rng.permutation(rows)[:n].astype(np.int32)
    idx[5] = -1
    dm, dv, dvar = _t(m), _t(v), _t(var)
    ops.lazy_adam(_t(g), _t(idx), dm, dv, dvar, 1e-3, 0.9, 0.999, 1e-7)
    port.lazy_adam(g, idx, m, v, var, 1e-3, 0.9, 0.999, 1e-7)
    for a, b in ((dm, m), (dv, v), (dvar, var)):
        np.testing.assert_array_equal(_np(a), b)


@pytest.mark.parametrize("wd", [None, 0.01])
def test_sgd(wd):
    from recsdk_b200 import ops

    rng = np.random.default_rng(8)
    rows, dim, n = 3000, 16, 1000
    var = rng.standard_normal((rows, dim)).astype(np.float32)
    g = rng.standard_normal((n, dim)).astype(np.float32)
    idx = rng.permutation(rows)[:n].astype(np.int64)  # unique: atomics land once per element -> bit-exact
    idx[3] = -1
    dvar = _t(var)
    ops.sgd(_t(g), _t(idx), dvar, 0.1, wd)
    port.sgd(g, idx, var, 0.1, wd)
    np.testing.assert_array_equal(_np(dvar), var)
    # duplicates accumulate (order of float atomics is free: 1e-6, relative to max(1, |x|))
    idx2 = rng.integers(0, 50, n).astype(np.int64)
    var2 = rng.standard_normal((rows, dim)).astype(np.float32)
    dvar2 = _t(var2)
    ops.sgd(_t(g), _t(idx2), dvar2, 0.1, wd)
    port.sgd(g, idx2, var2, 0.1, wd)
    np.testing.assert_allclose(_np(dvar2), var2, rtol=1e-6, atol=1e-6)


def test_restore():
    from recsdk_b200 import ops

    rng = np.random.default_rng(9)
    T = 4
    lens = rng.integers(0, 3000, T)
    lens[2] = 0
    tab_off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    uq, inv, uoff = [], [], [0]
    for t in range(T):
        ids = zipf_ids(rng, int(lens[t]), 500, 1.1) * 3 + t
        u = first_occurrence_unique(ids)
        lut = {int(x): k for k, x in enumerate(u)}
        inv.append(np.array([lut[int(x)] for x in ids], np.int64))
        uq.append(u)
        uoff.append(uoff[-1] + u.size)
    uq, inv, uoff = np.concatenate(uq), np.concatenate(inv), np.array(uoff, np.int64)
    exp = port.restore(uq, inv, uoff, tab_off)
    got = ops.restore(_t(uq), _t(inv), _t(uoff), tab_off.tolist())
    np.testing.assert_array_equal(_np(got), exp)


def test_long_churn_keeps_probe_chains_bounded():
    """Small tables under thousands of steps of churn (new keys every step, eviction every 4 steps, cache
    replacement): without compaction the EMPTY entries of the open-addressing tables run out; with it the results
    still match the CPU classes step by step and the longest displacement stays small."""
    from recsdk_b200.embcache import AdmitAndEvictConfig, EmbcacheManager, EmbConfig

    steps, n, interval, cache = 3000, 96, 4, 1024
    cfg = EmbConfig("t", emb_dim=4, optim_num=0, cache_size=cache, weight_init_max=1.0,
                    admit_and_evict_config=AdmitAndEvictConfig(-1, 0.0, 3, interval), filter_capacity=1024)
    mgr = EmbcacheManager([cfg], device=DEV)
    sw, fl = port.SwapManager(cache, 0), port.FeatureFilter(-1, 3, interval)
    rng = np.random.default_rng(77)
    recent = rng.integers(0, 2**62, size=n, dtype=np.int64)
    compactions = 0
    worst = 0
    for s in range(steps):
        fresh = rng.integers(0, 2**62, size=n // 2, dtype=np.int64)
        keys = np.concatenate([fresh, recent[rng.integers(0, recent.size, size=n - fresh.size)]])
        recent = np.concatenate([recent[-2 * n:], fresh])
        uq = first_occurrence_unique(keys)
        d_keys = torch.from_numpy(keys).to(DEV)
        mgr.record_timestamp(d_keys, [0, keys.size], torch.full((keys.size,), s, dtype=torch.int64, device=DEV))
        fl.record_timestamp(keys, np.full(keys.size, s, np.int64))
        if s > 0 and (s + 1) % interval == 0:
            before = mgr.feature_filters[0].table_stats()[1] + mgr.swap_managers[0].table_stats()[1]
            mgr.evict_features()
            after = mgr.feature_filters[0].table_stats()[1] + mgr.swap_managers[0].table_stats()[1]
            compactions += int(after < before)
            ev = fl.evict_keys()
            np.testing.assert_array_equal(np.sort(mgr.evicted_keys(0).cpu().numpy()), np.sort(ev))
            mgr.remove_embedding_table_info()
            sw.remove_keys(ev)
            fl.clear_evict()
        info = mgr.compute_swap_info(torch.from_numpy(uq).to(DEV), [0, uq.size])
        exp = sw.compute_swap_info(uq)
        np.testing.assert_array_equal(info.batch_offs.cpu().numpy(), exp[4])
        np.testing.assert_array_equal(info.swapout_keys[0].cpu().numpy(), exp[0])
        if s % 250 == 249:
            worst = max(worst, mgr.feature_filters[0].table_stats()[2], mgr.swap_managers[0].table_stats()[2])
    assert compactions > 0  # the tables were rebuilt along the way
    assert worst < 256  # displacement from the home entry stays far below the capacity (2048 / 4096 entries)


def test_bounded_wait_runs_out_cleanly():
    """The row mover's mbarrier waits are bounded.  With a poll limit of 0 the first wait gives up at once: the
    kernel must record RECSDK_ERR_CUDA in the status block and return (after letting its own copies land), and the
    context must stay usable -- the same call with the normal limit then moves the rows."""
    import ctypes as C

    from recsdk_b200 import _lib, ops

    lib = _lib.load()
    rng = np.random.default_rng(4)
    rows, dim, k = 4096, 64, 512
    table = _t(rng.standard_normal((rows, dim)).astype(np.float32))
    slots = _t(rng.permutation(rows)[:k].astype(np.int64))
    out = torch.zeros((k, dim), dtype=torch.float32, device=DEV)
    st = ops.new_status(DEV)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.recsdk_gather_rows_wait_limit(table.data_ptr(), slots.data_ptr(), k, dim, out.data_ptr(), rows, st.data_ptr(), 0,
                                           stream)
    assert rc == 0
    torch.cuda.synchronize()
    code = st.tolist()[0]
    assert code == _lib.ERR_CUDA
    with pytest.raises(RuntimeError):
        ops.raise_on_status(st)
    rc = lib.recsdk_gather_rows_wait_limit(table.data_ptr(), slots.data_ptr(), k, dim, out.data_ptr(), rows, st.data_ptr(),
                                           1 << 22, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert st.tolist()[0] == 0
    np.testing.assert_array_equal(_np(out), _np(table)[_np(slots)])
