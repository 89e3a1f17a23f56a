"""EmbcacheManager (policy tier of the hybrid-cache table interface) over two tables against the CPU classes
composed the way the reference manager composes them (embcache_manager.cpp:89-185): per-table key lists, slot
offsets shifted by the cache sizes of the tables before, table-local batch offsets."""
import numpy as np
import pytest
import torch

from oracle import port, ref
from tests.golden.driver import cache_driver_steps, first_occurrence_unique, run_cache_driver

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cpu_classes(cache, start, admit, thr, interval):
    try:
        if not ref.available():
            raise OSError
        return ref.SwapManager(cache, start), (ref.FeatureFilter(admit, thr, interval) if (admit != -1 or thr) else None)
    except OSError:
        return port.SwapManager(cache, start), (port.FeatureFilter(admit, thr, interval) if (admit != -1 or thr) else None)


@pytest.mark.parametrize("accumulate", [True, False])
def test_manager_matches_composed_reference_classes(accumulate):
    from recsdk_b200.embcache import AdmitAndEvictConfig, EmbcacheManager, EmbConfig

    steps, n, interval = 14, 4096, 4
    cfgs = [
        EmbConfig("t0", emb_dim=16, optim_num=2, cache_size=9000,
                  admit_and_evict_config=AdmitAndEvictConfig(2, 0.0, 3, interval), filter_capacity=1 << 17),
        EmbConfig("t1", emb_dim=16, optim_num=2, cache_size=7000),
    ]
    mgr = EmbcacheManager(cfgs, need_accumulate_offset=accumulate, device=DEV)
    streams = [cache_driver_steps(11, steps, n, 0.3), cache_driver_steps(12, steps, n // 2, 0.5)]
    # oracle side, table by table
    exp = []
    for t, (cache, start, admit, thr) in enumerate([(9000, 1, 2, 3), (7000, 0, -1, 0)]):
        sw, fl = _cpu_classes(cache, start, admit, thr, interval if thr else 0)
        exp.append(run_cache_driver(sw, fl, streams[t], interval if thr else 0))
    shift = [0, 9000 if accumulate else 0]
    for s in range(steps):
        raw = [streams[t][s] for t in range(2)]
        raw_cat = torch.from_numpy(np.concatenate(raw)).to(DEV)
        raw_offs = [0, raw[0].size, raw[0].size + raw[1].size]
        ts = torch.full((raw_cat.numel(),), s, dtype=torch.int64, device=DEV)
        mgr.record_timestamp(raw_cat, raw_offs, ts)
        if s > 0 and (s + 1) % interval == 0:
            n_evicted = mgr.evict_features()
            assert n_evicted == exp[0][s]["evicted"].size
            np.testing.assert_array_equal(np.sort(mgr.evicted_keys(0).cpu().numpy()), exp[0][s]["evicted"])
            mgr.remove_embedding_table_info()
        off_t = torch.tensor(raw_offs, dtype=torch.int64)
        for t in range(2):
            mgr.statistics_key_count(raw_cat, off_t, torch.empty(0, dtype=torch.int64, device=DEV), t)
        uniq = [first_occurrence_unique(k) for k in raw]
        keys = torch.from_numpy(np.concatenate(uniq)).to(DEV)
        offs = [0, uniq[0].size, uniq[0].size + uniq[1].size]
        info = mgr.compute_swap_info_async(keys, offs).get()
        np.testing.assert_array_equal(keys[:offs[1]].cpu().numpy(), exp[0][s]["filtered"])  # filtered in place
        for t in range(2):
            np.testing.assert_array_equal(info.swapout_keys[t].cpu().numpy(), exp[t][s]["swapout_keys"])
            np.testing.assert_array_equal(info.swapin_keys[t].cpu().numpy(), exp[t][s]["swapin_keys"])
        np.testing.assert_array_equal(info.swapout_offs.cpu().numpy(),
                                      np.concatenate([exp[t][s]["swapout_offs"] + shift[t] for t in range(2)]))
        np.testing.assert_array_equal(info.swapin_offs.cpu().numpy(),
                                      np.concatenate([exp[t][s]["swapin_offs"] + shift[t] for t in range(2)]))
        np.testing.assert_array_equal(info.batch_offs.cpu().numpy(),
                                      np.concatenate([exp[t][s]["batch_offs"] for t in range(2)]))
    assert mgr.swap_count == steps


def test_manager_argument_errors_and_host_tier():
    from recsdk_b200.embcache import EmbcacheManager, EmbConfig

    with pytest.raises(RuntimeError, match="Size of embConfigs must > 0"):
        EmbcacheManager([], device=DEV)
    mgr = EmbcacheManager([EmbConfig("a", cache_size=64, emb_dim=4, optim_num=1, weight_init_max=1.0),
                           EmbConfig("b", cache_size=64, emb_dim=4, optim_num=1, weight_init_max=1.0)], device=DEV)
    keys = torch.arange(10, dtype=torch.int64, device=DEV)
    with pytest.raises(RuntimeError, match="tableIndices size\\+1 must be equal to offsetPerKey size"):
        mgr.compute_swap_info_async(keys, [0, 10])
    with pytest.raises(RuntimeError, match="out of range"):
        mgr.compute_swap_info_async(keys, [0, 10], table_indices=[5])
    with pytest.raises(RuntimeError, match="must be of type int64_t"):
        mgr.compute_swap_info_async(keys.int(), [0, 5, 10])
    info = mgr.compute_swap_info(keys, [0, 10], table_indices=[1])  # only table 1
    assert info.swapin_keys[0].numel() == 10 and info.batch_offs.numel() == 10
    # host tier: the swap-in keys of table 1 get LINEAR rows and zero optimizer state, in pinned host tensors
    st = mgr.embedding_lookup_async(info, table_indices=[1]).get()
    assert st.swapin_embs.is_pinned() and st.jagged_offs.tolist() == [0, 40]
    np.testing.assert_array_equal(st.swapin_embs.view(10, 4).numpy(),
                                  np.tile(np.array([0, 1 / 3, 2 / 3, 1], np.float64).astype(np.float32), (10, 1)))
    assert len(st.swapin_optims) == 1 and torch.count_nonzero(st.swapin_optims[0]) == 0
    assert mgr.host_tables[1].size() == 10 and mgr.host_tables[0].size() == 0
    with pytest.raises(RuntimeError, match="tableIndices size must be equal"):
        mgr.embedding_lookup_async(info).get()  # one key list, two tables
