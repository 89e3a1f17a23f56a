"""Host tier + HBM cache as one table (`HybridCacheEmbeddingBag`): a hash-keyed table whose working set is four
times its HBM cache against the same table with everything in HBM -- every row that leaves the cache and comes
back must come back bit for bit, so pooled outputs and final rows are identical; and checkpoints in the
reference's layout: save -> fresh objects -> load -> the following steps equal the uninterrupted run."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
D, B, T = 32, 64, 2


def _make(cache_size, admit=-1):
    from recsdk_b200.embcache import AdmitAndEvictConfig, EmbConfig
    from recsdk_b200.hybrid_cache import HybridCacheEmbeddingBag
    from recsdk_b200.tbe import EmbOptimType, PoolingMode

    cfgs = [EmbConfig(f"table{i}", initializer_type=0, emb_dim=D, optim_num=2, cache_size=cache_size,
                      weight_init_min=-0.05, weight_init_max=0.05,
                      admit_and_evict_config=AdmitAndEvictConfig(admit_threshold=admit), filter_capacity=1 << 14)
            for i in range(T)]
    return HybridCacheEmbeddingBag(cfgs, optimizer=EmbOptimType.ADAM, pooling_mode=PoolingMode.SUM, device=DEV,
                                   learning_rate=0.05, eps=1e-8, beta1=0.9, beta2=0.999)


def _stream(seed, steps, universe, keys_per_step):
    """Per step and table: `keys_per_step` ids, 30 % never seen before, the rest from the keys issued so far (the
    dynamic-table config scaled down); bag lengths 0..3."""
    rng = np.random.default_rng(seed)
    issued = [rng.integers(0, 2**62, size=keys_per_step, dtype=np.int64) for _ in range(T)]
    out = []
    for _ in range(steps):
        keys, lens = [], []
        for t in range(T):
            ln = rng.integers(0, 4, size=B)
            n = int(ln.sum())
            fresh = rng.integers(0, 2**62, size=int(n * 0.3), dtype=np.int64)
            pool = issued[t][-universe:]
            k = np.concatenate([fresh, pool[rng.integers(0, pool.size, size=n - fresh.size)]])
            rng.shuffle(k)
            issued[t] = np.concatenate([issued[t], fresh])
            keys.append(k)
            lens.append(ln)
        offs = np.concatenate([[0], np.cumsum(np.concatenate(lens))]).astype(np.int64)
        grad = rng.standard_normal((B, T * D)).astype(np.float32)
        out.append((keys, offs, grad))
    return out


def _run(bag, stream):
    outs = []
    for keys, offs, grad in stream:
        o = bag.forward([torch.from_numpy(k).to(DEV) for k in keys], torch.from_numpy(offs).to(DEV))
        o.backward(torch.from_numpy(grad).to(DEV))
        outs.append(o.detach().cpu().numpy())
    return outs


def _rows_by_key(bag, table):
    bag.flush_to_host()
    k, e, o = bag.mgr.host_tables[table].export()
    order = np.argsort(k.numpy())
    return k.numpy()[order], e.numpy()[order], o[0].numpy()[order], o[1].numpy()[order]


def test_working_set_four_times_the_cache_matches_all_in_hbm():
    stream = _stream(11, steps=40, universe=600, keys_per_step=96)
    distinct = len(set(np.concatenate([k for s in stream for k in s[0]]).tolist()))
    small, big = _make(cache_size=256), _make(cache_size=8192)
    assert distinct > 4 * 256
    a, b = _run(small, stream), _run(big, stream)
    for x, y in zip(a, b):
        np.testing.assert_array_equal(x, y)
    for t in range(T):
        for u, v in zip(_rows_by_key(small, t), _rows_by_key(big, t)):
            np.testing.assert_array_equal(u, v)
    # rows did travel, one copy per array and direction per swap, on the copy stream
    labels = [e[0] for e in small.swap_events]
    assert labels.count("swap_out_d2h") > 10 and labels.count("swap_in_h2d") >= 40
    assert all(e[1].elapsed_time(e[2]) >= 0 for e in small.swap_events)


def test_checkpoint_resume_equals_uninterrupted_run(tmp_path):
    from recsdk_b200.checkpoint import Saver

    stream = _stream(12, steps=20, universe=400, keys_per_step=96)
    ref = _make(cache_size=256)
    expected = _run(ref, stream)
    first = _make(cache_size=256)
    got = _run(first, stream[:10])
    saver = Saver(rank=0)
    written = saver.save([(first.mgr, first.module)], str(tmp_path))
    assert written.startswith(str(tmp_path))
    resumed = _make(cache_size=256)
    saver.load([resumed.mgr], str(tmp_path))
    resumed.module.iter[0] = first.module.iter[0]  # the optimizer step count is the trainer's to carry
    resumed.module.step = first.module.step
    got += _run(resumed, stream[10:])
    for x, y in zip(got, expected):
        np.testing.assert_array_equal(x, y)
    for t in range(T):
        for u, v in zip(_rows_by_key(resumed, t), _rows_by_key(ref, t)):
            np.testing.assert_array_equal(u, v)


def test_checkpoint_carries_admission_counts_of_the_stored_keys(tmp_path):
    """With admission on, the checkpoint holds the count of every key that has a row in the host store (the keys
    that were admitted); the counts of keys seen but not yet admitted are not part of it -- in the reference either
    (embcache_manager.cpp:348-389: the count file is written for the keys of the embedding table)."""
    from recsdk_b200.checkpoint import Saver

    stream = _stream(13, steps=12, universe=300, keys_per_step=96)
    first = _make(cache_size=256, admit=2)
    _run(first, stream)
    Saver(rank=0).save([(first.mgr, first.module)], str(tmp_path))
    resumed = _make(cache_size=256, admit=2)
    Saver(rank=0).load([resumed.mgr], str(tmp_path))
    for t in range(T):
        k1, e1, o1 = first.mgr.host_tables[t].export()
        k2, e2, o2 = resumed.mgr.host_tables[t].export()
        a, b = np.argsort(k1.numpy()), np.argsort(k2.numpy())
        assert k1.numel() > 50
        np.testing.assert_array_equal(k1.numpy()[a], k2.numpy()[b])
        np.testing.assert_array_equal(e1.numpy()[a], e2.numpy()[b])
        np.testing.assert_array_equal(o1[1].numpy()[a], o2[1].numpy()[b])
        keys = k1[torch.from_numpy(a)].to(DEV)
        c1 = first.mgr.feature_filters[t].GetCounts(keys).cpu().numpy()
        c2 = resumed.mgr.feature_filters[t].GetCounts(keys).cpu().numpy()
        np.testing.assert_array_equal(c1, c2)
        assert (c1 >= 2).all()  # every stored key had been admitted
    _run(resumed, stream[:3])  # and training goes on from the loaded state
