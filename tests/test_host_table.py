"""Host (DRAM) tier of the hybrid cache on the CPU: the key -> [w | m | v] row store (`recsdk_host_table_*`) against
the semantics of Embcache::EmbTable (torchrec_embcache/csrc/emb_table/emb_table.h:54-179,300-330) and the LINEAR
initializer (emb_table/initializer.h:44-56), and a round trip through the checkpoint layout."""
import os

import numpy as np
import pytest
import torch

from recsdk_b200.embcache import AdmitAndEvictConfig, EmbConfig, HostEmbTable


def _cfg(dim=8, optim=2, init=0, lo=0.0, hi=1.0, seed=3):
    return EmbConfig("t0", initializer_type=init, emb_dim=dim, optim_num=optim, cache_size=16, weight_init_min=lo,
                     weight_init_max=hi, weight_init_mean=0.5, weight_init_stddev=0.5,
                     admit_and_evict_config=AdmitAndEvictConfig(), seed=seed)


def test_find_or_insert_linear_init_and_zero_state():
    t = HostEmbTable(_cfg())
    keys = torch.tensor([7, 2**62, 0, 7], dtype=torch.int64)
    e, m1, m2 = (torch.full((4 * 8,), 9.0) for _ in range(3))
    t.find_or_insert(keys, e, [m1, m2])
    lin = np.array([0.0 + 1.0 * i / 7 * 1.0 for i in range(8)]).astype(np.float32)  # GenLinear in double, stored float
    np.testing.assert_array_equal(e.view(4, 8).numpy(), np.tile(lin, (4, 1)))
    assert torch.count_nonzero(m1) == 0 and torch.count_nonzero(m2) == 0
    assert t.size() == 3  # the duplicate found the row the first occurrence made


def test_insert_or_assign_overwrites_and_creates():
    rng = np.random.default_rng(0)
    t = HostEmbTable(_cfg(dim=4, optim=1))
    keys = torch.tensor([5, 6, 5], dtype=torch.int64)
    e = torch.from_numpy(rng.standard_normal(12).astype(np.float32))
    m = torch.from_numpy(rng.standard_normal(12).astype(np.float32))
    t.insert_or_assign(keys, e, [m])
    oe, om = torch.empty(8), torch.empty(8)
    t.find_or_insert(torch.tensor([5, 6], dtype=torch.int64), oe, [om])
    np.testing.assert_array_equal(oe.view(2, 4).numpy(), e.view(3, 4).numpy()[[2, 1]])  # last assignment wins
    np.testing.assert_array_equal(om.view(2, 4).numpy(), m.view(3, 4).numpy()[[2, 1]])
    with pytest.raises(RuntimeError):
        t.insert_or_assign(keys, e, [])  # optimizer blocks must match optim_num


def test_remove_growth_and_export():
    rng = np.random.default_rng(1)
    t = HostEmbTable(_cfg(dim=4, optim=2))
    n = 50_000  # far beyond the initial key-table capacity: rows must survive the rebuilds
    keys = torch.from_numpy(rng.permutation(2**40)[:1].astype(np.int64)) if False else \
        torch.from_numpy(rng.choice(2**50, n, replace=False).astype(np.int64))
    e = torch.from_numpy(rng.standard_normal(n * 4).astype(np.float32))
    m1 = torch.from_numpy(rng.standard_normal(n * 4).astype(np.float32))
    m2 = torch.from_numpy(rng.standard_normal(n * 4).astype(np.float32))
    t.insert_or_assign(keys, e, [m1, m2])
    t.remove(keys[::2].contiguous())
    assert t.size() == n // 2
    t.insert_or_assign(keys[:10:2].contiguous(), e[:20], [m1[:20], m2[:20]])  # removed keys come back (free list)
    k, ee, oo = t.export()
    order = np.argsort(k.numpy())
    kept = np.concatenate([keys.numpy()[1::2], keys.numpy()[:10:2]])
    np.testing.assert_array_equal(k.numpy()[order], np.sort(kept))
    lut = {int(x): i for i, x in enumerate(keys.numpy())}
    for j in order[:200]:
        key = int(k[j])
        src = lut[key]
        if src < 10 and src % 2 == 0:
            src = [0, 2, 4, 6, 8].index(src)  # re-inserted from the first rows of the blocks
        np.testing.assert_array_equal(ee[j].numpy(), e.view(-1, 4)[src].numpy())
        np.testing.assert_array_equal(oo[1][j].numpy(), m2.view(-1, 4)[src].numpy())


def test_seeded_random_initializers_repeat_and_respect_bounds():
    for init in (1, 2):
        a, b = HostEmbTable(_cfg(dim=16, init=init, lo=-0.2, hi=0.3)), HostEmbTable(_cfg(dim=16, init=init, lo=-0.2, hi=0.3))
        keys = torch.arange(100, dtype=torch.int64)
        ea, eb = torch.empty(1600), torch.empty(1600)
        z = [torch.empty(1600), torch.empty(1600)]
        a.find_or_insert(keys, ea, z)
        b.find_or_insert(keys, eb, z)
        assert torch.equal(ea, eb) and float(ea.min()) >= -0.2 and float(ea.max()) <= 0.3
        assert float(ea.std()) > 0.01


def test_checkpoint_layout_round_trip(tmp_path):
    from recsdk_b200 import checkpoint

    rng = np.random.default_rng(2)
    cfg = _cfg(dim=4, optim=2)
    t = HostEmbTable(cfg)
    n = 300
    keys = torch.from_numpy(rng.choice(2**60, n, replace=False).astype(np.int64))
    blocks = [torch.from_numpy(rng.standard_normal(n * 4).astype(np.float32)) for _ in range(3)]
    t.insert_or_assign(keys, blocks[0], blocks[1:])
    prefix = os.path.join(str(tmp_path), "t0", "rank0")
    checkpoint.save_table(prefix, t, cfg, None)
    # the layout the reference writes: raw arrays and {element size, count[, dim]} attributes
    assert np.fromfile(os.path.join(prefix, "key", "slice.attribute"), np.int64).tolist() == [8, n]
    assert np.fromfile(os.path.join(prefix, "embedding", "slice.attribute"), np.int64).tolist() == [4, n, 4]
    assert np.fromfile(os.path.join(prefix, "momentum2", "slice.attribute"), np.int64).tolist() == [4, n, 4]
    assert os.path.getsize(os.path.join(prefix, "momentum1", "slice.data")) == n * 4 * 4
    saved_keys = np.fromfile(os.path.join(prefix, "key", "slice.data"), np.int64)
    assert sorted(saved_keys.tolist()) == sorted(keys.tolist())
    t2 = HostEmbTable(cfg)
    checkpoint.load_table(prefix, t2, cfg, None)
    k1, e1, o1 = t.export()
    k2, e2, o2 = t2.export()
    a, b = np.argsort(k1.numpy()), np.argsort(k2.numpy())
    np.testing.assert_array_equal(k1.numpy()[a], k2.numpy()[b])
    np.testing.assert_array_equal(e1.numpy()[a], e2.numpy()[b])
    np.testing.assert_array_equal(o1[1].numpy()[a], o2[1].numpy()[b])
    bad = _cfg(dim=8, optim=2)
    with pytest.raises(RuntimeError):
        checkpoint.load_table(prefix, HostEmbTable(bad), bad, None)  # dim of the files differs from the table's
