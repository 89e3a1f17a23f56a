"""Checkpoint files against the reference's OWN code (oracle/_ref/libref_manager.so = the reference's
EmbcacheManager compiled from its sources, driven through oracle/ref_manager_harness.cpp): a checkpoint written by
the reference loads here with every row intact, and a checkpoint written here loads in the reference, which writes
the same bytes back.  CPU only; skipped when the reference build is not present."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from recsdk_b200 import checkpoint
from recsdk_b200.embcache import AdmitAndEvictConfig, EmbConfig, HostEmbTable

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "oracle", "_ref", "libref_manager.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(LIB):
        pytest.skip("reference manager not built (oracle/build_ref.py)")
    lib = C.CDLL(LIB)
    lib.refmgr_new.restype = C.c_void_p
    lib.refmgr_new.argtypes = [C.c_char_p, C.c_int32, C.c_int32, C.c_int64, C.c_float, C.c_float, C.c_int64, C.c_uint64,
                               C.c_uint64]
    lib.refmgr_free.argtypes = [C.c_void_p]
    lib.refmgr_update.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.refmgr_statistics.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
    lib.refmgr_record_timestamp.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]
    lib.refmgr_save.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
    lib.refmgr_load.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
    return lib


DIM, N = 8, 500


def _rows(seed):
    rng = np.random.default_rng(seed)
    keys = rng.choice(2**60, N, replace=False).astype(np.int64)
    blocks = [rng.standard_normal((N, DIM)).astype(np.float32) for _ in range(3)]
    return keys, blocks


def _cfg(admit=-1, evict=0):
    return EmbConfig("tbl", initializer_type=0, emb_dim=DIM, optim_num=2, cache_size=64, weight_init_min=0.0,
                     weight_init_max=1.0, admit_and_evict_config=AdmitAndEvictConfig(admit, 0.0, evict, 10 if evict else 0))


def _sorted_table(prefix):
    keys = np.fromfile(os.path.join(prefix, "key", "slice.data"), np.int64)
    order = np.argsort(keys)
    out = [keys[order]]
    for name in ("embedding", "momentum1", "momentum2"):
        out.append(np.fromfile(os.path.join(prefix, name, "slice.data"), np.float32).reshape(-1, DIM)[order])
    return out


def test_checkpoint_written_by_the_reference_loads_here(ref, tmp_path):
    keys, blocks = _rows(1)
    m = ref.refmgr_new(b"tbl", DIM, 2, 64, 0.0, 1.0, 2, 50, 10)  # admission and eviction on: all six directories
    assert m
    assert ref.refmgr_update(m, keys.ctypes.data, N, DIM, *(b.ctypes.data for b in blocks)) == 0
    seen = np.concatenate([keys[:300], keys[:100]])  # counts 2 for the first 100, 1 for the next 200, absent for the rest
    assert ref.refmgr_statistics(m, seen.ctypes.data, seen.size) == 0
    ts = np.arange(N, dtype=np.int64) + 1000
    assert ref.refmgr_record_timestamp(m, keys.ctypes.data, ts.ctypes.data, N) == 0
    path = str(tmp_path / "by_ref")
    assert ref.refmgr_save(m, path.encode(), 3) == 0
    ref.refmgr_free(m)
    prefix = os.path.join(path, "tbl", "rank3")
    cfg = _cfg(admit=2, evict=50)
    t = HostEmbTable(cfg)
    checkpoint.load_table(prefix, t, cfg, None)
    k, e, o = t.export()
    order, want = np.argsort(k.numpy()), np.argsort(keys)
    np.testing.assert_array_equal(k.numpy()[order], keys[want])
    np.testing.assert_array_equal(e.numpy()[order], blocks[0][want])
    np.testing.assert_array_equal(o[0].numpy()[order], blocks[1][want])
    np.testing.assert_array_equal(o[1].numpy()[order], blocks[2][want])
    # admission / eviction files: the layout this package reads and writes
    saved_keys = np.fromfile(os.path.join(prefix, "key", "slice.data"), np.int64)
    counts = np.fromfile(os.path.join(prefix, "admit_count", "slice.data"), np.int64)
    assert np.fromfile(os.path.join(prefix, "admit_count", "slice.attribute"), np.int64).tolist() == [8, N]
    expect = {int(k_): (2 if i < 100 else 1 if i < 300 else -1) for i, k_ in enumerate(keys)}
    assert [expect[int(k_)] for k_ in saved_keys] == counts.tolist()
    ek = np.fromfile(os.path.join(prefix, "evict_timestamp", "slice_evict_key.data"), np.int64)
    et = np.fromfile(os.path.join(prefix, "evict_timestamp", "slice_evict_ts.data"), np.int64)
    assert np.fromfile(os.path.join(prefix, "evict_timestamp", "slice.attribute"), np.int64).tolist() == [8, N]
    assert dict(zip(ek.tolist(), et.tolist())) == dict(zip(keys.tolist(), ts.tolist()))


def test_checkpoint_written_here_loads_in_the_reference(ref, tmp_path):
    keys, blocks = _rows(2)
    cfg = _cfg()
    t = HostEmbTable(cfg)
    t.insert_or_assign(torch.from_numpy(keys), *(torch.from_numpy(b).reshape(-1) for b in blocks[:1]),
                       [torch.from_numpy(b).reshape(-1) for b in blocks[1:]])
    ours = str(tmp_path / "ours")
    checkpoint.save_table(os.path.join(ours, "tbl", "rank0"), t, cfg, None)
    m = ref.refmgr_new(b"tbl", DIM, 2, 64, 0.0, 1.0, -1, 0, 0)
    assert ref.refmgr_load(m, ours.encode(), 0) == 0
    back = str(tmp_path / "back")
    assert ref.refmgr_save(m, back.encode(), 0) == 0
    ref.refmgr_free(m)
    for a, b in zip(_sorted_table(os.path.join(ours, "tbl", "rank0")), _sorted_table(os.path.join(back, "tbl", "rank0"))):
        np.testing.assert_array_equal(a, b)
    for name, n in (("key", 2), ("embedding", 3), ("momentum1", 3), ("momentum2", 3)):
        a = np.fromfile(os.path.join(ours, "tbl", "rank0", name, "slice.attribute"), np.int64)
        b = np.fromfile(os.path.join(back, "tbl", "rank0", name, "slice.attribute"), np.int64)
        assert a.tolist() == b.tolist() and a.size == n
