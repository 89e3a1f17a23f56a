"""Checkpoints of the hybrid cache in the reference's on-disk layout
(torchrec_embcache/csrc/embedding_cache/embcache_manager.cpp: Save :342-389, WriteAttributeFile :423-458,
Load :460-530, admission / eviction state :824-947; driver torchrec_embcache/saver.py:63-107):

    <path>/<table>/rank<r>/key/slice.data                 int64 keys, host-table iteration order
    <path>/<table>/rank<r>/key/slice.attribute            int64 {8, count}
    <path>/<table>/rank<r>/embedding/slice.data           float32 [count, dim], same order as the keys
    <path>/<table>/rank<r>/embedding/slice.attribute      int64 {4, count, dim}
    <path>/<table>/rank<r>/momentum{1,2}/slice.{data,attribute}      like embedding, one per optimizer state
    <path>/<table>/rank<r>/admit_count/slice.attribute    int64 {8, count}            (admission enabled)
    <path>/<table>/rank<r>/admit_count/slice.data         int64 count per saved key, -1 = not in the count map
    <path>/<table>/rank<r>/evict_timestamp/slice.attribute          int64 {8, n}      (eviction enabled)
    <path>/<table>/rank<r>/evict_timestamp/slice_evict_key.data     int64 keys of the timestamp map
    <path>/<table>/rank<r>/evict_timestamp/slice_evict_ts.data      int64 timestamps, same order

All files are raw little-endian arrays, so a checkpoint written by the reference loads here and the other way
round.  One deviation, on purpose: the reference's chunked writers of the admission / eviction files skip the data
when there is exactly one record (their flush test is `i > 0 && ...`, :860,:904) while the attribute file says one;
here the record is written.

`Saver` mirrors torchrec_embcache/saver.py: a UTC timestamp directory per save, the latest one on load.
"""
from __future__ import annotations

import os
from datetime import datetime, timezone

import numpy as np
import torch

KEY_SIZE_MAX = 1 << 40
TIMESTAMP_FORMAT = "%Y%m%d%H%M%S"


def _write(path: str, array: np.ndarray) -> None:
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "wb") as f:
        f.write(np.ascontiguousarray(array).tobytes())


def _read_attr(path: str, n: int) -> np.ndarray:
    if not os.path.exists(path) or os.path.getsize(path) != 8 * n:
        raise RuntimeError(f"Read key attribute file error, file:{path}")
    return np.fromfile(path, dtype=np.int64)


def _read_i64(attr_path: str, data_path: str) -> np.ndarray:
    attr = _read_attr(attr_path, 2)
    count = int(attr[1])
    if count < 0 or count > KEY_SIZE_MAX:
        raise RuntimeError(f"Read key attribute file error, keys count is invalid:{count}, file:{attr_path}.")
    size = os.path.getsize(data_path) if os.path.exists(data_path) else -1
    if size != count * 8:
        raise RuntimeError(f"Key file bytes is not an integer multiple of type int64_t, key file:{data_path}")
    return np.fromfile(data_path, dtype=np.int64)


def _read_rows(prefix: str, name: str, count: int, dim: int) -> np.ndarray:
    attr = _read_attr(os.path.join(prefix, name, "slice.attribute"), 3)
    if int(attr[2]) != dim:
        raise RuntimeError(f"Embedding or momentum dim error, load data dim from attribute:{int(attr[2])}, current table "
                           f"dim:{dim}, file:{os.path.join(prefix, name, 'slice.attribute')}.")
    path = os.path.join(prefix, name, "slice.data")
    if os.path.getsize(path) < count * dim * 4:
        raise RuntimeError(f"Read data to file error, file:{path}")
    return np.fromfile(path, dtype=np.float32, count=count * dim).reshape(count, dim)


def save_table(prefix: str, host_table, cfg, feature_filter) -> None:
    """One table of one rank.  `host_table` is a HostEmbTable, `feature_filter` the table's FeatureFilter or None."""
    keys, embs, optims = host_table.export()
    count, dim = keys.numel(), int(cfg.emb_dim)
    _write(os.path.join(prefix, "key", "slice.data"), keys.numpy())
    _write(os.path.join(prefix, "key", "slice.attribute"), np.array([8, count], np.int64))
    _write(os.path.join(prefix, "embedding", "slice.data"), embs.numpy())
    _write(os.path.join(prefix, "embedding", "slice.attribute"), np.array([4, count, dim], np.int64))
    for i, o in enumerate(optims):
        _write(os.path.join(prefix, f"momentum{i + 1}", "slice.data"), o.numpy())
        _write(os.path.join(prefix, f"momentum{i + 1}", "slice.attribute"), np.array([4, count, dim], np.int64))
    aae = cfg.admit_and_evict_config
    if feature_filter is None:
        return
    if aae.is_admit_enabled():
        counts = feature_filter.GetCounts(keys.to(feature_filter.device)).cpu().numpy() if count else np.empty(0, np.int64)
        _write(os.path.join(prefix, "admit_count", "slice.attribute"), np.array([8, count], np.int64))
        _write(os.path.join(prefix, "admit_count", "slice.data"), counts)
    if aae.is_evict_enabled():
        tk, ts = feature_filter.timestamp_records()
        _write(os.path.join(prefix, "evict_timestamp", "slice.attribute"), np.array([8, tk.numel()], np.int64))
        _write(os.path.join(prefix, "evict_timestamp", "slice_evict_key.data"), tk.numpy())
        _write(os.path.join(prefix, "evict_timestamp", "slice_evict_ts.data"), ts.numpy())


def load_table(prefix: str, host_table, cfg, feature_filter) -> None:
    dim = int(cfg.emb_dim)
    keys = _read_i64(os.path.join(prefix, "key", "slice.attribute"), os.path.join(prefix, "key", "slice.data"))
    count = keys.size
    embs = _read_rows(prefix, "embedding", count, dim)
    optims = [_read_rows(prefix, f"momentum{i + 1}", count, dim) for i in range(int(cfg.optim_num))]
    host_table.insert_or_assign(torch.from_numpy(keys), torch.from_numpy(embs).reshape(-1),
                                [torch.from_numpy(o).reshape(-1) for o in optims])
    aae = cfg.admit_and_evict_config
    if feature_filter is None:
        return
    dev = feature_filter.device
    if aae.is_admit_enabled():
        counts = _read_i64(os.path.join(prefix, "admit_count", "slice.attribute"),
                           os.path.join(prefix, "admit_count", "slice.data"))
        if counts.size != count:
            raise RuntimeError("Failed to load key count info, vector size is not same between keys and counts.")
        feature_filter.load_feature_records(torch.from_numpy(keys).to(dev), torch.from_numpy(counts).to(dev))
    if aae.is_evict_enabled():
        attr = os.path.join(prefix, "evict_timestamp", "slice.attribute")
        tk = _read_i64(attr, os.path.join(prefix, "evict_timestamp", "slice_evict_key.data"))
        ts = _read_i64(attr, os.path.join(prefix, "evict_timestamp", "slice_evict_ts.data"))
        feature_filter.load_timestamp_records(torch.from_numpy(tk).to(dev), torch.from_numpy(ts).to(dev))


class Saver:
    """torchrec_embcache/saver.py:63-107 for a list of (manager, table module) pairs: every save goes to a new UTC
    timestamp directory under `path` (after the HBM cache rows were pushed to the host store), load reads the
    latest one."""

    def __init__(self, rank: int = 0):
        self.rank = int(rank)

    @staticmethod
    def is_timestamp_format(name: str) -> bool:
        try:
            datetime.strptime(name, TIMESTAMP_FORMAT)
            return True
        except ValueError:
            return False

    @staticmethod
    def get_latest_load_path(path: str) -> str:
        dirs = [d for d in os.listdir(path) if os.path.isdir(os.path.join(path, d)) and Saver.is_timestamp_format(d)]
        if not dirs:
            raise ValueError(f"expect a timestamp directory but empty in path:{path}")
        return os.path.join(os.path.realpath(path), max(dirs))

    def save(self, pairs, path: str, timestamp: str = None) -> str:
        """pairs: [(EmbcacheManager, table module with weights_dev / get_momentum())].  Returns the directory written.
        With several ranks pass the same `timestamp` on all of them (the reference broadcasts rank 0's)."""
        path = os.path.join(os.path.realpath(path), timestamp or datetime.now(tz=timezone.utc).strftime(TIMESTAMP_FORMAT))
        os.makedirs(path, exist_ok=True)
        for mgr, module in pairs:
            mgr.embedding_to_host(module.weights_dev.detach(), [m.detach() for m in module.get_momentum()])
            mgr.save(path, self.rank)
        return path

    def load(self, managers, path: str) -> str:
        path = self.get_latest_load_path(path)
        for mgr in managers:
            mgr.load(path, self.rank)
        return path
