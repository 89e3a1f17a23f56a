"""Hybrid-cache table interface: the policy tier of the reference's ``embcache_pybind`` module with its state in HBM.

Mirrors ``EmbConfig`` / ``AdmitAndEvictConfig`` / ``SwapInfo`` / ``EmbcacheManager``
(torchrec_embcache/src/torchrec_embcache/csrc/bind.cpp:19-115, embedding_cache/embcache_manager.cpp, common/common.h:55-110)
for the methods that decide WHERE a key lives: ``compute_swap_info(_async)``, ``statistics_key_count``,
``record_timestamp``, ``evict_features``, ``record_embedding_update_times``, ``remove_embedding_table_info``.
One SwapManager and (when admission or eviction is configured) one FeatureFilter per table, exactly as the
reference composes them (embcache_manager.cpp:42-63).

The host tier -- the DRAM key -> [w | m | v] row store behind ``embedding_lookup_async`` /
``embedding_update_async`` / ``embedding_to_host`` (emb_table/emb_table.h) -- is a C++ store inside the library
(`recsdk_host_table_*`); ``save`` / ``load`` write and read the reference's checkpoint layout
(recsdk_b200/checkpoint.py).  Keys and policy results are device tensors (the reference takes CPU tensors and returns
pinned ones); swapped rows cross in pinned host tensors as in the reference.
"""
from __future__ import annotations

import ctypes as C
import os
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from . import _lib, ops
from .tables import FeatureFilter, SwapManager

TABLE_NAME_LENGTH = 255


@dataclass
class AdmitAndEvictConfig:
    """common/common.h:55-83"""
    admit_threshold: int = -1
    not_admitted_default_value: float = 0.0
    evict_threshold: int = 0
    evict_step_interval: int = 0

    def is_admit_enabled(self) -> bool:
        return self.admit_threshold != -1

    def is_evict_enabled(self) -> bool:
        return self.evict_threshold != 0

    def is_feature_filter_enabled(self) -> bool:
        return self.is_admit_enabled() or self.is_evict_enabled()


@dataclass
class EmbConfig:
    """common/common.h:85-110.  The initializer fields describe the host store and are carried only."""
    table_name: str
    initializer_type: int = 0
    emb_dim: int = 0
    optim_num: int = 0
    cache_size: int = 0
    weight_init_min: float = 0.0
    weight_init_max: float = 0.0
    weight_init_mean: float = 0.0
    weight_init_stddev: float = 1.0
    admit_and_evict_config: AdmitAndEvictConfig = field(default_factory=AdmitAndEvictConfig)
    initializer_random_pool_size: int = -1
    seed: int = 0
    # capacity of the per-key admission / timestamp state kept in HBM (distinct keys tracked at once)
    filter_capacity: int = 1 << 22


@dataclass
class SwapInfo:
    """embcache_manager.h SwapInfo: per-table key lists, offsets concatenated over the tables."""
    swapout_keys: List[torch.Tensor]
    swapout_offs: torch.Tensor
    swapin_keys: List[torch.Tensor]
    swapin_offs: torch.Tensor
    batch_offs: torch.Tensor


@dataclass
class SwapinTensor:
    """embcache_manager.h SwapinTensor: pinned host tensors, tables one after the other."""
    swapin_embs: torch.Tensor
    swapin_optims: List[torch.Tensor]
    jagged_offs: torch.Tensor


class AsyncTask:
    """csrc/utils/async_task.h: the work runs on a pool thread; ``get()`` waits for it and re-raises its error."""

    def __init__(self, pool: ThreadPoolExecutor, fn):
        self._future = pool.submit(fn)

    def get(self):
        return self._future.result()


class HostEmbTable:
    """One table's host store (`recsdk_host_table_*`): AoS rows [w | m | v] keyed by int64, CPU tensors in and out
    (Embcache::EmbTable, emb_table/emb_table.h:32-52)."""

    def __init__(self, cfg: "EmbConfig"):
        self.emb_dim, self.optim_num = int(cfg.emb_dim), int(cfg.optim_num)
        init = int(getattr(cfg.initializer_type, "value", cfg.initializer_type))
        self._lib = _lib.load()
        self._h = self._lib.recsdk_host_table_create(self.emb_dim, self.optim_num, init, cfg.weight_init_min,
                                                     cfg.weight_init_max, cfg.weight_init_mean, cfg.weight_init_stddev,
                                                     int(cfg.seed), 0)
        if not self._h:
            raise RuntimeError(f"invalid host table configuration for {cfg.table_name}")

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.recsdk_host_table_destroy(self._h)
            self._h = None

    @staticmethod
    def _cpu(t: torch.Tensor, dtype) -> torch.Tensor:
        if t.is_cuda or t.dtype != dtype or not t.is_contiguous():
            raise RuntimeError("host table arguments are contiguous CPU tensors of the stated type")
        return t

    def _optim_ptrs(self, optims):
        if len(optims) != self.optim_num:
            raise RuntimeError("outOptims size is not equal to optimNum")
        ptrs = [self._cpu(o, torch.float32).data_ptr() for o in optims] + [None, None]
        return ptrs[0], ptrs[1]

    def size(self) -> int:
        return int(self._lib.recsdk_host_table_size(self._h))

    def find_or_insert(self, keys: torch.Tensor, out_embs: torch.Tensor, out_optims: Sequence[torch.Tensor]) -> None:
        n = self._cpu(keys, torch.int64).numel()
        if out_embs.numel() != n * self.emb_dim:
            raise RuntimeError("outEmbs has the wrong size")
        o1, o2 = self._optim_ptrs(out_optims)
        _lib.check(self._lib.recsdk_host_table_find_or_insert(self._h, keys.data_ptr(), n,
                                                              self._cpu(out_embs, torch.float32).data_ptr(), o1, o2),
                   "EmbTable.FindOrInsert")

    def insert_or_assign(self, keys: torch.Tensor, in_embs: torch.Tensor, in_optims: Sequence[torch.Tensor]) -> None:
        n = self._cpu(keys, torch.int64).numel()
        if in_embs.numel() != n * self.emb_dim:
            raise RuntimeError("inEmbs has the wrong size")
        o1, o2 = self._optim_ptrs(in_optims)
        _lib.check(self._lib.recsdk_host_table_insert_or_assign(self._h, keys.data_ptr(), n,
                                                                self._cpu(in_embs, torch.float32).data_ptr(), o1, o2),
                   "EmbTable.InsertOrAssign")

    def remove(self, keys: torch.Tensor) -> None:
        _lib.check(self._lib.recsdk_host_table_remove(self._h, self._cpu(keys, torch.int64).data_ptr(), keys.numel()),
                   "EmbTable.RemoveEmbedding")

    def export(self):
        """ForEachKey: (keys [n], embs [n, D], [optim [n, D]] ...) in the table's iteration order."""
        n = self.size()
        keys = torch.empty(n, dtype=torch.int64)
        arrays = [torch.empty((n, self.emb_dim), dtype=torch.float32) for _ in range(1 + self.optim_num)]
        ptrs = [a.data_ptr() for a in arrays] + [None, None]
        got = self._lib.recsdk_host_table_export(self._h, keys.data_ptr(), ptrs[0], ptrs[1], ptrs[2], n)
        if got != n:
            raise RuntimeError("host table changed while it was exported")
        return keys, arrays[0], arrays[1:]


def restore(unique_indices: torch.Tensor, unique_inverse: torch.Tensor, unique_offset: torch.Tensor,
            offsets_per_table: Sequence[int]) -> torch.Tensor:
    """embcache_pybind.restore (csrc/ops/restore.cpp:15-51): hash_indices[r] = unique_indices[unique_inverse[r] +
    unique_offset[t]] for the positions r of table t."""
    return ops.restore(unique_indices, unique_inverse, unique_offset, list(offsets_per_table))


def restore_async(unique_indices, unique_inverse, unique_offset, offsets_per_table) -> "AsyncResult":
    """The work is enqueued on the current stream; ``get()`` hands the device tensor over."""
    out = restore(unique_indices, unique_inverse, unique_offset, offsets_per_table)
    return AsyncResult(lambda: out)


class AsyncResult:
    """Stands in for the reference's AsyncTask (csrc/utils/async_task.h): work was enqueued on the current CUDA
    stream when the object was made; ``get()`` raises what the device reported and hands the result over."""

    def __init__(self, finish):
        self._finish = finish
        self._value = None
        self._done = False

    def get(self):
        if not self._done:
            self._value = self._finish()
            self._done = True
        return self._value


class EmbcacheManager:
    def __init__(self, emb_configs: Sequence[EmbConfig], need_accumulate_offset: bool = True, device="cuda"):
        if len(emb_configs) == 0:
            raise RuntimeError("ERROR, Size of embConfigs must > 0")
        for c in emb_configs:
            if len(c.table_name) > TABLE_NAME_LENGTH:
                raise RuntimeError("the length of table name is invalid.")
            if c.optim_num != emb_configs[0].optim_num:
                raise RuntimeError("optimNum must be the same for every table")
        self.emb_configs = list(emb_configs)
        self.emb_num = len(self.emb_configs)
        self.need_accumulate_offset = bool(need_accumulate_offset)
        self.device = torch.device(device)
        self.swap_managers: List[SwapManager] = []
        self.feature_filters: List[Optional[FeatureFilter]] = []
        for c in self.emb_configs:
            aae = c.admit_and_evict_config
            self.swap_managers.append(SwapManager(c.cache_size, 1 if aae.is_admit_enabled() else 0, device=self.device))
            self.feature_filters.append(
                FeatureFilter(c.table_name, aae.admit_threshold, aae.evict_threshold, aae.evict_step_interval,
                              capacity=c.filter_capacity, device=self.device)
                if aae.is_feature_filter_enabled() else None)
        self.swap_count = 0
        self.emb_update_count = 0
        self.optim_num = int(self.emb_configs[0].optim_num)
        # host (DRAM) tier: one key -> [w | m | v] row store per table (emb_table/emb_table.h)
        self.host_tables = [HostEmbTable(c) for c in self.emb_configs]
        self._evict_swap_count = [0] * self.emb_num
        self._pool = ThreadPoolExecutor(max_workers=2, thread_name_prefix="embcache")

    # ------------------------------------------------------------------ helpers
    def _tables(self, table_indices: Optional[Sequence[int]], n_offsets: int) -> List[int]:
        cur = list(table_indices) if table_indices else list(range(self.emb_num))
        if len(cur) + 1 != n_offsets:
            raise RuntimeError("tableIndices size+1 must be equal to offsetPerKey size")
        for idx in cur:
            if not 0 <= idx < self.emb_num:
                raise RuntimeError(f"table index {idx} is out of range [0, {self.emb_num})")
        return cur

    # ------------------------------------------------------------------ embcache_manager.cpp:89-185
    def compute_swap_info_async(self, batch_keys: torch.Tensor, jagged_offs: Sequence[int],
                                table_indices: Optional[Sequence[int]] = None) -> AsyncResult:
        """``batch_keys`` (int64, device, first-occurrence unique per table) is filtered IN PLACE like the
        reference's (not yet admitted keys become -1)."""
        if batch_keys.dtype != torch.int64:
            raise RuntimeError("batchKeys must be of type int64_t")
        if not batch_keys.is_contiguous():
            raise RuntimeError("batchKeys must be contiguous")
        offs = [int(o) for o in jagged_offs]
        cur = self._tables(table_indices, len(offs))
        n = batch_keys.numel()
        parts = []
        off_pre_sum = 0
        for i, idx in enumerate(cur):
            if offs[i] > n or offs[i + 1] > n:
                raise RuntimeError(f"offsetPerKey[{i}] is greater than keyNum")
            keys = batch_keys[offs[i]:offs[i + 1]]
            cfg = self.emb_configs[idx]
            if cfg.admit_and_evict_config.is_admit_enabled() and self.feature_filters[idx] is not None:
                self.feature_filters[idx].CountFilter(keys)
            sok, soo, sik, sio, bo, counts = self.swap_managers[idx].ComputeSwapInfoDevice(keys)
            parts.append((idx, sok, soo, sik, sio, bo, counts, off_pre_sum))
            if self.need_accumulate_offset:
                off_pre_sum += cfg.cache_size
        self.swap_count += 1

        def finish() -> SwapInfo:
            so_k, so_o, si_k, si_o, b_o = [], [], [], [], []
            for idx, sok, soo, sik, sio, bo, counts, shift in parts:
                self.swap_managers[idx].raise_if_error("ComputeSwapInfo")
                nin, nout = counts.tolist()
                so_k.append(sok[:nout])
                si_k.append(sik[:nin])
                so_o.append(soo[:nout] + shift)  # slots of table i are shifted by the cache sizes before it
                si_o.append(sio[:nin] + shift)
                b_o.append(bo)                   # batch offsets are table-local (embcache_manager.cpp:130-147)
            cat = (lambda xs: torch.cat(xs) if xs else torch.empty(0, dtype=torch.int64, device=self.device))
            return SwapInfo(so_k, cat(so_o), si_k, cat(si_o), cat(b_o))

        return AsyncResult(finish)

    def compute_swap_info(self, batch_keys, jagged_offs, table_indices=None) -> SwapInfo:
        return self.compute_swap_info_async(batch_keys, jagged_offs, table_indices).get()

    # ------------------------------------------------------------------ embcache_manager.cpp:777-822
    def statistics_key_count(self, batch_keys: torch.Tensor, offset: torch.Tensor, batch_key_counts: torch.Tensor,
                             table_index: int) -> None:
        if not 0 <= table_index < self.emb_num:
            raise RuntimeError(f"table index {table_index} is out of range [0, {self.emb_num}). embNum_={self.emb_num}")
        if not self.emb_configs[table_index].admit_and_evict_config.is_admit_enabled():
            return
        if offset.numel() <= table_index + 1:
            raise RuntimeError("param error, tableIndex need be smaller than offset length, but got equal or greater "
                               "than offset length.")
        have_counts = batch_key_counts is not None and batch_key_counts.numel() > 0
        if have_counts and batch_keys.numel() != batch_key_counts.numel():
            raise RuntimeError("batchKeys length should equal with batchKeyCounts length when batchKeyCounts is not "
                               "empty.")
        o = offset.tolist() if isinstance(offset, torch.Tensor) else list(offset)
        start, end = int(o[table_index]), int(o[table_index + 1])
        if end > batch_keys.numel():
            raise RuntimeError("offset exceeds the number of keys")
        f = self.feature_filters[table_index]
        if f is None:
            return
        f.StatisticsKeyCount(batch_keys[start:end], batch_key_counts[start:end] if have_counts else None)

    # ------------------------------------------------------------------ embcache_manager.cpp:663-688
    def record_timestamp(self, batch_keys: torch.Tensor, jagged_offs: Sequence[int], batch_timestamps: torch.Tensor,
                         table_indices: Optional[Sequence[int]] = None) -> None:
        offs = [int(o) for o in jagged_offs]
        cur = self._tables(table_indices, len(offs))
        for i, idx in enumerate(cur):
            f = self.feature_filters[idx]
            if self.emb_configs[idx].admit_and_evict_config.is_evict_enabled() and f is not None:
                f.RecordTimestamp(batch_keys[offs[i]:offs[i + 1]], batch_timestamps[offs[i]:offs[i + 1]])

    # ------------------------------------------------------------------ embcache_manager.cpp:690-715
    def evict_features(self) -> int:
        """Marks the cache slots of the keys the last evict scans collected as reusable; returns how many."""
        total = 0
        for i in range(self.emb_num):
            f = self.feature_filters[i]
            if not self.emb_configs[i].admit_and_evict_config.is_evict_enabled() or f is None:
                continue
            keys, count = f.GetEvictKeysDevice()
            self.swap_managers[i].RemoveKeys(keys, count)  # the count stays on the device: no synchronisation
            self._evict_swap_count[i] = self.swap_count  # evictFeatureRecord_.SetSwapCount (embcache_manager.cpp:710)
            total += int(count.item())
            # an eviction round turns entries of both tables into tombstones: rebuild them when they pile up
            f.compact_if_needed()
            self.swap_managers[i].compact_if_needed()
        return total

    def evicted_keys(self, table_index: int) -> torch.Tensor:
        f = self.feature_filters[table_index]
        return f.GetEvictKeys() if f is not None else torch.empty(0, dtype=torch.int64, device=self.device)

    def remove_embedding_table_info(self) -> None:
        """RemoveEmbeddingTableInfo (embcache_manager.cpp:754-775): the rows of the evicted keys leave the host store
        and the evict record is cleared."""
        for idx, f in enumerate(self.feature_filters):
            if f is None:
                continue
            keys = f.GetEvictKeys()
            if keys.numel() == 0:
                continue
            self.host_tables[idx].remove(keys.to("cpu").contiguous())
            f.ClearEvictInfo()
            self._evict_swap_count[idx] = 0

    def _need_evict_embedding_table(self) -> bool:
        """NeedEvictEmbeddingTable (:734-752): some table has evicted keys on record and the update count has reached
        the swap count at which evict_features recorded them."""
        for idx, f in enumerate(self.feature_filters):
            if f is None or not self.emb_configs[idx].admit_and_evict_config.is_evict_enabled():
                continue
            if self._evict_swap_count[idx] == self.emb_update_count and int(f.GetEvictKeysDevice()[1].item()) > 0:
                return True
        return False

    def record_embedding_update_times(self) -> None:
        self.emb_update_count += 1
        if self._need_evict_embedding_table():
            self.remove_embedding_table_info()

    # ------------------------------------------------------------------ host tier (embcache_manager.cpp:196-318)
    def _host_keys(self, key_lists, table_indices) -> List[int]:
        cur = list(table_indices) if table_indices else list(range(self.emb_num))
        if len(cur) != len(key_lists):
            raise RuntimeError("tableIndices size must be equal to swapinKeys size")
        return cur

    def embedding_lookup(self, swapin_keys: Sequence[torch.Tensor], table_indices=None) -> "SwapinTensor":
        """EmbeddingLookup (:196-235): FindOrInsert of every table's swap-in keys in the host store, rows copied out
        into pinned SoA tensors laid out table after table (``jagged_offs`` in elements)."""
        cur = self._host_keys(swapin_keys, table_indices)
        keys_h = [k.detach().to("cpu", torch.int64).contiguous() for k in swapin_keys]
        offs = [0]
        for k, idx in zip(keys_h, cur):
            offs.append(offs[-1] + k.numel() * self.emb_configs[idx].emb_dim)
        total = offs[-1]
        embs = torch.empty(total, dtype=torch.float32).pin_memory()
        optims = [torch.empty(total, dtype=torch.float32).pin_memory() for _ in range(self.optim_num)]
        for i, (k, idx) in enumerate(zip(keys_h, cur)):
            self.host_tables[idx].find_or_insert(k, embs[offs[i]:offs[i + 1]], [o[offs[i]:offs[i + 1]] for o in optims])
        return SwapinTensor(embs, optims, torch.tensor(offs, dtype=torch.int64).pin_memory())

    def embedding_lookup_async(self, swap_info: SwapInfo, table_indices=None) -> "AsyncTask":
        keys = [k.detach().to("cpu", torch.int64) for k in swap_info.swapin_keys]  # captured by value, like the reference
        return AsyncTask(self._pool, lambda: self.embedding_lookup(keys, table_indices))

    def embedding_update(self, swapout_keys: Sequence[torch.Tensor], swapout_embs: torch.Tensor,
                         swapout_optims: Sequence[torch.Tensor], table_indices=None) -> None:
        """EmbeddingUpdate (:245-282): InsertOrAssign of the swapped-out rows, then the bookkeeping of
        record_embedding_update_times (rows of evicted keys leave the host store when the update count reaches the
        swap count at which they were evicted)."""
        if len(swapout_optims) != self.optim_num:
            raise RuntimeError("Expected embedConfig.optimNum == (int32_t)swapoutOptims.size() to be true")
        for o in swapout_optims:
            if o.numel() != swapout_embs.numel() or o.dtype != torch.float32:
                raise RuntimeError("swapoutOptims must be float32 and as large as swapoutEmbs")
        if swapout_embs.dtype != torch.float32:
            raise RuntimeError("swapoutEmbs must be float32")
        cur = self._host_keys(swapout_keys, table_indices)
        embs = swapout_embs.detach().reshape(-1).to("cpu").contiguous()
        optims = [o.detach().reshape(-1).to("cpu").contiguous() for o in swapout_optims]
        off = 0
        for k, idx in zip(swapout_keys, cur):
            kh = k.detach().to("cpu", torch.int64).contiguous()
            n = kh.numel() * self.emb_configs[idx].emb_dim
            self.host_tables[idx].insert_or_assign(kh, embs[off:off + n], [o[off:off + n] for o in optims])
            off += n
        self.record_embedding_update_times()

    def embedding_update_async(self, swap_info: SwapInfo, swapout_embs: torch.Tensor,
                               swapout_optims: Sequence[torch.Tensor], table_indices=None) -> "AsyncTask":
        keys = [k.detach().to("cpu", torch.int64) for k in swap_info.swapout_keys]
        embs = swapout_embs.detach().to("cpu")
        optims = [o.detach().to("cpu") for o in swapout_optims]
        return AsyncTask(self._pool, lambda: self.embedding_update(keys, embs, optims, table_indices))

    def embedding_to_host(self, weights_dev: torch.Tensor, momentum_devs: Sequence[torch.Tensor]) -> None:
        """Embedding2Host (:284-318): every occupied cache slot's row goes to the host store under the key that holds
        the slot.  ``weights_dev`` is the flat cache of all tables, table i's part cache_size_i * emb_dim_i long."""
        for m in momentum_devs:
            if m.numel() != weights_dev.numel() or m.dtype != torch.float32:
                raise RuntimeError("momentumDevs must be float32 and as large as weightsDev")
        if weights_dev.dtype != torch.float32:
            raise RuntimeError("weightsDev must be float32")
        w = weights_dev.detach().reshape(-1)
        ms = [m.detach().reshape(-1) for m in momentum_devs]
        off = 0
        for idx, cfg in enumerate(self.emb_configs):
            sm = self.swap_managers[idx]
            start, end = sm.GetMemStartOffset(), sm.GetOccupiedNum()
            lo, hi = off + start * cfg.emb_dim, off + end * cfg.emb_dim
            keys = sm.slot_keys()[start:end].to("cpu").contiguous()
            self.host_tables[idx].insert_or_assign(keys, w[lo:hi].to("cpu").contiguous(),
                                                   [m[lo:hi].to("cpu").contiguous() for m in ms])
            off += cfg.cache_size * cfg.emb_dim

    # ------------------------------------------------------------------ checkpoints (embcache_manager.cpp:342-389,
    # 423-458, 460-530, 824-947): <path>/<table>/rank<r>/{key,embedding,momentum1,momentum2,admit_count,
    # evict_timestamp}/slice.{data,attribute}
    def save(self, path: str, rank: int) -> None:
        from . import checkpoint

        if os.path.abspath(path) != path:
            raise RuntimeError(f"File path is invalid, it is not an absolute path:{path}.")
        for idx, cfg in enumerate(self.emb_configs):
            checkpoint.save_table(os.path.join(path, cfg.table_name, f"rank{rank}"), self.host_tables[idx], cfg,
                                  self.feature_filters[idx])

    def load(self, path: str, rank: int) -> None:
        from . import checkpoint

        for idx, cfg in enumerate(self.emb_configs):
            checkpoint.load_table(os.path.join(path, cfg.table_name, f"rank{rank}"), self.host_tables[idx], cfg,
                                  self.feature_filters[idx])
