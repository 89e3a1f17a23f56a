"""Hybrid-cache table interface: the policy tier of the reference's ``embcache_pybind`` module with its state in HBM.

Mirrors ``EmbConfig`` / ``AdmitAndEvictConfig`` / ``SwapInfo`` / ``EmbcacheManager``
(torchrec_embcache/src/torchrec_embcache/csrc/bind.cpp:19-115, embedding_cache/embcache_manager.cpp, common/common.h:55-110)
for the methods that decide WHERE a key lives: ``compute_swap_info(_async)``, ``statistics_key_count``,
``record_timestamp``, ``evict_features``, ``record_embedding_update_times``, ``remove_embedding_table_info``.
One SwapManager and (when admission or eviction is configured) one FeatureFilter per table, exactly as the
reference composes them (embcache_manager.cpp:42-63).

The host tier -- the DRAM key/value store behind ``embedding_lookup_async`` / ``embedding_update_async`` /
``embedding_to_host`` / ``save`` / ``load`` -- is not part of this package; those methods raise
NotImplementedError.  Keys and results are device tensors (the reference takes CPU tensors and returns pinned
ones); nothing here synchronises except the ``get()`` of a result.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

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
            total += int(count.item())
        return total

    def evicted_keys(self, table_index: int) -> torch.Tensor:
        f = self.feature_filters[table_index]
        return f.GetEvictKeys() if f is not None else torch.empty(0, dtype=torch.int64, device=self.device)

    def remove_embedding_table_info(self) -> None:
        """The reference drops the evicted keys' host rows here and clears the evict record
        (embcache_manager.cpp RemoveEmbeddingTableInfo); with no host tier only the record is cleared."""
        for f in self.feature_filters:
            if f is not None:
                f.ClearEvictInfo()

    def record_embedding_update_times(self) -> None:
        self.emb_update_count += 1

    # ------------------------------------------------------------------ host tier (not part of this package)
    def _host_tier(self, name: str):
        raise NotImplementedError(f"EmbcacheManager.{name}: the host (DRAM) embedding store is not part of recsdk_b200; "
                                  "move rows with gather_embs / scatter_update_embs of the table module")

    def embedding_lookup_async(self, *a, **k):
        self._host_tier("embedding_lookup_async")

    def embedding_update_async(self, *a, **k):
        self._host_tier("embedding_update_async")

    def embedding_to_host(self, *a, **k):
        self._host_tier("embedding_to_host")

    def save(self, *a, **k):
        self._host_tier("save")

    def load(self, *a, **k):
        self._host_tier("load")
