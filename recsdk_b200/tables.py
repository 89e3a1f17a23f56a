"""HBM-resident key tables behind the reference's host-side interfaces.

``IdsMapper``      mirrors ``torch.classes.hybrid.IdsMapper``
                   (hybrid_torchrec/src/ids_process/ids_mapper.h:30-102, bind_torch_lib.cpp:9-19)
``SwapManager``    mirrors ``Embcache::SwapManager``
                   (torchrec_embcache/csrc/embedding_cache/swap_manager.h:28-55)
``FeatureFilter``  mirrors ``Embcache::FeatureFilter``
                   (torchrec_embcache/csrc/feature_filter/feature_filter.h:26-60)

Same method names, argument meaning and error behaviour; tensors are CUDA
tensors and all state lives in device memory owned by these objects.  Methods
that the reference implements with a raise (negative key, table full, cache
too small) synchronise on a device status block and raise RuntimeError with the
reference's message; pass ``check=False`` to skip the synchronisation and call
``raise_if_error()`` later.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib
from .ops import _chk, _ptr, _stream, _workspace, new_status, raise_on_status


def _pow2_at_least(x: int) -> int:
    p = 16
    while p < x:
        p <<= 1
    return p


class IdsMapper:
    """key -> slot with first-come slot numbering; state in HBM.

    ``initMaxIndex`` slots are provisioned.  Unlike the host reference, which lets
    the map grow past ``initMaxIndex`` when ``onlyDeviceMem`` is False, this mapper
    never grows: running out of slots is an error in both modes.
    """

    def __init__(self, initMaxIndex: int, onlyDeviceMem: bool = True, device="cuda", load_factor: float = 0.5):
        self._lib = _lib.load()
        self.device = torch.device(device)
        self.initMaxIndex = int(initMaxIndex)
        self.onlyDeviceMem = bool(onlyDeviceMem)
        cap = _pow2_at_least(int(self.initMaxIndex / load_factor) + 1)
        self._table = torch.empty(cap * 2, dtype=torch.int64, device=self.device)
        self._slot_key = torch.empty(self.initMaxIndex, dtype=torch.int64, device=self.device)
        self._mark = torch.empty(self.initMaxIndex, dtype=torch.int32, device=self.device)
        self._counters = torch.zeros(4, dtype=torch.int64, device=self.device)
        # the status block with one more word behind it: the unique count of ids2indices_unique, so that status and
        # count come back in ONE device-to-host read
        self._status_and_count = torch.zeros(_lib.STATUS_WORDS + 1, dtype=torch.int64, device=self.device)
        self._status = self._status_and_count[:_lib.STATUS_WORDS]
        self._c = _lib.MapperT(_ptr(self._table), cap, _ptr(self._slot_key), _ptr(self._mark), _ptr(self._counters),
                               self.initMaxIndex, int(self.onlyDeviceMem))
        self._ws: Optional[torch.Tensor] = None
        with torch.cuda.device(self.device):
            _lib.check(self._lib.recsdk_mapper_init(C.byref(self._c), _stream()), "recsdk_mapper_init")

    # -- helpers
    def _workspace_for(self, n: int) -> torch.Tensor:
        need = self._lib.recsdk_mapper_workspace_bytes(n)
        if self._ws is None or self._ws.numel() < need:
            self._ws = _workspace(need, self.device)
        return self._ws

    def raise_if_error(self, where: str = "IdsMapper") -> None:
        raise_on_status(self._status, where)

    def size(self) -> int:
        """Number of keys mapped so far (maxIndex)."""
        return int(self._counters[0].item())

    def slot_keys(self) -> torch.Tensor:
        """indice2id: key of every assigned slot."""
        return self._slot_key[: self.size()]

    # -- reference interface
    def ids2indices_unique(self, ids: torch.Tensor, check: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(hash_indices, unique (sorted), inverse) -- ids_mapper.cpp:27-61."""
        _chk(ids, torch.int64, "globalIds")
        n = ids.numel()
        hi = torch.empty(n, dtype=torch.int64, device=self.device)
        uq = torch.empty(max(n, 1), dtype=torch.int64, device=self.device)
        inv = torch.empty(max(n, 1), dtype=torch.int64, device=self.device)
        cnt = self._status_and_count[_lib.STATUS_WORDS:]
        ws = self._workspace_for(n)
        _lib.check(self._lib.recsdk_mapper_ids2indices_unique(C.byref(self._c), _ptr(ids), n, _ptr(hi), _ptr(uq),
                                                              _ptr(inv), _ptr(cnt), _ptr(self._status), _ptr(ws),
                                                              ws.numel(), _stream()), "ids2indices_unique")
        host = self._status_and_count.tolist()  # the one synchronisation of the call
        if check and host[0] != 0:
            self.raise_if_error("ids2indices_unique")
        u = int(host[_lib.STATUS_WORDS])
        return hi, uq[:u], inv[:n]

    def ids2indices_unique_out(self, ids, hash_indices, offset, unique, unique_ids, unique_inverse, unique_offset,
                               table_id: int, check: bool = True) -> None:
        """ids_mapper.cpp:63-174.  ``offset`` may be a CPU tensor/list (segment bounds are host scalars here)."""
        _chk(ids, torch.int64, "globalIds")
        _chk(hash_indices, torch.int64, "hashIndices")
        _chk(unique, torch.int64, "unique")
        _chk(unique_ids, torch.int64, "uniqueIds")
        _chk(unique_inverse, torch.int64, "uniqueInverse")
        _chk(unique_offset, torch.int64, "uniqueOffset")
        offs = offset.tolist() if isinstance(offset, torch.Tensor) else list(offset)
        if not (len(offs) - 1 > table_id):
            raise RuntimeError("offset must be equal to table size + 1")
        start, end = int(offs[table_id]), int(offs[table_id + 1])
        ws = self._workspace_for(end - start)
        _lib.check(self._lib.recsdk_mapper_unique_out(C.byref(self._c), _ptr(ids), _ptr(hash_indices), start,
                                                      end - start, _ptr(unique), _ptr(unique_ids),
                                                      _ptr(unique_inverse), _ptr(unique_offset), table_id,
                                                      _ptr(self._status), _ptr(ws), ws.numel(), _stream()),
                   "ids2indices_unique_out")
        if check:
            self.raise_if_error("ids2indices_unique_out")

    @staticmethod
    def parallel_ids2indices_unique_out(mappers: Sequence["IdsMapper"], ids, hash_indices, offsets, unique,
                                        unique_ids, unique_inverse, unique_offset, check: bool = True) -> None:
        """ids_mapper.cpp:227-285: one mapper per table; tables are enqueued back to back on the stream."""
        offs = offsets.tolist() if isinstance(offsets, torch.Tensor) else list(offsets)
        for t, m in enumerate(mappers):
            m.ids2indices_unique_out(ids, hash_indices, offs, unique, unique_ids, unique_inverse, unique_offset, t,
                                     check=False)
        if check:
            for m in mappers:
                m.raise_if_error("parallel_ids2indices_unique_out")


class _KeyTableCare:
    """Load statistics and tombstone compaction shared by the three key tables (`self._table`, `self._cap`,
    `self._entry_words`, `self._max_live`, `self._status`, `self._lib`, `self.device`)."""

    def table_stats(self):
        """(live entries, tombstones, longest displacement, capacity) of the key table; synchronises."""
        st = torch.zeros(4, dtype=torch.int64, device=self.device)
        _lib.check(self._lib.recsdk_key_table_stats(_ptr(self._table), self._cap, self._entry_words, _ptr(st), _stream()),
                   "recsdk_key_table_stats")
        live, tomb, disp, _ = st.tolist()
        return live, tomb, disp, self._cap

    def compact(self) -> None:
        """Rebuild the key table without tombstones (stream-ordered; nothing else may run on the table meanwhile)."""
        need = self._lib.recsdk_key_table_rebuild_workspace_bytes(self._max_live, self._entry_words)
        ws = _workspace(need, self.device)
        _lib.check(self._lib.recsdk_key_table_rebuild(_ptr(self._table), self._cap, self._entry_words, self._max_live,
                                                      _ptr(self._status), _ptr(ws), ws.numel(), _stream()),
                   "recsdk_key_table_rebuild")

    def compact_if_needed(self, threshold: float = 0.75) -> bool:
        """Compacts when live + tombstones exceed `threshold` of the capacity (one host read).  The callers that own
        a natural point for it (after an eviction round, every so many slot-policy steps) call this themselves."""
        live, tomb, _, cap = self.table_stats()
        if tomb > 0 and live + tomb > threshold * cap:
            self.compact()
            return True
        return False


class SwapManager(_KeyTableCare):
    """Slot policy of the HBM cache (hit / append / clock-sweep replacement)."""

    def __init__(self, cacheSize: int, memStartOffset: int = 0, device="cuda", load_factor: float = 0.5):
        self._lib = _lib.load()
        self.device = torch.device(device)
        self.cacheSize = int(cacheSize)
        self.memStartOffset = int(memStartOffset)
        cap = _pow2_at_least(int(self.cacheSize / load_factor) + 1)
        self._table = torch.empty(cap * 2, dtype=torch.int64, device=self.device)
        self._slot_key = torch.empty(self.cacheSize, dtype=torch.int64, device=self.device)
        self._slot_version = torch.empty(self.cacheSize, dtype=torch.int64, device=self.device)
        self._counters = torch.zeros(4, dtype=torch.int64, device=self.device)
        self._status = new_status(self.device)
        self._c = _lib.SwapT(_ptr(self._table), cap, _ptr(self._slot_key), _ptr(self._slot_version),
                             _ptr(self._counters), self.cacheSize, self.memStartOffset)
        self._ws: Optional[torch.Tensor] = None
        self._cap, self._entry_words, self._max_live = cap, 2, self.cacheSize
        self._calls_since_check = 0
        with torch.cuda.device(self.device):
            _lib.check(self._lib.recsdk_swap_init(C.byref(self._c), _stream()), "recsdk_swap_init")

    def raise_if_error(self, where: str = "SwapManager") -> None:
        raise_on_status(self._status, where)

    def ComputeSwapInfoDevice(self, keys: torch.Tensor):
        """Device-resident result, no synchronisation: (swapout_keys[n], swapout_offs[n], swapin_keys[n],
        swapin_offs[n], batch_offs[n], counts[2] = {n_swapin, n_swapout})."""
        _chk(keys, torch.int64, "keys")
        n = keys.numel()
        dev = self.device
        m = max(n, 1)
        bo, sik, sio, sok, soo = (torch.empty(m, dtype=torch.int64, device=dev) for _ in range(5))
        counts = torch.zeros(2, dtype=torch.int64, device=dev)
        need = self._lib.recsdk_swap_workspace_bytes(n, self.cacheSize)
        if self._ws is None or self._ws.numel() < need:
            self._ws = _workspace(need, dev)
        _lib.check(self._lib.recsdk_swap_compute(C.byref(self._c), _ptr(keys), n, _ptr(bo), _ptr(sik), _ptr(sio),
                                                 _ptr(sok), _ptr(soo), _ptr(counts), _ptr(self._status),
                                                 _ptr(self._ws), self._ws.numel(), _stream()), "ComputeSwapInfo")
        return sok, soo, sik, sio, bo[:n], counts

    def ComputeSwapInfo(self, keys: torch.Tensor):
        """(swapoutKeys, swapoutOffs, swapinKeys, swapinOffs, batchOffs) -- swap_manager.cpp:32-139.
        Raises RuntimeError("cacheSize_ too small") like the reference."""
        sok, soo, sik, sio, bo, counts = self.ComputeSwapInfoDevice(keys)
        self.raise_if_error("ComputeSwapInfo")
        nin, nout = counts.tolist()
        self._calls_since_check += 1
        if self._calls_since_check >= 256:  # replacement and RemoveKeys leave tombstones: look now and then
            self._calls_since_check = 0
            self.compact_if_needed()
        return sok[:nout], soo[:nout], sik[:nin], sio[:nin], bo

    def RemoveKeys(self, keys: torch.Tensor, n_keys_dev: Optional[torch.Tensor] = None) -> None:
        _chk(keys, torch.int64, "keys")
        _lib.check(self._lib.recsdk_swap_remove(C.byref(self._c), _ptr(keys), keys.numel(), _ptr(n_keys_dev),
                                                _stream()), "RemoveKeys")

    def GetOccupiedNum(self) -> int:
        return int(self._counters[0].item())

    def GetMemStartOffset(self) -> int:
        return self.memStartOffset

    def slot_keys(self) -> torch.Tensor:
        """Key of every slot up to the occupied count (cache_[off].key, swap_manager.h:41-54); slots freed by
        RemoveKeys keep the key they last held, as in the reference."""
        return self._slot_key[: self.GetOccupiedNum()]

    def GetKey(self, off: int) -> int:
        occ = self.GetOccupiedNum()
        if not (0 <= off < occ):
            raise RuntimeError(f"off is out of bounds: {off}, occupiedNum: {occ}")
        return int(self._slot_key[off].item())


class FeatureFilter(_KeyTableCare):
    """Count-based admission and timestamp eviction, per-key state in HBM.

    ``capacity`` bounds the number of distinct keys tracked at once (admitted or not)."""

    def __init__(self, tableName: str, admitThreshold: int = -1, evictThreshold: int = 0, evictStepInterval: int = 0,
                 capacity: int = 1 << 20, device="cuda", load_factor: float = 0.5, evict_list_capacity: int = 0):
        self._lib = _lib.load()
        self.device = torch.device(device)
        self.tableName = tableName
        cap = _pow2_at_least(int(capacity / load_factor) + 1)
        self._table = torch.empty(cap * 4, dtype=torch.int64, device=self.device)
        self._counters = torch.zeros(4, dtype=torch.int64, device=self.device)
        self._status = new_status(self.device)
        self._cap, self._entry_words, self._max_live = cap, 4, int(capacity)
        self._evict_cap = int(evict_list_capacity or capacity)
        self._evict_keys = torch.empty(self._evict_cap, dtype=torch.int64, device=self.device)
        self._c = _lib.FilterT(_ptr(self._table), cap, _ptr(self._counters), int(admitThreshold), int(evictThreshold),
                               int(evictStepInterval))
        self._ws: Optional[torch.Tensor] = None
        with torch.cuda.device(self.device):
            _lib.check(self._lib.recsdk_filter_init(C.byref(self._c), _stream()), "recsdk_filter_init")

    def IsAdmitEnabled(self) -> bool:
        return self._c.admit_threshold != -1

    def raise_if_error(self, where: str = "FeatureFilter") -> None:
        raise_on_status(self._status, where)

    def StatisticsKeyCount(self, keys: torch.Tensor, counts: Optional[torch.Tensor] = None) -> None:
        _chk(keys, torch.int64, "batchKeys")
        if counts is not None and counts.numel() > 0:
            _chk(counts, torch.int64, "batchKeyCounts")
            if counts.numel() != keys.numel():
                raise RuntimeError("batchKeys length should equal with batchKeyCounts length when batchKeyCounts "
                                   "is not empty.")
        else:
            counts = None
        _lib.check(self._lib.recsdk_filter_statistics(C.byref(self._c), _ptr(keys), _ptr(counts), keys.numel(),
                                                      _ptr(self._status), _stream()), "StatisticsKeyCount")

    def CountFilter(self, keys: torch.Tensor) -> torch.Tensor:
        """In place: keys not admitted yet become -1 (feature_filter.cpp:140-160)."""
        _chk(keys, torch.int64, "featureData")
        _lib.check(self._lib.recsdk_filter_count_filter(C.byref(self._c), _ptr(keys), keys.numel(), _stream()),
                   "CountFilter")
        return keys

    def RecordTimestamp(self, keys: torch.Tensor, timestamps: torch.Tensor) -> None:
        _chk(keys, torch.int64, "featureData")
        _chk(timestamps, torch.int64, "timestampData")
        n = keys.numel()
        need = self._lib.recsdk_filter_workspace_bytes(n)
        if self._ws is None or self._ws.numel() < need:
            self._ws = _workspace(need, self.device)
        _lib.check(self._lib.recsdk_filter_record_timestamp(C.byref(self._c), _ptr(keys), _ptr(timestamps), n,
                                                            _ptr(self._evict_keys), self._evict_cap,
                                                            _ptr(self._status), _ptr(self._ws), self._ws.numel(),
                                                            _stream()), "RecordTimestamp")

    def GetEvictKeysDevice(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(evict key buffer, device count) without synchronising."""
        return self._evict_keys, self._counters[2:3]

    def GetEvictKeys(self) -> torch.Tensor:
        """Keys collected by the evict scans since the last ClearEvictInfo (order unspecified, as in the reference)."""
        self.raise_if_error("FeatureEvict")
        n = int(self._counters[2].item())
        return self._evict_keys[:n]

    def ClearEvictInfo(self) -> None:
        _lib.check(self._lib.recsdk_filter_clear_evict(C.byref(self._c), _stream()), "ClearEvictInfo")

    def timestamp_records(self):
        """(keys, timestamps) of every key in the timestamp map (GetFeatureTimestampMap, feature_filter.h), read
        back from the table; order unspecified.  Synchronises."""
        t = self._table.view(-1, 4).cpu()
        sel = (t[:, 0] >= 0) & (t[:, 2] != torch.iinfo(torch.int64).min)
        return t[sel, 0].contiguous(), t[sel, 2].contiguous()

    def load_feature_records(self, keys: torch.Tensor, counts: torch.Tensor) -> None:
        """LoadFeatureRecords (feature_filter.cpp:92-100) on a fresh filter: count[key] = counts[i].  Keys saved
        with -1 (not in the count map when the checkpoint was written) stay absent."""
        keep = counts >= 0
        if bool(keep.any()):
            self.StatisticsKeyCount(keys[keep].contiguous(), counts[keep].contiguous())

    def load_timestamp_records(self, keys: torch.Tensor, timestamps: torch.Tensor) -> None:
        """LoadTimestampRecords (feature_filter.cpp:102-110): timestamp[key] = ts; the latest-timestamp and
        batch counters stay as they are, as in the reference."""
        if keys.numel() == 0:
            return
        before = self._counters[:2].clone()
        saved_interval = self._c.evict_step_interval
        self._c.evict_step_interval = 0  # no evict scan while loading
        try:
            self.RecordTimestamp(keys, timestamps)
        finally:
            self._c.evict_step_interval = saved_interval
        self._counters[:2].copy_(before)

    def GetCounts(self, keys: torch.Tensor) -> torch.Tensor:
        """count of each key, -1 where the key is not in the count map."""
        _chk(keys, torch.int64, "keys")
        out = torch.empty(keys.numel(), dtype=torch.int64, device=self.device)
        _lib.check(self._lib.recsdk_filter_count_of(C.byref(self._c), _ptr(keys), keys.numel(), _ptr(out), _stream()),
                   "GetCounts")
        return out
