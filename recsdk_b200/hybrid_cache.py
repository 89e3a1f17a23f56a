"""Hash-keyed embedding table larger than its HBM cache: rows live in the host store, the rows of the keys in flight
live in an HBM cache of ``cache_size`` slots, and every step swaps rows between the two.

The step the reference's pipeline runs per batch (torchrec_embcache/distributed/train_pipeline.py:445-561 swap-out /
swap-in around the lookup, :591-735 the overlapped schedule; torchrec_embcache/distributed/embedding_bag.py:651-655
unique keys -> compute_swap_info -> restore):

    keys (with duplicates) -> first-occurrence unique + inverse
    admission statistics / timestamps (FeatureFilter), slot policy (SwapManager)        -> SwapInfo
    swap-out: gather rows [w | m | v] at swapout_offs -> pinned host buffers (copy stream) -> host store InsertOrAssign
    swap-in : host store FindOrInsert (new keys get the initializer) -> pinned -> H2D (copy stream) -> scatter at
              swapin_offs
    lookup  : pooled gather over the cache with batch_offs[inverse] as indices; backward updates the cache rows

The device work of one swap is two row kernels per array (`recsdk_gather_rows` / `recsdk_scatter_rows`, bulk
asynchronous copies) and ONE asynchronous copy per array and direction; the host-store work runs on the manager's
pool thread while the GPU proceeds.  Not the reference's 4-6 batch software pipeline: swaps of consecutive batches are
not overlapped with each other here.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import ops
from .embcache import EmbcacheManager, EmbConfig
from .tbe import EmbOptimType, HybridSplitTableBatchedEmbeddingBagsCodegen, PoolingMode


class HybridCacheEmbeddingBag:
    """Tables of equal dim behind one flat HBM cache (table i's slots are shifted by the cache sizes before it)."""

    def __init__(self, emb_configs: Sequence[EmbConfig], optimizer: EmbOptimType = EmbOptimType.ADAM,
                 pooling_mode: PoolingMode = PoolingMode.SUM, device="cuda", **optimizer_kwargs):
        self.device = torch.device(device)
        self.cfgs = list(emb_configs)
        dims = {c.emb_dim for c in self.cfgs}
        if len(dims) != 1:
            raise ValueError("Mixed dimensions are not supported.")
        self.dim = dims.pop()
        self.mgr = EmbcacheManager(self.cfgs, need_accumulate_offset=True, device=self.device)
        total_slots = sum(c.cache_size for c in self.cfgs)
        # one table of all cache slots; every feature reads it through slot numbers that are already shifted
        self.module = HybridSplitTableBatchedEmbeddingBagsCodegen(
            [(total_slots, self.dim)], feature_table_map=[0] * len(self.cfgs), optimizer=optimizer,
            pooling_mode=pooling_mode, device=self.device, **optimizer_kwargs)
        self.optim_num = self.mgr.optim_num
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self.swap_events: List[tuple] = []  # (label, start, stop) CUDA events of the copies, for overlap evidence
        self._pending_update = None

    # ------------------------------------------------------------------ one batch
    def lookup_slots(self, keys_per_table: Sequence[torch.Tensor], timestamps: Optional[Sequence[torch.Tensor]] = None):
        """keys_per_table[i]: the raw int64 keys of table i's bags (duplicates allowed).  Runs admission statistics,
        timestamps, the slot policy and the swap; returns (indices [N] = cache slot of every key occurrence,
        n_per_table)."""
        dev = self.device
        uniq, inv, offs = [], [], [0]
        for k in keys_per_table:
            u, i = _first_occurrence_unique(k)
            uniq.append(u)
            inv.append(i)
            offs.append(offs[-1] + u.numel())
        batch_keys = torch.cat(uniq) if uniq else torch.empty(0, dtype=torch.int64, device=dev)
        offs_t = torch.tensor(offs, dtype=torch.int64, device=dev)
        for i in range(len(self.cfgs)):
            self.mgr.statistics_key_count(batch_keys, offs_t, None, i)
        if timestamps is not None:
            ts = torch.cat([t[_first_positions(k)] for t, k in zip(timestamps, keys_per_table)])
            self.mgr.record_timestamp(batch_keys, offs, ts)
        info = self.mgr.compute_swap_info(batch_keys, offs)
        self.swap(info)
        slots, n_per_table = [], []
        for i, iv in enumerate(inv):
            slots.append(info.batch_offs[offs[i]:offs[i + 1]][iv] + self._shift(i))
            n_per_table.append(iv.numel())
        return torch.cat(slots) if slots else torch.empty(0, dtype=torch.int64, device=dev), n_per_table

    def _shift(self, table: int) -> int:
        return sum(c.cache_size for c in self.cfgs[:table])

    def swap(self, info) -> None:
        """Swap-out then swap-in for one SwapInfo (offsets already shifted per table)."""
        dev, D = self.device, self.dim
        main = torch.cuda.current_stream(dev)
        m = self.module
        if self._pending_update is not None:  # the previous batch's host update must be in the store before lookups
            self._pending_update.get()
            self._pending_update = None
        n_out = info.swapout_offs.numel()
        if n_out:
            rows = [m.gather_embs(info.swapout_offs)] + m.gather_momentum(info.swapout_offs)
            ready = torch.cuda.Event()
            ready.record(main)
            host = [torch.empty(n_out * D, dtype=torch.float32).pin_memory() for _ in rows]
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(self.copy_stream):
                self.copy_stream.wait_event(ready)
                ev0.record(self.copy_stream)
                for h, r in zip(host, rows):
                    h.copy_(r, non_blocking=True)  # one copy per array
                    r.record_stream(self.copy_stream)
                ev1.record(self.copy_stream)
            self.swap_events.append(("swap_out_d2h", ev0, ev1))
            ev1.synchronize()
            self._pending_update = self.mgr.embedding_update_async(info, host[0], host[1:])
        n_in = info.swapin_offs.numel()
        if n_in:
            if self._pending_update is not None:  # a key swapped out and in again in one batch reads its new row
                self._pending_update.get()
                self._pending_update = None
            st = self.mgr.embedding_lookup_async(info).get()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(self.copy_stream):
                ev0.record(self.copy_stream)
                d_rows = [t.to(dev, non_blocking=True) for t in [st.swapin_embs] + list(st.swapin_optims)]
                ev1.record(self.copy_stream)
            self.swap_events.append(("swap_in_h2d", ev0, ev1))
            main.wait_event(ev1)
            for r in d_rows:
                r.record_stream(main)
            m.scatter_update_embs(info.swapin_offs, d_rows[0])
            m.scatter_update_momentum(info.swapin_offs, d_rows[1:])

    def forward(self, keys_per_table: Sequence[torch.Tensor], offsets: torch.Tensor,
                timestamps: Optional[Sequence[torch.Tensor]] = None) -> torch.Tensor:
        """offsets [T*B+1] feature-major over the concatenated keys.  Returns the autograd-tracked pooled rows."""
        slots, _ = self.lookup_slots(keys_per_table, timestamps)
        return self.module(slots, offsets)

    def flush_to_host(self) -> None:
        """Every cached row goes to the host store (what a checkpoint does first)."""
        if self._pending_update is not None:
            self._pending_update.get()
            self._pending_update = None
        self.mgr.embedding_to_host(self.module.weights_dev.data, self.module.get_momentum())


def _first_occurrence_unique(keys: torch.Tensor):
    """(unique keys in first-occurrence order, inverse) -- the order the reference hands to compute_swap_info
    (torchrec_embcache/distributed/embedding_bag.py:651-655)."""
    su, sinv = torch.unique(keys, sorted=True, return_inverse=True)
    n = keys.numel()
    first = torch.full((su.numel(),), n, dtype=torch.int64, device=keys.device)
    first.scatter_reduce_(0, sinv, torch.arange(n, device=keys.device), reduce="amin")
    order = torch.argsort(first)
    rank = torch.empty_like(order)
    rank[order] = torch.arange(order.numel(), device=keys.device)
    return su[order].contiguous(), rank[sinv].contiguous()


def _first_positions(keys: torch.Tensor) -> torch.Tensor:
    su, sinv = torch.unique(keys, sorted=True, return_inverse=True)
    n = keys.numel()
    first = torch.full((su.numel(),), n, dtype=torch.int64, device=keys.device)
    first.scatter_reduce_(0, sinv, torch.arange(n, device=keys.device), reduce="amin")
    return torch.sort(first).values
