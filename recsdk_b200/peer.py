"""Peer-mapped sample-sharded buffers: the in-kernel replacement for the two pooled-row all-to-alls.

With table-wise sharding the reference pools on the table owner and then moves the pooled rows to the sample
owners with torchrec's PooledEmbeddingsAllToAll (hybrid_torchrec/hybrid_torchrec/distributed/embeddingbag.py:550-593;
sharding in distributed/sharding/hybrid_tw_sharding.py:43-82), and the gradients back the same way.  On one
NVSwitch box every GPU can address every other GPU's memory, so here each rank keeps ONE buffer with the pooled
rows of its own samples ([B_local, sum_t D_t]) and one with their gradients; the owners' forward kernels store
into the peers' buffers directly and their backward kernels read gradient rows from them directly.

The mappings are made once with CUDA IPC handles exchanged over the process group's store; the kernels use plain
loads and stores on them (no multicast objects).  Ordering between ranks is by stream-ordered collectives on tiny
tensors (`fence`), never by kernels spinning on each other.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from . import _lib
from .ops import SampleShards, check


class PeerMappedBuffer:
    """A float32 buffer of identical shape on every rank, addressable from every rank.

    ``local`` is this rank's tensor; ``ptrs[r]`` is the address of rank r's buffer in THIS process.
    """

    def __init__(self, shape, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.local = torch.zeros(shape, dtype=torch.float32, device=device)
        lib = _lib.load()
        handle = (C.c_ubyte * 64)()
        offset = C.c_int64(0)
        check(lib.recsdk_peer_export(self.local.data_ptr(), handle, C.byref(offset)), "recsdk_peer_export")
        mine = (bytes(handle), int(offset.value))
        gathered: List = [None] * self.world
        dist.all_gather_object(gathered, mine, group=group)
        self._imported = []
        self.ptrs: List[int] = []
        for r, (h, off) in enumerate(gathered):
            if r == self.rank:
                self.ptrs.append(self.local.data_ptr())
                continue
            out = C.c_void_p()
            buf = (C.c_ubyte * 64).from_buffer_copy(h)
            check(lib.recsdk_peer_import(buf, off, C.byref(out)), "recsdk_peer_import")
            self._imported.append((out.value, off))
            self.ptrs.append(out.value)

    def close(self) -> None:
        """Unmap the peers' buffers.  Call on every rank after the last kernel that uses them has finished and
        before the owning tensors are freed."""
        lib = _lib.load()
        torch.cuda.synchronize()
        for ptr, off in self._imported:
            check(lib.recsdk_peer_release(ptr, off), "recsdk_peer_release")
        self._imported = []


class FusedTableWiseExchange:
    """Sample-sharded pooled-output and gradient buffers for a table-wise sharded lookup.

    Column layout of a rank's buffer: tables in `TableWiseSharding.output_table_order` (grouped by owner rank),
    so `pooled.local` is directly the [B_local, sum_t D_t] input of the dense part.
    """

    def __init__(self, sharding, B_local: int, device: torch.device):
        self.sh = sharding
        self.B_local = B_local
        dims = sharding.dims
        total = sum(dims)
        col_of_table = {}
        o = 0
        for t in sharding.output_table_order:
            col_of_table[t] = o
            o += dims[t]
        self.row_stride = total
        self.col_offsets = torch.tensor([col_of_table[t] for t in sharding.local_tables], dtype=torch.int32, device=device)
        self.pooled = PeerMappedBuffer((B_local, total), device, sharding.group)
        self.grads = PeerMappedBuffer((B_local, total), device, sharding.group)
        self.out_shards = SampleShards(self.pooled.ptrs, B_local, total, self.col_offsets)
        self.grad_shards = SampleShards(self.grads.ptrs, B_local, total, self.col_offsets)
        self._token = torch.zeros(1, dtype=torch.float32, device=device)

    def fence(self) -> None:
        """Stream-ordered barrier across the ranks: work enqueued on this stream after the call starts only after
        every rank's work enqueued before its own call has finished (a one-element all-reduce)."""
        dist.all_reduce(self._token, group=self.sh.group)

    def close(self) -> None:
        self.pooled.close()
        self.grads.close()
