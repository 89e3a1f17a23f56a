"""The two sharded lookups of the path as modules: row-wise (row `id` on rank ``id % W``,
hybrid_torchrec/src/ids_process/bucketize.cpp:44-48) and table-wise with distinct-row fetch (whole tables on ranks,
hybrid_torchrec/hybrid_torchrec/distributed/sharding/hybrid_tw_sharding.py:43-82).  Both are the device-driven
dedup exchange of `recsdk_b200.exchange` with a placement chosen; with a process group (one process per GPU) the
constructor maps the peers' buffers, without one (world 1) the same kernels run on the local buffers.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch.distributed as dist

from .exchange import DedupExchange, connect_local  # noqa: F401  (re-exported for callers of this module)
from .tbe import EmbOptimType, PoolingMode


class RowWiseShardedEmbeddingBag(DedupExchange):
    """F tables of equal dim, rows split over the ranks by ``id % W``; pooled (or sequence) lookups for this rank's
    ``batch_size`` samples."""

    def __init__(self, rows: Sequence[int], dim: int, world: int, rank: int, group: Optional[dist.ProcessGroup] = None,
                 batch_size: int = 1, optimizer: EmbOptimType = EmbOptimType.ADAM,
                 pooling_mode: PoolingMode = PoolingMode.SUM, device="cuda", connect: bool = True, **kwargs):
        super().__init__(rows, dim, world, rank, partition="row", batch_size=batch_size, optimizer=optimizer,
                         pooling_mode=pooling_mode, device=device, **kwargs)
        if world > 1 and connect:
            self.connect_processes(group)


class TableWiseDedupEmbeddingBag(DedupExchange):
    """Whole tables on ranks (`owner[f]`), equal dim.  Instead of moving one pooled row per (sample, table) to the
    sample owners, each rank fetches the DISTINCT rows its samples need and pools locally; gradients travel back
    summed per distinct row.  With one id per field and skewed ids this cuts the bytes on the links by the
    duplicate factor of the batch (about 5x for Zipf(1.1) batches of 65536)."""

    def __init__(self, rows: Sequence[int], dim: int, owner: Sequence[int], world: int, rank: int,
                 group: Optional[dist.ProcessGroup] = None, batch_size: int = 1,
                 optimizer: EmbOptimType = EmbOptimType.ADAM, pooling_mode: PoolingMode = PoolingMode.SUM,
                 device="cuda", connect: bool = True, **kwargs):
        super().__init__(rows, dim, world, rank, partition="table", owner=owner, batch_size=batch_size,
                         optimizer=optimizer, pooling_mode=pooling_mode, device=device, **kwargs)
        if world > 1 and connect:
            self.connect_processes(group)
