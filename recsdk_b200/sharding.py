"""Table-wise sharding of the embedding path across the GPUs of one box.

One process per GPU.  Tables are placed whole on ranks (greedy byte balance -- the reference delegates
placement to the torchrec planner, hybrid_torchrec/hybrid_torchrec/distributed/sharding/hybrid_tw_sharding.py:43-82).
Per step there are three exchanges, all `all_to_all_single` with split sizes (NCCL on GPUs, gloo in the CPU
tests):

  ids        every rank sends, to each table owner, the ids of ITS samples for the owner's tables
             (the reference's KJT all-to-all, hybrid_tw_sharding.py:59-68) -> the owner holds [T_owner, W*B]
  outputs    the owner's pooled rows [W*B, T_owner*D] go back to the sample owners -> [B, sum_t D_t]
             (torchrec PooledEmbeddingsAllToAll in the reference, embeddingbag.py:550-593)
  gradients  the transposed exchange

The exchanges only move data; the hot path (gather, dedup, segment-sum, optimizer) runs locally on each owner,
so there is no other collective on the data path.  Everything here is device-agnostic tensor plumbing.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def greedy_table_placement(rows: Sequence[int], dims: Sequence[int], world: int,
                           loads: Optional[Sequence[float]] = None, bytes_cap: Optional[int] = None,
                           bytes_per_element: int = 12) -> List[int]:
    """Whole tables onto ranks.  Deterministic on every rank.

    Without `loads`: every table receives the same number of ids per step, so the lookup / update work of a rank is
    taken as proportional to its table COUNT while its memory is proportional to its table BYTES: biggest table
    first onto the rank with the fewest tables so far, ties to the rank with the fewest bytes.  Counts differ by at
    most one and the big tables are spread out.

    With `loads` (one number per table, e.g. the distinct rows a profile batch touches -- what the owner of a table
    serves to the other ranks and updates once per step): heaviest table first onto the rank with the least load so
    far among those where the table still fits under `bytes_cap` (weights + optimizer state, `bytes_per_element`
    bytes per element; no cap when None); a table that fits nowhere goes to the rank with the fewest bytes."""
    count = [0] * world
    load = [0] * world
    owner = [0] * len(rows)
    if loads is None:
        for t in sorted(range(len(rows)), key=lambda i: (-rows[i] * dims[i], i)):
            r = min(range(world), key=lambda k: (count[k], load[k], k))
            owner[t] = r
            count[r] += 1
            load[r] += rows[t] * dims[t]
        return owner
    if len(loads) != len(rows):
        raise ValueError("loads must have one entry per table")
    work = [0.0] * world
    for t in sorted(range(len(rows)), key=lambda i: (-float(loads[i]), -rows[i] * dims[i], i)):
        size = rows[t] * dims[t] * bytes_per_element
        fits = [k for k in range(world) if bytes_cap is None or load[k] + size <= bytes_cap]
        r = min(fits, key=lambda k: (work[k], load[k], k)) if fits else min(range(world), key=lambda k: (load[k], k))
        owner[t] = r
        work[r] += float(loads[t])
        load[r] += size
    return owner


class TableWiseSharding:
    """Exchange plan for one-id-per-field or fixed-length bags: every (table, sample) carries `L` ids."""

    def __init__(self, rows: Sequence[int], dims: Sequence[int], world: int, rank: int,
                 group: Optional[dist.ProcessGroup] = None, owner: Optional[Sequence[int]] = None):
        self.rows, self.dims = list(rows), list(dims)
        self.world, self.rank, self.group = world, rank, group
        self.owner = list(owner) if owner is not None else greedy_table_placement(rows, dims, world)
        self.tables_of = [[t for t in range(len(rows)) if self.owner[t] == r] for r in range(world)]
        self.local_tables = self.tables_of[rank]
        self.dim_of_rank = [sum(self.dims[t] for t in self.tables_of[r]) for r in range(world)]
        # column order of the assembled [B, sum D] output: by owner rank, then the owner's table order
        self.output_table_order = [t for r in range(world) for t in self.tables_of[r]]

    def _a2a(self, out: torch.Tensor, inp: torch.Tensor, out_splits: List[int], in_splits: List[int]) -> None:
        if self.world == 1:
            out.copy_(inp)
            return
        dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group)

    # ------------------------------------------------------------------ ids
    def exchange_ids(self, ids: torch.Tensor, owner_ordered: bool = False) -> torch.Tensor:
        """ids [T_total, B_local, L] (this rank's samples, every table) -> [T_local, W*B_local, L] on the owner,
        sample s*B_local + b being sample b of rank s.  owner_ordered=True: the tables of `ids` are already in
        `output_table_order` (grouped by owner), so the tensor is sent as it lies."""
        T, B, L = ids.shape
        W = self.world
        if owner_ordered or W == 1:
            send = ids.reshape(-1)
        else:
            send = torch.cat([ids[self.tables_of[r]].reshape(-1) for r in range(W)])
        in_splits = [len(self.tables_of[r]) * B * L for r in range(W)]
        Tl = len(self.local_tables)
        out_splits = [Tl * B * L] * W
        recv = torch.empty(W * Tl * B * L, dtype=ids.dtype, device=ids.device)
        self._a2a(recv, send, out_splits, in_splits)
        return recv.view(W, Tl, B, L).permute(1, 0, 2, 3).reshape(Tl, W * B, L).contiguous()

    # ------------------------------------------------------------------ pooled outputs
    def exchange_outputs(self, pooled: torch.Tensor, B_local: int, assemble: bool = True):
        """pooled [W*B_local, D_local] on the owner -> [B_local, sum_r D_r] on the sample owner
        (columns ordered as `output_table_order`).  With assemble=False the result stays blocked by owner rank
        (a list of [B_local, D_r] views of one receive buffer) and no second copy is made."""
        W = self.world
        Dl = self.dim_of_rank[self.rank]
        assert pooled.shape == (W * B_local, Dl)
        in_splits = [B_local * Dl] * W
        out_splits = [B_local * self.dim_of_rank[r] for r in range(W)]
        recv = torch.empty(sum(out_splits), dtype=pooled.dtype, device=pooled.device)
        self._a2a(recv, pooled.reshape(-1), out_splits, in_splits)
        parts, o = [], 0
        for r in range(W):
            parts.append(recv[o:o + out_splits[r]].view(B_local, self.dim_of_rank[r]))
            o += out_splits[r]
        if not assemble:
            return parts
        return torch.cat(parts, dim=1) if W > 1 else parts[0]

    # ------------------------------------------------------------------ gradients
    def blocked_gradient_buffer(self, B_local: int, device, dtype=torch.float32) -> torch.Tensor:
        """Flat buffer holding the upstream gradient blocked by owner rank: [B_local, D_0] | [B_local, D_1] | ..."""
        return torch.empty(B_local * sum(self.dim_of_rank), dtype=dtype, device=device)

    def exchange_gradients(self, grad: torch.Tensor, blocked: bool = False) -> torch.Tensor:
        """grad [B_local, sum_r D_r] (columns as `output_table_order`) -> [W*B_local, D_local] on the owner.
        blocked=True: `grad` is already the flat owner-blocked buffer (see blocked_gradient_buffer), sent as is."""
        W = self.world
        Dl = self.dim_of_rank[self.rank]
        if blocked:
            B = grad.numel() // sum(self.dim_of_rank)
            send = grad
        else:
            B = grad.shape[0]
            cols, o = [], 0
            for r in range(W):
                cols.append(grad[:, o:o + self.dim_of_rank[r]].reshape(-1))
                o += self.dim_of_rank[r]
            send = torch.cat(cols) if W > 1 else cols[0]
        in_splits = [B * self.dim_of_rank[r] for r in range(W)]
        out_splits = [B * Dl] * W
        recv = torch.empty(W * B * Dl, dtype=grad.dtype, device=grad.device)
        self._a2a(recv, send, out_splits, in_splits)
        return recv.view(W * B, Dl)
