"""Row-wise sharded lookup over the GPUs of one box: row `id` of every table lives on rank ``id % W`` at local row
``id // W`` (hybrid_torchrec/src/ids_process/bucketize.cpp:44-48).

Per step (one process per GPU, `torch.distributed` all-to-alls for the exchange steps, every compute step is one
of this package's kernels):

  forward   bucketize + per-(destination, feature) first-occurrence dedup of this rank's ids (`recsdk_bucketize`)
            -> all-to-all of the unique ids -> the owner gathers one row per received id (forward kernel, NONE
            pooling; the (source rank, feature) groups are features that share the owner's table)
            -> all-to-all of the rows back -> the sample owner pools them per bag (forward kernel again, with the
            received rows as the table and the dedup positions as indices).
  backward  the sample owner sums the bag gradients per unique row it fetched (fused backward with plain SGD,
            lr = -1, on a zeroed buffer: 0 - (-1 * g) = g) -> all-to-all of those gradient rows to the owners
            -> the owner's fused backward (NONE pooling) merges the rows that several ranks asked for, in
            source-rank order, and applies the optimizer once per row.

This is the exchange pattern of the reference's row-wise path (local unique, "restore vector second" on the owner,
all2all of unique rows and of summed gradients: `ascendc_op/.../lccl/v220/op_kernel/all2all_uss.h:319-381`), built
from the table-batched kernels instead of a dedicated collective.  Sizes of the exchanges depend on the batch, so
the two split-size reads synchronise with the host, as the reference's input dist does.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from . import ops
from .tbe import EmbOptimType, HybridSplitTableBatchedEmbeddingBagsCodegen, PoolingMode


def _running(xs):
    s = 0
    for x in xs:
        s += x
        yield s


def _a2a(out: torch.Tensor, inp: torch.Tensor, out_splits: List[int], in_splits: List[int], group) -> None:
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_to_all_single(out, inp, out_splits, in_splits, group=group)
    else:
        out.copy_(inp)


class _DedupExchangeLookup:
    """Shared machinery: this rank's ids are reduced to the distinct rows it needs, grouped by owner; only those
    ids, one row per id, and one summed gradient row per id cross between GPUs.  Subclasses say who owns a row
    (`_partition`) and where the owner keeps it (`_owner_rows`); `G` is the number of groups an owner sees per
    source rank (they become features that share the owner's tables)."""

    def _init_common(self, F: int, dim: int, world: int, rank: int, group, pooling_mode, device) -> None:
        if pooling_mode == PoolingMode.NONE:
            raise ValueError("pooled modes only")
        self.F, self.dim, self.world, self.rank, self.group = F, int(dim), world, rank, group
        self.pooling_mode = pooling_mode
        self.device = torch.device(device)
        self._zeros_F = torch.zeros(F, dtype=torch.int64, device=self.device)
        self._D_offsets = (torch.arange(F + 1, dtype=torch.int32, device=self.device) * self.dim).contiguous()
        self._ctx = None

    def _feature_of_position(self, offsets: torch.Tensor, N: int, B: int) -> torch.Tensor:
        return torch.searchsorted(offsets[B::B].contiguous(), torch.arange(N, device=self.device), right=True)

    # ------------------------------------------------------------------ forward
    def forward(self, indices: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
        """indices [N] int64 (global row ids), offsets [F*B+1] feature-major -> pooled [B, F*dim]."""
        F, D, W, G, dev = self.F, self.dim, self.world, self.G, self.device
        uniq_buf, perm, send_counts = self._partition(indices, offsets)
        recv_counts = torch.empty_like(send_counts)
        _a2a(recv_counts.view(-1), send_counts.view(-1).contiguous(), [G] * W, [G] * W, self.group)
        # the one host read of the forward: how many ids go to / come from every rank
        splits = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).tolist()
        send_splits, recv_splits = [int(x) for x in splits[0]], [int(x) for x in splits[1]]
        n_u, n_recv = sum(send_splits), sum(recv_splits)
        uniq = uniq_buf[:n_u]
        recv_ids = torch.empty(n_recv, dtype=torch.int64, device=dev)
        _a2a(recv_ids, uniq, recv_splits, send_splits, self.group)
        # owner: one row per received id; group (s, g) is feature s*G + g of the owner's module
        local = self._owner_rows(recv_ids)
        owner_offsets = torch.zeros(W * G + 1, dtype=torch.int64, device=dev)
        owner_offsets[1:] = torch.cumsum(recv_counts.view(-1), 0)
        rows_out = torch.empty((n_recv, D), dtype=torch.float32, device=dev)
        if n_recv:
            self.owner.forward_into(local, owner_offsets, rows_out)
        fetched = torch.empty((n_u, D), dtype=torch.float32, device=dev)
        _a2a(fetched.view(-1), rows_out.view(-1), [s * D for s in send_splits], [r * D for r in recv_splits], self.group)
        # sample owner: pool the fetched rows per bag (the fetched rows are the table, dedup positions the indices)
        out = ops.tbe_forward(fetched.view(-1), self._zeros_F, self._D_offsets, perm, offsets, F * D, D,
                              int(self.pooling_mode), bounds_check=True)
        self._ctx = (perm, offsets, n_u, send_splits, recv_splits, local, owner_offsets, n_recv)
        return out

    # ------------------------------------------------------------------ backward + optimizer
    def backward(self, grad_output: torch.Tensor, update_events=None) -> None:
        """grad_output [B, F*dim]: gradient of this rank's pooled rows.  Updates the owners' tables in place.
        ``update_events``: passed to the owner's fused backward (events around its row-update kernel)."""
        perm, offsets, n_u, send_splits, recv_splits, local, owner_offsets, n_recv = self._ctx
        F, D, dev = self.F, self.dim, self.device
        # per fetched row: sum of the bag gradients that used it (SGD with lr = -1 on zeros yields the sum itself)
        fetched_grad = torch.zeros(max(n_u, 1) * D, dtype=torch.float32, device=dev)
        hs = torch.zeros(F + 1, dtype=torch.int64, device=dev)
        hs[F] = n_u
        ops.tbe_backward(grad_output, fetched_grad, None, None, self._zeros_F, self._D_offsets, hs, perm, offsets,
                         F * D, D, int(self.pooling_mode), ops.OPT_SGD, -1.0,
                         total_hash_size_bits=max(1, int(n_u).bit_length()), bounds_check=True)
        recv_grad = torch.empty((n_recv, D), dtype=torch.float32, device=dev)
        _a2a(recv_grad.view(-1), fetched_grad[:n_u * D], [r * D for r in recv_splits], [s * D for s in send_splits],
             self.group)
        if n_recv:
            self.owner.backward_from(recv_grad, local, owner_offsets, update_events=update_events)
        else:
            self.owner.iter[0] += 1



class RowWiseShardedEmbeddingBag(_DedupExchangeLookup):
    """F tables of equal dim, rows split over the ranks by ``id % W``; pooled lookups for this rank's samples."""

    def __init__(self, rows: Sequence[int], dim: int, world: int, rank: int, group: Optional[dist.ProcessGroup] = None,
                 optimizer: EmbOptimType = EmbOptimType.ADAM, pooling_mode: PoolingMode = PoolingMode.SUM,
                 device="cuda", **optimizer_kwargs):
        self.rows = list(rows)
        self._init_common(len(self.rows), dim, world, rank, group, pooling_mode, device)
        self.G = self.F
        self.local_rows = [max((r - rank + world - 1) // world, 1) for r in self.rows]
        # feature (source rank s, table f) -> table f: rows asked for by several ranks are merged by the backward
        ftm = [f for _ in range(world) for f in range(self.F)]
        self.owner = HybridSplitTableBatchedEmbeddingBagsCodegen(
            [(r, self.dim) for r in self.local_rows], feature_table_map=ftm, optimizer=optimizer,
            pooling_mode=PoolingMode.NONE, device=self.device, **optimizer_kwargs)

    def _partition(self, indices, offsets):
        F, W, dev = self.F, self.world, self.device
        N = indices.numel()
        B = (offsets.numel() - 1) // F
        lengths = (offsets[1:] - offsets[:-1]).contiguous()
        _, uniq_buf, perm, _, num_out = ops.bucketize(lengths, indices, F, W, do_unique=True)
        # (destination, feature) group of every unique id: scatter the group of the inputs that map to it
        grp_in = (indices % W) * F + self._feature_of_position(offsets, N, B)
        # entries of `grp` past the number of unique ids keep the sentinel and fall into the extra bin
        grp = torch.full((N,), W * F, dtype=torch.int64, device=dev)
        grp[perm] = grp_in
        return uniq_buf, perm, torch.bincount(grp, minlength=W * F + 1)[:W * F].view(W, F)

    def _owner_rows(self, recv_ids):
        return torch.div(recv_ids, self.world, rounding_mode="floor")

    def local_table(self, f: int) -> torch.Tensor:
        """[local_rows_f, dim] view of this rank's shard of table f: local row j is global row j*W + rank."""
        return self.owner.split_embedding_weights()[f]


class TableWiseDedupEmbeddingBag(_DedupExchangeLookup):
    """Whole tables on ranks (`owner[f]`), equal dim.  Instead of moving one pooled row per (sample, table) to the
    sample owners, each rank fetches the DISTINCT rows its samples need and pools locally; gradients travel back
    summed per distinct row.  With one id per field and skewed ids this cuts the bytes on the links by the
    duplicate factor of the batch (about 5x for Zipf(1.1) batches of 65536).  The owner keeps its tables as one
    flat table (equal dims), addressed by a linear row number."""

    def __init__(self, rows: Sequence[int], dim: int, owner: Sequence[int], world: int, rank: int,
                 group: Optional[dist.ProcessGroup] = None, optimizer: EmbOptimType = EmbOptimType.ADAM,
                 pooling_mode: PoolingMode = PoolingMode.SUM, device="cuda", **optimizer_kwargs):
        self.rows, self.owner_of = list(rows), list(owner)
        self._init_common(len(self.rows), dim, world, rank, group, pooling_mode, device)
        self.G = 1
        # linear row numbering: tables ordered by owner rank (then table number); rank_base[r] = first row of rank r
        order = sorted(range(self.F), key=lambda f: (self.owner_of[f], f))
        base, acc = [0] * self.F, 0
        rank_base = [0] * (world + 1)
        for f in order:
            base[f] = acc
            acc += self.rows[f]
            rank_base[self.owner_of[f] + 1] = acc
        for r in range(1, world + 1):
            rank_base[r] = max(rank_base[r], rank_base[r - 1])
        self.table_base = torch.tensor(base, dtype=torch.int64, device=self.device)
        self.rank_base = torch.tensor(rank_base, dtype=torch.int64, device=self.device)
        self._rank_base_host = rank_base
        self.key_bits = max(1, int(acc).bit_length())
        self.local_tables = [f for f in order if self.owner_of[f] == rank]
        n_local = max(rank_base[rank + 1] - rank_base[rank], 1)
        # W features (one per source rank) that share the owner's single flat table
        self.owner = HybridSplitTableBatchedEmbeddingBagsCodegen(
            [(n_local, self.dim)], feature_table_map=[0] * world, optimizer=optimizer, pooling_mode=PoolingMode.NONE,
            device=self.device, **optimizer_kwargs)

    # ------------------------------------------------------------------ peer-pull variant of the two row exchanges
    def enable_peer_pull(self, max_ids_per_table_per_rank: int) -> None:
        """Replace the all-to-alls of rows and of gradient rows by copies out of peer-mapped buffers: the owner
        gathers the requested rows into a buffer every rank can address and each requester pulls its segment
        (copy engines over NVLink); gradients travel the same way in the other direction.  Buffers are sized for
        the worst case (every id of a rank's batch distinct: ``max_ids_per_table_per_rank`` is the largest number
        of ids one rank's batch can hold for one table, the batch size for one id per bag); call once, on every
        rank, after construction."""
        from .peer import PeerMappedBuffer

        W, D = self.world, self.dim
        max_tables = max(sum(1 for o in self.owner_of if o == r) for r in range(W))
        self._rows_stage = PeerMappedBuffer((max_tables * W * max_ids_per_table_per_rank, D), self.device, self.group)
        self._grad_stage = PeerMappedBuffer((self.F * max_ids_per_table_per_rank, D), self.device, self.group)
        self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._peer_pull = True

    def _fence(self) -> None:
        dist.all_reduce(self._token, group=self.group)  # stream-ordered barrier across the ranks

    def _pull(self, dst: torch.Tensor, src_ptr: int, rows: int) -> None:
        from . import _lib
        from .ops import _stream, check

        check(_lib.load().recsdk_peer_copy(dst.data_ptr(), src_ptr, rows * self.dim * 4, _stream()), "recsdk_peer_copy")

    def forward(self, indices: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
        if not getattr(self, "_peer_pull", False):
            return super().forward(indices, offsets)
        F, D, W, dev, me = self.F, self.dim, self.world, self.device, self.rank
        uniq_buf, perm, send_counts = self._partition(indices, offsets)
        mat = torch.empty(W * W, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(mat, send_counts.view(-1).contiguous(), group=self.group)
        M = mat.view(W, W).tolist()  # M[q][r]: distinct rows rank q asks of rank r (the one host read of the forward)
        send_splits, recv_splits = [int(x) for x in M[me]], [int(M[q][me]) for q in range(W)]
        n_u, n_recv = sum(send_splits), sum(recv_splits)
        # every rank sees the whole matrix, so a buffer that is too small is an error on all ranks at once
        worst_owner = max(sum(int(M[q][r]) for q in range(W)) for r in range(W))
        worst_asker = max(sum(int(x) for x in M[q]) for q in range(W))
        if worst_owner > self._rows_stage.local.shape[0] or worst_asker > self._grad_stage.local.shape[0]:
            raise RuntimeError(f"peer-pull buffers too small: {worst_owner} rows at an owner / {worst_asker} at a "
                               f"requester, capacities {self._rows_stage.local.shape[0]} / "
                               f"{self._grad_stage.local.shape[0]}")
        recv_ids = torch.empty(n_recv, dtype=torch.int64, device=dev)
        _a2a(recv_ids, uniq_buf[:n_u], recv_splits, send_splits, self.group)
        local = self._owner_rows(recv_ids)
        owner_offsets = torch.tensor([0] + list(_running(recv_splits)), dtype=torch.int64, device=dev)
        stage = self._rows_stage.local[:max(n_recv, 1)]
        if n_recv:
            self.owner.forward_into(local, owner_offsets, stage[:n_recv])
        self._fence()  # every owner's rows are in its buffer
        fetched = torch.empty((n_u, D), dtype=torch.float32, device=dev)
        seg = 0
        for r in range(W):
            n = send_splits[r]
            if n:
                start_in_r = sum(int(M[q][r]) for q in range(me))  # rows of lower ranks come first in r's buffer
                self._pull(fetched[seg:seg + n], self._rows_stage.ptrs[r] + start_in_r * D * 4, n)
            seg += n
        out = ops.tbe_forward(fetched.view(-1), self._zeros_F, self._D_offsets, perm, offsets, F * D, D,
                              int(self.pooling_mode), bounds_check=True)
        self._ctx = (perm, offsets, n_u, send_splits, recv_splits, local, owner_offsets, n_recv, M)
        return out

    def backward(self, grad_output: torch.Tensor, update_events=None) -> None:
        if not getattr(self, "_peer_pull", False):
            return super().backward(grad_output, update_events)
        perm, offsets, n_u, send_splits, recv_splits, local, owner_offsets, n_recv, M = self._ctx
        F, D, W, dev, me = self.F, self.dim, self.world, self.device, self.rank
        fetched_grad = self._grad_stage.local.view(-1)[:max(n_u, 1) * D]
        fetched_grad.zero_()
        hs = torch.zeros(F + 1, dtype=torch.int64, device=dev)
        hs[F] = n_u
        ops.tbe_backward(grad_output, fetched_grad, None, None, self._zeros_F, self._D_offsets, hs, perm, offsets,
                         F * D, D, int(self.pooling_mode), ops.OPT_SGD, -1.0,
                         total_hash_size_bits=max(1, int(n_u).bit_length()), bounds_check=True)
        self._fence()  # every requester's per-row sums are in its buffer
        recv_grad = torch.empty((n_recv, D), dtype=torch.float32, device=dev)
        seg = 0
        for q in range(W):
            n = recv_splits[q]
            if n:
                start_in_q = sum(int(M[q][r]) for r in range(me))  # q's rows for lower owners come first in its buffer
                self._pull(recv_grad[seg:seg + n], self._grad_stage.ptrs[q] + start_in_q * D * 4, n)
            seg += n
        if n_recv:
            self.owner.backward_from(recv_grad, local, owner_offsets, update_events=update_events)
        else:
            self.owner.iter[0] += 1

    def close(self) -> None:
        if getattr(self, "_peer_pull", False):
            self._rows_stage.close()
            self._grad_stage.close()
            self._peer_pull = False

    def _partition(self, indices, offsets):
        F, dev = self.F, self.device
        N = indices.numel()
        B = (offsets.numel() - 1) // F
        if N == F * B:  # one id per bag: the feature of a position is position // B
            lin = (indices.view(F, B) + self.table_base.view(F, 1)).view(-1)
        else:
            lin = indices + self.table_base[self._feature_of_position(offsets, N, B)]
        # the unused tail of the buffer holds INT64_MAX, so the whole buffer is sorted and can be searched
        uniq_buf, inv, _ = ops.unique_sorted(lin, key_bits=self.key_bits, fill=torch.iinfo(torch.int64).max)
        # ascending linear rows are grouped by owner rank already
        bounds = torch.searchsorted(uniq_buf, self.rank_base)
        return uniq_buf, inv, (bounds[1:] - bounds[:-1]).view(self.world, 1)

    def _owner_rows(self, recv_ids):
        return recv_ids - self._rank_base_host[self.rank]

    def local_table(self, f: int) -> torch.Tensor:
        """[rows_f, dim] view of table f (which this rank must own)."""
        start = int(self.table_base[f].item()) - self._rank_base_host[self.rank]
        return self.owner.split_embedding_weights()[0][start:start + self.rows[f]]
