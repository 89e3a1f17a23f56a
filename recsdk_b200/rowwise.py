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


def _a2a(out: torch.Tensor, inp: torch.Tensor, out_splits: List[int], in_splits: List[int], group) -> None:
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_to_all_single(out, inp, out_splits, in_splits, group=group)
    else:
        out.copy_(inp)


class RowWiseShardedEmbeddingBag:
    """F tables of equal dim, rows split over the ranks by ``id % W``; pooled lookups for this rank's samples."""

    def __init__(self, rows: Sequence[int], dim: int, world: int, rank: int, group: Optional[dist.ProcessGroup] = None,
                 optimizer: EmbOptimType = EmbOptimType.ADAM, pooling_mode: PoolingMode = PoolingMode.SUM,
                 device="cuda", **optimizer_kwargs):
        if pooling_mode == PoolingMode.NONE:
            raise ValueError("pooled modes only")
        self.rows, self.dim, self.world, self.rank, self.group = list(rows), int(dim), world, rank, group
        self.F = len(self.rows)
        self.pooling_mode = pooling_mode
        self.device = torch.device(device)
        self.local_rows = [max((r - rank + world - 1) // world, 1) for r in self.rows]
        # feature (source rank s, table f) -> table f: rows asked for by several ranks are merged by the backward
        ftm = [f for _ in range(world) for f in range(self.F)]
        self.owner = HybridSplitTableBatchedEmbeddingBagsCodegen(
            [(r, self.dim) for r in self.local_rows], feature_table_map=ftm, optimizer=optimizer,
            pooling_mode=PoolingMode.NONE, device=self.device, **optimizer_kwargs)
        F, D = self.F, self.dim
        self._zeros_F = torch.zeros(F, dtype=torch.int64, device=self.device)
        self._D_offsets = (torch.arange(F + 1, dtype=torch.int32, device=self.device) * D).contiguous()
        self._ctx = None

    # ------------------------------------------------------------------ forward
    def forward(self, indices: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
        """indices [N] int64 (global row ids), offsets [F*B+1] feature-major -> pooled [B, F*dim]."""
        F, D, W, dev = self.F, self.dim, self.world, self.device
        N = indices.numel()
        B = (offsets.numel() - 1) // F
        lengths = (offsets[1:] - offsets[:-1]).contiguous()
        _, uniq_buf, perm, _, num_out = ops.bucketize(lengths, indices, F, W, do_unique=True)
        # (destination, feature) group of every unique id: scatter the group of the inputs that map to it
        feat = torch.searchsorted(offsets[B::B].contiguous(), torch.arange(N, device=dev), right=True)
        grp_in = (indices % W) * F + feat
        n_u = int(num_out.item())
        grp = torch.empty(n_u, dtype=torch.int64, device=dev)
        grp[perm] = grp_in
        send_counts = torch.bincount(grp, minlength=W * F).view(W, F)
        recv_counts = torch.empty_like(send_counts)
        _a2a(recv_counts.view(-1), send_counts.view(-1).contiguous(), [F] * W, [F] * W, self.group)
        send_splits = send_counts.sum(1).tolist()
        recv_splits = recv_counts.sum(1).tolist()
        n_recv = int(sum(recv_splits))
        recv_ids = torch.empty(n_recv, dtype=torch.int64, device=dev)
        _a2a(recv_ids, uniq_buf[:n_u].contiguous(), recv_splits, send_splits, self.group)
        # owner: one row per received id; group (s, f) is feature s*F + f of the owner's module
        local = torch.div(recv_ids, W, rounding_mode="floor")
        owner_offsets = torch.zeros(W * F + 1, dtype=torch.int64, device=dev)
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
    def backward(self, grad_output: torch.Tensor) -> None:
        """grad_output [B, F*dim]: gradient of this rank's pooled rows.  Updates the owners' tables in place."""
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
            self.owner.backward_from(recv_grad, local, owner_offsets)
        else:
            self.owner.iter[0] += 1

    # ------------------------------------------------------------------ helpers
    def local_table(self, f: int) -> torch.Tensor:
        """[local_rows_f, dim] view of this rank's shard of table f: local row j is global row j*W + rank."""
        return self.owner.split_embedding_weights()[f]
